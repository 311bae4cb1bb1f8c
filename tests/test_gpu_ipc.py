"""Process boundary end to end: a llis_server process on the GPU, requests through the client library
(shared-memory rings, request pool in POSIX shm registered with CUDA by the server), results compared
with the oracle; and the llis_app_client load generator against the same server."""
import ctypes as C
import os
import subprocess
import time

import numpy as np
import pytest

from oracle import graph as og
from paella_b200 import capi, packer

pytestmark = pytest.mark.gpu
BIN = os.path.join(os.path.dirname(capi.LIB_PATH), "bin")


_SERVERS = [0]


def _start_server(models_dir):
    _SERVERS[0] += 1
    name = f"pbsrv{os.getpid()}n{_SERVERS[0]}"      # a fresh name per server: a killed server leaves its rings in /dev/shm
    env = dict(os.environ, LLIS_MODELS_DIR=models_dir, CUDA_DEVICE_MAX_CONNECTIONS="32")
    p = subprocess.Popen([os.path.join(BIN, "llis_server"), "--name", name, "--sched", "full3", "--num_streams", "64", "--gpu", "0"],
                         env=env, stderr=subprocess.PIPE, text=True)
    deadline = time.time() + 60
    while not os.path.exists(f"/dev/shm/llis:channel:c2s:{name}"):
        assert p.poll() is None, p.stderr.read()
        assert time.time() < deadline, "llis_server did not come up"
        time.sleep(0.05)
    return name, p


def _stop_server(name, p):
    if p.poll() is None:
        p.terminate()
        p.wait(10)
    for f in os.listdir("/dev/shm"):
        if f.startswith("llis:") and f.endswith(name) or f":{name}:" in f:
            try:
                os.unlink(os.path.join("/dev/shm", f))
            except OSError:
                pass


@pytest.fixture()
def server(models_dir):
    name, p = _start_server(models_dir)
    yield name, p
    _stop_server(name, p)


def test_a_launch_that_fails_is_answered_and_the_server_lives_on(tmp_path):
    """The models directory holds the MNIST pack only.  A ResNet-18 request cannot be initialised (its pack is
    missing): the client's wait() must return for it at once instead of blocking for ever, the server must stay up,
    and MNIST requests sent before and after it are served correctly."""
    packer.mnist_cnn(seed=1234).save(str(tmp_path / packer.pack_file_name("mnist")))
    name, proc = _start_server(str(tmp_path))
    try:
        L = capi.load()
        client = C.c_void_p()
        capi.check(L.pb_client_connect(name.encode(), C.byref(client)), "pb_client_connect")
        inst = {}
        for plugin in ("tvm_mnist", "tvm_resnet18"):
            j, ib, ob = C.c_uint32(), C.c_size_t(), C.c_size_t()
            capi.check(L.pb_client_register_job(client, capi.plugin_path(plugin).encode(), C.byref(j), C.byref(ib), C.byref(ob)), "register_job")
            i, pin, pout = C.c_uint64(), C.c_void_p(), C.c_void_p()
            capi.check(L.pb_client_create_instance(client, j.value, C.byref(i), C.byref(pin), C.byref(pout)), "create_instance")
            inst[plugin] = (i.value, pin.value, pout.value, ob.value)
        x = np.random.default_rng(3).random((1, 28, 28), dtype=np.float32)
        ref = og.run(og.Pack(packer.mnist_cnn(seed=1234).to_bytes()), x)
        C.memmove(inst["tvm_mnist"][1], x.ctypes.data, x.nbytes)
        got = C.c_uint64()
        for plugin in ("tvm_mnist", "tvm_resnet18", "tvm_resnet18", "tvm_mnist"):
            if plugin == "tvm_mnist":
                C.memset(inst[plugin][2], 0, inst[plugin][3])
            capi.check(L.pb_client_launch(client, inst[plugin][0]), "launch")
            deadline = time.time() + 30
            rc = 0
            while rc != 1 and time.time() < deadline:
                assert proc.poll() is None, proc.stderr.read()
                rc = L.pb_client_wait(client, 100, C.byref(got))
            assert rc == 1 and got.value == inst[plugin][0], f"no answer for the {plugin} request"
            if plugin == "tvm_mnist":
                y = np.frombuffer((C.c_char * inst[plugin][3]).from_address(inst[plugin][2]), np.float32).copy()
                assert float(np.abs(y - ref).max()) <= 1e-5 * float(np.abs(ref).max())
        capi.check(L.pb_client_kill_server(client), "kill_server")
        assert proc.wait(30) == 0
        L.pb_client_close(client)
    finally:
        _stop_server(name, proc)


def test_requests_through_a_server_process(server):
    name, proc = server
    L = capi.load()
    client = C.c_void_p()
    capi.check(L.pb_client_connect(name.encode(), C.byref(client)), "pb_client_connect")
    jobs = {}
    for plugin, shape in (("tvm_mnist", (1, 28, 28)), ("tvm_resnet18", (3, 224, 224))):
        j, ib, ob = C.c_uint32(), C.c_size_t(), C.c_size_t()
        capi.check(L.pb_client_register_job(client, capi.plugin_path(plugin).encode(), C.byref(j), C.byref(ib), C.byref(ob)), "register_job")
        jobs[plugin] = (j.value, shape, ib.value, ob.value)
    packs = {"tvm_mnist": og.Pack(packer.mnist_cnn(seed=1234).to_bytes()), "tvm_resnet18": og.Pack(packer.resnet18(seed=1234).to_bytes())}
    pending = {}
    for plugin, count in (("tvm_mnist", 12), ("tvm_resnet18", 3)):
        j, shape, ib, ob = jobs[plugin]
        for k in range(count):
            inst, pin, pout = C.c_uint64(), C.c_void_p(), C.c_void_p()
            capi.check(L.pb_client_create_instance(client, j, C.byref(inst), C.byref(pin), C.byref(pout)), "create_instance")
            rng = np.random.default_rng(1000 + len(pending))
            x = rng.random(shape, dtype=np.float32) if plugin == "tvm_mnist" else rng.standard_normal(shape, dtype=np.float32)
            C.memmove(pin.value, x.ctypes.data, x.nbytes)
            pending[inst.value] = (plugin, x, pout.value, ob)
    for rnd in range(2):                       # the second round reuses the server's pooled job instances
        for inst in pending:
            capi.check(L.pb_client_launch(client, inst), "launch")
        done = set()
        got = C.c_uint64()
        deadline = time.time() + 120
        while len(done) < len(pending) and time.time() < deadline:
            assert proc.poll() is None, proc.stderr.read()
            if L.pb_client_wait(client, 100, C.byref(got)) == 1:
                done.add(got.value)
        assert done == set(pending)
        for inst, (plugin, x, pout, ob) in pending.items():
            y = np.frombuffer((C.c_char * ob).from_address(pout), np.float32).copy()
            ref = og.run(packs[plugin], x)
            tol = 1e-5 if plugin == "tvm_mnist" else 1e-2
            assert float(np.abs(y - ref).max()) <= tol * float(np.abs(ref).max())
            assert int(y.argmax()) == int(ref.argmax())
    capi.check(L.pb_client_kill_server(client), "kill_server")
    assert proc.wait(30) == 0
    L.pb_client_close(client)


def test_app_client_load_generator(server, tmp_path):
    name, proc = server
    prefix = str(tmp_path / "run")
    out = subprocess.run([os.path.join(BIN, "llis_app_client"), "--server_name", name, "--iat", "200", "--concurrency", "32", "--num_jobs", "2000",
                          "--start_record_num", "200", "--seed", "1", "--prefix", prefix,
                          capi.plugin_path("tvm_mnist"), "0.9", "16", capi.plugin_path("tvm_resnet18"), "0.1", "4"],
                         capture_output=True, text=True, timeout=300, env=dict(os.environ))
    assert out.returncode == 0, out.stderr
    fields = open(prefix + ".txt").read().strip().split(",")
    assert len(fields) == 3 + 7 * 3                   # iat, jobs, elapsed + 7 stats overall and per model
    assert float(fields[0]) == 200.0 and int(fields[1]) == 2000
    thr = 2000 / (float(fields[2]) * 1e-6)
    assert 3000 < thr < 5500                          # open loop at 5000 req/s
    assert 0 < float(fields[4]) < 5000                # overall p50 latency (us)


def test_bursts_and_a_second_client_on_the_same_server(server, tmp_path):
    """More completions in flight than the client's datagram queue holds (the wake-ups must queue in the
    server, not block it), then a second client process after the first has exited."""
    name, proc = server
    for run, (iat, conc) in enumerate([("25", "48"), ("25", "48")]):
        prefix = str(tmp_path / f"burst{run}")
        out = subprocess.run([os.path.join(BIN, "llis_app_client"), "--server_name", name, "--iat", iat, "--concurrency", conc,
                              "--num_jobs", "6000", "--start_record_num", "500", "--seed", str(run + 1), "--prefix", prefix,
                              capi.plugin_path("tvm_mnist"), "0.9", "40", capi.plugin_path("tvm_resnet18"), "0.1", "8"],
                             capture_output=True, text=True, timeout=120, env=dict(os.environ))
        assert out.returncode == 0, out.stderr
        assert proc.poll() is None, "the server must survive a client that left"
        fields = open(prefix + ".txt").read().strip().split(",")
        assert int(fields[1]) == 6000
        assert 6000 / (float(fields[2]) * 1e-6) > 15000          # offered 40k req/s
