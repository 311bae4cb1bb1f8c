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


@pytest.fixture()
def server(models_dir):
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
    yield name, p
    if p.poll() is None:
        p.terminate()
        p.wait(10)
    for f in os.listdir("/dev/shm"):
        if f.startswith("llis:") and f.endswith(name) or f":{name}:" in f:
            try:
                os.unlink(os.path.join("/dev/shm", f))
            except OSError:
                pass


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
