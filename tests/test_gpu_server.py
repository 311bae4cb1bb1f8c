"""The serving path end to end on one GPU: plugins loaded by path, requests launched with pinned
host slots, kernels released one at a time by the scheduler from ring notifications, results read
back from the slots and compared with the oracle."""
import ctypes as C
import os
import time

import numpy as np
import pytest

from oracle import graph as og
from paella_b200 import capi, packer

pytestmark = pytest.mark.gpu


def _server(models_dir, monkeypatch, sched=b"full3", streams=64):
    monkeypatch.setenv("LLIS_MODELS_DIR", models_dir)
    L = capi.load()
    cfg = capi.ServerConfig()
    L.pb_server_config_default(C.byref(cfg))
    cfg.num_streams = streams
    cfg.scheduler = sched
    s = C.c_void_p()
    capi.check(L.pb_server_create(C.byref(cfg), C.byref(s)), "pb_server_create")
    return L, s


def _pinned(nbytes):
    import torch
    return torch.zeros(nbytes, dtype=torch.uint8).pin_memory()


def _run_until(L, s, n, timeout=60.0):
    done = {}
    cookies, errs = (C.c_uint64 * 64)(), (C.c_int32 * 64)()
    t0 = time.time()
    while len(done) < n and time.time() - t0 < timeout:
        assert L.pb_server_step(s, 256) >= 0, L.pb_last_error()
        k = L.pb_server_poll_done(s, cookies, errs, 64)
        for i in range(k):
            done[cookies[i]] = errs[i]
    return done


@pytest.mark.parametrize("sched", [b"full3", b"fifo2", b"fifo"])
def test_mnist_requests_through_the_server(models_dir, monkeypatch, sched):
    monkeypatch.setenv("PB_PRECISION", "0")
    L, s = _server(models_dir, monkeypatch, sched)
    jid = C.c_uint32()
    capi.check(L.pb_server_register_job(s, capi.plugin_path("tvm_mnist").encode(), C.byref(jid)), "register")
    ib, ob, sb = C.c_size_t(), C.c_size_t(), C.c_size_t()
    L.pb_server_job_io_bytes(s, jid, C.byref(ib), C.byref(ob), C.byref(sb))
    assert (ib.value, ob.value, sb.value) == (3136, 40, 3176)
    n = 24
    slots = _pinned(sb.value * n)
    base = slots.data_ptr()
    host = slots.numpy()
    xs = []
    for i in range(n):
        x = np.random.default_rng(100 + i).random((1, 28, 28), dtype=np.float32)
        xs.append(x)
        host[i * sb.value: i * sb.value + 3136] = np.frombuffer(x.tobytes(), np.uint8)
    for rnd in range(2):          # second round reuses pooled instances (reset_internal + init)
        for i in range(n):
            capi.check(L.pb_server_launch(s, jid, base + i * sb.value, 1000 * rnd + i), "launch")
        done = _run_until(L, s, n)
        assert len(done) == n and all(e == 0 for e in done.values())
        pack = og.Pack(packer.mnist_cnn(seed=1234).to_bytes())
        for i in range(n):
            y = np.frombuffer(host[i * sb.value + 3136: i * sb.value + 3176].tobytes(), np.float32)
            ref = og.run(pack, xs[i])
            assert float(np.abs(y - ref).max()) <= 1e-5 * float(np.abs(ref).max())
    assert L.pb_server_jobs_in_flight(s) == 0
    L.pb_server_destroy(s)


def test_mixed_models_and_synthetic_jobs(models_dir, monkeypatch):
    monkeypatch.delenv("PB_PRECISION", raising=False)
    monkeypatch.setenv("PB_VEC_ADD_N", str(1 << 20))
    L, s = _server(models_dir, monkeypatch)
    ids = {}
    for job in ["tvm_mnist", "tvm_resnet18", "vec_add", "dummy_short"]:
        j = C.c_uint32()
        capi.check(L.pb_server_register_job(s, capi.plugin_path(job).encode(), C.byref(j)), "register " + job)
        ids[job] = j.value
    sizes = {}
    for job, j in ids.items():
        ib, ob, sb = C.c_size_t(), C.c_size_t(), C.c_size_t()
        L.pb_server_job_io_bytes(s, j, C.byref(ib), C.byref(ob), C.byref(sb))
        sizes[job] = (ib.value, ob.value, sb.value)
    plan = [("tvm_resnet18", 3), ("tvm_mnist", 10), ("vec_add", 3), ("dummy_short", 4)]
    bufs, cookie, meta = [], 0, {}
    for job, cnt in plan:
        ib, ob, sb = sizes[job]
        for k in range(cnt):
            t = _pinned(sb)
            h = t.numpy()
            rng = np.random.default_rng(cookie)
            if job == "tvm_resnet18":
                x = rng.standard_normal((3, 224, 224), dtype=np.float32)
            elif job == "tvm_mnist":
                x = rng.random((1, 28, 28), dtype=np.float32)
            else:
                x = rng.uniform(-1, 1, ib // 4 if ib >= 4 else 1).astype(np.float32)
            nb = min(ib, x.nbytes)
            h[:nb] = np.frombuffer(x.tobytes(), np.uint8)[:nb]
            bufs.append(t)
            meta[cookie] = (job, x, t)
            capi.check(L.pb_server_launch(s, ids[job], t.data_ptr(), cookie), "launch")
            cookie += 1
    done = _run_until(L, s, cookie, 120.0)
    assert len(done) == cookie and all(e == 0 for e in done.values()), done
    r18 = og.Pack(packer.resnet18(seed=1234).to_bytes())
    mn = og.Pack(packer.mnist_cnn(seed=1234).to_bytes())
    for ck, (job, x, t) in meta.items():
        ib, ob, sb = sizes[job]
        off = (ib + 7) // 8 * 8
        if job == "tvm_resnet18":
            y = np.frombuffer(t.numpy()[off: off + ob].tobytes(), np.float32)
            ref = og.run(r18, x)
            assert float(np.abs(y - ref).max()) <= 1e-2 * float(np.abs(ref).max())
            assert int(y.argmax()) == int(ref.argmax())
        elif job == "tvm_mnist":
            y = np.frombuffer(t.numpy()[off: off + ob].tobytes(), np.float32)
            ref = og.run(mn, x)
            # the pack's own precision hint is fp32 for MNIST
            assert float(np.abs(y - ref).max()) <= 1e-5 * float(np.abs(ref).max())
    L.pb_server_destroy(s)


def test_loadgen_open_and_closed_loop(models_dir, monkeypatch):
    monkeypatch.setenv("LLIS_MODELS_DIR", models_dir)
    L = capi.load()
    cfg = capi.LoadgenConfig()
    L.pb_loadgen_config_default(C.byref(cfg))
    cfg.num_gpus = 1
    cfg.num_types = 2
    cfg.plugin_paths[0] = capi.plugin_path("tvm_mnist").encode()
    cfg.plugin_paths[1] = capi.plugin_path("tvm_resnet18").encode()
    cfg.proportions[0], cfg.proportions[1] = 0.9, 0.1
    cfg.max_outstanding[0], cfg.max_outstanding[1] = 16, 4
    cfg.concurrency = 16
    cfg.num_jobs, cfg.warmup_jobs = 300, 50
    cfg.server.num_streams = 64
    res = capi.LoadgenResult()
    capi.check(L.pb_loadgen_run(C.byref(cfg), C.byref(res)), "closed loop")
    assert res.errors == 0 and res.all.count == 300
    assert res.per_type[0].count + res.per_type[1].count == 300 and res.per_type[1].count > 5
    assert res.throughput_rps > 100 and res.all.p99_us >= res.all.p50_us > 0
    assert res.h2d_bytes == res.per_type[0].count * 3136 + res.per_type[1].count * 602112
    cfg.mean_interarrival_us = 500.0      # open loop, Poisson, 2000 req/s
    res2 = capi.LoadgenResult()
    capi.check(L.pb_loadgen_run(C.byref(cfg), C.byref(res2)), "open loop")
    assert res2.errors == 0 and res2.all.count == 300
    assert 1000 < res2.throughput_rps < 3000
    cfg.device_resident = 1
    res3 = capi.LoadgenResult()
    capi.check(L.pb_loadgen_run(C.byref(cfg), C.byref(res3)), "device resident")
    assert res3.errors == 0 and res3.h2d_bytes == 0 and res3.d2h_bytes == 0


def test_reference_protocol_copy_stages_one_kernel_per_stage(tmp_path, monkeypatch):
    """PB_COPY_STAGES=1 + PB_STAGE_GROUP=1: H2D copy stage, one scheduler stage per kernel, D2H copy
    stage - the reference adapters' protocol - gives the same logits."""
    from paella_b200 import packer as pk
    d = tmp_path / "models_ref_protocol"      # own directory: plugins cache loaded models by path
    d.mkdir()
    pk.write_all(str(d), ["mnist", "resnet18"])
    monkeypatch.setenv("PB_COPY_STAGES", "1")
    monkeypatch.setenv("PB_STAGE_GROUP", "1")
    monkeypatch.setenv("PB_FUSE_MNIST", "0")
    L, s = _server(str(d), monkeypatch)
    ids = {}
    for job in ["tvm_mnist", "tvm_resnet18"]:
        j = C.c_uint32()
        capi.check(L.pb_server_register_job(s, capi.plugin_path(job).encode(), C.byref(j)), "register")
        ids[job] = j.value
    bufs = {}
    for job, shape, nout in (("tvm_mnist", (1, 28, 28), 10), ("tvm_resnet18", (3, 224, 224), 1000)):
        x = np.random.default_rng(77).standard_normal(shape).astype(np.float32)
        nb = x.nbytes
        t = _pinned((nb + 7) // 8 * 8 + nout * 4 + 8)
        t.numpy()[:nb] = np.frombuffer(x.tobytes(), np.uint8)
        bufs[job] = (x, t, (nb + 7) // 8 * 8, nout)
        capi.check(L.pb_server_launch(s, ids[job], t.data_ptr(), ids[job]), "launch")
    done = _run_until(L, s, 2, 120.0)
    assert len(done) == 2 and all(e == 0 for e in done.values())
    assert L.pb_server_num_decisions(s) == (6 + 2) + (24 + 2)      # kernels + two copy stages, per request
    for job, pack in (("tvm_mnist", pk.mnist_cnn(seed=1234)), ("tvm_resnet18", pk.resnet18(seed=1234))):
        x, t, off, nout = bufs[job]
        y = np.frombuffer(t.numpy()[off: off + 4 * nout].tobytes(), np.float32)
        ref = og.run(og.Pack(pack.to_bytes()), x)
        assert float(np.abs(y - ref).max()) <= 1e-2 * float(np.abs(ref).max())
        assert int(y.argmax()) == int(ref.argmax())
    L.pb_server_destroy(s)


def test_headline_mix_inception_v3_and_mnist_concurrently(models_dir, monkeypatch):
    """The benchmark's workload with its outputs checked: 16 Inception-v3 (299x299) and 48 MNIST requests in
    flight together through the server, host-buffer mode (the 1 MB inputs go through the copy engine, the
    results are written into the pinned slots), every slot with its own seeded input, two rounds so pooled
    instances are reused.  Every slot's logits are compared with the oracle: <= 1e-2 of the largest |logit|
    and the same argmax for the bf16 tensor-core path, 1e-5 for fp32 MNIST.  A race between instances
    (shared scratch, launch slots, grouped-launch tables) would show up as a wrong slot."""
    monkeypatch.delenv("PB_PRECISION", raising=False)
    L, s = _server(models_dir, monkeypatch, streams=128)
    ids, sizes = {}, {}
    for job in ["tvm_mnist", "tvm_inception_v3"]:
        j = C.c_uint32()
        capi.check(L.pb_server_register_job(s, capi.plugin_path(job).encode(), C.byref(j)), "register " + job)
        ids[job] = j.value
        ib, ob, sb = C.c_size_t(), C.c_size_t(), C.c_size_t()
        L.pb_server_job_io_bytes(s, j, C.byref(ib), C.byref(ob), C.byref(sb))
        sizes[job] = (ib.value, ob.value, sb.value)
    assert sizes["tvm_inception_v3"][0] == 3 * 299 * 299 * 4
    n_inc, n_mn = 16, 48
    reqs = []                      # (job, x, pinned tensor)
    for i in range(n_inc + n_mn):
        # interleaved: three MNIST requests after every Inception request
        job = "tvm_inception_v3" if i % 4 == 0 else "tvm_mnist"
        rng = np.random.default_rng(5000 + i)
        # every Inception input at its own amplitude: with random weights the logits of two N(0,1) images differ by
        # only 1.5 % of the largest logit, too close to the tolerance to tell one slot's result from another's
        x = (rng.standard_normal((3, 299, 299), dtype=np.float32) * np.float32(0.5 + 0.1 * (i // 4))
             if job == "tvm_inception_v3" else rng.random((1, 28, 28), dtype=np.float32))
        t = _pinned(sizes[job][2])
        t.numpy()[:x.nbytes] = np.frombuffer(x.tobytes(), np.uint8)
        reqs.append((job, x, t))
    inc = og.Pack(packer.inception_v3(seed=1234).to_bytes())
    mn = og.Pack(packer.mnist_cnn(seed=1234).to_bytes())
    refs = [og.run(inc if job == "tvm_inception_v3" else mn, x) for job, x, _ in reqs]
    worst = 0.0
    for rnd in range(2):
        for job, x, t in reqs:      # outputs of the previous round must not survive by accident
            ib, ob, sb = sizes[job]
            t.numpy()[(ib + 7) // 8 * 8:] = 0
        for i, (job, x, t) in enumerate(reqs):
            capi.check(L.pb_server_launch(s, ids[job], t.data_ptr(), 1000 * rnd + i), "launch")
        done = _run_until(L, s, len(reqs), 120.0)
        assert len(done) == len(reqs) and all(e == 0 for e in done.values()), done
        flag = C.c_uint32(0)
        capi.check(L.pb_device_error_flag(0, C.byref(flag), 1), "pb_device_error_flag")
        assert flag.value == 0
        for (job, x, t), ref in zip(reqs, refs):
            ib, ob, sb = sizes[job]
            off = (ib + 7) // 8 * 8
            y = np.frombuffer(t.numpy()[off: off + ob].tobytes(), np.float32)
            rel = float(np.abs(y - ref).max() / np.abs(ref).max())
            if job == "tvm_inception_v3":
                worst = max(worst, rel)
                assert rel <= 1e-2, (rnd, rel)
                assert int(y.argmax()) == int(ref.argmax())
            else:
                assert rel <= 1e-5, (rnd, rel)
    assert L.pb_server_jobs_in_flight(s) == 0
    L.pb_server_destroy(s)
