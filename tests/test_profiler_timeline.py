"""The job-event timeline: the overhead-stack rules on a hand-made timeline (CPU), the PROFILER_CMD wire
messages against a played server (CPU), and a recorded timeline of real requests (GPU)."""
import ctypes as C
import os
import struct
import threading

import numpy as np
import pytest

from paella_b200 import capi, overhead_stack as ost


def test_overhead_stack_rules(tmp_path):
    # one job with two stages (codes of include/llis/server/profiler.h:15-23 of the reference)
    ev = [(0, 100.0), (1, 110.0), (3, 111.0), (4, 114.0), (5, 150.0), (1, 152.0), (3, 153.5), (4, 155.5), (5, 200.0), (6, 201.0)]
    r = ost.job_stack(ev, send_time=90.0)
    assert r["ipc_latency"] == 10.0 and r["queueing_delay"] == 10.0
    assert r["scheduling_overhead"] == pytest.approx(1.0 + 1.5)
    assert r["kernel_launch_overhead"] == pytest.approx(3.0 + 2.0)
    assert r["kernel_runtime"] == pytest.approx(36.0 + 44.5)
    assert r["kernel_interval"] == pytest.approx(3.5)          # finish of stage 0 -> submit of stage 1
    assert r["total"] == 101.0 and r["stages"] == 2
    p = tmp_path / "x_job_events.txt"
    p.write_text(" ".join(f"{e} {t:f}" for e, t in ev) + " \n" + "0 5.0 1 6.0 3 6.5 4 7.0 5 9.0 6 9.5 \n")
    jobs = ost.read_job_events(str(p))
    assert len(jobs) == 2 and jobs[1][-1] == (6, 9.5)
    s = ost.overhead_stack(jobs)
    assert s["jobs"] == 2 and s["stages_per_job"] == 1.5
    assert s["kernel_runtime"] == pytest.approx((80.5 + 2.0) / 2)
    assert ost.overhead_stack(jobs, stages=1)["jobs"] == 1


def test_profiler_cmd_wire_messages():
    """PROFILER_CMD {u32 6} + sub-command {u32}; SAVE {u32 12} is followed by the path as {size_t n, bytes}
    (src/client/profiler_client.cpp of the reference)."""
    from tests.test_ipc import _open, _read, _uniq, _write      # the played-server helpers
    L = capi.load()
    server = _uniq("prf")
    c2s = _open("c2s:" + server, 1024)
    client = C.c_void_p()
    res = {}
    t = threading.Thread(target=lambda: res.setdefault("rc", L.pb_client_connect(server.encode(), C.byref(client))))
    t.start()
    msg, tmp_id = struct.unpack("<II", _read(c2s, 8))
    tmp = _open(f"s2c:{server}:{tmp_id}")
    s2c = _open(f"s2c:{server}:0", 4096)
    _write(tmp, struct.pack("<I", 0))
    t.join(30)
    assert res["rc"] == 0
    capi.check(L.pb_client_profiler_cmd(client, 8, None), "SET_RECORD_JOB_EVENTS")
    assert struct.unpack("<II", _read(c2s, 8)) == (6, 8)
    capi.check(L.pb_client_profiler_cmd(client, 12, b"/tmp/some_prefix"), "SAVE")
    assert struct.unpack("<II", _read(c2s, 8)) == (6, 12)
    n = struct.unpack("<Q", _read(c2s, 8))[0]
    assert _read(c2s, n) == b"/tmp/some_prefix"
    assert L.pb_client_profiler_cmd(client, 12, None) != 0       # SAVE without a path is refused locally
    assert L.pb_client_profiler_cmd(client, 13, None) != 0
    L.pb_client_close(client)
    for h in (tmp, s2c, c2s):
        L.pb_shm_channel_close(h)


@pytest.mark.gpu
def test_recorded_timeline_of_real_requests(models_dir, tmp_path, monkeypatch):
    import ctypes
    monkeypatch.setenv("LLIS_MODELS_DIR", models_dir)
    L = capi.load()
    cfg = capi.ServerConfig()
    L.pb_server_config_default(C.byref(cfg))
    cfg.extra_kernels = 8
    srv = C.c_void_p()
    capi.check(L.pb_server_create(C.byref(cfg), C.byref(srv)), "pb_server_create")
    ids = {}
    for job in ("tvm_mnist", "tvm_resnet18"):
        jid = C.c_uint32()
        capi.check(L.pb_server_register_job(srv, capi.plugin_path(job).encode(), C.byref(jid)), "register")
        ids[job] = jid.value
    capi.check(L.pb_server_profiler_cmd(srv, 8, None), "record job events")
    capi.check(L.pb_server_profiler_cmd(srv, 6, None), "record run_next times")
    import torch
    bufs = []
    plan = [("tvm_mnist", 28 * 28)] * 6 + [("tvm_resnet18", 3 * 224 * 224)] * 2
    for k, (job, n_in) in enumerate(plan):
        b = torch.zeros(n_in + 1008, dtype=torch.float32).pin_memory()
        b[:n_in] = torch.rand(n_in)
        bufs.append(b)
        capi.check(L.pb_server_launch(srv, ids[job], ctypes.c_void_p(b.data_ptr()), k), "launch")
    done, cookies, errs = 0, (C.c_uint64 * 16)(), (C.c_int32 * 16)()
    import time
    t0 = time.time()
    while done < len(plan) and time.time() - t0 < 60:
        assert L.pb_server_step(srv, 64) >= 0
        done += L.pb_server_poll_done(srv, cookies, errs, 16)
    assert done == len(plan)
    prefix = str(tmp_path / "tl")
    capi.check(L.pb_server_profiler_cmd(srv, 12, prefix.encode()), "save")
    L.pb_server_destroy(srv)
    jobs = ost.read_job_events(prefix + "_job_events.txt")
    assert len(jobs) == len(plan)
    for ev in jobs:
        codes = [e for e, _ in ev]
        times = [t for _, t in ev]
        assert codes[0] == 0 and codes[-1] == 6
        assert times == sorted(times)
        n_stage = codes.count(3)
        assert n_stage >= 1 and codes.count(1) == n_stage and codes.count(4) == n_stage and codes.count(5) == n_stage
    s = ost.overhead_stack(jobs)
    assert s["jobs"] == len(plan) and s["kernel_runtime"] > 0 and s["kernel_launch_overhead"] > 0
    lines = open(prefix + "_run_next_times.txt").read().strip().splitlines()
    assert len(lines) == sum(ev.count(3) if False else [e for e, _ in ev].count(3) for ev in jobs)
