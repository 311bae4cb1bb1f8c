"""GPU->host notification ring, notifiers and the synthetic instrumented kernels, through the C ABI."""
import ctypes as C
import time
from collections import Counter

import numpy as np
import pytest

from oracle import graph as og
from oracle import scheduler as osch
from paella_b200 import capi

pytestmark = pytest.mark.gpu


@pytest.fixture()
def ring_env():
    L = capi.load()
    ring, nf = C.c_void_p(), C.c_void_p()
    capi.check(L.pb_ring_create(0, 1 << 16, C.byref(ring)), "pb_ring_create")
    capi.check(L.pb_notifier_create_array(ring, 4, C.byref(nf)), "pb_notifier_create_array")
    yield L, ring, nf
    L.pb_notifier_free_array(nf)
    L.pb_ring_destroy(ring)


def _drain(L, ring, want, timeout=10.0):
    recs = []
    buf = (C.c_uint64 * 256)()
    t0 = time.time()
    while len(recs) < want and time.time() - t0 < timeout:
        n = L.pb_ring_poll(ring, buf, 256)
        assert n >= 0, L.pb_last_error()
        recs += [buf[i] for i in range(n)]
    return recs


def _unpack(v):
    return dict(is_start=v & 0xff, smid=(v >> 8) & 0xff, num=(v >> 16) & 0xff, status=(v >> 24) & 0xff, job_id=v >> 32)


@pytest.mark.parametrize("g", [1, 5, 16, 17, 148, 200, 4736])
def test_aggregated_notifications_match_notifier_arithmetic(ring_env, g):
    L, ring, nf = ring_env
    want = osch.notifier_records(g)
    capi.check(L.pb_launch_notify_probe(None, g, 64, 77, nf, 1), "probe")
    recs = [_unpack(r) for r in _drain(L, ring, 2 * len(want))]
    assert len(recs) == 2 * len(want)
    assert all(r["job_id"] == 77 for r in recs)
    starts = [r["num"] for r in recs if r["is_start"] == 1]
    ends = [r["num"] for r in recs if r["is_start"] == 0]
    # per kind, records appear in ticket order: the 16s first, then the remainder
    assert Counter(starts) == Counter(want) and Counter(ends) == Counter(want)
    assert sum(starts) == g and sum(ends) == g
    # the notifier's counters wrapped back to zero: a second kernel on the same notifier gives the same records
    capi.check(L.pb_launch_notify_probe(None, g, 64, 78, nf, 1), "probe")
    recs2 = [_unpack(r) for r in _drain(L, ring, 2 * len(want))]
    assert sum(r["num"] for r in recs2 if r["is_start"] == 1) == g
    assert sum(r["num"] for r in recs2 if r["is_start"] == 0) == g
    assert L.pb_ring_poll(ring, (C.c_uint64 * 4)(), 4) == 0


@pytest.mark.parametrize("g", [1, 100, 1184])
def test_per_block_notifications_count_is_two_per_block(ring_env, g):
    """The invariant the reference's GPU ring benchmark relies on
    (tests/ipc/shm_channel/latency/shmpc_latency_gpu.cu:46-52)."""
    L, ring, nf = ring_env
    capi.check(L.pb_launch_notify_probe(None, g, 32, 5, nf, 0), "probe")
    recs = [_unpack(r) for r in _drain(L, ring, 2 * g)]
    assert len(recs) == 2 * g
    assert sum(r["is_start"] == 1 for r in recs) == g
    assert all(r["num"] == 1 and r["smid"] < 160 for r in recs)
    assert L.pb_ring_poll(ring, (C.c_uint64 * 4)(), 4) == 0


def test_ring_wraps_and_tags_laps():
    L = capi.load()
    ring, nf = C.c_void_p(), C.c_void_p()
    capi.check(L.pb_ring_create(0, 64, C.byref(ring)), "pb_ring_create")
    capi.check(L.pb_notifier_create_array(ring, 1, C.byref(nf)), "pb_notifier_create_array")
    total = 0
    for it in range(40):   # 40 x 24 = 960 records through 64 slots = 15 laps
        capi.check(L.pb_launch_notify_probe(None, 12, 32, it, nf, 0), "probe")
        recs = [_unpack(r) for r in _drain(L, ring, 24)]
        assert len(recs) == 24 and all(r["job_id"] == it for r in recs)
        for i, r in enumerate(recs):
            assert r["status"] == 1 + ((total + i) // 64) % 255
        total += 24
    assert L.pb_ring_records_read(ring) == total
    L.pb_notifier_free_array(nf)
    L.pb_ring_destroy(ring)


def test_ring_overflow_is_detected_not_silent():
    import torch
    L = capi.load()
    ring, nf = C.c_void_p(), C.c_void_p()
    capi.check(L.pb_ring_create(0, 16, C.byref(ring)), "pb_ring_create")
    capi.check(L.pb_notifier_create_array(ring, 1, C.byref(nf)), "pb_notifier_create_array")
    capi.check(L.pb_launch_notify_probe(None, 20, 32, 1, nf, 0), "probe")   # 40 records into 16 slots
    torch.cuda.synchronize()
    buf = (C.c_uint64 * 64)()
    rc, seen = 0, 0
    for _ in range(8):
        rc = L.pb_ring_poll(ring, buf, 64)
        if rc < 0:
            break
        seen += rc
    assert rc == -3, f"expected PB_ERR_RING_OVERFLOW, read {seen} records"
    L.pb_notifier_free_array(nf)
    L.pb_ring_destroy(ring)


def test_mem_done_record(ring_env):
    L, ring, nf = ring_env
    capi.check(L.pb_launch_mem_done(None, 1234, nf), "mem_done")
    recs = [_unpack(r) for r in _drain(L, ring, 1)]
    assert recs == [dict(is_start=2, smid=0, num=1, status=1, job_id=1234)]


@pytest.mark.parametrize("n", [1, 7, 1000003, 1 << 20, 1 << 24])
def test_vec_add_matches_oracle(ring_env, n):
    import torch
    L, ring, nf = ring_env
    rng = np.random.default_rng(n)
    a = rng.uniform(-1, 1, n).astype(np.float32)
    b = rng.uniform(-1, 1, n).astype(np.float32)
    out, inp = torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda()
    li = capi.LaunchInfo()
    capi.check(L.pb_vec_add_info(n, C.byref(li)), "info")
    assert li.bytes == 12 * n
    capi.check(L.pb_vec_add_launch(out.data_ptr(), inp.data_ptr(), n, None, 9, nf), "vec_add")
    torch.cuda.synchronize()
    ref = a.copy()
    og.lib().orc_vec_add(ref.ctypes.data_as(C.POINTER(C.c_float)), b.ctypes.data_as(C.POINTER(C.c_float)), n)
    np.testing.assert_array_equal(out.cpu().numpy(), ref)       # one fp32 add per element: bit exact
    want = osch.notifier_records(li.num_blocks)
    recs = [_unpack(r) for r in _drain(L, ring, 2 * len(want))]
    assert sum(r["num"] for r in recs if r["is_start"] == 0) == li.num_blocks


def test_spin_kernel_holds_its_slot_for_the_requested_time(ring_env):
    import torch
    L, ring, nf = ring_env
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s = torch.cuda.current_stream().cuda_stream
    capi.check(L.pb_spin_launch(148, 10000, None, s, 3, nf), "spin warm-up")
    e0.record()
    capi.check(L.pb_spin_launch(148, 1000000, None, s, 3, nf), "spin")
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    assert 0.99 <= ms < 5.0, ms
    assert L.pb_spin_launch(1, 10 ** 9, None, s, 3, nf) == -2      # refuses absurd durations
    _drain(L, ring, 2 * 2 * len(osch.notifier_records(148)))


def test_ring_latency_probe_and_clock_calibration(ring_env):
    L, ring, nf = ring_env
    cal = (C.c_uint64 * 3)()
    capi.check(L.pb_clock_calibrate(0, cal), "calibrate")
    assert cal[2] >= cal[0] and cal[1] > 0
    capi.check(L.pb_launch_latency_probe(None, 8, nf), "latency probe")
    assert len(_drain(L, ring, 8)) == 8


def test_a_device_wait_that_runs_out_reports_status_and_leaves_the_context_usable():
    """The bounded-wait rule, checked on the kernel that waits for the host: with a ping that never comes it gives
    up after its poll limit, reports status 2 and returns; nothing faults and the next kernel runs normally."""
    L = capi.load()
    status, recs = C.c_uint32(0), C.c_uint32(7)
    capi.check(L.pb_ring_wait_expiry_probe(0, 2000, C.byref(status), C.byref(recs)), "pb_ring_wait_expiry_probe")
    assert status.value == 2 and recs.value == 0
    n = 200
    rtt = (C.c_double * n)()
    capi.check(L.pb_ring_roundtrip_bench(0, n, rtt), "round trip after the expired wait")
    assert all(0 < rtt[i] < 1e5 for i in range(n))
