"""Host-side multi-GPU logic, on CPU: the request router's partition of one global arrival stream, and
the benchmark's reduction over ranks (max time, summed counts) with two gloo ranks."""
import ctypes as C
import os
import sys

import numpy as np
import pytest

from paella_b200 import capi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _plan(num_replicas, replica, jobs=500, warm=50, iat=100.0, seed=3, props=(0.9, 0.1), sigma=0.0):
    L = capi.load()
    cfg = capi.LoadgenConfig()
    L.pb_loadgen_config_default(C.byref(cfg))
    cfg.num_gpus = num_replicas
    cfg.num_types = len(props)
    for i, p in enumerate(props):
        cfg.proportions[i] = p
    cfg.num_jobs, cfg.warmup_jobs, cfg.seed = jobs, warm, seed
    cfg.mean_interarrival_us = iat
    cfg.lognormal_sigma = sigma
    n = C.c_uint32()
    cap = jobs + warm
    types = (C.c_uint32 * cap)()
    arr = (C.c_double * cap)()
    meas = (C.c_uint8 * cap)()
    capi.check(L.pb_loadgen_plan(C.byref(cfg), replica, types, arr, meas, cap, C.byref(n)), "pb_loadgen_plan")
    assert n.value == cap
    return np.array(types[:]), np.array(arr[:]), np.array(meas[:])


def test_router_deals_one_global_stream_round_robin():
    G = 4
    parts = [_plan(G, g) for g in range(G)]
    single_t, single_a, single_m = _plan(1, 0, jobs=500 * G, warm=50 * G, iat=100.0 / G)
    # replica g gets requests g, g+G, g+2G ... of the global stream: interleaving them restores it
    glob_t = np.stack([p[0] for p in parts], axis=1).ravel()
    glob_a = np.stack([p[1] for p in parts], axis=1).ravel()
    np.testing.assert_array_equal(glob_t, single_t)
    np.testing.assert_allclose(glob_a, single_a, rtol=0, atol=0)
    assert parts[0][1][0] == 0.0 and parts[0][1][50] == 0.0
    for t, a, m in parts:
        assert m[:50].sum() == 0 and m[50:].all()                 # warm-up first, then measured
        assert a[0] < 200.0 and a[50] < 200.0 and a[50] < a[49]   # each phase restarts its clock at t = 0
        assert (np.diff(a[50:]) >= 0).all()
        # per replica the arrival rate is 1 / iat: mean gap = G * (iat / G)
        assert abs(np.diff(a[50:]).mean() - 100.0) < 15.0
        assert 0.05 < (t[50:] == 1).mean() < 0.16                 # 10 % of the mix


def test_router_is_deterministic_and_seeded():
    a = _plan(2, 1, seed=7)
    b = _plan(2, 1, seed=7)
    c = _plan(2, 1, seed=8)
    np.testing.assert_array_equal(a[0], b[0])
    np.testing.assert_array_equal(a[1], b[1])
    assert not np.array_equal(a[1], c[1])
    # closed loop: no arrival times; lognormal keeps the requested mean
    assert (_plan(2, 0, iat=0.0)[1] == 0).all()
    ln = _plan(1, 0, jobs=4000, warm=0, iat=50.0, sigma=1.5)[1]
    assert 30.0 < np.diff(ln).mean() < 80.0


def _rank_main(rank, world, port, out_path):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    sys.path.insert(0, ROOT)
    import torch.distributed as dist

    import bench
    dist.init_process_group("gloo", rank=rank, world_size=world)
    ms, sums = bench.reduce_over_ranks(dist, 10.0 + rank, [100.0 * (rank + 1), 7.0, float(rank)])
    dist.barrier()
    if rank == 0:
        with open(out_path, "w") as f:
            f.write(repr((ms, sums)))
    dist.destroy_process_group()


def test_rank_reduction_with_two_gloo_ranks(tmp_path):
    import torch.multiprocessing as mp
    out = tmp_path / "reduced.txt"
    port = 29650 + (os.getpid() % 200)
    mp.spawn(_rank_main, args=(2, port, str(out)), nprocs=2, join=True)
    ms, sums = eval(out.read_text())
    assert ms == 11.0                       # max over ranks
    assert sums == [300.0, 14.0, 1.0]       # summed over ranks


def test_single_process_reduction_is_identity():
    sys.path.insert(0, ROOT)
    import bench
    assert bench.reduce_over_ranks(None, 5.0, [1.0, 2.0]) == (5.0, [1.0, 2.0])
