"""Deterministic replay: the product scheduler (C++, through pb_sched_replay) must make the
same decisions, bit for bit, as the oracle's restatement of the reference scheduler on the
same event trace - job, stage, copy/compute, over-subscription flag, stream and notifier
slot, and the priority's 64 bits."""
import ctypes as C
import random
import struct

import pytest

from oracle import scheduler as osch
from paella_b200 import capi

B200_TOTALS = (148 * 65536, 148 * 233472, 148 * 2048, 148 * 32)   # regs, smem, threads, block slots


def _replay(types_spec, events, num_streams, unfair, extra, totals):
    L = capi.load()
    keep = []
    rtypes = (capi.ReplayType * len(types_spec))()
    for i, st in enumerate(types_spec):
        n = len(st)
        a_mem = (C.c_uint8 * n)(*[int(s.is_mem) for s in st])
        a_pre = (C.c_uint8 * n)(*[int(s.pre_notify) for s in st])
        a_blk = (C.c_uint32 * n)(*[s.blocks for s in st])
        a_thr = (C.c_uint32 * n)(*[s.threads for s in st])
        a_smem = (C.c_uint32 * n)(*[s.smem for s in st])
        a_regs = (C.c_uint32 * n)(*[s.regs for s in st])
        keep += [a_mem, a_pre, a_blk, a_thr, a_smem, a_regs]
        rtypes[i] = capi.ReplayType(n, a_mem, a_pre, a_blk, a_thr, a_smem, a_regs)
    evs = (capi.ReplayEvent * len(events))(*[capi.ReplayEvent(k, a, b, t) for (k, a, b, t) in events])
    cfg = capi.ReplayConfig(num_streams, extra, unfair, *totals)
    cap = 8 * len(events) + 64
    dec = (capi.ReplayDecision * cap)()
    nd, nf = C.c_uint32(0), C.c_uint32(0)
    capi.check(L.pb_sched_replay(C.byref(cfg), rtypes, len(types_spec), evs, len(events), dec, cap, C.byref(nd), C.byref(nf)),
               "pb_sched_replay")
    assert nd.value <= cap
    out = [(d.event_index, d.job_id, d.type, d.stage, d.is_mem, d.unfit, d.stream_slot, d.notifier_slot, d.priority)
           for d in dec[: nd.value]]
    return out, nf.value


def _bits(x):
    return struct.pack("<d", x)


CASES = [
    # seed, types, jobs, streams, unfair, extra, totals, mean_iat, big
    dict(seed=1, ntypes=2, jobs=300, streams=500, unfair=1e6, extra=2, totals=B200_TOTALS, iat=30.0),
    dict(seed=2, ntypes=3, jobs=400, streams=8, unfair=1e6, extra=2, totals=B200_TOTALS, iat=5.0),
    dict(seed=3, ntypes=4, jobs=400, streams=64, unfair=0.5, extra=2, totals=B200_TOTALS, iat=4.0),     # fairness path
    dict(seed=4, ntypes=3, jobs=300, streams=64, unfair=1e6, extra=2, totals=(40 * 65536, 40 * 65536, 40 * 1024, 40 * 16),
         iat=3.0, big=True),                                                                            # over-subscription
    dict(seed=5, ntypes=5, jobs=500, streams=3, unfair=2.0, extra=1, totals=(40 * 65536, 40 * 65536, 40 * 1024, 40 * 16),
         iat=2.0, big=True),
    dict(seed=6, ntypes=2, jobs=200, streams=500, unfair=0.01, extra=2, totals=B200_TOTALS, iat=1.0),
]


@pytest.mark.parametrize("case", CASES, ids=[f"seed{c['seed']}" for c in CASES])
def test_product_scheduler_replays_oracle_decisions(case):
    rng = random.Random(case["seed"] * 7919)
    types_spec = [osch.model_like_type(rng, rng.choice([1, 4, 9, 20]), big=case.get("big", False) and i % 2 == 0)
                  for i in range(case["ntypes"])]
    weights = [rng.choice([1, 3, 9]) for _ in types_spec]
    events, ref_dec, ref_fin = osch.make_trace(types_spec, case["jobs"], case["seed"], case["streams"], case["unfair"],
                                               case["extra"], case["totals"], case["iat"], weights)
    assert ref_fin == case["jobs"]
    got, fin = _replay(types_spec, events, case["streams"], case["unfair"], case["extra"], case["totals"])
    assert fin == ref_fin
    assert len(got) == len(ref_dec)
    for g, r in zip(got, ref_dec):
        assert g[:8] == r[:8], (g, r)
        assert _bits(g[8]) == _bits(r[8]), (g, r)
    if case.get("big"):
        assert any(d[5] for d in ref_dec), "case was meant to exercise over-subscribed dispatch"


def test_fairness_override_changes_order():
    """With a low threshold the decisions differ from pure priority order (the override is live)."""
    rng = random.Random(11)
    types_spec = [osch.model_like_type(rng, 12), osch.model_like_type(rng, 2)]
    a = osch.make_trace(types_spec, 200, 9, 4, 1e6, 2, B200_TOTALS, 2.0)[1]
    b = osch.make_trace(types_spec, 200, 9, 4, 0.2, 2, B200_TOTALS, 2.0)[1]
    assert [d[1:4] for d in a] != [d[1:4] for d in b]


def test_notifier_record_arithmetic():
    """floor(G/16) records of 16 and one of G%16 (if non-zero), in that order; sums to G."""
    for g in [1, 5, 15, 16, 17, 31, 32, 148, 200, 4736]:
        recs = osch.notifier_records(g)
        assert recs == [16] * (g // 16) + ([g % 16] if g % 16 else [])
        assert sum(recs) == g


def test_reference_ring_model_delivers_in_order():
    """The reference's own ring fixture: ints 0..9999 in order through a small ring
    (tests/ipc/shm_channel/shmc_read_write.cpp:6-14, 64-byte ring of 8-byte records)."""
    ring = osch.RefRing(8)
    got, nxt = [], 0
    while len(got) < 10000:
        while nxt < 10000 and nxt - len(got) < 8:
            ring.write(nxt)
            nxt += 1
        while ring.can_read():
            got.append(ring.read())
    assert got == list(range(10000))


def test_jain_index():
    assert osch.jain_index([1, 1, 1, 1]) == 1.0
    assert abs(osch.jain_index([1, 0, 0, 0]) - 0.25) < 1e-12
