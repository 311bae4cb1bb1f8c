"""The ready queue against the reference's own JobQueue class.

oracle/ref_jobqueue/ compiles the reference's JobQueue (include/llis/server/scheduler_full3.h:26-208) from the
header where it lies, with stand-in headers for everything else that header includes, into oracle/_ref/.  Random
push / top / pop sequences then run through three queues at once: that build, the Python restatement the
scheduler oracle uses (oracle/scheduler.py:RefJobQueue), and the product's queue (include/llis/server/job_queue.h,
built behind the same C entry points).  All three must name the same job at every top() and pop().

Sequences cover: many equal priorities (ties resolve by insertion order), types that drain and come back (their
deficit counter is forgotten), thresholds low enough that the fairness override fires on most pops, and
thresholds so high that it never does."""
import ctypes as C
import os
import subprocess

import numpy as np
import pytest

from oracle import scheduler as osch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_DIR = os.path.join(ROOT, "oracle", "_ref")
REFERENCE = os.environ.get("PAELLA_REFERENCE", "/root/reference")


def _load(name):
    path = os.path.join(REF_DIR, name)
    if not os.path.exists(path) and os.path.exists(os.path.join(REFERENCE, "include", "llis", "server", "scheduler_full3.h")):
        subprocess.check_call(["make", "-s", "-C", os.path.join(ROOT, "oracle", "ref_jobqueue"), f"REFERENCE={REFERENCE}"])
    if not os.path.exists(path):
        pytest.skip(f"{name} is not built and the reference's sources are not on this machine")
    L = C.CDLL(path)
    L.jq_create.restype = C.c_void_p
    L.jq_create.argtypes = [C.c_double]
    L.jq_destroy.argtypes = [C.c_void_p]
    L.jq_push.argtypes = [C.c_void_p, C.c_uint32, C.c_double, C.c_uint64]
    for f in (L.jq_top, L.jq_pop, L.jq_size):
        f.restype = C.c_uint64
        f.argtypes = [C.c_void_p]
    return L


class _PyJob:
    def __init__(self, type_id, priority, tag):
        self.type_id, self.priority, self.tag = type_id, priority, tag


def _fuzz(seed, n_ops, n_types, threshold, distinct_priorities, push_bias):
    ref, prod = _load("libjobqueue_ref.so"), _load("libjobqueue_product.so")
    hr, hp = ref.jq_create(threshold), prod.jq_create(threshold)
    py = osch.RefJobQueue(threshold)
    rng = np.random.default_rng(seed)
    size, tag, fair_pops = 0, 0, 0
    try:
        for step in range(n_ops):
            # drain completely now and then so that every type forgets its counter and re-registers
            drain = size > 0 and rng.random() < 0.01
            for _ in range(size if drain else 1):
                if not drain and (size == 0 or rng.random() < push_bias):
                    t = int(rng.integers(0, n_types))
                    pr = float(rng.integers(0, distinct_priorities)) * 0.25 - 3.0
                    ref.jq_push(hr, t, pr, tag)
                    prod.jq_push(hp, t, pr, tag)
                    py.push(_PyJob(t, pr, tag))
                    tag += 1
                    size += 1
                else:
                    want = ref.jq_top(hr)
                    assert prod.jq_top(hp) == want and py.top().tag == want, f"top() differs at step {step}"
                    fair_pops += int(py._fair())
                    got = ref.jq_pop(hr)
                    assert got == want
                    assert prod.jq_pop(hp) == want, f"product pop() differs at step {step}"
                    assert py.pop().tag == want, f"restatement pop() differs at step {step}"
                    size -= 1
                assert ref.jq_size(hr) == size == prod.jq_size(hp)
    finally:
        ref.jq_destroy(hr)
        prod.jq_destroy(hp)
    return fair_pops, tag


@pytest.mark.parametrize("seed", range(6))
@pytest.mark.parametrize("threshold", [0.0, 1.5, 10.0, 1e6])
def test_three_queues_agree_on_random_sequences(seed, threshold):
    fair, pushed = _fuzz(seed, 4000, n_types=1 + seed, threshold=threshold, distinct_priorities=5 + 40 * (seed % 2), push_bias=0.55)
    assert pushed > 1000
    if threshold == 1e6:
        assert fair == 0
    if threshold == 0.0 and seed > 0:
        assert fair > 100        # the override really ran


def test_bursts_of_one_type_then_a_latecomer():
    """One type floods the queue, a second type arrives late: with a threshold of 2 the latecomer's jobs overtake
    once the flood has been served twice more than its share."""
    fair, _ = _fuzz(99, 3000, n_types=2, threshold=2.0, distinct_priorities=3, push_bias=0.7)
    assert fair > 0
