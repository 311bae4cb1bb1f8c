"""The product scheduler driven call by call on the CPU (pb_sched_sim_*): the test plays the clients and the GPU.
Covers what a recorded trace cannot: gangs, deferred dispatch, a plugin whose run_next() fails, the stage watchdog.
The record stream per dispatch is the notifier's (floor(G/16) records of 16 and one of G mod 16 per direction)."""
import ctypes as C
import heapq

import pytest

from oracle import scheduler as osch
from paella_b200 import capi

B200 = (148 * 65536, 148 * 233472, 148 * 2048, 148 * 32)


class Sim:
    def __init__(self, types, fails=None, streams=64, extra=2, unfair=1e6, totals=B200, gang=1, cap=1, deferred=0, sched=b"full3",
                 wd_factor=0.0, wd_floor=0.0):
        self.L = capi.load()
        self.keep = []
        n_types = len(types)
        self.rtypes = (capi.ReplayType * n_types)()
        for i, st in enumerate(types):
            n = len(st)
            arrs = [(C.c_uint8 * n)(*[int(s["mem"]) for s in st]), (C.c_uint8 * n)(*[int(i2 == n - 1) for i2 in range(n)]),
                    (C.c_uint32 * n)(*[s["blocks"] for s in st]), (C.c_uint32 * n)(*[s.get("threads", 256) for s in st]),
                    (C.c_uint32 * n)(*[s.get("smem", 1024) for s in st]), (C.c_uint32 * n)(*[s.get("regs", 32) for s in st])]
            self.keep += arrs
            self.rtypes[i] = capi.ReplayType(n, *arrs)
        fl = None
        if fails:
            fl = (C.POINTER(C.c_uint8) * n_types)()
            for i, st in enumerate(types):
                a = (C.c_uint8 * len(st))(*[int(j in fails.get(i, ())) for j in range(len(st))])
                self.keep.append(a)
                fl[i] = a
        cfg = capi.SimConfig(capi.ReplayConfig(streams, extra, unfair, *totals), sched, gang, cap, deferred, wd_factor, wd_floor)
        self.h = C.c_void_p()
        capi.check(self.L.pb_sched_sim_create(C.byref(cfg), self.rtypes, n_types, fl, C.byref(self.h)), "pb_sched_sim_create")
        self.types = types
        self.now = 0.0
        self.events = []          # heap of (time, seq, kind, job_id, num)
        self.seq = 0
        self.done = {}
        self.log = []
        self.drop_end_of = set()  # cookies whose stages never report their last end record

    def close(self):
        self.L.pb_sched_sim_destroy(self.h)

    def submit(self, typ, cookie):
        capi.check(self.L.pb_sched_sim_new_job(self.h, typ, self.now, cookie), "new_job")

    def _post(self, t, kind, job_id, num):
        heapq.heappush(self.events, (t, self.seq, kind, job_id, num))
        self.seq += 1

    def collect(self):
        """Reads new dispatches, queues their records on the toy GPU; reads finished jobs."""
        dec = (capi.SimDecision * 256)()
        while True:
            n = self.L.pb_sched_sim_take_decisions(self.h, dec, 256)
            for d in dec[:n]:
                self.log.append((d.job_id, d.type, d.stage, d.is_mem, d.unfit, d.num_blocks, d.gang_size, d.cookie))
                if d.failed:
                    continue              # the launch failed: a GPU sends nothing for it
                if d.is_mem:
                    self._post(self.now + 5.0, 3, d.job_id, 1)
                    continue
                recs = osch.notifier_records(d.num_blocks)
                t = self.now + 1.0
                for r in recs:
                    self._post(t, 1, d.job_id, r)
                    t += 0.1
                t = self.now + 20.0
                for i, r in enumerate(recs):
                    if d.cookie in self.drop_end_of and i == len(recs) - 1:
                        continue          # the kernel never reports its last blocks
                    self._post(t, 2, d.job_id, r)
                    t += 0.1
            if n < 256:
                break
        ck, er = (C.c_uint64 * 256)(), (C.c_int32 * 256)()
        while True:
            n = self.L.pb_sched_sim_take_finished(self.h, ck, er, 256)
            for i in range(n):
                assert ck[i] not in self.done, "a request finished twice"
                self.done[ck[i]] = er[i]
            if n < 256:
                break

    def run(self, until=None, flush_every_record=True):
        """Plays queued records in time order until the toy GPU is idle (or `until`)."""
        failed = self.L.pb_sched_sim_flush(self.h, self.now)
        self.collect()
        while self.events and (until is None or self.events[0][0] <= until):
            t, _, kind, job_id, num = heapq.heappop(self.events)
            self.now = max(self.now, t)
            capi.check(self.L.pb_sched_sim_record(self.h, kind, job_id, num, self.now), "record")
            if flush_every_record:
                failed += self.L.pb_sched_sim_flush(self.h, self.now)
            self.collect()
        if until is not None:
            self.now = max(self.now, until)
        failed += self.L.pb_sched_sim_flush(self.h, self.now)
        self.collect()
        return failed

    def in_flight(self):
        return self.L.pb_sched_sim_jobs_in_flight(self.h)


MODEL = [dict(mem=False, blocks=40), dict(mem=False, blocks=100), dict(mem=False, blocks=7)]
SMALL = [dict(mem=False, blocks=1)]
COPIES = [dict(mem=True, blocks=0), dict(mem=False, blocks=33), dict(mem=True, blocks=0)]


@pytest.mark.parametrize("sched", [b"full3", b"fifo2", b"fifo"])
def test_failing_run_next_drains_the_job_with_its_error(sched):
    """run_next() of stage 1 of type 0 enqueues nothing and raises the job's error flag: the scheduler closes the
    stage with records of its own, the job runs (and fails) through its remaining stages, ends with the error, and
    its stream, notifier and occupancy come back - the other type is not disturbed.  A failing copy stage likewise."""
    s = Sim([MODEL, SMALL, COPIES], fails={0: (1,), 2: (0,)}, streams=4, sched=sched)
    for i in range(6):
        s.submit(0, 100 + i)
        s.submit(1, 200 + i)
        s.submit(2, 300 + i)
    s.run()
    assert len(s.done) == 18 and s.in_flight() == 0
    for i in range(6):
        assert s.done[100 + i] == -1 and s.done[300 + i] == -1 and s.done[200 + i] == 0
    # every stage of the failing jobs was still dispatched (they drain, they are not dropped)
    assert sum(1 for e in s.log if e[1] == 0) == 6 * 3 and sum(1 for e in s.log if e[1] == 2) == 6 * 3
    # and the pools are whole: a second wave runs
    for i in range(8):
        s.submit(1, 400 + i)
    s.run()
    assert all(s.done[400 + i] == 0 for i in range(8))
    s.close()


def test_gangs_form_from_what_is_queued_and_end_together():
    s = Sim([MODEL, SMALL], gang=4, cap=8)
    for i in range(10):
        s.submit(0, 100 + i)
    for i in range(5):
        s.submit(1, 200 + i)
    assert s.L.pb_sched_sim_take_decisions(s.h, (capi.SimDecision * 4)(), 4) == 0      # nothing is dispatched before the flush
    s.run()
    assert len(s.done) == 15 and all(e == 0 for e in s.done.values()) and s.in_flight() == 0
    first = [e for e in s.log if e[1] == 0 and e[2] == 0]
    assert sorted(e[6] for e in first) == [2, 4, 4]                   # 10 jobs -> gangs of 4, 4, 2
    for e in s.log:
        if e[1] == 0:
            assert e[5] == MODEL[e[2]]["blocks"] * e[6]               # a gang of n declares n times the blocks
    assert sum(1 for e in s.log if e[1] == 0) == 3 * 3                # 3 gangs x 3 stages, not 10 x 3
    assert sorted(e[6] for e in s.log if e[1] == 1) == [1, 4]         # max_gang caps the MNIST-like type too
    # a gang never takes a job that has already started: jobs submitted later run on their own
    s.submit(0, 300)
    s.run()
    assert s.done[300] == 0 and [e[6] for e in s.log if e[7] == 300] == [1, 1, 1]
    s.close()


def test_gang_capacity_of_the_plugin_limits_the_gang():
    s = Sim([MODEL], gang=8, cap=2)
    for i in range(5):
        s.submit(0, i)
    s.run()
    assert len(s.done) == 5 and sorted(e[6] for e in s.log if e[2] == 0) == [1, 2, 2]
    s.close()


def test_a_failing_leader_fails_its_gang():
    s = Sim([MODEL], fails={0: (2,)}, gang=4, cap=4)
    for i in range(4):
        s.submit(0, i)
    s.run()
    assert s.done == {0: -1, 1: -1, 2: -1, 3: -1} and s.in_flight() == 0
    s.close()


def test_deferred_dispatch_runs_the_same_jobs():
    """Dispatch once per batch of records instead of inside every record: same requests, same number of stage
    dispatches, all complete."""
    out = []
    for deferred, every in ((0, True), (1, True), (1, False)):
        s = Sim([MODEL, SMALL, COPIES], streams=6, deferred=deferred)
        for i in range(30):
            s.submit(i % 3, i)
        s.run(flush_every_record=every)
        if not every:                      # records only queue work up; the final flush of run() dispatched one batch
            while s.in_flight():
                s.run()
        assert len(s.done) == 30 and all(e == 0 for e in s.done.values())
        out.append(len(s.log))
        s.close()
    assert out[0] == out[1] == out[2] == 10 * (3 + 1 + 3)


def test_stage_watchdog_gives_up_a_stage_that_never_ends():
    """The toy GPU withholds the last end record of one request's stages (a wedged kernel).  With the watchdog on,
    that request ends with PB_ERR_TIMEOUT once its stage is 10 x over its learned length (at least 1 ms here), its
    occupancy is released, the other requests are not held up, and its job id is never handed out again: the late
    record is ignored."""
    s = Sim([MODEL, SMALL], streams=8, wd_factor=10.0, wd_floor=1000.0)
    for i in range(4):                     # learn the stage lengths first
        s.submit(0, i)
    assert s.run() == 0 and len(s.done) == 4
    s.drop_end_of.add(50)
    s.submit(0, 50)
    s.submit(0, 51)
    s.submit(1, 52)
    assert s.run() == 0                    # nothing has run out yet
    assert s.done.get(51) == 0 and s.done.get(52) == 0 and 50 not in s.done and s.in_flight() == 1
    stuck_id = [e[0] for e in s.log if e[7] == 50][-1]
    assert s.run(until=s.now + 900.0) == 0 and 50 not in s.done      # below the 1 ms floor
    assert s.run(until=s.now + 200.0) == 1                            # above it
    assert s.done[50] == -5 and s.in_flight() == 0
    # the record that comes after all is a stray; the id stays out of circulation
    capi.check(s.L.pb_sched_sim_record(s.h, 2, stuck_id, MODEL[0]["blocks"] % 16 or 16, s.now + 1.0), "late record")
    for i in range(12):
        s.submit(0, 100 + i)
    s.run()
    assert all(s.done[100 + i] == 0 for i in range(12))
    assert stuck_id not in [e[0] for e in s.log if e[7] >= 100]
    s.close()


def test_a_tight_occupancy_gate_makes_waiting_requests_leave_as_a_gang():
    """The GPU of this test holds one and a half stages of TWO at a time.  With no over-subscribed stage allowed, the
    first request is dispatched alone; three more arrive one after the other while it runs, do not fit, wait in the
    queue - and when the first request is through they leave together as ONE gang.  With a wide-open gate (64
    over-subscribed stages) the same arrivals are dispatched one by one the moment they arrive.  This is the mechanism
    behind the benchmark's gate of 18 stages: under load, requests meet in the queue."""
    TWO = [dict(mem=False, blocks=100), dict(mem=False, blocks=100)]
    tight = (150 * 256 * 32, 148 * 233472, 150 * 256, 148 * 32)      # registers, shared memory, threads, block slots
    for extra, want in ((0, [1, 3]), (64, [1, 1, 1, 1])):
        s = Sim([TWO], streams=16, extra=extra, totals=tight, gang=4, cap=8)
        s.submit(0, 1)
        s.run(until=0.5)                       # dispatched; its first stage is in flight (block records come later)
        assert [e[6] for e in s.log if e[2] == 0] == [1]
        for k, t in ((2, 3.0), (3, 6.0), (4, 9.0)):
            s.submit(0, k)
            s.run(until=t)
        s.run()
        assert len(s.done) == 4 and all(v == 0 for v in s.done.values())
        assert sorted(e[6] for e in s.log if e[2] == 0) == want, (extra, s.log)
        s.close()
