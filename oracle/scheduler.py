"""Oracle for the notification arithmetic and the kernel-level scheduler.

TEST INFRASTRUCTURE ONLY (never imported by the paella_b200 package).

Restates, structure for structure, the reference's
  * notifier batching          include/llis/job/finished_block_notifier.h:27-43,65-81
  * ring slot/status protocol  include/llis/ipc/shm_primitive_channel_impl.h:18-64
  * JobQueue                   include/llis/server/scheduler_full3.h:26-208
  * SmResources                src/server/sm_resources.cpp:36-57, include/llis/server/sm_resources.h:29-31
  * RegisteredJob tables       src/server/registered_job.cpp:112-182
  * Job stage state            include/llis/job/job.h:138-191,278-292
  * SchedulerFull3             src/server/scheduler_full3.cpp:123-459
with std::multimap emulated by a sorted list that inserts at the upper bound of equal
keys (what std::multimap::emplace/insert do), so tie-breaking is the reference's.

Pins available upstream: the reference has no scheduler tests.  What it does pin is
"exactly 2*num_blocks un-aggregated records per kernel"
(tests/ipc/shm_channel/latency/shmpc_latency_gpu.cu:46-52) and in-order delivery of
0..9999 through a small ring (tests/ipc/shm_channel/shmc_read_write.cpp:6-14); both are
reproduced in tests/ against this file.  Scheduler decisions are otherwise "parity
unpinned" upstream: the restatement below is the pin.
"""
from __future__ import annotations

import heapq
import math
import random
from dataclasses import dataclass, field

DBL_MAX = 1.7976931348623157e308
NOTI_BATCH = 16


# --------------------------------------------------------------------------- notifier
def notifier_records(num_blocks: int, order=None):
    """Records one direction of a kernel of `num_blocks` blocks emits, in ticket order:
    the t-th block to take a ticket (t = 1..G) emits num=16 when t % 16 == 0, and the last
    one emits the remainder (finished_block_notifier.h:27-43)."""
    out = []
    for total in range(1, num_blocks + 1):
        batch = total % NOTI_BATCH
        if batch == 0:
            out.append(NOTI_BATCH)
        elif total == num_blocks:
            out.append(batch)
    return out


class RefRing:
    """Host model of the reference ring: writer takes ticket = inc-with-wrap(count-1), stores a
    record with status 1; reader polls slot[read_pos].status, clears it, advances
    (shm_primitive_channel_impl.h:18-64)."""

    def __init__(self, count):
        self.count = count
        self.slots = [None] * count
        self.write_pos = 0
        self.read_pos = 0

    def write(self, rec):
        pos = self.write_pos
        self.write_pos = 0 if pos >= self.count - 1 else pos + 1   # atomicInc(ptr, count-1)
        self.slots[pos] = rec

    def can_read(self):
        return self.slots[self.read_pos] is not None

    def read(self):
        rec = self.slots[self.read_pos]
        self.slots[self.read_pos] = None
        self.read_pos = 0 if self.read_pos == self.count - 1 else self.read_pos + 1
        return rec


# --------------------------------------------------------------------------- multimap
class MultiMap:
    """std::multimap<double, V, std::greater<double>>: descending keys; equal keys keep
    insertion order (insert at upper bound)."""

    def __init__(self):
        self.items = []   # [key, handle, value]
        self._next = 0

    def emplace(self, key, value):
        i = 0
        while i < len(self.items) and self.items[i][0] >= key:
            i += 1
        h = self._next
        self._next += 1
        self.items.insert(i, [key, h, value])
        return h

    def begin(self):
        return self.items[0]

    def erase(self, handle):
        for i, it in enumerate(self.items):
            if it[1] == handle:
                return self.items.pop(i)
        raise KeyError(handle)

    def __len__(self):
        return len(self.items)


class RefJobQueue:
    """include/llis/server/scheduler_full3.h:26-208"""

    def __init__(self, unfairness_threshold):
        self.unfairness_threshold = float(unfairness_threshold)
        self.new_type_deficit = 0.0
        self.num_types = 0
        self.all_map = MultiMap()
        self.per_type = []      # dict(deficit, job_map, it)
        self.type_map = MultiMap()

    def push(self, job):
        t = job.type_id
        it_all = self.all_map.emplace(job.priority, {"job": job})
        if t >= len(self.per_type):
            orig = len(self.per_type)
            for _ in range(orig, t + 1):
                self.per_type.append({"deficit": DBL_MAX, "job_map": MultiMap(), "it": None})
            self.per_type[t]["deficit"] = self.new_type_deficit
            self.num_types += 1
        elif self.per_type[t]["deficit"] == DBL_MAX:
            self.per_type[t]["deficit"] = self.new_type_deficit
            self.num_types += 1
        te = self.per_type[t]
        if len(te["job_map"]) == 0:
            te["it"] = self.type_map.emplace(te["deficit"], te)
        it_pt = te["job_map"].emplace(job.priority, {"job": job, "other": it_all})
        for it in self.all_map.items:
            if it[1] == it_all:
                it[2]["other"] = it_pt

    def _fair(self):
        return self.type_map.begin()[0] >= self.unfairness_threshold

    def top(self):
        if self._fair():
            return self.type_map.begin()[2]["job_map"].begin()[2]["job"]
        return self.all_map.begin()[2]["job"]

    def pop(self):
        if self._fair():
            jm = self.type_map.begin()[2]["job_map"]
            entry = jm.begin()[2]
            jm.erase(jm.begin()[1])
            self.all_map.erase(entry["other"])
        else:
            entry = self.all_map.begin()[2]
            self.all_map.erase(self.all_map.begin()[1])
            self.per_type[entry["job"].type_id]["job_map"].erase(entry["other"])
        fair_share = 1.0 / float(self.num_types)
        self.new_type_deficit -= fair_share
        self.unfairness_threshold -= fair_share
        te = self.per_type[entry["job"].type_id]
        if len(te["job_map"]) == 0:
            te["deficit"] = DBL_MAX
            self.num_types -= 1
            self.type_map.erase(te["it"])
        else:
            key, _, val = self.type_map.erase(te["it"])
            te["it"] = self.type_map.emplace(key - 1.0, val)
        return entry["job"]

    def empty(self):
        return len(self.all_map) == 0


# --------------------------------------------------------------------------- jobs
@dataclass
class StageSpec:
    is_mem: bool
    pre_notify: bool
    blocks: int = 0
    threads: int = 0
    smem: int = 0
    regs: int = 0


@dataclass
class RefType:
    """RegisteredJob tables (registered_job.cpp:112-182) + LIFO instance pool (:61-93)."""
    type_id: int
    stages: list
    stage_lengths: list = field(default_factory=list)
    stage_resources: list = field(default_factory=list)
    unused: list = field(default_factory=list)

    def update_stage_length(self, stage, length):
        if len(self.stage_lengths) > stage:
            self.stage_lengths[stage] = (self.stage_lengths[stage] + length) / 2
        else:
            self.stage_lengths.append(length)

    def has_stage_resource(self, stage):
        return len(self.stage_resources) > stage

    def set_stage_resource(self, stage, res):
        if len(self.stage_resources) <= stage:
            self.stage_resources.append(res)

    def remaining_rl(self, frm):
        s = 0.0
        for i in range(frm, len(self.stage_lengths)):
            s += self.stage_lengths[i] * (self.stage_resources[i] if i < len(self.stage_resources) else 0.0)
        return s


class RefJob:
    """Scheduler-visible job state (job.h) for a table-driven job that follows the adapters'
    stage protocol (tvm_mnist.cpp:35-47: next stage declared before run_next returns)."""

    def __init__(self, typ: RefType):
        self.typ = typ
        self.type_id = typ.type_id
        self.reset()

    def reset(self):
        self.is_running = False
        self.has_started = False
        self.is_mem = False
        self.is_pre_notify = False
        self.cur_stage = -1
        self.is_unfit = False
        self.next_idx = 0
        self._declare()

    def _declare(self):
        if self.next_idx < len(self.typ.stages):
            s = self.typ.stages[self.next_idx]
            self.is_mem = s.is_mem
            if s.pre_notify:
                self.is_pre_notify = True
            self.num_blocks, self.threads, self.smem, self.regs = s.blocks, s.threads, s.smem, s.regs

    def has_next(self):
        return self.next_idx < len(self.typ.stages)

    def run_next(self):
        self.next_idx += 1
        self._declare()

    def set_running(self, stream, now):
        self.is_running = True
        self.stream = stream
        self.num_running_blocks = self.num_blocks
        self.num_pending_blocks = self.num_blocks
        self.cur = (self.num_blocks, self.threads, self.smem, self.regs)
        self.stage_start = now
        self.cur_stage += 1

    def set_stage_lengths_resources(self, total, lengths, resources):
        self.cur_rl = total
        self.stage_lengths = list(lengths)
        self.stage_resources = list(resources)

    def dec_cur_rl(self):
        i = self.cur_stage + 1
        if len(self.stage_lengths) > 0 and i < len(self.stage_lengths) and i < len(self.stage_resources):
            # the reference indexes without a bounds check (job.h:288-292); out of range counts as 0 here
            self.cur_rl -= self.stage_lengths[i] * self.stage_resources[i]


class RefSmResources:
    def __init__(self, regs, smem, threads, blocks):
        self.regs, self.smem, self.threads, self.blocks = regs, smem, threads, blocks

    def job_fits(self, j):
        return (self.regs >= j.regs * j.threads * j.num_blocks and self.smem >= j.smem * j.num_blocks and
                self.threads >= j.threads * j.num_blocks and self.blocks >= j.num_blocks)

    def _apply(self, j, num):
        nb, th, sm, rg = j.cur
        self.regs += rg * th * num
        self.threads += th * num
        self.smem += sm * num
        self.blocks += num

    def acquire(self, j, num):
        self._apply(j, -num)

    def release(self, j, num):
        self._apply(j, num)


class RefSchedulerFull3:
    """src/server/scheduler_full3.cpp:123-459.  `now` is set by the driver before each event;
    on_run(job, is_mem) is called where the reference calls job->run_next()."""

    def __init__(self, types, num_streams, unfair, extra_kernels, totals, on_run=None):
        self.types = types
        self.streams = list(range(num_streams))
        self.notifiers = list(range(num_streams))
        self.queue = RefJobQueue(unfair)
        self.jobs = []
        self.unused_ids = []
        self.res = RefSmResources(*totals)
        self.num_jobs = 0
        self.num_outstanding = 0
        self.max_outstanding = extra_kernels
        self.now = 0.0
        self.event_index = 0
        self.decisions = []
        self.finished = 0
        self.on_run = on_run

    # -- registered-job services ------------------------------------------------
    def _ensure_resource(self, job):
        if not job.typ.has_stage_resource(job.cur_stage + 1):
            job.typ.set_stage_resource(job.cur_stage + 1, 1.0)

    @staticmethod
    def _priority(job):
        rl = job.cur_rl
        job.dec_cur_rl()
        return -rl

    def new_job(self, type_id):
        typ = self.types[type_id]
        if typ.unused:
            job = typ.unused.pop()
            job.reset()
        else:
            job = RefJob(typ)
        self.handle_new_job(job)

    def handle_new_job(self, job):
        if not job.has_next():
            job.typ.unused.append(job)
            return
        if not self.unused_ids:
            job.id = len(self.jobs)
            self.jobs.append(job)
        else:
            job.id = self.unused_ids.pop()
            self.jobs[job.id] = job
        self._ensure_resource(job)
        job.set_stage_lengths_resources(job.typ.remaining_rl(0), job.typ.stage_lengths, job.typ.stage_resources)
        job.priority = self._priority(job)
        self.queue.push(job)
        self.num_jobs += 1
        self.schedule_job()

    def handle_block_start(self, job_id, num):
        job = self.jobs[job_id]
        job.num_pending_blocks -= num
        if job.num_pending_blocks == 0:
            if job.is_unfit:
                job.is_unfit = False
                self.num_outstanding -= 1
                self.schedule_job()

    def _stage_finished(self, job):
        length = self.now - job.stage_start
        job.typ.update_stage_length(job.cur_stage, length)
        if job.has_next():
            self._ensure_resource(job)
            job.priority = self._priority(job)
            self.queue.push(job)
        else:
            self.finished += 1
            self.num_jobs -= 1

    def handle_block_finish(self, job_id, num):
        job = self.jobs[job_id]
        job.num_running_blocks -= num
        if job.num_running_blocks <= 0:
            job.is_running = False
        done = not job.is_running
        if done:
            self._stage_finished(job)
            if job.is_unfit:
                job.is_unfit = False
                self.num_outstanding -= 1
            self.streams.append(job.stream)
            self.notifiers.append(job.notifier)
        self.res.release(job, num)
        if done and not job.has_next():
            self.unused_ids.append(job.id)
            self.jobs[job.id] = None
            job.typ.unused.append(job)
        self.schedule_job()

    def handle_mem_finish(self, job_id):
        job = self.jobs[job_id]
        job.is_running = False
        self._stage_finished(job)
        self.streams.append(job.stream)
        if not job.has_next():
            self.unused_ids.append(job.id)
            self.jobs[job.id] = None
            job.typ.unused.append(job)
        self.schedule_job()

    def schedule_job(self):
        if not self.streams or self.queue.empty():
            return
        while True:
            job = self.queue.top()
            is_mem = job.is_mem
            unfit = False
            if not is_mem and not self.res.job_fits(job):
                if self.num_outstanding >= self.max_outstanding:
                    break
                self.num_outstanding += 1
                job.is_unfit = True
                unfit = True
            self.queue.pop()
            job.has_started = True
            job.set_running(self.streams.pop(), self.now)
            nslot = 0xFFFFFFFF
            if not is_mem:
                job.notifier = self.notifiers.pop()
                nslot = job.notifier
                self.res.acquire(job, job.cur[0])
            self.decisions.append((self.event_index, job.id, job.type_id, job.cur_stage, int(is_mem), int(unfit),
                                   job.stream, nslot, job.priority))
            stage = job.cur_stage
            job.run_next()
            if self.on_run:
                self.on_run(job, stage, is_mem)
            if not self.streams:
                break
            if self.queue.empty():
                break


# --------------------------------------------------------------------------- trace generation
def make_trace(types_spec, num_jobs, seed, num_streams, unfair, extra_kernels, totals, mean_iat=30.0,
               type_weights=None):
    """Runs the oracle scheduler against a toy GPU (each stage takes a pseudo-random time; block
    start/end records arrive in the notifier's batches) and returns (events, decisions, finished).
    events: list of (kind, a, b, time_us) with kind 0 NEW_JOB(type) 1 START(job,num) 2 END(job,num) 3 MEM(job)."""
    rng = random.Random(seed)
    types = [RefType(i, st) for i, st in enumerate(types_spec)]
    pending = []   # heap of (time, seq, kind, a, b)
    seq = [0]

    def post(t, kind, a, b=0):
        heapq.heappush(pending, (t, seq[0], kind, a, b))
        seq[0] += 1

    sched = None

    def on_run(job, stage, is_mem):
        now = sched.now
        spec = job.typ.stages[stage]
        if is_mem:
            post(now + 3.0 + rng.random() * 5.0, 3, job.id)
            return
        dur = 2.0 + rng.random() * 20.0 + spec.blocks * 0.01
        t_start = now + 1.5 + rng.random()
        for n in notifier_records(spec.blocks):
            t_start += rng.random() * 0.2
            post(t_start, 1, job.id, n)
        t_end = max(t_start, now + dur)
        for n in notifier_records(spec.blocks):
            t_end += rng.random() * 0.2
            post(t_end, 2, job.id, n)

    sched = RefSchedulerFull3(types, num_streams, unfair, extra_kernels, totals, on_run)
    t = 0.0
    weights = type_weights or [1.0] * len(types)
    for _ in range(num_jobs):
        t += rng.expovariate(1.0 / mean_iat)
        post(t, 0, rng.choices(range(len(types)), weights)[0])

    events = []
    while pending:
        tm, _, kind, a, b = heapq.heappop(pending)
        sched.now = tm
        sched.event_index = len(events)
        events.append((kind, a, b, tm))
        if kind == 0:
            sched.new_job(a)
        elif kind == 1:
            sched.handle_block_start(a, b)
        elif kind == 2:
            sched.handle_block_finish(a, b)
        else:
            sched.handle_mem_finish(a)
    return events, sched.decisions, sched.finished


def model_like_type(rng, n_kernels, big=False):
    """H2D copy, n kernels, D2H copy with pre-notify: the adapters' stage protocol."""
    st = [StageSpec(True, False)]
    for _ in range(n_kernels):
        blocks = rng.choice([1, 5, 13, 16, 17, 48, 148, 333]) * (40 if big else 1)
        st.append(StageSpec(False, False, blocks, rng.choice([128, 160, 256]), rng.choice([0, 4096, 49152, 98304]),
                            rng.choice([32, 40, 64])))
    st.append(StageSpec(True, True))
    return st


def jain_index(xs):
    """(sum x)^2 / (n sum x^2): tools/calculate_jains_fairness_index.py:17-21"""
    xs = list(xs)
    return (sum(xs) ** 2) / (len(xs) * sum(x * x for x in xs)) if xs else math.nan
