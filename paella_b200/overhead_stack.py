"""Where a job's latency goes, from a server's job-event timeline.

Input: "<prefix>_job_events.txt" as written by pb_server_profiler_cmd(SAVE) / llis_server on a SAVE
command: one line per finished job, "code time_us" pairs with the codes of the reference's
Profiler::JobEvent (include/llis/server/profiler.h:15-23).  Output: the six means of the reference's
tools/calculate_overhead_stack.py:36-96 (IPC latency only when client send times are given), computed
by the same event-pair rules, as a dict / one CSV line; jobs with ragged lines are handled (that tool
needs every job to have the same number of events).  No plotting.

    python -m paella_b200.overhead_stack run_job_events.txt [--send-times send.txt] [--min-events N]
"""
import argparse
import json
from enum import IntEnum


class JobEvent(IntEnum):
    JOB_SUBMITTED = 0
    KERNEL_SCHED_START = 1
    KERNEL_SCHED_ABORT = 2
    KERNEL_SUBMIT_START = 3
    KERNEL_SUBMIT_END = 4
    KERNEL_FINISHED = 5
    JOB_FINISHED = 6


def read_job_events(path):
    jobs = []
    with open(path) as f:
        for line in f:
            v = line.split()
            if len(v) < 2:
                continue
            jobs.append([(int(v[i]), float(v[i + 1])) for i in range(0, len(v) - 1, 2)])
    return jobs


def job_stack(events, send_time=None):
    """The six components of one job, microseconds."""
    ipc = queueing = None
    sched = launch = runtime = interval = 0.0
    prev_e = prev_t = None
    last_finish = None
    for e, t in events:
        if prev_e is None and e == JobEvent.JOB_SUBMITTED and send_time is not None:
            ipc = t - send_time
        if prev_e == JobEvent.JOB_SUBMITTED and e == JobEvent.KERNEL_SCHED_START:
            queueing = t - prev_t
        if prev_e == JobEvent.KERNEL_SCHED_START and e in (JobEvent.KERNEL_SCHED_ABORT, JobEvent.KERNEL_SUBMIT_START):
            sched += t - prev_t
        if prev_e == JobEvent.KERNEL_SUBMIT_START and e == JobEvent.KERNEL_SUBMIT_END:
            launch += t - prev_t
        if prev_e == JobEvent.KERNEL_SUBMIT_END and e == JobEvent.KERNEL_FINISHED:
            runtime += t - prev_t
        if e == JobEvent.KERNEL_FINISHED:
            last_finish = t
        if e == JobEvent.KERNEL_SUBMIT_START and last_finish is not None:
            interval += t - last_finish
        prev_e, prev_t = e, t
    total = events[-1][1] - events[0][1] if events else 0.0
    return {"ipc_latency": ipc, "queueing_delay": queueing or 0.0, "scheduling_overhead": sched,
            "kernel_launch_overhead": launch, "kernel_runtime": runtime, "kernel_interval": interval, "total": total,
            "stages": sum(1 for e, _ in events if e == JobEvent.KERNEL_SUBMIT_START)}


def overhead_stack(jobs, send_times=None, min_events=0, stages=None):
    """Means over the jobs (optionally only those with `stages` scheduler stages, e.g. one model of a mix)."""
    rows = []
    for i, ev in enumerate(jobs):
        if len(ev) < max(2, min_events):
            continue
        r = job_stack(ev, send_times[i] if send_times is not None else None)
        if stages is not None and r["stages"] != stages:
            continue
        rows.append(r)
    if not rows:
        return {"jobs": 0}
    keys = ["queueing_delay", "scheduling_overhead", "kernel_launch_overhead", "kernel_runtime", "kernel_interval", "total"]
    out = {"jobs": len(rows), "unit": "us"}
    for k in keys:
        out[k] = round(sum(r[k] for r in rows) / len(rows), 3)
    if send_times is not None:
        out["ipc_latency"] = round(sum(r["ipc_latency"] or 0.0 for r in rows) / len(rows), 3)
    out["stages_per_job"] = round(sum(r["stages"] for r in rows) / len(rows), 2)
    return out


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("job_events")
    ap.add_argument("--send-times", default=None, help="one client send time (us, same clock) per job line")
    ap.add_argument("--min-events", type=int, default=0)
    ap.add_argument("--stages", type=int, default=None, help="only jobs with this many scheduler stages")
    a = ap.parse_args()
    st = [float(x) for x in open(a.send_times).read().split()] if a.send_times else None
    print(json.dumps(overhead_stack(read_job_events(a.job_events), st, a.min_events, a.stages)))
