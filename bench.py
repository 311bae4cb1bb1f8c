#!/usr/bin/env python
"""Serving benchmark: mixed MNIST + Inception-v3 (9:1 by request count), requests/s and p50/p99.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

A "step" is one batch of --batch requests per GPU (default 1000: ~900 MNIST + ~100 Inception-v3)
pushed through the serving path: plugin -> scheduler -> one kernel at a time per job, released
by ring notifications.  W un-timed warm-up steps are fully drained, then exactly K steps are
timed between a device synchronise on both sides (CUDA events, max over GPUs/ranks).

  value : req/s with request inputs already resident in HBM (copy stages skipped)
  e2e   : the same through host buffers: pinned H2D copy of every input and D2H copy of every
          result inside the timed region
  roofline     : the tcgen05 implicit-GEMM convolution over the Inception-v3 layers, timed here
                 with CUDA events (L2 flushed before every launch)
  cpu_baseline : the CPU oracle (fp32, OpenMP) on a bounded sample of the same mix

Under torchrun (WORLD_SIZE > 1) every rank drives the GPU LOCAL_RANK with its own scheduler and
pools; there is no data-path collective.  Ranks meet at a gloo barrier before the timed region
and reduce (max time, sum requests) after it.  Without torchrun, --gpus N runs N replicas as
threads of this process.
"""
import argparse
import ctypes as C
import json
import os
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "requests/s at p99 SLO, mixed MNIST + Inception-v3 (9:1)"
WORKLOADS = {
    # the headline configuration
    "mix": [("tvm_mnist", "mnist", 0.9), ("tvm_inception_v3", "inception_v3", 0.1)],
    # single-model configuration
    "resnet18": [("tvm_resnet18", "resnet18", 1.0)],
    # the two halves of the headline mix, each alone (to see which one bounds the mix)
    "mnist": [("tvm_mnist", "mnist", 1.0)],
    "inception_v3": [("tvm_inception_v3", "inception_v3", 1.0)],
    # further model adapters, each alone
    "resnet34": [("tvm_resnet34", "resnet34", 1.0)],
    "googlenet": [("tvm_googlenet", "googlenet", 1.0)],
    "squeezenet1_1": [("tvm_squeezenet1_1", "squeezenet1_1", 1.0)],
    "densenet121": [("tvm_densenet121", "densenet121", 1.0)],
    "arcfaceresnet100": [("tvm_arcfaceresnet100", "arcfaceresnet100", 1.0)],
    "ultraface320": [("tvm_ultraface320", "ultraface320", 1.0)],
    # the reference's face pipeline mix (tools/run_ultraface_arcface.sh:27): detector 0.7, embedding 0.3
    "ultraface_arcface": [("tvm_ultraface320", "ultraface320", 0.7), ("tvm_arcfaceresnet100", "arcfaceresnet100", 0.3)],
    # depthwise + bottleneck mix
    "mobilenet_resnet50": [("tvm_mobilenet", "mobilenet", 0.5), ("tvm_resnet50", "resnet50", 0.5)],
    # the reference's eight-model mix (sosp23_artifact/gen_data_fig11_paella.sh:81-90) and its ResNet-18 : Inception-v3
    # pair (gen_data_fig12_paella.sh:82-84): proportions here, per-model instance caps and client count in PAPER_MIXES
    "fig11": [("tvm_mobilenet", "mobilenet", 0.257), ("tvm_densenet121", "densenet121", 0.0706), ("tvm_googlenet", "googlenet", 0.0546),
              ("tvm_inception_v3", "inception_v3", 0.0138), ("tvm_resnet18", "resnet18", 0.272), ("tvm_resnet34", "resnet34", 0.168),
              ("tvm_resnet50", "resnet50", 0.0745), ("tvm_squeezenet1_1", "squeezenet1_1", 0.0895)],
    "fig12": [("tvm_resnet18", "resnet18", 0.952), ("tvm_inception_v3", "inception_v3", 0.048)],
    # scheduler stress (vec_add of 2^22 floats x 10 launches, 148-block spin kernels of 10 us / 1 ms)
    "stress": [("vec_add", None, 1 / 3), ("dummy_short", None, 1 / 3), ("dummy_long", None, 1 / 3)],
}
# instances (max outstanding) per model in the order of WORKLOADS, clients in flight, and the lognormal sigmas of the
# arrival process, as the reference's scripts give them
PAPER_MIXES = {"fig11": {"caps": [36, 10, 8, 2, 38, 24, 10, 13], "concurrency": 141, "ln_sigma": (1.5, 2.0)},
               "fig12": {"caps": [119, 6], "concurrency": 125, "ln_sigma": (1.5, 2.0)}}
MIX = WORKLOADS["mix"]
GANG, DEFERRED = 1, 0      # set from the command line


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d.get("hbm_gbs", 6650.0), d.get("bf16_tflops", 1590.0), "measured"
    return 6650.0, 1590.0, "fallback"


class ClockSampler:
    """nvidia-smi clock/throttle samples during the timed region."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.proc, self.lines = None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "200"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for ln in self.proc.stdout:
            self.lines.append(ln.strip())

    def stop(self, gpu_ids):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        sm, mx, reasons = [], [], set()
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9 or not f[0].isdigit() or int(f[0]) not in gpu_ids:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def reduce_over_ranks(dist, ms, sums):
    """Max of the per-rank elapsed time and element-wise sum of the per-rank counters (gloo, CPU tensors).
    With dist None (single process) returns its arguments."""
    if dist is None:
        return ms, list(sums)
    import torch
    t = torch.tensor([ms], dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    c = torch.tensor(list(sums), dtype=torch.float64)
    dist.all_reduce(c, op=dist.ReduceOp.SUM)
    return float(t[0]), [float(v) for v in c]


def packer_name(model):
    from paella_b200 import packer
    return packer.pack_file_name(model)


def write_packs(models_dir):
    from paella_b200 import packer
    graphs = {}
    for _, model, _ in MIX:
        if model is None:
            continue
        g = packer.MODELS[model](seed=1234)
        g.save(os.path.join(models_dir, packer.pack_file_name(model)))
        graphs[model] = g
    return graphs


def run_load(L, capi, devices, batch, steps, warmup, resident, concurrency, caps, iat_us=0.0, seed=1, extra_kernels=2, mix=None,
             sched="full3", streams=500, gang=None, deferred=None, samples_per_type=0, cpus=None, ln_sigma=0.0):
    """One load-generator run (one replica thread per entry of `devices`).  Returns the result struct and, with
    samples_per_type > 0, the sampled request slots [(type index, slot, input float32 array, output float32 array)]."""
    import numpy as np
    mix = mix or MIX
    cfg = capi.LoadgenConfig()
    L.pb_loadgen_config_default(C.byref(cfg))
    cfg.num_gpus = len(devices)
    for i, d in enumerate(devices):
        cfg.devices[i] = d
        cfg.cpu_of_replica[i] = cpus[i] if cpus else -1
    cfg.num_types = len(mix)
    for i, (job, model, prop) in enumerate(mix):
        cfg.plugin_paths[i] = capi.plugin_path(job).encode()
        cfg.proportions[i] = prop
        cfg.max_outstanding[i] = caps[i]
        cfg.input_uniform[i] = 1 if model == "mnist" else 0      # U[0,1) images for MNIST, N(0,1) for the others
    cfg.concurrency = concurrency
    cfg.mean_interarrival_us = iat_us
    cfg.lognormal_sigma = ln_sigma
    cfg.num_jobs = max(1, int(batch * steps))
    cfg.warmup_jobs = int(batch * warmup)
    cfg.seed = seed
    cfg.device_resident = 1 if resident else 0
    cfg.server.num_streams = streams
    cfg.server.scheduler = sched.encode()
    cfg.server.extra_kernels = extra_kernels
    cfg.server.max_gang = GANG if gang is None else gang
    cfg.server.deferred_schedule = DEFERRED if deferred is None else deferred
    buf = None
    if samples_per_type and not resident:
        buf = np.zeros(len(mix) * samples_per_type * (1 << 21) // 4, np.float32)      # <= 2 MB per sample
        cfg.samples_per_type = samples_per_type
        cfg.sample_buf = buf.ctypes.data
        cfg.sample_buf_bytes = buf.nbytes
    res = capi.LoadgenResult()
    capi.check(L.pb_loadgen_run(C.byref(cfg), C.byref(res)), "pb_loadgen_run")
    if res.errors:
        raise RuntimeError(f"{res.errors} requests reported an error")
    if buf is None:
        return res
    raw, off, samples = buf.view(np.uint8), 0, []
    for _ in range(res.samples):
        t, slot = (int(v) for v in raw[off:off + 8].view(np.uint32))
        nin, nout = (int(v) for v in raw[off + 8:off + 24].view(np.uint64))
        pin, pout = (nin + 7) // 8 * 8, (nout + 7) // 8 * 8
        x = raw[off + 24:off + 24 + nin].view(np.float32).copy()
        y = raw[off + 24 + pin:off + 24 + pin + nout].view(np.float32).copy()
        samples.append((t, slot, x, y))
        off += 24 + pin + pout
    return res, samples


def roofline_leg(L, capi, models_dir, iters=20, only="", batch=1):
    """Times every stage of Inception-v3 alone, at the batch the serving path runs it with (a gang of `batch`
    requests per launch), L2 flushed before every launch.  The tensor-core convolutions are timed through
    pb_conv_umma_time on the kernel the stage graphs use (the persistent one); the other kinds through the
    instance.  Returns the convolution aggregate and a per-kind table."""
    from paella_b200 import packer
    hbm, tf, how = measured_peaks()
    model, inst = C.c_void_p(), C.c_void_p()
    path = os.path.join(models_dir, packer.pack_file_name("inception_v3"))
    capi.check(L.pb_model_load(path.encode(), 0, 1, C.byref(model)), "pb_model_load")
    capi.check(L.pb_instance_create_batched(model, batch, 0, C.byref(inst)), "pb_instance_create_batched")
    li, us = capi.LaunchInfo(), C.c_double()
    per_kind = {}
    layers = []
    persist = os.environ.get("PB_CONV_PERSIST", "0") == "1"
    for s in range(L.pb_model_num_stages(model)):
        capi.check(L.pb_model_stage_info_batched(model, s, batch, C.byref(li)), "pb_model_stage_info_batched")
        name = L.pb_model_stage_name(model, s).decode()
        if only and only not in name:
            continue
        k = capi.STAGE_NAMES[li.kind]
        if li.kind == capi.STAGE_CONV_UMMA:
            p = capi.OpParams()
            capi.check(L.pb_instance_stage_params(inst, s, batch, C.byref(p)), "pb_instance_stage_params")
            capi.check(L.pb_conv_umma_time(C.byref(p), 1 if persist else 0, iters, 192 << 20, C.byref(us)), "pb_conv_umma_time")
        else:
            capi.check(L.pb_instance_time_stage_batched(inst, s, batch, iters, 192 << 20, C.byref(us)), "pb_instance_time_stage_batched")
        d = per_kind.setdefault(k, {"launches": 0, "us": 0.0, "flops": 0, "bytes": 0})
        d["launches"] += 1; d["us"] += us.value; d["flops"] += li.flops; d["bytes"] += li.bytes
        layers.append((name, k, us.value, li.flops, li.bytes, li.num_blocks))
    L.pb_instance_destroy(inst)
    L.pb_model_destroy(model)
    conv = per_kind.get("conv_umma", {"launches": 0, "us": 1.0, "flops": 0, "bytes": 0})
    achieved = conv["flops"] / (conv["us"] * 1e-6) / 1e12 if conv["launches"] else 0.0
    total_us = sum(d["us"] for d in per_kind.values())
    # DRAM bytes per launch, from the ncu captures summarised in profiles/conv_umma_tma_kernel__inception_v3_layers.md:
    # 1 image per launch: the mean over the Mixed_* layers (818 185 B against 856 300 B algorithmic); 8 images per
    # launch: the captured layer's ratio of DRAM traffic to algorithmic bytes (3.91 MB / 4.73 MB: the output stays in
    # L2), scaled to this leg's mean algorithmic bytes per launch.  Other batches: no capture, null.
    alg_per_launch = conv["bytes"] / max(conv["launches"], 1)
    traffic = None
    if not only and batch == 1:
        traffic = 818185
    elif not only and batch == 8:
        traffic = int(alg_per_launch * 3.912704 / 4.73472)
    kern = ("conv_umma_persist_kernel (tcgen05 implicit GEMM, TMA im2col, several tiles per CTA, two TMEM accumulators)" if persist
            else "conv_umma_tma_kernel (tcgen05 implicit GEMM, TMA im2col, one tile per CTA)")
    roof = {"bound": "tensor", "kernel": f"{kern}: every Inception-v3 conv layer launched alone, {batch} image(s) per launch as served, L2 flushed",
            "achieved": round(achieved, 3), "peak": tf, "unit": "TFLOP/s", "frac": round(achieved / tf, 5), "of": how,
            "traffic": traffic, "algorithmic_bytes_per_launch": int(conv["bytes"] / max(conv["launches"], 1)),
            "launches": conv["launches"], "avg_launch_us": round(conv["us"] / max(conv["launches"], 1), 3),
            "images_per_launch": batch,
            "hbm_gbs_same_kernel": round(conv["bytes"] / (conv["us"] * 1e-6) / 1e9, 1),
            "time_share_of_request": round(conv["us"] / total_us, 4) if total_us else None}
    table = {k: {"launches": d["launches"], "us": round(d["us"], 2), "share": round(d["us"] / total_us, 4),
                 "gbs": round(d["bytes"] / (d["us"] * 1e-6) / 1e9, 1), "tflops": round(d["flops"] / (d["us"] * 1e-6) / 1e12, 3)}
             for k, d in per_kind.items()}
    return roof, table, layers


def fairness_leg(L, capi, device, mix, mixed_result, cpus=None):
    """Jain's index over per-model slowdowns (mean latency in the mix / mean latency alone, one client):
    tools/calculate_jains_fairness_index.py:17-21 of the reference."""
    iso, slow = {}, []
    for i, (job, model, _) in enumerate(mix):
        r = run_load(L, capi, [device], 60 if model != "mnist" else 300, 1, 0.2, False, 1, [1], mix=[(job, model, 1.0)], gang=1, cpus=cpus)
        iso[model or job] = r.all.mean_us
        slow.append(mixed_result.per_type[i].mean_us / r.all.mean_us)
    jain = (sum(slow) ** 2) / (len(slow) * sum(x * x for x in slow))
    return {"jain_index": round(jain, 4), "slowdown": {(m or j): round(x, 3) for (j, m, _), x in zip(mix, slow)},
            "isolated_mean_us": {k: round(v, 1) for k, v in iso.items()}}


def extras_leg(L, capi, device):
    """Ring round trip, vec_add bandwidth, scheduler decisions/s under the synthetic stress mix."""
    hbm, _, how = measured_peaks()
    n = 2000
    rtt = (C.c_double * n)()
    capi.check(L.pb_ring_roundtrip_bench(device, n, rtt), "pb_ring_roundtrip_bench")
    v = sorted(rtt[100:])
    out = {"ring_roundtrip_us": {"p50": round(v[len(v) // 2], 2), "p99": round(v[int(len(v) * 0.99)], 2), "min": round(v[0], 2),
                                 "note": "host ping (mapped memory) -> one-thread kernel -> record -> host poll; sum of both directions"}}
    us = C.c_double()
    va = {}
    for lg in (20, 22, 24, 26):
        capi.check(L.pb_vec_add_bench(device, 1 << lg, 10, 192 << 20, C.byref(us)), "pb_vec_add_bench")
        gbs = 12.0 * (1 << lg) / (us.value * 1e-6) / 1e9
        va[f"2^{lg}"] = {"us": round(us.value, 2), "GB/s": round(gbs, 1), "frac_of_hbm_peak": round(gbs / hbm, 4)}
    out["vec_add"] = {"bytes_per_element": 12, "peak_GB/s": hbm, "of": how, "sizes": va}
    return out


def membound_leg(L, capi, device, scale="large", iters=10):
    """The memory-bound operator kernels (depthwise convolution, pooling, elementwise, GEMV, layout
    conversion, vec_add) on tensors larger than the 126 MB L2, through pb_op_launch, timed with CUDA events.

    The batch-1 tensors of the served models are a few MB: at that size these kernels are launch- and
    latency-bound whatever their code does.  This leg answers the other question, whether the kernels
    themselves stream at HBM speed: bf16 channels-last tensors of 128 channels x H x W, every launch
    reading and writing more than the L2 holds, algorithmic bytes (each input and output once, from
    pb_op_info) over the CUDA-event time, against the measured copy bandwidth."""
    import torch
    hbm, _, how = measured_peaks()
    torch.cuda.set_device(device)
    hw = 1024 if scale == "large" else 768          # 128 ch x hw^2 x 2 B = 256 MB / 144 MB per tensor
    Cc = 128
    dev = torch.device("cuda", device)
    x = torch.randn(hw * hw * Cc, device=dev, dtype=torch.float32).to(torch.bfloat16)
    x2 = torch.randn(hw * hw * Cc, device=dev, dtype=torch.float32).to(torch.bfloat16)
    y = torch.empty(hw * hw * Cc, device=dev, dtype=torch.bfloat16)
    w9 = torch.randn(9 * Cc, device=dev, dtype=torch.float32).to(torch.bfloat16)
    fb = torch.randn(Cc, device=dev, dtype=torch.float32)
    fs = torch.randn(Cc, device=dev, dtype=torch.float32)

    def prm(kind, R=1, S=1, st=1, pad=0, groups=1, act=0, flags=0):
        p = capi.OpParams()
        p.dtype = 1
        p.C, p.H, p.W, p.Cs = Cc, hw, hw, Cc
        P = (hw + 2 * pad - R) // st + 1
        p.K, p.P, p.Q, p.Ks = Cc, P, P, Cc
        p.R, p.S, p.stride_h, p.stride_w, p.pad_h, p.pad_w, p.groups = R, S, st, st, pad, pad, groups
        p.act, p.flags = act, flags
        p.x, p.y = x.data_ptr(), y.data_ptr()
        return p

    cases = []
    p = prm(capi.STAGE_DWCONV, 3, 3, 1, 1, groups=Cc, act=2); p.w, p.bias = w9.data_ptr(), fb.data_ptr()
    cases.append(("dwconv 3x3 s1 (+bias, ReLU6)", capi.STAGE_DWCONV, p))
    p = prm(capi.STAGE_DWCONV, 3, 3, 2, 1, groups=Cc, act=2); p.w, p.bias = w9.data_ptr(), fb.data_ptr()
    cases.append(("dwconv 3x3 s2 (+bias, ReLU6)", capi.STAGE_DWCONV, p))
    cases.append(("maxpool 3x3 s2", capi.STAGE_MAXPOOL, prm(capi.STAGE_MAXPOOL, 3, 3, 2, 0)))
    cases.append(("maxpool 2x2 s2", capi.STAGE_MAXPOOL, prm(capi.STAGE_MAXPOOL, 2, 2, 2, 0)))
    cases.append(("avgpool 3x3 s1 p1", capi.STAGE_AVGPOOL, prm(capi.STAGE_AVGPOOL, 3, 3, 1, 1, flags=1)))
    p = prm(capi.STAGE_ADD, act=1); p.residual, p.res_Cs = x2.data_ptr(), Cc
    cases.append(("add (+ReLU)", capi.STAGE_ADD, p))
    p = prm(capi.STAGE_AFFINE, act=1); p.w, p.bias = fs.data_ptr(), fb.data_ptr()
    cases.append(("affine (batch-norm + ReLU)", capi.STAGE_AFFINE, p))
    # GEMV: rows x cols bf16 weights = the x2 buffer; input vector = head of x; fp32 results into y
    cols = 16384
    rows = (hw * hw * Cc) // cols
    p = capi.OpParams()
    p.dtype, p.C, p.H, p.W, p.Cs, p.K, p.P, p.Q, p.Ks = 1, cols, 1, 1, cols, rows, 1, 1, rows
    p.R = p.S = p.stride_h = p.stride_w = p.groups = 1
    p.x, p.w, p.y = x.data_ptr(), x2.data_ptr(), y.data_ptr()
    cases.append((f"dense GEMV {rows}x{cols}", capi.STAGE_DENSE, p))
    # NCHW fp32 -> channels-last bf16 (3 channels padded to 8): input = x viewed as fp32
    # the output (8 bf16 per pixel = 16 B) is the larger side and has to fit y
    side = int(((hw * hw * Cc * 2) // 16) ** 0.5) // 16 * 16
    p = capi.OpParams()
    p.dtype, p.C, p.H, p.W, p.Cs, p.K, p.P, p.Q, p.Ks = 1, 3, side, side, 8, 3, side, side, 8
    p.R = p.S = p.stride_h = p.stride_w = p.groups = 1
    p.x, p.y = x.data_ptr(), y.data_ptr()
    cases.append((f"input layout 3x{side}x{side} fp32 -> channels-last bf16", capi.STAGE_INPUT, p))

    out = {}
    li = capi.LaunchInfo()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for name, kind, p in cases:
        capi.check(L.pb_op_info(kind, C.byref(p), C.byref(li)), "pb_op_info")
        for _ in range(3):
            capi.check(L.pb_op_launch(kind, C.byref(p), None, 0, None), name)
        torch.cuda.synchronize(device)
        e0.record()
        for _ in range(iters):
            capi.check(L.pb_op_launch(kind, C.byref(p), None, 0, None), name)
        e1.record()
        torch.cuda.synchronize(device)
        us = e0.elapsed_time(e1) * 1000.0 / iters
        gbs = li.bytes / (us * 1e-6) / 1e9
        out[name] = {"us": round(us, 1), "algorithmic_MB": round(li.bytes / 1e6, 1), "GB/s": round(gbs, 1),
                     "frac_of_hbm_peak": round(gbs / hbm, 4)}
    del x, x2, y
    torch.cuda.empty_cache()
    us = C.c_double()
    n = 1 << (26 if scale == "large" else 25)
    capi.check(L.pb_vec_add_bench(device, n, iters, 0, C.byref(us)), "pb_vec_add_bench")
    gbs = 12.0 * n / (us.value * 1e-6) / 1e9
    out[f"vec_add 2^{n.bit_length() - 1} fp32"] = {"us": round(us.value, 1), "algorithmic_MB": round(12.0 * n / 1e6, 1),
                                                  "GB/s": round(gbs, 1), "frac_of_hbm_peak": round(gbs / hbm, 4)}
    return {"what": f"bf16 channels-last tensors of {Cc} x {hw} x {hw} ({hw * hw * Cc * 2 >> 20} MB each, larger than L2), "
                    f"{iters} launches back to back after 3 warm-up launches, CUDA events",
            "peak_GB/s": hbm, "of": how, "kernels": out}


def ipc_leg(capi, models_dir, rates=(50000, 75000, 100000)):
    """The same mix through the PROCESS boundary: a llis_server process on GPU 0 and the llis_app_client load
    generator (open loop, Poisson) talking to it over the shared-memory rings and the pinned request pool."""
    bindir = os.path.join(os.path.dirname(capi.LIB_PATH), "bin")
    name = f"pbbench{os.getpid()}"
    env = dict(os.environ, LLIS_MODELS_DIR=models_dir, CUDA_DEVICE_MAX_CONNECTIONS="32")
    srv = subprocess.Popen([os.path.join(bindir, "llis_server"), "--name", name, "--sched", "full3", "--num_streams", "128",
                            "--extra_kernels", "64", "--gpu", "0"], env=env, stderr=subprocess.PIPE, text=True)
    out = []
    try:
        t0 = time.time()
        while not os.path.exists(f"/dev/shm/llis:channel:c2s:{name}"):
            if srv.poll() is not None or time.time() - t0 > 60:
                return {"error": "llis_server did not come up"}
            time.sleep(0.05)
        for rate in rates:
            prefix = os.path.join(models_dir, f"ipc_{rate}")
            n = 30000
            r = subprocess.run([os.path.join(bindir, "llis_app_client"), "--server_name", name, "--iat", f"{1e6 / rate:.3f}",
                                "--concurrency", "96", "--num_jobs", str(n), "--start_record_num", "3000", "--seed", "1", "--prefix", prefix,
                                capi.plugin_path("tvm_mnist"), "0.9", "64", capi.plugin_path("tvm_inception_v3"), "0.1", "32"],
                               capture_output=True, text=True, timeout=120, env=env)
            if r.returncode != 0:
                out.append({"offered_rps": rate, "error": r.stderr[-300:]})
                continue
            f = open(prefix + ".txt").read().strip().split(",")
            # iat, jobs, elapsed_us, then mean,p50,p90,p95,p99,max,sd overall / MNIST / Inception-v3
            out.append({"offered_rps": rate, "achieved_rps": round(n / (float(f[2]) * 1e-6)),
                        "mnist_p50_p99_us": [round(float(f[11])), round(float(f[14]))],
                        "inception_v3_p50_p99_us": [round(float(f[18])), round(float(f[21]))]})
    finally:
        if srv.poll() is None:
            srv.terminate()
            try:
                srv.wait(10)
            except subprocess.TimeoutExpired:
                srv.kill()
    return {"what": "llis_server process + llis_app_client process (open loop, Poisson), 9:1 MNIST : Inception-v3, one GPU", "points": out}


def cpu_sample(graphs, samples=None, names=None, repeats=3):
    """Oracle (CPU fp32, OpenMP over all cores) on a bounded sample of the mix; returns req/s of the 9:1 mix, the
    seconds spent, the requests run and - when `samples` (sampled request slots of the GPU run) are given - the
    comparison of the serving path's outputs with the oracle's on the same inputs."""
    # torchrun pins OMP_NUM_THREADS=1 in its workers; the CPU leg is meant to use every host core
    os.environ["OMP_NUM_THREADS"] = str(os.cpu_count() or 1)
    import numpy as np
    from oracle import graph as og
    og.build()
    packs = {m: og.Pack(g.to_bytes()) for m, g in graphs.items()}
    shapes = {"mnist": (1, 28, 28), "inception_v3": (3, 299, 299)}
    rng = np.random.default_rng(0)
    inputs = {"mnist": [], "inception_v3": []}
    gpu_out = {"mnist": [], "inception_v3": []}
    for (t, slot, x, y) in (samples or []):
        m = names[t]
        if m in inputs:
            inputs[m].append(x.reshape(shapes[m])); gpu_out[m].append(y)
    have_samples = all(len(v) > 0 for v in inputs.values())
    if not have_samples:
        inputs = {"mnist": [rng.random((1, 28, 28), dtype=np.float32)], "inception_v3": [rng.standard_normal((3, 299, 299), dtype=np.float32)]}
    og.run(packs["mnist"], inputs["mnist"][0])
    t_model, n = {}, 0
    refs = {"mnist": [], "inception_v3": []}
    t_all0 = time.perf_counter()
    for m in ("mnist", "inception_v3"):
        reps = repeats * (9 if m == "mnist" else 1)
        t0 = time.perf_counter()
        for r in range(reps):
            for x in inputs[m]:
                y = og.run(packs[m], x); n += 1
                if r == 0:
                    refs[m].append(y)
        t_model[m] = (time.perf_counter() - t0) / (reps * len(inputs[m]))
    dt = time.perf_counter() - t_all0
    rps = 10.0 / (9 * t_model["mnist"] + t_model["inception_v3"])
    parity = {}
    if have_samples:
        rel, same = {}, True
        for m in refs:
            worst = 0.0
            for y, ref in zip(gpu_out[m], refs[m]):
                worst = max(worst, float(np.abs(y - ref).max() / max(float(np.abs(ref).max()), 1e-30)))
                same = same and int(y.argmax()) == int(ref.argmax())
            rel[m] = worst
        tol = {"mnist": 1e-5, "inception_v3": 1e-2}
        parity = {"parity_checked": sum(len(v) for v in refs.values()),
                  "parity_max_rel": {m: float(f"{v:.3g}") for m, v in rel.items()},
                  "parity_argmax_equal": bool(same),
                  "parity_ok": bool(same and all(rel[m] <= tol[m] for m in rel)),
                  "parity_what": "outputs left in sampled request slots by the timed closed-loop host-buffer run vs the CPU oracle on the same "
                                 "slot inputs; tolerance 1e-5 (MNIST, fp32) / 1e-2 of the largest logit and same argmax (Inception-v3, bf16)"}
    return rps, dt, n, parity


def pick_cpu(device, index):
    """A CPU of the GPU's NUMA node for replica `index` (reads sysfs only): the i-th allowed CPU of the node's list, skipping
    its first one.  -1 (no pinning) when the topology cannot be read."""
    try:
        out = subprocess.run(["nvidia-smi", "--query-gpu=index,pci.bus_id", "--format=csv,noheader"], capture_output=True, text=True, timeout=20).stdout
        bdf = None
        for ln in out.splitlines():
            f = [x.strip() for x in ln.split(",")]
            if len(f) == 2 and f[0].isdigit() and int(f[0]) == device:
                bdf = f[1].lower()
        if bdf is None:
            return -1
        if bdf.startswith("00000000:"):
            bdf = bdf[4:]
        txt = open(f"/sys/bus/pci/devices/{bdf}/local_cpulist").read().strip()
        local = []
        for part in txt.split(","):
            a, _, b = part.partition("-")
            local += list(range(int(a), int(b or a) + 1))
        allowed = sorted(set(local) & set(os.sched_getaffinity(0))) or sorted(os.sched_getaffinity(0))
        if len(allowed) < 2:
            return -1
        # ranks that share a node must not share a core: spread by the GPU index as well
        return allowed[(1 + 2 * (device + index)) % len(allowed)]
    except Exception:
        return -1


def granularity_sweep(args):
    """Scheduling granularity on the same kernels: layers per scheduler stage (PB_STAGE_GROUP), one child process per
    point because the grouping is fixed when a model is loaded.  1 = one kernel per stage with H2D / D2H copy stages,
    the reference's protocol."""
    pts = []
    for g in (1, 4, 12, 24, 48):
        env = dict(os.environ, PB_STAGE_GROUP=str(g))
        if g == 1:
            env["PB_COPY_STAGES"] = "1"
        cmd = [sys.executable, os.path.abspath(__file__), "--granularity-child", str(g), "--steps", "3", "--warmup", "3",
               "--batch", str(1000 if g == 1 else 4000), "--gang", str(1 if g == 1 else args.gang), "--concurrency", str(args.concurrency),
               "--inception-instances", str(args.inception_instances), "--extra-kernels", "64", "--sched", args.sched]
        try:
            r = subprocess.run(cmd, capture_output=True, text=True, timeout=180, env=env)
            pts.append(json.loads(r.stdout.strip().splitlines()[-1]) if r.returncode == 0 and r.stdout.strip() else
                       {"layers_per_stage": g, "error": (r.stderr or "no output")[-200:]})
        except Exception as e:      # a point that fails does not take the headline down with it
            pts.append({"layers_per_stage": g, "error": str(e)[:200]})
    return {"what": "closed loop, host buffers, same mix and clients; layers_per_stage = 1 also restores the H2D / D2H copy stages "
                    "(the reference's protocol: one scheduler decision and one set of block records per kernel)", "points": pts}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--batch", type=int, default=0, help="requests per GPU per step (default 12000 for the mix, so that 20 steps last about a second)")
    ap.add_argument("--concurrency", type=int, default=0, help="clients per replica: requests in flight at most (closed loop: always); default 192 "
                                                                 "(fig11: 141, fig12: 125, the reference's)")
    ap.add_argument("--inception-instances", type=int, default=96, help="Inception-v3 instances (max outstanding) per replica")
    ap.add_argument("--replicas-per-gpu", type=int, default=1,
                    help="independent scheduler+pool replicas (one busy-polling host thread each) sharing every GPU")
    ap.add_argument("--extra-kernels", type=int, default=0,
                    help="scheduler: over-subscribed stages allowed in flight (--extra_kernels); default 18 for the headline mix (under Poisson "
                         "arrivals the gate makes requests queue into gangs when the GPU is busy: measured best of 6..64), 64 otherwise")
    ap.add_argument("--sched", default="full3", choices=["full3", "fifo", "fifo2"],
                    help="full3 = the kernel-level scheduler; fifo (job by job) and fifo2 (stage by stage, arrival order) are the ablations")
    ap.add_argument("--streams", type=int, default=500, help="scheduler stream pool (--num_streams); 1 with --sched fifo = single-stream baseline")
    ap.add_argument("--gang", type=int, default=8, help="scheduler: up to this many queued requests of one model run as one launch per stage (1 = never)")
    ap.add_argument("--deferred", type=int, default=0, help="scheduler: 1 = dispatch loop once per batch of notifications (implied by --gang > 1)")
    ap.add_argument("--workload", default="mix", choices=sorted(WORKLOADS), help="mix = the headline (MNIST : Inception-v3 = 9 : 1)")
    ap.add_argument("--extras", action="store_true", help="also measure ring round trip and vec_add bandwidth")
    ap.add_argument("--iat-us", type=float, default=0.0, help="open loop: mean inter-arrival per replica in us (Poisson); 0 = closed loop")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-roofline", action="store_true")
    ap.add_argument("--no-fairness", action="store_true", help="skip the isolated runs behind Jain's index")
    ap.add_argument("--no-sweep", action="store_true", help="skip the open-loop Poisson rate sweep of the mix (headline = closed loop)")
    ap.add_argument("--no-granularity", action="store_true", help="skip the layers-per-scheduler-stage sweep (child processes)")
    ap.add_argument("--no-membound", action="store_true", help="skip the memory-bound operator kernels on tensors larger than L2")
    ap.add_argument("--no-pin", dest="pin", action="store_false", help="do not pin the replica threads to CPUs of their GPU's NUMA node")
    ap.add_argument("--parity-samples", type=int, default=4, help="request slots per model whose outputs are compared with the CPU oracle")
    ap.add_argument("--granularity-child", type=int, default=None, help=argparse.SUPPRESS)
    ap.add_argument("--layers", default="", help="write the per-layer timing table to this file")
    ap.add_argument("--only-roofline", default=None, metavar="SUBSTR",
                    help="skip the serving legs; time only the Inception-v3 stages whose name contains SUBSTR "
                         "('' = all).  Small enough to run under ncu.")
    ap.add_argument("--iters", type=int, default=20, help="timed launches per stage in the roofline leg")
    ap.add_argument("--only-membound", default=None, choices=["large", "small"],
                    help="skip the serving legs; time only the memory-bound operator kernels on tensors larger than L2 "
                         "(large: 256 MB per tensor; small: 144 MB per tensor, 3 launches each, for an ncu capture)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.batch <= 0:
        args.batch = {"mix": 12000, "mnist": 20000, "fig11": 8000, "fig12": 8000}.get(args.workload, 1500)
    paper = PAPER_MIXES.get(args.workload)
    if args.extra_kernels <= 0:
        args.extra_kernels = 18 if args.workload == "mix" else 64
    if args.concurrency <= 0:
        args.concurrency = paper["concurrency"] if paper else 192
    global MIX, GANG, DEFERRED
    MIX = WORKLOADS[args.workload]
    GANG, DEFERRED = args.gang, args.deferred
    names = [m or j for j, m, _ in MIX]

    args.replicas_per_gpu = max(1, args.replicas_per_gpu)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    wl_text = {"mix": "mixed MNIST-CNN : Inception-v3@299 = 9:1 by request count, batch 1, random He-normal weights (headline configuration)",
               "resnet18": "ResNet-18 v1, batch 1, 224x224, BN folded, random He-normal weights",
               "mnist": "MNIST-CNN alone, batch 1, 28x28, fp32",
               "inception_v3": "Inception-v3 alone, batch 1, 299x299, BN folded, random He-normal weights",
               "resnet34": "ResNet-34 v1 alone, batch 1, 224x224, BN folded, random He-normal weights",
               "googlenet": "GoogLeNet (torchvision form) alone, batch 1, 224x224, BN folded, random He-normal weights",
               "squeezenet1_1": "SqueezeNet 1.1 alone, batch 1, 224x224, random He-normal weights",
               "densenet121": "DenseNet-121 alone, batch 1, 224x224, random He-normal weights",
               "arcfaceresnet100": "ArcFace LResNet100E-IR alone, batch 1, 112x112, random He-normal weights",
               "ultraface320": "320x240 receptive-field-block face detector alone, batch 1, random He-normal weights",
               "ultraface_arcface": "face detector : ArcFace LResNet100E-IR = 0.7 : 0.3, batch 1",
               "mobilenet_resnet50": "MobileNetV2 : ResNet-50 = 1:1, batch 1, 224x224",
               "fig11": "the reference's eight-model mix by its proportions and per-model instance caps: MobileNetV2 .257, DenseNet-121 .0706, "
                        "GoogLeNet .0546, Inception-v3 .0138, ResNet-18 .272, ResNet-34 .168, ResNet-50 .0745, SqueezeNet 1.1 .0895; batch 1",
               "fig12": "ResNet-18 : Inception-v3 = 0.952 : 0.048 with the reference's instance caps (119 / 6), batch 1",
               "stress": "vec_add : dummy_short : dummy_long = 1:1:1 synthetic scheduler stress"}[args.workload]
    config = {"workload": wl_text,
              "batch_per_step_per_replica": args.batch, "clients_per_replica": args.concurrency,
              "instances_per_replica": dict(zip(names, paper["caps"])) if paper else
                                       {names[0]: args.concurrency, **({names[-1]: args.inception_instances} if len(names) > 1 else {})},
              "scheduler": args.sched, "max_gang": args.gang, "deferred_schedule": int(args.deferred or args.gang > 1), "num_streams": args.streams, "extra_kernels": args.extra_kernels, "replicas_per_gpu": args.replicas_per_gpu,
              "precision": "MNIST fp32; other models bf16 x bf16 -> fp32 (tcgen05)",
              "replicas": "one scheduler+pools per GPU, requests dealt round-robin, no collective",
              "l2": "not flushed between requests: the working set per GPU (47.6 MB of bf16 weights + 19 MB of activations "
                    "per in-flight Inception instance x instances) exceeds the 126 MB L2; the roofline leg flushes L2 "
                    "before every launch"}

    # ----------------------------------------------------------------- reference arm: CPU
    if args.impl == "reference":
        if rank != 0:
            return
        with tempfile.TemporaryDirectory() as d:
            graphs = write_packs(d)
        times, n_per = [], 10
        for _ in range(args.warmup):
            cpu_sample(graphs, repeats=1)
        for _ in range(args.steps):
            rps, dt, n_per, _ = cpu_sample(graphs, repeats=3)
            times.append(dt)
        total = sum(times)
        value = n_per * len(times) / total
        cores = os.cpu_count()
        line = {"impl": "reference", "metric": METRIC, "value": round(value, 3),
                "unit": "req/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
                "ms_per_step": round(1000 * total / len(times), 2), "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": config,
                "cpu_baseline": {"value": round(value, 3), "unit": "req/s", "cores": cores, "kind": "port",
                                 "sample": "each step = 3 x (9 MNIST + 1 Inception-v3) requests run back to back by the CPU "
                                           "oracle (fp32 C operators, OpenMP over all host cores); the reference's own "
                                           "TVM CPU build is unavailable on this box"},
                "e2e": {"value": round(value, 3), "unit": "req/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
        print(json.dumps(line))
        return

    # ----------------------------------------------------------------- our arm: GPU
    import paella_b200 as pb
    from paella_b200 import capi
    L = pb.load()
    if L.pb_device_count() < 1:
        raise SystemExit("bench.py needs a CUDA device (paella_b200 has no CPU path)")
    tmp = tempfile.TemporaryDirectory()
    os.environ["LLIS_MODELS_DIR"] = tmp.name
    graphs = write_packs(tmp.name)
    caps = [args.concurrency] * (len(MIX) - 1) + [args.inception_instances] if len(MIX) > 1 else [args.concurrency]
    if paper:
        caps = list(paper["caps"])
    if args.workload == "stress":
        os.environ.setdefault("PB_VEC_ADD_N", str(1 << 22))
        caps = [args.inception_instances] * 3

    dist = None
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("gloo", rank=rank, world_size=world)
        devices = [local_rank] * args.replicas_per_gpu
        n_gpus = world
    else:
        devices = [d for d in range(args.gpus) for _ in range(args.replicas_per_gpu)]
        n_gpus = args.gpus

    if args.only_membound is not None:
        print(json.dumps({"membound": membound_leg(L, capi, devices[0], args.only_membound,
                                                   10 if args.only_membound == "large" else 3)}))
        return
    if args.granularity_child is not None:
        # one point of the granularity sweep: closed loop through host buffers, this process's PB_STAGE_GROUP
        r = run_load(L, capi, devices[:1], args.batch, args.steps, args.warmup, False, args.concurrency, caps,
                     extra_kernels=args.extra_kernels, sched=args.sched, streams=args.streams, cpus=[pick_cpu(devices[0], 0)] if args.pin else None)
        t = max(r.host_launch_us + r.host_sched_us + r.host_idle_us, 1e-9)
        sec = r.elapsed_event_ms * 1e-3
        mh = C.c_void_p()
        capi.check(L.pb_model_load(os.path.join(tmp.name, packer_name("inception_v3")).encode(), devices[0], -1, C.byref(mh)), "pb_model_load")
        stages = L.pb_model_num_groups(mh) + (2 if os.environ.get("PB_COPY_STAGES") == "1" else 0)
        L.pb_model_destroy(mh)
        print(json.dumps({"layers_per_stage": args.granularity_child, "inception_v3_scheduler_stages": stages, "max_gang": args.gang,
                          "extra_kernels": args.extra_kernels,
                          "rps": round(r.all.count / sec),
                          "mnist_p50_p99_us": [round(r.per_type[0].p50_us), round(r.per_type[0].p99_us)],
                          "inception_v3_p50_p99_us": [round(r.per_type[1].p50_us), round(r.per_type[1].p99_us)],
                          "decisions_per_s": round(r.decisions / sec), "records_per_s": round(r.records_consumed / sec),
                          "host_time_share": {"launch": round(r.host_launch_us / t, 3), "sched": round(r.host_sched_us / t, 3),
                                              "idle": round(r.host_idle_us / t, 3)}}))
        return
    if args.only_roofline is not None:
        roof, table, layers = roofline_leg(L, capi, tmp.name, args.iters, args.only_roofline, batch=max(1, args.gang))
        print(json.dumps({"roofline": roof, "kernel_table_inception_v3": table,
                          "layers": [(n, k, round(u, 2), nb) for (n, k, u, _, _, nb) in layers]}))
        return

    cpus = None
    if args.pin:
        cpus = [pick_cpu(d, i) for i, d in enumerate(devices)]
        config["replica_cpus"] = cpus
    sampler = ClockSampler()
    load_kw = dict(extra_kernels=args.extra_kernels, sched=args.sched, streams=args.streams, cpus=cpus)
    leg_seconds = {}

    def leg(name, resident, iat_us, steps, seed=1, samples=0, warmup=None, ln_sigma=0.0):
        """One load run on every rank (barrier first); returns rank-reduced numbers."""
        import numpy as np
        if dist:
            dist.barrier()
        t0 = time.time()
        out = run_load(L, capi, devices, args.batch, steps, args.warmup if warmup is None else warmup, resident, args.concurrency, caps,
                       iat_us=iat_us, seed=seed, samples_per_type=samples, ln_sigma=ln_sigma, **load_kw)
        r, smp = out if isinstance(out, tuple) else (out, [])
        leg_seconds[name] = round(time.time() - t0, 1)
        nt = len(MIX)
        sums = [float(r.all.count), float(r.h2d_bytes), float(r.d2h_bytes), float(r.records_consumed), float(r.decisions)] + \
               [float(r.per_type[i].count) for i in range(nt)]
        ms, sums = reduce_over_ranks(dist, r.elapsed_event_ms, sums)
        # per-model tails: the worst rank's (an SLO has to hold on every GPU)
        p99 = [r.per_type[i].p99_us for i in range(nt)]
        p50 = [r.per_type[i].p50_us for i in range(nt)]
        mean = [r.per_type[i].mean_us for i in range(nt)]
        per_rank = None
        if dist:
            import torch
            t = torch.tensor(p99 + p50, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            p99, p50 = [float(v) for v in t[:nt]], [float(v) for v in t[nt:]]
            tt = max(r.host_launch_us + r.host_sched_us + r.host_idle_us, 1e-9)
            mine = torch.tensor([r.all.count / (r.elapsed_event_ms * 1e-3), r.host_launch_us / tt, r.host_sched_us / tt, r.host_idle_us / tt],
                                dtype=torch.float64)
            allr = [torch.zeros(4, dtype=torch.float64) for _ in range(world)]
            dist.all_gather(allr, mine)
            per_rank = [{"rps": round(float(a[0])), "launch": round(float(a[1]), 3), "sched": round(float(a[2]), 3), "idle": round(float(a[3]), 3)}
                        for a in allr]
        return {"r": r, "n": sums[0], "ms": ms, "rps": sums[0] / (ms * 1e-3), "h2d": sums[1], "d2h": sums[2], "records": sums[3],
                "decisions": sums[4], "counts": sums[5:], "p99": p99, "p50": p50, "mean": mean, "samples": smp, "per_rank": per_rank}

    slo = {"inception_v3_p99_ms": 5.0, "mnist_p99_ms": 1.0}
    is_mix = args.workload == "mix"

    def meets_slo(x):
        return (not is_mix) or (x["p99"][1] <= slo["inception_v3_p99_ms"] * 1e3 and x["p99"][0] <= slo["mnist_p99_ms"] * 1e3)

    def point(x, offered=None):
        d = {"achieved_rps": round(x["rps"]), "slo_met": bool(meets_slo(x))}
        if offered is not None:
            d["offered_rps"] = round(offered)
        for i, nm in enumerate(names):
            d[f"{nm}_p50_p99_us"] = [round(x["p50"][i]), round(x["p99"][i])]
        return d

    if rank == 0:
        sampler.start()
    # ---- closed loop: the capacity of the serving path, inputs resident in HBM and through host buffers ----
    closed_dev = leg("closed_resident", True, 0.0, args.steps)
    closed_e2e = leg("closed_e2e", False, 0.0, args.steps, samples=args.parity_samples if rank == 0 else 0)
    open_loop = args.iat_us > 0 or (is_mix and not args.no_sweep)
    sweep_pts = []
    head_dev, head_e2e = closed_dev, closed_e2e
    if args.iat_us > 0:
        head_dev = leg("poisson_resident", True, args.iat_us, args.steps, seed=7)
        head_e2e = leg("poisson_e2e", False, args.iat_us, args.steps, seed=7)
    elif open_loop:
        # ---- open loop (the configuration's arrivals): Poisson at fractions of the closed-loop rate, highest first; the
        # headline is the highest offered rate whose per-model p99s stay inside the SLO (the first failing point
        # above it brackets the knee).  Every point is a full K-step run timed like the others. ----
        def sweep(resident, cap_rps, tag):
            best = None
            for frac in (1.05, 1.0, 0.975, 0.95, 0.925, 0.9, 0.85, 0.8, 0.7, 0.5):
                offered = frac * cap_rps
                x = leg(f"poisson_{tag}_{frac}", resident, 1e6 * n_gpus * args.replicas_per_gpu / offered, args.steps, seed=7)
                sweep_pts.append(dict(point(x, offered), inputs=tag, fraction_of_closed_loop=frac))
                if meets_slo(x) and x["rps"] >= 0.97 * offered:
                    best = x
                    break
            return best
        b = sweep(False, closed_e2e["rps"], "host_buffers")
        if b is not None:
            head_e2e = b
        b = sweep(True, closed_dev["rps"], "resident")
        if b is not None:
            head_dev = b
    lognormal_pts = []
    if paper and args.iat_us <= 0:
        # ---- the reference's arrival process for these mixes: lognormal inter-arrival times (sigma 1.5 and 2) at two
        # offered rates below the closed-loop capacity; per-model mean and tail latency at each ----
        for sigma in paper["ln_sigma"]:
            for frac in (0.5, 0.8):
                offered = frac * closed_e2e["rps"]
                x = leg(f"lognormal_{sigma}_{frac}", False, 1e6 * n_gpus * args.replicas_per_gpu / offered, args.steps, seed=7, ln_sigma=sigma)
                d = dict(point(x, offered), ln_sigma=sigma, fraction_of_closed_loop=frac, inputs="host_buffers")
                for i, nm in enumerate(names):
                    d[f"{nm}_mean_us"] = round(x["mean"][i])
                lognormal_pts.append(d)
    clocks = sampler.stop(set(range(n_gpus))) if rank == 0 else None

    fairness = None
    if args.workload in ("mix", "mobilenet_resnet50") and not args.no_fairness:
        # every rank measures its own GPU: isolated mean latency per model, then Jain's index over the slowdowns
        t0 = time.time()
        f = fairness_leg(L, capi, devices[0], MIX, head_e2e["r"], cpus=cpus[:1] if cpus else None)
        leg_seconds["fairness"] = round(time.time() - t0, 1)
        if dist:
            import torch
            allj = [torch.zeros(1, dtype=torch.float64) for _ in range(world)]
            dist.all_gather(allj, torch.tensor([f["jain_index"]], dtype=torch.float64))
            f["jain_index_per_gpu"] = [round(float(a[0]), 4) for a in allj]
            f["jain_index"] = round(min(f["jain_index_per_gpu"]), 4)
        fairness = f

    if rank != 0:
        dist.barrier()
        return

    # kernels of ours inside the timed region: every measured request runs all launches of its model's plan
    # (a stage group replayed as a CUDA graph still launches each of its kernels on the device; independent
    # tensor-core convolutions that share a launch count once; the requests of a gang share their launches)
    kernels_per_request = {}
    layers_per_request = {}
    for job, model, _ in MIX:
        if model is None:     # synthetic jobs: PB_*_KERNELS launches per request (10 by default)
            kernels_per_request[job] = (10, 10)
            continue
        mh = C.c_void_p()
        capi.check(L.pb_model_load(os.path.join(tmp.name, packer_name(model)).encode(), devices[0], -1, C.byref(mh)), "pb_model_load")
        n_stages, n_groups, n_launches = L.pb_model_num_stages(mh), L.pb_model_num_groups(mh), 0
        for g in range(n_groups):
            order, launch = (C.c_int32 * n_stages)(), (C.c_int32 * n_stages)()
            k = L.pb_model_group_plan(mh, g, order, launch, n_stages)
            n_launches += (launch[k - 1] + 1) if k > 0 else 0
        kernels_per_request[model] = (n_launches, n_groups)
        layers_per_request[model] = n_stages
        L.pb_model_destroy(mh)
    counts = head_dev["counts"]          # measured requests per model, summed over GPUs
    # dispatches the schedulers made = stage launches; launches per stage from the plan (gangs make fewer dispatches)
    stages_if_alone = sum(c * kernels_per_request[m or j][1] for c, (j, m, _) in zip(counts, MIX))
    launches_if_alone = sum(c * kernels_per_request[m or j][0] for c, (j, m, _) in zip(counts, MIX))
    gpu_launches = int(launches_if_alone * head_dev["decisions"] / max(stages_if_alone, 1))
    config["kernels_per_request"] = {m: k[0] for m, k in kernels_per_request.items()}
    config["layers_per_request"] = layers_per_request
    config["scheduler_stages_per_request"] = {m: k[1] for m, k in kernels_per_request.items()}
    config["mean_gang_size"] = round(stages_if_alone / max(head_dev["decisions"], 1), 2)
    config["slo"] = slo
    config["arrivals"] = ("closed loop" if head_e2e is closed_e2e else "Poisson (exponential inter-arrival), latency = completion - scheduled arrival; "
                          "headline = highest offered rate of the sweep whose per-model p99s meet the SLO")

    def lat(x):
        r = x["r"]
        d = {"all": r.all.as_dict()}
        for i, nm in enumerate(names):
            d[nm] = r.per_type[i].as_dict()
        return d

    r_e2e = head_e2e["r"]
    host_t = max(r_e2e.host_launch_us + r_e2e.host_sched_us + r_e2e.host_idle_us, 1e-9)
    line = {"metric": METRIC if is_mix else f"requests/s, {args.workload}", "slo_met": bool(meets_slo(head_e2e)),
            "value": round(head_dev["rps"], 2), "unit": "req/s",
            "n_gpus": n_gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(head_dev["ms"] / args.steps, 3),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": config, "clocks": clocks, "gpu_launches": gpu_launches,
            "e2e": {"value": round(head_e2e["rps"], 2), "unit": "req/s", "h2d_bytes_per_step": int(head_e2e["h2d"] / args.steps),
                    "d2h_bytes_per_step": int(head_e2e["d2h"] / args.steps), "ms_per_step": round(head_e2e["ms"] / args.steps, 3),
                    "latency_us": lat(head_e2e)},
            "latency_us": lat(head_dev),
            "closed_loop": {"resident": point(closed_dev), "host_buffers": point(closed_e2e)},
            "timing": "CUDA events on each GPU around the measured requests (device idle on both sides), max over GPUs",
            "records_consumed": int(head_dev["records"]), "decisions": int(head_dev["decisions"]),
            "scheduler_decisions_per_s": round(head_dev["decisions"] / (head_dev["ms"] * 1e-3)),
            "notification_records_per_s": round(head_dev["records"] / (head_dev["ms"] * 1e-3)),
            # rank 0's replica threads during the e2e leg: share of their time inside CUDA launch calls, in
            # notification handling + scheduling, and polling with nothing to do (GPU-bound when large)
            "host_time_share": {"launch": round(r_e2e.host_launch_us / host_t, 3), "sched": round(r_e2e.host_sched_us / host_t, 3),
                                "idle": round(r_e2e.host_idle_us / host_t, 3)},
            "leg_seconds": leg_seconds}
    if head_e2e["per_rank"]:
        line["per_rank_e2e"] = head_e2e["per_rank"]
    if sweep_pts:
        line["poisson_sweep"] = {"arrivals": "Poisson, exponential inter-arrival, latency = completion - scheduled arrival; points in the order run "
                                             "(highest offered rate first, stopping at the first that meets the SLO and keeps up)",
                                 "points": sweep_pts}
    if fairness:
        line["fairness"] = fairness
    if lognormal_pts:
        line["lognormal_arrivals"] = {"what": "open loop, lognormal inter-arrival times with the mean of the offered rate (mu = ln(mean) - sigma^2/2), "
                                              "latency = completion - scheduled arrival, host buffers",
                                      "points": lognormal_pts}

    if is_mix and not dist and not args.no_granularity:
        # ---- scheduling granularity: layers per scheduler stage (1 = the reference's kernel-by-kernel release) ----
        t0 = time.time()
        line["granularity_sweep"] = granularity_sweep(args)
        leg_seconds["granularity_sweep"] = round(time.time() - t0, 1)
    if args.extras and not dist and is_mix:
        # Job-event timeline of a short e2e run (the server records it when PB_PROFILE_PREFIX is set) and the
        # reference's overhead stack computed from it, per model (MNIST = 1 scheduler stage per request).
        from paella_b200 import overhead_stack as ost
        prefix = os.path.join(tmp.name, "timeline")
        os.environ["PB_PROFILE_PREFIX"] = prefix
        try:
            run_load(L, capi, devices[:1], 4000, 1, 0.25, False, args.concurrency, caps, seed=11, **load_kw)
        finally:
            del os.environ["PB_PROFILE_PREFIX"]
        jobs = ost.read_job_events(prefix + "_job_events.txt")
        # lines are in completion order: the first ones are the instance warm-ups (which wait for every model
        # to load) and the un-timed quarter of the run
        jobs = jobs[len(jobs) - 3000:] if len(jobs) > 3000 else jobs
        n_inc_stages = kernels_per_request[names[1]][1]
        line["overhead_stack"] = {"what": "means per request from the server's job-event timeline (closed loop, host buffers): queueing = "
                                          "submission -> first dispatch, scheduling = dispatch -> run_next(), launch = inside run_next(), "
                                          "runtime = run_next() returned -> stage's last block-end record handled, interval = stage finished -> "
                                          "next stage submitted",
                                  "mnist": ost.overhead_stack(jobs, stages=1), "inception_v3": ost.overhead_stack(jobs, stages=n_inc_stages)}
    if args.extras and not dist:
        line["extras"] = extras_leg(L, capi, devices[0])
        if is_mix:
            line["extras"]["ipc"] = ipc_leg(capi, tmp.name)
    if n_gpus == 1 and not dist and not args.no_membound:
        t0 = time.time()
        line["membound"] = membound_leg(L, capi, devices[0], "large", 5)
        leg_seconds["membound"] = round(time.time() - t0, 1)
    if n_gpus == 1 and not args.no_roofline and is_mix:
        t0 = time.time()
        roof, table, layers = roofline_leg(L, capi, tmp.name, args.iters, batch=max(1, args.gang))
        # The same kernel while the GPU serves the whole mix: tensor-core convolution FLOPs retired per second of
        # the timed region (many launches of many requests overlap, so there is no per-launch duration here).
        conv_flops = sum(fl for (_, k, _, fl, _, _) in layers if k == "conv_umma") / max(1, args.gang)
        inc_rps = closed_dev["counts"][1] / (closed_dev["ms"] * 1e-3)
        roof["under_load"] = {"achieved": round(conv_flops * inc_rps / 1e12, 2), "unit": "TFLOP/s",
                              "frac": round(conv_flops * inc_rps / 1e12 / roof["peak"], 4),
                              "inception_v3_per_s": round(inc_rps, 1), "conv_flops_per_request": int(conv_flops),
                              "leg": "closed loop, inputs resident"}
        line["roofline"] = roof
        line["kernel_table_inception_v3"] = table
        leg_seconds["roofline"] = round(time.time() - t0, 1)
        if args.layers:
            with open(args.layers, "w") as f:
                f.write("stage\tkind\tus\tflops\tbytes\tblocks\tTFLOP/s\tGB/s\n")
                for (nm, k, us, fl, by, nb) in layers:
                    f.write(f"{nm}\t{k}\t{us:.2f}\t{fl}\t{by}\t{nb}\t{fl / us / 1e6:.3f}\t{by / us / 1e3:.1f}\n")
        # ---- CPU baseline + output check: the oracle runs the sampled request slots' own inputs ----
        t0 = time.time()
        rps, dt, n, parity = cpu_sample(graphs, closed_e2e["samples"], names)
        leg_seconds["cpu_baseline"] = round(time.time() - t0, 1)
        line["cpu_baseline"] = {"value": round(rps, 3), "unit": "req/s", "cores": os.cpu_count(), "kind": "port",
                                "sample": f"{n} requests (9:1 MNIST : Inception-v3, the inputs of request slots of the timed host-buffer run) "
                                          f"by the CPU oracle, fp32, OpenMP on all host cores, {dt:.1f} s"}
        line.update(parity)
    print(json.dumps(line))
    if dist:
        dist.barrier()


if __name__ == "__main__":
    main()
