"""ctypes bindings of the C ABI declared in include/paella_b200.h."""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libpaella_b200.so")
_LIB = None

PB_MAX_JOB_TYPES = 8
PB_MAX_GPUS = 8

(STAGE_INPUT, STAGE_CONV_SIMT, STAGE_CONV_UMMA, STAGE_DWCONV, STAGE_DENSE, STAGE_MAXPOOL, STAGE_AVGPOOL,
 STAGE_GAP, STAGE_ADD, STAGE_SOFTMAX, STAGE_MNIST_FUSED, STAGE_AFFINE, STAGE_DETECT) = range(13)
STAGE_NAMES = ["input", "conv_simt", "conv_umma", "dwconv", "dense", "maxpool", "avgpool", "gap", "add", "softmax",
               "mnist_fused", "affine", "detect"]


class PbError(RuntimeError):
    pass


class LaunchInfo(C.Structure):
    _fields_ = [("num_blocks", C.c_uint32), ("threads_per_block", C.c_uint32), ("smem_per_block", C.c_uint32),
                ("regs_per_thread", C.c_uint32), ("tmem_cols_per_block", C.c_uint32), ("kind", C.c_uint32),
                ("flops", C.c_uint64), ("bytes", C.c_uint64), ("scratch_bytes", C.c_uint64)]


class OpParams(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("dtype", "C", "H", "W", "Cs", "K", "P", "Q", "Ks", "out_c_off", "R", "S",
                                         "stride_h", "stride_w", "pad_h", "pad_w", "groups", "act", "flags", "res_Cs")] + \
               [("x", C.c_void_p), ("w", C.c_void_p), ("bias", C.c_void_p), ("residual", C.c_void_p), ("y", C.c_void_p),
                ("scratch", C.c_void_p), ("scratch_bytes", C.c_uint64),
                ("batch", C.c_int32), ("dil_h", C.c_int32), ("dil_w", C.c_int32), ("reserved", C.c_int32)]


class ServerConfig(C.Structure):
    _fields_ = [("device", C.c_int32), ("num_streams", C.c_uint32), ("extra_kernels", C.c_uint32),
                ("unfairness_threshold", C.c_float), ("sched_sleep", C.c_uint32), ("ring_capacity", C.c_uint64),
                ("scheduler", C.c_char_p), ("device_resident", C.c_int32), ("max_gang", C.c_uint32), ("deferred_schedule", C.c_uint32),
                ("watchdog_factor", C.c_float), ("watchdog_floor_ms", C.c_float)]


class LoadgenConfig(C.Structure):
    _fields_ = [("num_gpus", C.c_int32), ("devices", C.c_int32 * PB_MAX_GPUS), ("num_types", C.c_int32),
                ("plugin_paths", C.c_char_p * PB_MAX_JOB_TYPES), ("proportions", C.c_float * PB_MAX_JOB_TYPES),
                ("max_outstanding", C.c_uint32 * PB_MAX_JOB_TYPES), ("concurrency", C.c_uint32),
                ("mean_interarrival_us", C.c_double), ("lognormal_sigma", C.c_double), ("num_jobs", C.c_uint32),
                ("warmup_jobs", C.c_uint32), ("seed", C.c_uint32), ("device_resident", C.c_int32),
                ("server", ServerConfig), ("samples_per_type", C.c_uint32), ("sample_buf", C.c_void_p),
                ("sample_buf_bytes", C.c_uint64), ("cpu_of_replica", C.c_int32 * PB_MAX_GPUS),
                ("input_uniform", C.c_int32 * PB_MAX_JOB_TYPES)]


class LatencyStats(C.Structure):
    _fields_ = [("count", C.c_uint64)] + [(n, C.c_double) for n in
                                         ("mean_us", "p50_us", "p90_us", "p95_us", "p99_us", "max_us", "sd_us")]

    def as_dict(self):
        return {n: getattr(self, n) for n, _ in self._fields_}


class LoadgenResult(C.Structure):
    _fields_ = [("elapsed_us", C.c_double), ("elapsed_event_ms", C.c_double), ("throughput_rps", C.c_double), ("all", LatencyStats),
                ("per_type", LatencyStats * PB_MAX_JOB_TYPES), ("per_gpu_rps", C.c_double * PB_MAX_GPUS),
                ("kernels_launched", C.c_uint64), ("records_consumed", C.c_uint64), ("decisions", C.c_uint64),
                ("h2d_bytes", C.c_uint64), ("d2h_bytes", C.c_uint64), ("errors", C.c_int32),
                ("host_launch_us", C.c_double), ("host_sched_us", C.c_double), ("host_idle_us", C.c_double),
                ("samples", C.c_uint32), ("sample_bytes", C.c_uint64)]


class ReplayType(C.Structure):
    _fields_ = [("num_stages", C.c_uint32), ("stage_is_mem", C.POINTER(C.c_uint8)),
                ("stage_pre_notify", C.POINTER(C.c_uint8)), ("stage_blocks", C.POINTER(C.c_uint32)),
                ("stage_threads", C.POINTER(C.c_uint32)), ("stage_smem", C.POINTER(C.c_uint32)),
                ("stage_regs", C.POINTER(C.c_uint32))]


class ReplayEvent(C.Structure):
    _fields_ = [("kind", C.c_uint32), ("a", C.c_uint32), ("b", C.c_uint32), ("time_us", C.c_double)]


class ReplayDecision(C.Structure):
    _fields_ = [("event_index", C.c_uint32), ("job_id", C.c_uint32), ("type", C.c_uint32), ("stage", C.c_uint32),
                ("is_mem", C.c_uint32), ("unfit", C.c_uint32), ("stream_slot", C.c_uint32),
                ("notifier_slot", C.c_uint32), ("priority", C.c_double)]


class ReplayConfig(C.Structure):
    _fields_ = [("num_streams", C.c_uint32), ("extra_kernels", C.c_uint32), ("unfairness_threshold", C.c_double),
                ("total_regs", C.c_int32), ("total_smem", C.c_int32), ("total_threads", C.c_int32),
                ("total_blocks", C.c_int32)]


class SimConfig(C.Structure):
    _fields_ = [("base", ReplayConfig), ("scheduler", C.c_char_p), ("max_gang", C.c_uint32), ("gang_capacity", C.c_uint32),
                ("deferred", C.c_uint32), ("watchdog_factor", C.c_double), ("watchdog_floor_us", C.c_double)]


class SimDecision(C.Structure):
    _fields_ = [(n, C.c_uint32) for n in ("job_id", "type", "stage", "is_mem", "unfit", "num_blocks", "gang_size", "failed")] + \
               [("cookie", C.c_uint64)]


# name -> (restype, argtypes); every symbol include/paella_b200.h declares
_VP, _U32, _U64, _I, _SZ = C.c_void_p, C.c_uint32, C.c_uint64, C.c_int, C.c_size_t
_PP = C.POINTER(C.c_void_p)
SIGNATURES = {
    "pb_last_error": (C.c_char_p, []),
    "pb_version": (C.c_char_p, []),
    "pb_device_count": (_I, []),
    "pb_ring_create": (_I, [_I, _U64, _PP]),
    "pb_ring_destroy": (None, [_VP]),
    "pb_ring_capacity": (_U64, [_VP]),
    "pb_ring_poll": (_I, [_VP, C.POINTER(_U64), _I]),
    "pb_ring_records_read": (_U64, [_VP]),
    "pb_ring_device_view": (_I, [_VP, _VP, _SZ]),
    "pb_notifier_create_array": (_I, [_VP, _U32, _PP]),
    "pb_notifier_free_array": (None, [_VP]),
    "pb_notifier_size": (_SZ, []),
    "pb_launch_notify_probe": (_I, [_VP, _U32, _U32, _U32, _VP, _I]),
    "pb_launch_mem_done": (_I, [_VP, _U32, _VP]),
    "pb_launch_latency_probe": (_I, [_VP, _U32, _VP]),
    "pb_clock_calibrate": (_I, [_I, C.POINTER(_U64)]),
    "pb_ring_roundtrip_bench": (_I, [_I, _U32, C.POINTER(C.c_double)]),
    "pb_ring_wait_expiry_probe": (_I, [_I, _U32, C.POINTER(_U32), C.POINTER(_U32)]),
    "pb_vec_add_bench": (_I, [_I, _U64, _I, _SZ, C.POINTER(C.c_double)]),
    "pb_vec_add_info": (_I, [_U64, C.POINTER(LaunchInfo)]),
    "pb_vec_add_launch": (_I, [_VP, _VP, _U64, _VP, _U32, _VP]),
    "pb_spin_info": (_I, [_U32, C.POINTER(LaunchInfo)]),
    "pb_spin_launch": (_I, [_U32, _U64, _VP, _VP, _U32, _VP]),
    "pb_op_info": (_I, [_I, C.POINTER(OpParams), C.POINTER(LaunchInfo)]),
    "pb_op_launch": (_I, [_I, C.POINTER(OpParams), _VP, _U32, _VP]),
    "pb_op_pack_weights": (C.c_int64, [_I, C.POINTER(OpParams), _VP, _VP]),
    "pb_conv_umma_supported": (_I, [C.POINTER(OpParams)]),
    "pb_conv2d_umma_noalloc": (_I, [C.POINTER(OpParams), _VP, _U32, _VP]),
    "pb_device_error_flag": (_I, [_I, C.POINTER(_U32), _I]),
    "pb_set_conv_split_gain_us": (None, [C.c_double]),
    "pb_conv_umma_time": (_I, [C.POINTER(OpParams), _I, _I, _SZ, C.POINTER(C.c_double)]),
    "pb_instance_create_batched": (_I, [_VP, _I, _I, _PP]),
    "pb_instance_capacity": (_I, [_VP]),
    "pb_model_group_info_batched": (_I, [_VP, _I, _I, C.POINTER(LaunchInfo)]),
    "pb_model_stage_info_batched": (_I, [_VP, _I, _I, C.POINTER(LaunchInfo)]),
    "pb_instance_launch_group_batched": (_I, [_VP, _I, _I, _VP, _U32, _VP, _PP, _PP]),
    "pb_instance_run_batch_sync": (_I, [_VP, _I, _I, _VP, _VP]),
    "pb_instance_stage_params": (_I, [_VP, _I, _I, C.POINTER(OpParams)]),
    "pb_instance_time_stage_batched": (_I, [_VP, _I, _I, _I, _SZ, C.POINTER(C.c_double)]),
    "pb_model_load": (_I, [C.c_char_p, _I, _I, _PP]),
    "pb_model_destroy": (None, [_VP]),
    "pb_model_input_bytes": (_SZ, [_VP]),
    "pb_model_output_bytes": (_SZ, [_VP]),
    "pb_model_num_stages": (_I, [_VP]),
    "pb_model_stage_info": (_I, [_VP, _I, C.POINTER(LaunchInfo)]),
    "pb_model_stage_name": (C.c_char_p, [_VP, _I]),
    "pb_instance_create": (_I, [_VP, _PP]),
    "pb_instance_destroy": (None, [_VP]),
    "pb_instance_input_dev": (_VP, [_VP]),
    "pb_instance_output_dev": (_VP, [_VP]),
    "pb_instance_launch_stage": (_I, [_VP, _I, _VP, _U32, _VP]),
    "pb_instance_run_sync": (_I, [_VP, _VP, _VP]),
    "pb_instance_run_groups_sync": (_I, [_VP, _VP, _VP]),
    "pb_model_num_groups": (_I, [_VP]),
    "pb_model_group_info": (_I, [_VP, _I, C.POINTER(LaunchInfo)]),
    "pb_model_group_stages": (_I, [_VP, _I, C.POINTER(_I), C.POINTER(_I)]),
    "pb_model_group_plan": (_I, [_VP, _I, C.POINTER(C.c_int32), C.POINTER(C.c_int32), _I]),
    "pb_instance_launch_group": (_I, [_VP, _I, _VP, _U32, _VP, _VP, _VP]),
    "pb_instance_read_tensor": (_I, [_VP, _I, _VP, _SZ]),
    "pb_instance_time_stage": (_I, [_VP, _I, _I, _SZ, C.POINTER(C.c_double)]),
    "pb_server_config_default": (None, [C.POINTER(ServerConfig)]),
    "pb_server_create": (_I, [C.POINTER(ServerConfig), _PP]),
    "pb_server_destroy": (None, [_VP]),
    "pb_server_register_job": (_I, [_VP, C.c_char_p, C.POINTER(_U32)]),
    "pb_server_job_io_bytes": (_I, [_VP, _U32, C.POINTER(_SZ), C.POINTER(_SZ), C.POINTER(_SZ)]),
    "pb_server_launch": (_I, [_VP, _U32, _VP, _U64]),
    "pb_server_step": (_I, [_VP, _I]),
    "pb_server_poll_done": (_I, [_VP, C.POINTER(_U64), C.POINTER(C.c_int32), _I]),
    "pb_server_num_decisions": (_U64, [_VP]),
    "pb_server_jobs_in_flight": (_U32, [_VP]),
    "pb_loadgen_config_default": (None, [C.POINTER(LoadgenConfig)]),
    "pb_loadgen_run": (_I, [C.POINTER(LoadgenConfig), C.POINTER(LoadgenResult)]),
    "pb_loadgen_plan": (_I, [C.POINTER(LoadgenConfig), _I, C.POINTER(_U32), C.POINTER(C.c_double), C.POINTER(C.c_uint8),
                             _U32, C.POINTER(_U32)]),
    "pb_shm_channel_open": (_I, [C.c_char_p, _SZ, _PP]),
    "pb_shm_channel_close": (None, [_VP]),
    "pb_shm_channel_write": (_I, [_VP, _VP, _SZ, _U64]),
    "pb_shm_channel_read": (_I, [_VP, _VP, _SZ, _U64]),
    "pb_shm_channel_can_read": (_I, [_VP]),
    "pb_shm_channel_lock": (None, [_VP]),
    "pb_shm_channel_unlock": (None, [_VP]),
    "pb_client_connect": (_I, [C.c_char_p, _PP]),
    "pb_client_close": (None, [_VP]),
    "pb_client_id": (_U32, [_VP]),
    "pb_client_register_job": (_I, [_VP, C.c_char_p, C.POINTER(_U32), C.POINTER(_SZ), C.POINTER(_SZ)]),
    "pb_client_create_instance": (_I, [_VP, _U32, C.POINTER(_U64), _PP, _PP]),
    "pb_client_launch": (_I, [_VP, _U64]),
    "pb_client_wait": (_I, [_VP, _I, C.POINTER(_U64)]),
    "pb_client_kill_server": (_I, [_VP]),
    "pb_client_profiler_cmd": (_I, [_VP, _U32, C.c_char_p]),
    "pb_server_profiler_cmd": (_I, [_VP, _U32, C.c_char_p]),
    "pb_sched_sim_create": (_I, [C.POINTER(SimConfig), C.POINTER(ReplayType), _U32, C.POINTER(C.POINTER(C.c_uint8)), _PP]),
    "pb_sched_sim_destroy": (None, [_VP]),
    "pb_sched_sim_new_job": (_I, [_VP, _U32, C.c_double, _U64]),
    "pb_sched_sim_record": (_I, [_VP, _U32, _U32, _U32, C.c_double]),
    "pb_sched_sim_flush": (_I, [_VP, C.c_double]),
    "pb_sched_sim_take_decisions": (_I, [_VP, C.POINTER(SimDecision), _I]),
    "pb_sched_sim_take_finished": (_I, [_VP, C.POINTER(_U64), C.POINTER(C.c_int32), _I]),
    "pb_sched_sim_jobs_in_flight": (_U32, [_VP]),
    "pb_sched_replay": (_I, [C.POINTER(ReplayConfig), C.POINTER(ReplayType), _U32, C.POINTER(ReplayEvent), _U32,
                             C.POINTER(ReplayDecision), _U32, C.POINTER(_U32), C.POINTER(_U32)]),
}


def load():
    """Loads the native library; raises if it has not been built (no fallback exists)."""
    global _LIB
    if _LIB is None:
        if not os.path.exists(LIB_PATH):
            raise PbError(f"{LIB_PATH} is missing: build it with `make -C {_HERE}` "
                          "(or __graft_entry__.build()); paella_b200 has no CPU fallback")
        # More hardware queues than the default 8, as the reference's scripts set
        # (sosp23_artifact/gen_data_fig11_paella.sh:29); must precede CUDA initialisation.
        os.environ.setdefault("CUDA_DEVICE_MAX_CONNECTIONS", "32")
        L = C.CDLL(LIB_PATH, mode=C.RTLD_GLOBAL)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args
        _LIB = L
    return _LIB


def lib():
    return load()


def check(rc, what=""):
    if rc is not None and rc < 0:
        raise PbError(f"{what} failed ({rc}): {lib().pb_last_error().decode()}")
    return rc


def plugin_path(job: str) -> str:
    """Path of a job plugin, e.g. plugin_path('tvm_mnist') -> .../jobs/libjob_tvm_mnist.so"""
    p = os.path.join(_HERE, "jobs", f"libjob_{job}.so")
    if not os.path.exists(p):
        raise PbError(f"job plugin {p} is missing: build it with `make -C {_HERE}`")
    return p
