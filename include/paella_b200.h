/*
 * paella_b200 C ABI.
 *
 * Everything the host side (the C++ scheduler/server, the job plugins, and the
 * Python tests and benchmark through ctypes) needs from the CUDA library goes
 * through these functions: plain pointers and sizes, no C++ or torch types.
 * Streams are passed as `void*` holding a `cudaStream_t`; device buffers as
 * `void*` device addresses.  Every function returns PB_OK (0) or a negative
 * pb_status, and never aborts the process.  pb_last_error() returns a
 * thread-local description of the most recent failure.
 *
 * File references name the interface of the reference implementation that each
 * group replaces (paths inside the eniac/paella tree).
 */
#ifndef PAELLA_B200_H
#define PAELLA_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define PB_API __attribute__((visibility("default")))

typedef enum pb_status {
    PB_OK = 0,
    PB_ERR_CUDA = -1,          /* a CUDA runtime/driver call failed */
    PB_ERR_INVALID = -2,       /* bad argument / unsupported shape */
    PB_ERR_RING_OVERFLOW = -3, /* device writer lapped the host reader */
    PB_ERR_IO = -4,            /* pack file missing or malformed */
    PB_ERR_TIMEOUT = -5,       /* a bounded wait ran out */
    PB_ERR_NO_DEVICE = -6,     /* no CUDA device / library built without one */
    PB_ERR_DEVICE_FLAG = -7    /* a kernel raised its error flag (bounded wait expired on device) */
} pb_status;

PB_API const char* pb_last_error(void);
PB_API const char* pb_version(void);
PB_API int pb_device_count(void);

/* Launch geometry and per-block resources of one kernel launch: what a job stage
 * declares to the scheduler (include/llis/job/job.h:62-135 in the reference). */
typedef struct pb_launch_info {
    uint32_t num_blocks;
    uint32_t threads_per_block;
    uint32_t smem_per_block;     /* static + dynamic bytes */
    uint32_t regs_per_thread;
    uint32_t tmem_cols_per_block;
    uint32_t kind;               /* pb_stage_kind */
    uint64_t flops;              /* algorithmic 2*MAC */
    uint64_t bytes;              /* algorithmic bytes: inputs + weights + outputs once */
    uint64_t scratch_bytes;      /* scratch memory the launch can use (0 = none); see pb_op_params.scratch */
} pb_launch_info;

/* ------------------------------------------------------------------------ *
 * GPU -> host notification ring and notifiers.
 * Replaces ShmPrimitiveChannelGpu<uint64_t> (include/llis/ipc/shm_primitive_channel.h:11-68,
 * include/llis/ipc/shm_primitive_channel_impl.h:18-64, src/ipc/shm_primitive_channel.cu:49-131)
 * and FinishedBlockNotifier::create_array/free_array (src/job/finished_block_notifier.cu:21-48).
 * ------------------------------------------------------------------------ */
typedef struct pb_ring pb_ring;

/* capacity is rounded up to a power of two (reference default: 1 024 000 records). */
PB_API int pb_ring_create(int device, uint64_t capacity, pb_ring** out);
PB_API void pb_ring_destroy(pb_ring* ring);
PB_API uint64_t pb_ring_capacity(const pb_ring* ring);
/* Non-blocking read of up to `max` records (8 bytes each, layout of
 * llis::job::InstrumentInfo).  Returns the number read (>= 0) or PB_ERR_RING_OVERFLOW. */
PB_API int pb_ring_poll(pb_ring* ring, uint64_t* records, int max);
PB_API uint64_t pb_ring_records_read(const pb_ring* ring);
/* Fills a llis::ipc::Gpu2SchedChannelDev (24 bytes) for embedding in device objects. */
PB_API int pb_ring_device_view(const pb_ring* ring, void* view_out, size_t view_size);
/* n notifiers (device memory) bound to the ring; element size = pb_notifier_size(). */
PB_API int pb_notifier_create_array(pb_ring* ring, uint32_t n, void** dev_array_out);
PB_API void pb_notifier_free_array(void* dev_array);
PB_API size_t pb_notifier_size(void);

/* Microbenchmark kernel of the reference's tests/ipc/shm_channel/latency/shmpc_latency_gpu.cu:7-32:
 * a grid of `num_blocks` x `threads` that only emits start/end notifications.
 * aggregated != 0 uses the notifier (1 record / 16 blocks), else one record per block
 * with the SM id (include/llis/job/instrument.h:9-63). */
PB_API int pb_launch_notify_probe(void* stream, uint32_t num_blocks, uint32_t threads, uint32_t job_id,
                                  void* notifier, int aggregated);
/* One-block kernel that writes a kMemDone record for `job_id`: follows an async copy
 * stage in stream order (replaces cudaLaunchHostFunc + the mem2sched CPU ring,
 * src/server/scheduler_full3.cpp:429-431,465-468). */
PB_API int pb_launch_mem_done(void* stream, uint32_t job_id, void* notifier_or_ring_view);
/* Ring latency probe: like the notify probe, but the record's job_id field carries the
 * low 32 bits of %globaltimer (ns) at the time of the write. */
PB_API int pb_launch_latency_probe(void* stream, uint32_t num_blocks, void* notifier);
/* Reads %globaltimer on the device and the host monotonic clock around it:
 * out[0] = host ns before, out[1] = device globaltimer ns, out[2] = host ns after. */
PB_API int pb_clock_calibrate(int device, uint64_t out[3]);

/* Ring round trip: a one-thread kernel answers `iters` host pings (a counter in host-mapped memory)
 * with one record each; rtt_us_out[i] = host store of ping i -> host sees record i.  It is the sum
 * of host->GPU visibility (the kernel's poll of host memory) and the GPU->host record; every device
 * wait is bounded.  Counterpart of the reference's tests/ipc/shm_channel/latency/shmpc_latency_gpu.cu. */
PB_API int pb_ring_roundtrip_bench(int device, uint32_t iters, double* rtt_us_out);
/* A device-side wait that runs out, on purpose and harmlessly: the round-trip kernel is launched with a ping that
 * never comes and a limit of `max_polls` polls (<= 65536, i.e. well under a second); it gives up, reports status 2
 * in *status_out (1 would mean it saw the ping) and returns.  *records_out = records it wrote (0 expected). */
PB_API int pb_ring_wait_expiry_probe(int device, uint32_t max_polls, uint32_t* status_out, uint32_t* records_out);
/* vec_add over n floats on private buffers, `iters` timed launches between CUDA events with an L2
 * flush (a write of flush_bytes) before each; mean microseconds per launch in *us_out. */
PB_API int pb_vec_add_bench(int device, uint64_t n, int iters, size_t flush_bytes, double* us_out);

/* ------------------------------------------------------------------------ *
 * Synthetic jobs of the scheduler stress configuration.
 * vec_add:  jobs/vec_add_coroutine/vec_add_coroutine.cu:8-20  (out[i] += in[i])
 * spin:     jobs/dummy_short/dummy_short.cu:8-27 and jobs/dummy_long (occupy SMs for a known time);
 *           each block spins on %globaltimer until `spin_ns` elapsed (bounded, never waits on the host).
 * ------------------------------------------------------------------------ */
PB_API int pb_vec_add_info(uint64_t n, pb_launch_info* out);
PB_API int pb_vec_add_launch(float* out_dev, const float* in_dev, uint64_t n, void* stream, uint32_t job_id,
                             void* notifier);
PB_API int pb_spin_info(uint32_t num_blocks, pb_launch_info* out);
PB_API int pb_spin_launch(uint32_t num_blocks, uint64_t spin_ns, uint32_t* sink_dev, void* stream, uint32_t job_id,
                          void* notifier);

/* ------------------------------------------------------------------------ *
 * Inference operators (the kernels the reference's TVM job adapters launch:
 * jobs/tvm_<model>/tvm_<model>.cpp:24-47 -> generated conv / dense / pool /
 * depthwise / elementwise kernels).  Device tensors are channels-last
 * [H][W][Cs] with Cs = channel count rounded up to a 16-byte vector; dtype 0 = fp32,
 * 1 = bf16.  Each launcher enqueues exactly one kernel on `stream`; every block of it
 * reports start/end on `notifier` (may be NULL) for `job_id`.
 * ------------------------------------------------------------------------ */
typedef enum pb_stage_kind {
    PB_STAGE_INPUT = 0,      /* NCHW fp32 -> channels-last dtype */
    PB_STAGE_CONV_SIMT = 1,
    PB_STAGE_CONV_UMMA = 2,  /* tcgen05 implicit GEMM */
    PB_STAGE_DWCONV = 3,
    PB_STAGE_DENSE = 4,
    PB_STAGE_MAXPOOL = 5,
    PB_STAGE_AVGPOOL = 6,
    PB_STAGE_GAP = 7,
    PB_STAGE_ADD = 8,
    PB_STAGE_SOFTMAX = 9,
    PB_STAGE_MNIST_FUSED = 10,
    PB_STAGE_AFFINE = 11,    /* per-channel scale + bias (+ activation): a batch-norm that precedes its convolution (DenseNet) */
    PB_STAGE_DETECT = 12     /* detection head over one feature map: x = [H][W][6A] (2A class logits, then 4A box regressions),
                              * w = fp32 priors [H*W*A][4] (cx, cy, w, h), bias = {centre variance, size variance}, K = priors of
                              * the whole model, out_c_off = first prior of this map; writes softmax scores to y[(first+i)*2..]
                              * and corner-form boxes to y[K*2 + (first+i)*4..] of the fp32 model output (K*6 floats) */
} pb_stage_kind;

typedef struct pb_op_params {
    int32_t dtype;            /* 0 fp32, 1 bf16 (activations and weights) */
    int32_t C, H, W, Cs;      /* input: channels, height, width, channel stride */
    int32_t K, P, Q, Ks;      /* output: channels written, height, width, channel stride of the output tensor */
    int32_t out_c_off;        /* first output channel written (concatenation slice) */
    int32_t R, S, stride_h, stride_w, pad_h, pad_w, groups;
    int32_t act;              /* 0 none, 1 relu, 2 relu6, 3 prelu (dense convolutions only: `bias` then holds 2*K floats,
                               *   the K biases followed by the K per-channel slopes) */
    int32_t flags;            /* bit0 count_include_pad (avg pool); bit1 output is fp32 */
    int32_t res_Cs;           /* channel stride of the residual tensor (0 = none) */
    const void* x;            /* input activations */
    const void* w;            /* weights in the layout pb_op_weight_layout reports */
    const float* bias;        /* fp32 [K] or NULL */
    const void* residual;     /* same dtype as x, [P][Q][res_Cs], or NULL */
    void* y;                  /* output tensor base (slice offset applied by the kernel) */
    /* Scratch memory (device, 16-byte aligned, zero-filled before its first use, private to one
     * in-flight launch).  The tensor-core convolution splits its reduction over several thread
     * blocks when given at least pb_launch_info.scratch_bytes here; NULL = no split. */
    void* scratch;
    uint64_t scratch_bytes;
    /* Images per launch (0 or 1 = one).  A batch is how a gang of requests of one model runs as one
     * launch: x, residual and y then hold `batch` images back to back without padding ([batch][H][W][Cs]),
     * the weights are shared.  The kernels that read the request input or write the fp32 model output
     * take image i at offset i * (C*H*W) resp. i * K floats from x / y. */
    int32_t batch;
    int32_t dil_h, dil_w;     /* filter dilation (0 or 1 = dense filter); tensor-core and direct convolutions only */
    int32_t reserved;
} pb_op_params;

/* Geometry/resources the launch of `kind` with `p` will use. */
PB_API int pb_op_info(int kind, const pb_op_params* p, pb_launch_info* out);
PB_API int pb_op_launch(int kind, const pb_op_params* p, void* stream, uint32_t job_id, void* notifier);
/* Converts OIHW fp32 host weights into the device layout `kind` expects.  Returns the byte
 * size needed when dst_host is NULL, else fills dst_host (host memory) and returns the size. */
PB_API int64_t pb_op_pack_weights(int kind, const pb_op_params* p, const float* w_oihw, void* dst_host);
/* 1 if the tcgen05 implicit-GEMM kernel supports this convolution. */
PB_API int pb_conv_umma_supported(const pb_op_params* p);
/* The tensor-core convolution splits a long reduction over several thread blocks (partial tiles meet in
 * scratch memory) when its cost model expects to save at least this many microseconds on a lone launch
 * (default 6, or PB_CONV_SPLIT_GAIN_US from the environment; 0 = split whenever it pays at all, a large
 * value = never; negative = back to the default).  Read at every pb_op_info / pb_op_launch, and when a model
 * instance builds its launches for a batch size: instances built before a change keep their split. */
PB_API void pb_set_conv_split_gain_us(double us);
/* Mean microseconds of one launch of the tensor-core convolution `p` (any batch): 3 warm-up launches, then `iters`
 * launches on a private stream between CUDA events, a write of flush_bytes before each (0 = none).  mode 0 = the
 * one-tile-per-CTA kernel pb_op_launch uses, 1 = the persistent kernel the model stage graphs use. */
PB_API int pb_conv_umma_time(const pb_op_params* p, int mode, int iters, size_t flush_bytes, double* us_out);
/* Tensor-core convolution for callers that must not allocate: code running inside a CUDA memory-pool
 * or allocator callback, a latency-critical thread that may not take the allocator's locks, or a host
 * that pre-partitions all device memory and leaves none to ask for.  It has no counterpart in the
 * reference (which allocates freely); it is the same kernel as pb_op_launch(PB_STAGE_CONV_UMMA) with its
 * split-K scratch taken from a buffer built into the library instead of p->scratch.
 *  - p->scratch / p->scratch_bytes are ignored.  Inputs, weights and outputs are still the caller's.
 *  - Limit: the built-in buffer is 4 MiB (and is held by every GPU that loads the library until the
 *    process exits).  A convolution whose split needs more (pb_launch_info.scratch_bytes) is refused
 *    with PB_ERR_INVALID and a message; nothing is launched.
 *  - The first call on each device looks up the buffer's device address and sets the kernels' shared
 *    memory limit; make that first call outside any stream capture.
 *  - All calls on a device share the one buffer: the tile counters are cleared (stream-ordered) at the
 *    start of every call, the rest keeps the previous call's contents.  Two calls whose kernels can
 *    overlap on the GPU (different streams, no dependency) race on it: keep them on one stream or
 *    order them yourself.
 *  - Never calls cudaMalloc, cudaFree or any allocating routine, on the host heap either. */
PB_API int pb_conv2d_umma_noalloc(const pb_op_params* p, void* stream, uint32_t job_id, void* notifier);
/* Device-side error flag raised by bounded waits inside kernels (0 = none): the OR of the library's flag and of
 * the one pb_conv2d_umma_noalloc keeps for itself.  Reading and resetting use plain synchronous copies: synchronise
 * the streams that may still be running kernels (pb_conv2d_umma_noalloc included) before a reset, or a flag raised
 * in between is lost. */
PB_API int pb_device_error_flag(int device, uint32_t* flag_out, int reset);

/* ------------------------------------------------------------------------ *
 * Model packs and instances: the graph executor behind the model job adapters
 * (replaces tvm::runtime::Module::LoadFromFile + "run"/"get_input"/"get_output",
 * jobs/tvm_mnist/tvm_mnist.cpp:24-33).
 * ------------------------------------------------------------------------ */
typedef struct pb_model pb_model;
typedef struct pb_instance pb_instance;

/* precision: -1 = the pack's own hint, 0 = fp32 SIMT kernels, 1 = bf16 (tcgen05 where supported). */
PB_API int pb_model_load(const char* pack_path, int device, int precision, pb_model** out);
PB_API void pb_model_destroy(pb_model* m);
PB_API size_t pb_model_input_bytes(const pb_model* m);   /* NCHW fp32 */
PB_API size_t pb_model_output_bytes(const pb_model* m);  /* fp32 vector */
PB_API int pb_model_num_stages(const pb_model* m);       /* compute stages (kernels) per request */
PB_API int pb_model_stage_info(const pb_model* m, int stage, pb_launch_info* out);
PB_API const char* pb_model_stage_name(const pb_model* m, int stage);
PB_API int pb_instance_create(pb_model* m, pb_instance** out);
PB_API void pb_instance_destroy(pb_instance* inst);
PB_API void* pb_instance_input_dev(pb_instance* inst);   /* device staging buffer, NCHW fp32 */
PB_API void* pb_instance_output_dev(pb_instance* inst);  /* device fp32 output */
PB_API int pb_instance_launch_stage(pb_instance* inst, int stage, void* stream, uint32_t job_id, void* notifier);
/* Stage groups: consecutive kernels that the job adapter presents to the scheduler as ONE stage
 * (default up to 48 kernels, PB_STAGE_GROUP=1 gives the reference's one-kernel-per-stage granularity).
 * A multi-kernel group is replayed as a CUDA graph - one driver call instead of one per kernel - and
 * only its last kernel reports block start/end on the notifier, so pb_model_group_info's block count
 * is that kernel's grid and its per-block resources are the group's largest footprint spread over
 * those blocks.  io_in / io_out: this request's input (NCHW fp32) and output buffers, device memory
 * or host-mapped pinned memory; the first kernel reads io_in and the last writes io_out directly
 * (no separate copy stages).  NULL = the instance's own device buffers. */
PB_API int pb_model_num_groups(const pb_model* m);
PB_API int pb_model_group_info(const pb_model* m, int group, pb_launch_info* out);
PB_API int pb_model_group_stages(const pb_model* m, int group, int* first_stage, int* num_stages);
/* The group's launch plan: its stages in launch order (dependence depth first, then program order) and,
 * for each, the index of the launch it belongs to.  Stages that share a launch index are independent
 * tensor-core convolutions issued as ONE grid (the parallel branches of an Inception block, a ResNet
 * shortcut beside the block's first convolution); the group's last launch is the one that notifies, so
 * pb_model_group_info's block count is the sum of its stages' grids.  Returns the number of stages
 * written (<= max_stages).  PB_FUSE_BRANCHES=0 at load time: program order, one stage per launch.
 * No counterpart in the reference (it launches one TVM kernel at a time). */
PB_API int pb_model_group_plan(const pb_model* m, int group, int32_t* stage_order, int32_t* launch_index, int max_stages);
PB_API int pb_instance_launch_group(pb_instance* inst, int group, void* stream, uint32_t job_id, void* notifier,
                                    const void* io_in, void* io_out);
/* Batches: an instance created with capacity `cap` (<= PB_MAX_GANG) runs any number nb <= cap of requests
 * of its model as ONE set of launches - a "gang".  Its activation tensors hold cap images back to back, the
 * tensor-core convolutions then see nb * pixels rows (fuller 128-row tiles, the weights pulled once for the
 * gang), every other kernel puts the image on blockIdx.y, and the number of launches is that of one request.
 * What depends on nb (descriptors, scratch, executable graphs) is built on the first use of that nb, or for
 * every nb at creation with prepare_all != 0 (a build takes milliseconds: do it outside the serving path).
 * pb_model_group_info_batched / pb_model_stage_info_batched give the launch geometry a stage declares for a
 * gang of nb.  io_in[i] / io_out[i]: member i's request buffers (NULL entries or NULL arrays: the instance's
 * own device buffers, image i).  Results are those of nb separate runs; they are bit-identical to them when
 * the split of the reduction is the same (see pb_set_conv_split_gain_us).
 * No counterpart in the reference, which runs one request per launch (its paper argues against batching by
 * waiting; a gang only takes requests that are already queued). */
#define PB_MAX_GANG 8
PB_API int pb_instance_create_batched(pb_model* m, int capacity, int prepare_all, pb_instance** out);
PB_API int pb_instance_capacity(const pb_instance* inst);
PB_API int pb_model_group_info_batched(const pb_model* m, int group, int batch, pb_launch_info* out);
PB_API int pb_model_stage_info_batched(const pb_model* m, int stage, int batch, pb_launch_info* out);
PB_API int pb_instance_launch_group_batched(pb_instance* inst, int group, int batch, void* stream, uint32_t job_id, void* notifier,
                                            const void* const* io_in, void* const* io_out);
/* Convenience for tests: H2D of `batch` inputs (back to back), the model kernel by kernel (by_groups = 0) or
 * group by group, D2H of the `batch` outputs, then synchronise. */
PB_API int pb_instance_run_batch_sync(pb_instance* inst, int batch, int by_groups, const float* inputs_host, float* outputs_host);
/* The operator parameters (device pointers resolved, batch set) stage `stage` of the instance is launched with for a
 * gang of `batch`: what pb_op_launch / pb_conv_umma_time take, for layer-by-layer measurements. */
PB_API int pb_instance_stage_params(pb_instance* inst, int stage, int batch, pb_op_params* out);
PB_API int pb_instance_time_stage_batched(pb_instance* inst, int stage, int batch, int iters, size_t flush_bytes, double* us_out);
/* Convenience for tests: H2D, every group, D2H on one stream, then synchronise. */
PB_API int pb_instance_run_groups_sync(pb_instance* inst, const float* input_host, float* output_host);
/* Convenience for tests: H2D, every stage, D2H on one stream, then synchronise. */
PB_API int pb_instance_run_sync(pb_instance* inst, const float* input_host, float* output_host);
/* Copies tensor `t` of the pack (as NCHW fp32) to host; for layer-by-layer parity tests. */
PB_API int pb_instance_read_tensor(pb_instance* inst, int tensor, float* dst_host, size_t dst_floats);
/* Times stage `stage` alone: `iters` launches on a private stream between CUDA events, with an
 * L2 flush (a write of flush_bytes) before each; returns mean microseconds in *us_out. */
PB_API int pb_instance_time_stage(pb_instance* inst, int stage, int iters, size_t flush_bytes, double* us_out);

/* ------------------------------------------------------------------------ *
 * Server: scheduler + job registry + in-process client endpoint.
 * Replaces llis_server's main loop and scheduler (src/server/server.cpp:29-35,43-80,
 * src/server/scheduler_full3.cpp, src/server/registered_job.cpp:26-137,
 * src/server/sm_resources.cpp).  One server per GPU; all calls on one thread.
 * ------------------------------------------------------------------------ */
typedef struct pb_server pb_server;

typedef struct pb_server_config {
    int32_t device;
    uint32_t num_streams;        /* --num_streams, default 500 */
    uint32_t extra_kernels;      /* --extra_kernels, default 2 */
    float unfairness_threshold;  /* --unfair, default 1e6 */
    uint32_t sched_sleep;        /* --sched_sleep, default 0 */
    uint64_t ring_capacity;      /* 0 = 1<<20 */
    const char* scheduler;       /* "full3" (default), "fifo", "fifo2" */
    int32_t device_resident;     /* 1: model jobs skip their host<->device copies (inputs already in HBM) */
    uint32_t max_gang;           /* full3 only: up to this many queued requests of one model run as ONE launch per stage
                                  * (a gang, <= PB_MAX_GANG); 0 or 1 = one request per launch, as in the reference */
    uint32_t deferred_schedule;  /* 0: the dispatch loop runs inside every launch / notification, as in the reference
                                  * (src/server/scheduler_full3.cpp:64-99,272-313).  1 (implied by max_gang > 1): launches
                                  * and notifications only update the queue and the occupancy model; the dispatch loop runs
                                  * once per pb_server_step batch (<= 64 records) */
    float watchdog_factor;       /* 0 = off (the reference: a kernel that never reports its last block wedges the server).
                                  * > 0: a stage in flight longer than max(factor x its learned length, watchdog_floor_ms)
                                  * is given up - the request (and its gang) ends with PB_ERR_TIMEOUT, its job id, stream
                                  * and notifier are not reused */
    float watchdog_floor_ms;     /* 0 = 100 ms */
} pb_server_config;

PB_API void pb_server_config_default(pb_server_config* cfg);
PB_API int pb_server_create(const pb_server_config* cfg, pb_server** out);
PB_API void pb_server_destroy(pb_server* s);
/* REGISTER_JOB: dlopen the plugin and call init_job (src/server/registered_job.cpp:26-59). */
PB_API int pb_server_register_job(pb_server* s, const char* plugin_path, uint32_t* job_ref_id_out);
/* Pinned I/O slot size the plugin asks for (include/llis/job/job.h:54-60). */
PB_API int pb_server_job_io_bytes(pb_server* s, uint32_t job_ref_id, size_t* in_bytes, size_t* out_bytes,
                                  size_t* slot_bytes);
/* LAUNCH_JOB: io_ptr is a pinned host slot (input at 0, output at align8(input size));
 * cookie comes back from pb_server_poll_done when the job ends. */
PB_API int pb_server_launch(pb_server* s, uint32_t job_ref_id, void* io_ptr, uint64_t cookie);
/* One iteration of the serve loop: at most `max_records` ring records, then return. */
PB_API int pb_server_step(pb_server* s, int max_records);
/* Completed jobs since the last call: fills cookies/errors, returns the count. */
PB_API int pb_server_poll_done(pb_server* s, uint64_t* cookies, int32_t* errors, int max);
PB_API uint64_t pb_server_num_decisions(const pb_server* s);
PB_API uint32_t pb_server_jobs_in_flight(const pb_server* s);
/* Job-event timeline and run_next() timings of the reference's Profiler (include/llis/server/profiler.h:15-23,
 * src/server/profiler.cpp:10-131).  `cmd` is a llis::ProfilerMsgType value: 8 / 9 start / stop recording job
 * events (0 JOB_SUBMITTED, 1 KERNEL_SCHED_START, 3 KERNEL_SUBMIT_START, 4 KERNEL_SUBMIT_END, 5 KERNEL_FINISHED,
 * 6 JOB_FINISHED with steady-clock microseconds), 6 / 7 run_next() timings, 12 SAVE writes
 * "<path>_job_events.txt" (one line per finished job: "code time " pairs) and "<path>_run_next_times.txt"
 * ("start end duration blocks") in the reference's formats; the other commands are accepted and record nothing.
 * PB_PROFILE_PREFIX=<path> in the environment records from server creation and saves at destruction. */
PB_API int pb_server_profiler_cmd(pb_server* s, uint32_t cmd, const char* path);

/* ------------------------------------------------------------------------ *
 * Load generator + request router over one server per GPU
 * (workload semantics of app/client.cpp:123-212,393-495).
 * ------------------------------------------------------------------------ */
#define PB_MAX_JOB_TYPES 8
#define PB_MAX_GPUS 8

typedef struct pb_loadgen_config {
    int32_t num_gpus;
    int32_t devices[PB_MAX_GPUS];
    int32_t num_types;
    const char* plugin_paths[PB_MAX_JOB_TYPES];
    float proportions[PB_MAX_JOB_TYPES];          /* request mix, sums to 1 */
    uint32_t max_outstanding[PB_MAX_JOB_TYPES];   /* per type and per GPU (instances in its pool) */
    uint32_t concurrency;          /* total outstanding cap per GPU */
    double mean_interarrival_us;   /* per GPU stream of arrivals; <= 0 = closed loop at `concurrency` */
    double lognormal_sigma;        /* 0 = exponential (Poisson) arrivals */
    uint32_t num_jobs;             /* measured requests per GPU */
    uint32_t warmup_jobs;          /* un-measured requests per GPU issued first */
    uint32_t seed;
    int32_t device_resident;       /* 1: inputs already in HBM, copy stages skipped */
    pb_server_config server;
    /* Output check by the caller (host-buffer runs only): after the measured phase replica 0 copies, for each job
     * type, the first `samples_per_type` request slots in which a measured request completed into sample_buf as
     * records { u32 type, u32 slot, u64 in_bytes, u64 out_bytes, input (padded to 8), output (padded to 8) }. */
    uint32_t samples_per_type;
    void* sample_buf;
    uint64_t sample_buf_bytes;
    /* CPU placement: replica g's thread (it submits, polls and launches for GPU g) is pinned to cpu_of_replica[g]
     * when >= 0 (sched_setaffinity on the thread only; nothing of the GPU is changed).  -1 = leave it to the OS. */
    int32_t cpu_of_replica[PB_MAX_GPUS];
    /* Request inputs are filled once per slot from the seed: N(0,1) floats, or U[0,1) for the types marked here
     * (the MNIST configuration's input range). */
    int32_t input_uniform[PB_MAX_JOB_TYPES];
} pb_loadgen_config;

typedef struct pb_latency_stats {
    uint64_t count;
    double mean_us, p50_us, p90_us, p95_us, p99_us, max_us, sd_us;
} pb_latency_stats;

typedef struct pb_loadgen_result {
    double elapsed_us;               /* host clock: last completion - first arrival of the measured requests, over all GPUs */
    double elapsed_event_ms;         /* max over GPUs of the CUDA-event time around the measured phase */
    double throughput_rps;           /* total measured jobs / elapsed */
    pb_latency_stats all;
    pb_latency_stats per_type[PB_MAX_JOB_TYPES];
    double per_gpu_rps[PB_MAX_GPUS];
    uint64_t kernels_launched;       /* compute stages dispatched in the measured window */
    uint64_t records_consumed;
    uint64_t decisions;
    uint64_t h2d_bytes, d2h_bytes;
    int32_t errors;
    /* where the replicas' host threads spent the measured phase, summed over replicas (us):
     * inside the plugins' run_next() (CUDA launches), inside notification handling and scheduling
     * around it, and in polls that found nothing to do (the GPU was the slower side) */
    double host_launch_us, host_sched_us, host_idle_us;
    uint32_t samples;                /* records written to sample_buf */
    uint64_t sample_bytes;
} pb_loadgen_result;

PB_API void pb_loadgen_config_default(pb_loadgen_config* cfg);
PB_API int pb_loadgen_run(const pb_loadgen_config* cfg, pb_loadgen_result* out);
/* The router alone (no GPU needed): the requests replica `replica` of cfg->num_gpus would play - job
 * type, scheduled arrival (us from its phase start) and whether it is measured - in submission order. */
PB_API int pb_loadgen_plan(const pb_loadgen_config* cfg, int replica, uint32_t* types, double* arrivals_us,
                           uint8_t* measured, uint32_t max, uint32_t* n_out);

/* ------------------------------------------------------------------------ *
 * Client <-> server IPC (process boundary): the byte ring in POSIX shared memory
 * (include/llis/ipc/shm_channel.h:59-130 of the reference; "llis:channel:<name>") and the client
 * library (src/client/client.cpp, job_ref.cpp, job_instance_ref.cpp) against a running llis_server.
 * ------------------------------------------------------------------------ */
typedef struct pb_shm_channel pb_shm_channel;
typedef struct pb_client pb_client;

/* size > 0 creates ring "llis:channel:<name>" (name "" = anonymous, same process); size == 0 attaches. */
PB_API int pb_shm_channel_open(const char* name, size_t size, pb_shm_channel** out);
PB_API void pb_shm_channel_close(pb_shm_channel* ch);
/* Blocking copies; max_spins > 0 bounds every wait (PB_ERR_TIMEOUT when it runs out). */
PB_API int pb_shm_channel_write(pb_shm_channel* ch, const void* buf, size_t n, uint64_t max_spins);
PB_API int pb_shm_channel_read(pb_shm_channel* ch, void* buf, size_t n, uint64_t max_spins);
PB_API int pb_shm_channel_can_read(pb_shm_channel* ch);
PB_API void pb_shm_channel_lock(pb_shm_channel* ch);     /* multi-writer spin lock */
PB_API void pb_shm_channel_unlock(pb_shm_channel* ch);

/* REGISTER_CLIENT handshake with the server named `server_name`. */
PB_API int pb_client_connect(const char* server_name, pb_client** out);
PB_API void pb_client_close(pb_client* c);
PB_API uint32_t pb_client_id(const pb_client* c);
/* REGISTER_JOB + first GROW_POOL; *job_out indexes this client's registered jobs. */
PB_API int pb_client_register_job(pb_client* c, const char* plugin_path, uint32_t* job_out, size_t* in_bytes, size_t* out_bytes);
/* A request slot in the shared pool; in_ptr/out_ptr are this process's addresses of its input and output. */
PB_API int pb_client_create_instance(pb_client* c, uint32_t job, uint64_t* instance_out, void** in_ptr, void** out_ptr);
PB_API int pb_client_launch(pb_client* c, uint64_t instance);                         /* LAUNCH_JOB */
/* Next finished request: 1 and *instance_out set, 0 on timeout (timeout_ms < 0 blocks). */
PB_API int pb_client_wait(pb_client* c, int timeout_ms, uint64_t* instance_out);
PB_API int pb_client_profiler_cmd(pb_client* c, uint32_t cmd, const char* path);      /* PROFILER_CMD + sub-command (+ path for SAVE = 12) */
PB_API int pb_client_kill_server(pb_client* c);                                       /* EXIT_CMD */

/* ------------------------------------------------------------------------ *
 * Scheduler replay (no GPU needed): feeds a recorded event trace to the product
 * scheduler with fake streams/notifiers and returns its decision log, to be
 * compared bit-for-bit with the oracle's restatement of
 * src/server/scheduler_full3.cpp:123-459 and include/llis/server/scheduler_full3.h:26-208.
 * ------------------------------------------------------------------------ */
typedef struct pb_replay_type {
    uint32_t num_stages;
    const uint8_t* stage_is_mem;        /* [num_stages] */
    const uint8_t* stage_pre_notify;    /* [num_stages] */
    const uint32_t* stage_blocks;       /* [num_stages] */
    const uint32_t* stage_threads;
    const uint32_t* stage_smem;
    const uint32_t* stage_regs;
} pb_replay_type;

typedef struct pb_replay_event {
    uint32_t kind;      /* 0 NEW_JOB(type = a), 1 BLOCK_START(job_id = a, num = b), 2 BLOCK_END, 3 MEM_FINISH(job_id = a) */
    uint32_t a, b;
    double time_us;
} pb_replay_event;

typedef struct pb_replay_decision {
    uint32_t event_index;   /* event being handled when the dispatch happened */
    uint32_t job_id, type, stage;
    uint32_t is_mem, unfit, stream_slot, notifier_slot;
    double priority;
} pb_replay_decision;

typedef struct pb_replay_config {
    uint32_t num_streams, extra_kernels;
    double unfairness_threshold;
    int32_t total_regs, total_smem, total_threads, total_blocks;  /* whole-GPU aggregate (sm_resources.cpp:17-34) */
} pb_replay_config;

PB_API int pb_sched_replay(const pb_replay_config* cfg, const pb_replay_type* types, uint32_t num_types,
                           const pb_replay_event* events, uint32_t num_events, pb_replay_decision* decisions,
                           uint32_t max_decisions, uint32_t* num_decisions_out, uint32_t* num_finished_out);

/* Interactive form of the same (no GPU needed): the caller plays the clients and the GPU call by call - it
 * submits jobs, is told every dispatch (with the blocks the stage declared and the size of the gang it serves)
 * and feeds back the start / end / copy-done records, or withholds them.  For the scheduler features a recorded
 * trace cannot express: gangs (max_gang, jobs that can lead `gang_capacity` members), deferred dispatch, plugins
 * whose run_next() fails (stage_fails[type][stage] != 0) and the stage watchdog.  pb_sched_sim_flush runs the
 * deferred dispatch loop and the watchdog at `now_us` and returns how many jobs the watchdog failed. */
typedef struct pb_sched_sim pb_sched_sim;
typedef struct pb_sim_config {
    pb_replay_config base;
    const char* scheduler;          /* NULL = "full3" */
    uint32_t max_gang, gang_capacity, deferred;
    double watchdog_factor, watchdog_floor_us;
} pb_sim_config;
typedef struct pb_sim_decision {
    uint32_t job_id, type, stage, is_mem, unfit, num_blocks, gang_size;
    uint32_t failed;                /* the plugin's run_next() raised its error flag: nothing was enqueued, no record will come */
    uint64_t cookie;
} pb_sim_decision;
PB_API int pb_sched_sim_create(const pb_sim_config* cfg, const pb_replay_type* types, uint32_t num_types,
                               const uint8_t* const* stage_fails, pb_sched_sim** out);
PB_API void pb_sched_sim_destroy(pb_sched_sim* sim);
PB_API int pb_sched_sim_new_job(pb_sched_sim* sim, uint32_t type, double now_us, uint64_t cookie);
/* kind: 1 block start, 2 block end, 3 copy done */
PB_API int pb_sched_sim_record(pb_sched_sim* sim, uint32_t kind, uint32_t job_id, uint32_t num, double now_us);
PB_API int pb_sched_sim_flush(pb_sched_sim* sim, double now_us);
PB_API int pb_sched_sim_take_decisions(pb_sched_sim* sim, pb_sim_decision* out, int max);
PB_API int pb_sched_sim_take_finished(pb_sched_sim* sim, uint64_t* cookies, int32_t* errors, int max);
PB_API uint32_t pb_sched_sim_jobs_in_flight(const pb_sched_sim* sim);

#ifdef __cplusplus
}
#endif
#endif /* PAELLA_B200_H */
