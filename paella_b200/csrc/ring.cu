// Host side of the GPU->host notification ring, notifier arrays, and the small
// instrumented kernels (notification probes, mem-done marker, vec_add, bounded spin).
#include <llis/ipc/shm_primitive_channel.h>
#include <llis/job/finished_block_notifier.h>
#include <llis/job/instrument.h>

#include <time.h>

#include <cstdlib>
#include <cstring>
#include <mutex>
#include <new>

#include "launch_slot.cuh"
#include "ops.h"
#include "pb_common.h"

using llis::ipc::Gpu2SchedChannelDev;
using llis::job::FinishedBlockNotifier;
using llis::job::InstrumentInfo;

namespace pb {

static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}

static uint32_t* g_flag[16] = {};
static std::mutex g_flag_mu;

uint32_t* device_error_flag_ptr(int device) {
    if (device < 0 || device >= 16) return nullptr;
    std::lock_guard<std::mutex> lk(g_flag_mu);
    if (!g_flag[device]) {
        int prev = 0;
        cudaGetDevice(&prev);
        cudaSetDevice(device);
        uint32_t* p = nullptr;
        if (cudaMalloc(&p, sizeof(uint32_t)) == cudaSuccess) {
            cudaMemset(p, 0, sizeof(uint32_t));
            g_flag[device] = p;
        }
        cudaSetDevice(prev);
    }
    return g_flag[device];
}

}  // namespace pb

struct pb_ring {
    int device = 0;
    uint64_t capacity = 0;
    uint32_t log2_capacity = 0;
    uint64_t* slots_host = nullptr;   // pinned, mapped
    uint64_t* slots_dev = nullptr;    // device-visible alias
    unsigned long long* ticket_dev = nullptr;
    uint64_t read_pos = 0;            // monotonic; owned by the single reader
};

extern "C" {

const char* pb_last_error(void) { return pb::g_err; }
const char* pb_version(void) { return "paella_b200 0.1 (sm_100a)"; }

int pb_device_count(void) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    return n;
}

int pb_ring_create(int device, uint64_t capacity, pb_ring** out) {
    PB_REQUIRE(out != nullptr, "pb_ring_create: out is NULL");
    PB_REQUIRE(capacity >= 2 && capacity <= (1ull << 28), "pb_ring_create: capacity %llu out of range",
               (unsigned long long)capacity);
    PB_CUDA(cudaSetDevice(device));
    uint32_t lg = 1;
    while ((1ull << lg) < capacity) ++lg;
    pb_ring* r = new (std::nothrow) pb_ring();
    PB_REQUIRE(r != nullptr, "out of host memory");
    r->device = device;
    r->capacity = 1ull << lg;
    r->log2_capacity = lg;
    cudaError_t e = cudaHostAlloc((void**)&r->slots_host, r->capacity * sizeof(uint64_t),
                                  cudaHostAllocMapped | cudaHostAllocPortable);
    if (e != cudaSuccess) { delete r; return pb::cuda_fail(e, "cudaHostAlloc(ring)", __FILE__, __LINE__); }
    memset(r->slots_host, 0, r->capacity * sizeof(uint64_t));
    e = cudaHostGetDevicePointer((void**)&r->slots_dev, r->slots_host, 0);
    if (e == cudaSuccess) e = cudaMalloc((void**)&r->ticket_dev, sizeof(unsigned long long));
    if (e == cudaSuccess) e = cudaMemset(r->ticket_dev, 0, sizeof(unsigned long long));
    if (e != cudaSuccess) {
        cudaFreeHost(r->slots_host);
        if (r->ticket_dev) cudaFree(r->ticket_dev);
        delete r;
        return pb::cuda_fail(e, "ring device set-up", __FILE__, __LINE__);
    }
    *out = r;
    return PB_OK;
}

void pb_ring_destroy(pb_ring* r) {
    if (!r) return;
    cudaSetDevice(r->device);
    cudaDeviceSynchronize();
    cudaFree(r->ticket_dev);
    cudaFreeHost(r->slots_host);
    delete r;
}

uint64_t pb_ring_capacity(const pb_ring* r) { return r ? r->capacity : 0; }
uint64_t pb_ring_records_read(const pb_ring* r) { return r ? r->read_pos : 0; }

int pb_ring_poll(pb_ring* r, uint64_t* records, int max) {
    int n = 0;
    const uint64_t mask = r->capacity - 1;
    while (n < max) {
        const uint64_t pos = r->read_pos;
        const uint64_t v = __atomic_load_n(&r->slots_host[pos & mask], __ATOMIC_ACQUIRE);
        const uint8_t status = (uint8_t)((v >> 24) & 0xff);
        const uint8_t want = InstrumentInfo::status_for(pos, r->log2_capacity);
        if (status == want) {
            records[n++] = v;
            r->read_pos = pos + 1;
            continue;
        }
        // Not written yet in this lap: the slot still holds the previous lap's tag (or 0 on lap 0).
        const uint64_t lap = pos >> r->log2_capacity;
        const uint8_t prev = lap == 0 ? 0 : InstrumentInfo::status_for(pos - r->capacity, r->log2_capacity);
        if (status != prev) {
            pb::set_error("notification ring overflow at record %llu (slot tag %u, expected %u or %u)",
                          (unsigned long long)pos, status, want, prev);
            return PB_ERR_RING_OVERFLOW;
        }
        break;
    }
    return n;
}

int pb_ring_device_view(const pb_ring* r, void* view_out, size_t view_size) {
    PB_REQUIRE(r && view_out && view_size == sizeof(Gpu2SchedChannelDev), "pb_ring_device_view: bad arguments");
    Gpu2SchedChannelDev v;
    v.slots = r->slots_dev;
    v.ticket = r->ticket_dev;
    v.mask = (uint32_t)(r->capacity - 1);
    v.log2_capacity = r->log2_capacity;
    memcpy(view_out, &v, sizeof(v));
    return PB_OK;
}

size_t pb_notifier_size(void) { return sizeof(FinishedBlockNotifier); }

int pb_notifier_create_array(pb_ring* r, uint32_t n, void** dev_array_out) {
    PB_REQUIRE(r && dev_array_out && n > 0, "pb_notifier_create_array: bad arguments");
    PB_CUDA(cudaSetDevice(r->device));
    FinishedBlockNotifier* host = (FinishedBlockNotifier*)calloc(n, sizeof(FinishedBlockNotifier));
    PB_REQUIRE(host != nullptr, "out of host memory");
    for (uint32_t i = 0; i < n; ++i) {
        pb_ring_device_view(r, &host[i].channel_, sizeof(Gpu2SchedChannelDev));
        host[i].agg_counter_start_ = 0;
        host[i].agg_counter_end_ = 0;
    }
    void* dev = nullptr;
    cudaError_t e = cudaMalloc(&dev, n * sizeof(FinishedBlockNotifier));
    if (e == cudaSuccess) e = cudaMemcpy(dev, host, n * sizeof(FinishedBlockNotifier), cudaMemcpyHostToDevice);
    free(host);
    if (e != cudaSuccess) {
        if (dev) cudaFree(dev);
        return pb::cuda_fail(e, "notifier array set-up", __FILE__, __LINE__);
    }
    *dev_array_out = dev;
    return PB_OK;
}

void pb_notifier_free_array(void* dev_array) {
    if (dev_array) cudaFree(dev_array);
}

int pb_device_error_flag(int device, uint32_t* flag_out, int reset) {
    uint32_t* p = pb::device_error_flag_ptr(device);
    PB_REQUIRE(p != nullptr, "no error flag for device %d", device);
    PB_CUDA(cudaSetDevice(device));
    if (flag_out) PB_CUDA(cudaMemcpy(flag_out, p, sizeof(uint32_t), cudaMemcpyDeviceToHost));
    if (reset) PB_CUDA(cudaMemset(p, 0, sizeof(uint32_t)));
    // the no-allocation convolution path keeps its own flag (it may not share one that was cudaMalloc'ed)
    if (uint32_t* q = pb::noalloc_error_flag_ptr(device)) {
        uint32_t v = 0;
        PB_CUDA(cudaMemcpy(&v, q, sizeof(uint32_t), cudaMemcpyDeviceToHost));
        if (flag_out) *flag_out |= v;      // both flags are reported: neither hides the other
        if (reset) PB_CUDA(cudaMemset(q, 0, sizeof(uint32_t)));
    }
    return PB_OK;
}

}  // extern "C"

// ---------------------------------------------------------------------------
// Kernels
// ---------------------------------------------------------------------------
namespace {

__device__ __forceinline__ unsigned long long globaltimer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__global__ void notify_probe_agg(uint32_t job_id, FinishedBlockNotifier* n) {
    n->start(job_id);
    n->end(job_id);
}

__global__ void notify_probe_per_block(uint32_t job_id, FinishedBlockNotifier* n) {
    llis::job::kernel_start(job_id, &n->channel_);
    llis::job::kernel_end(job_id, &n->channel_);
}

__global__ void mem_done_kernel(uint32_t job_id, const Gpu2SchedChannelDev* ch) {
    if (threadIdx.x == 0) ch->write(InstrumentInfo::kMemDone, 0, 1, job_id, true);
}

__global__ void latency_probe_kernel(FinishedBlockNotifier* n) {
    if (threadIdx.x == 0) {
        const uint32_t t = (uint32_t)globaltimer_ns();
        n->channel_.write(InstrumentInfo::kEnd, (uint8_t)llis::job::pb_smid(), 1, t, true);
    }
}

__global__ void read_globaltimer_kernel(unsigned long long* out) { *out = globaltimer_ns(); }

// Ring round-trip probe: one thread answers `iters` host "pings" (a counter in host-mapped memory)
// with one record each.  Every wait is bounded: after `max_polls` polls without the expected value
// the kernel writes status 2 and returns.
__global__ void ring_pingpong_kernel(const volatile uint32_t* ping, uint32_t iters, uint32_t max_polls, FinishedBlockNotifier* n,
                                     uint32_t* status) {
    if (threadIdx.x != 0 || blockIdx.x != 0) return;
    for (uint32_t i = 1; i <= iters; ++i) {
        uint32_t polls = 0;
        while (*ping != i) {
            if (++polls > max_polls) { *status = 2; return; }
        }
        n->channel_.write(InstrumentInfo::kEnd, 0, 1, i, true);
    }
    *status = 1;
}

// out[i] += in[i]; 128-bit vectors, grid-stride.
__global__ void __launch_bounds__(256) vec_add_kernel(float* __restrict__ out, const float* __restrict__ in,
                                                      uint64_t n, uint32_t job_id, FinishedBlockNotifier* nf) {
    if (nf) nf->start(job_id);
    const uint64_t n4 = n >> 2;
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    float4* o4 = reinterpret_cast<float4*>(out);
    const float4* i4 = reinterpret_cast<const float4*>(in);
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
        float4 a = __ldcs(o4 + i);
        const float4 b = __ldcs(i4 + i);
        a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
        __stcs(o4 + i, a);
    }
    for (uint64_t i = (n4 << 2) + (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) out[i] += in[i];
    if (nf) nf->end(job_id);
}

// Occupies its SM slot for spin_ns, bounded by the device clock; never waits on anything external.
__global__ void __launch_bounds__(256) spin_kernel(uint64_t spin_ns, uint32_t* sink, uint32_t job_id,
                                                   FinishedBlockNotifier* nf) {
    if (nf) nf->start(job_id);
    const unsigned long long t0 = globaltimer_ns();
    uint32_t acc = threadIdx.x;
    // Iteration cap: even if the timer misbehaved the loop ends (2^26 polls ~ tens of ms).
    for (uint32_t it = 0; it < (1u << 26); ++it) {
        if (globaltimer_ns() - t0 >= spin_ns) break;
        acc = acc * 1664525u + 1013904223u;
    }
    if (sink && acc == 0xdeadbeefu) sink[0] = acc;
    if (nf) nf->end(job_id);
}

}  // namespace

extern "C" {

int pb_launch_notify_probe(void* stream, uint32_t num_blocks, uint32_t threads, uint32_t job_id, void* notifier,
                           int aggregated) {
    PB_REQUIRE(notifier && num_blocks > 0 && threads > 0 && threads <= 1024, "pb_launch_notify_probe: bad arguments");
    if (aggregated)
        notify_probe_agg<<<num_blocks, threads, 0, (cudaStream_t)stream>>>(job_id, (FinishedBlockNotifier*)notifier);
    else
        notify_probe_per_block<<<num_blocks, threads, 0, (cudaStream_t)stream>>>(job_id, (FinishedBlockNotifier*)notifier);
    return pb::launch_check("notify_probe");
}

int pb_launch_mem_done(void* stream, uint32_t job_id, void* notifier_or_ring_view) {
    PB_REQUIRE(notifier_or_ring_view != nullptr, "pb_launch_mem_done: NULL channel");
    // A notifier starts with its channel view, so either pointer works.
    mem_done_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(job_id, (const Gpu2SchedChannelDev*)notifier_or_ring_view);
    return pb::launch_check("mem_done");
}

int pb_launch_latency_probe(void* stream, uint32_t num_blocks, void* notifier) {
    PB_REQUIRE(notifier && num_blocks > 0, "pb_launch_latency_probe: bad arguments");
    latency_probe_kernel<<<num_blocks, 32, 0, (cudaStream_t)stream>>>((FinishedBlockNotifier*)notifier);
    return pb::launch_check("latency_probe");
}

int pb_clock_calibrate(int device, uint64_t out[3]) {
    PB_CUDA(cudaSetDevice(device));
    unsigned long long* host = nullptr;
    PB_CUDA(cudaHostAlloc((void**)&host, sizeof(*host), cudaHostAllocMapped));
    unsigned long long* dev = nullptr;
    cudaError_t e = cudaHostGetDevicePointer((void**)&dev, host, 0);
    if (e != cudaSuccess) { cudaFreeHost(host); return pb::cuda_fail(e, "cudaHostGetDevicePointer", __FILE__, __LINE__); }
    uint64_t best[3] = {0, 0, ~0ull};
    for (int i = 0; i < 20; ++i) {
        cudaDeviceSynchronize();
        struct timespec a, b;
        clock_gettime(CLOCK_MONOTONIC, &a);
        read_globaltimer_kernel<<<1, 1>>>(dev);
        cudaDeviceSynchronize();
        clock_gettime(CLOCK_MONOTONIC, &b);
        const uint64_t ta = (uint64_t)a.tv_sec * 1000000000ull + a.tv_nsec;
        const uint64_t tb = (uint64_t)b.tv_sec * 1000000000ull + b.tv_nsec;
        if (tb - ta < best[2] - best[0]) { best[0] = ta; best[1] = *host; best[2] = tb; }
    }
    cudaFreeHost(host);
    out[0] = best[0]; out[1] = best[1]; out[2] = best[2];
    return PB_OK;
}

int pb_ring_roundtrip_bench(int device, uint32_t iters, double* rtt_us_out) {
    PB_REQUIRE(rtt_us_out && iters > 0 && iters <= 100000, "pb_ring_roundtrip_bench: bad arguments");
    PB_CUDA(cudaSetDevice(device));
    pb_ring* ring = nullptr;
    void* nf = nullptr;
    int rc = pb_ring_create(device, 1 << 12, &ring);
    if (rc != PB_OK) return rc;
    rc = pb_notifier_create_array(ring, 1, &nf);
    if (rc != PB_OK) { pb_ring_destroy(ring); return rc; }
    volatile uint32_t* ping = nullptr;
    uint32_t* status = nullptr;
    cudaStream_t st = nullptr;
    cudaError_t e = cudaHostAlloc((void**)&ping, 64, cudaHostAllocMapped);
    if (e == cudaSuccess) e = cudaHostAlloc((void**)&status, 64, cudaHostAllocMapped);
    if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking);
    if (e != cudaSuccess) {
        if (ping) cudaFreeHost((void*)ping);
        if (status) cudaFreeHost(status);
        pb_notifier_free_array(nf);
        pb_ring_destroy(ring);
        return pb::cuda_fail(e, "round-trip probe set-up", __FILE__, __LINE__);
    }
    *ping = 0;
    *status = 0;
    // about one second of polling per ping at most (a poll of host memory takes ~1 us)
    ring_pingpong_kernel<<<1, 32, 0, st>>>(ping, iters, 1u << 20, (FinishedBlockNotifier*)nf, status);
    rc = pb::launch_check("ring_pingpong");
    uint64_t rec = 0;
    for (uint32_t i = 1; rc == PB_OK && i <= iters; ++i) {
        struct timespec a, b;
        clock_gettime(CLOCK_MONOTONIC, &a);
        __atomic_store_n((uint32_t*)ping, i, __ATOMIC_RELEASE);
        int n = 0;
        for (uint64_t spins = 0; n == 0 && spins < (1ull << 28); ++spins) n = pb_ring_poll(ring, &rec, 1);
        clock_gettime(CLOCK_MONOTONIC, &b);
        if (n != 1) { pb::set_error("ring round trip %u: no record (status %u)", i, *status); rc = n < 0 ? n : PB_ERR_TIMEOUT; break; }
        rtt_us_out[i - 1] = ((double)(b.tv_sec - a.tv_sec) * 1e9 + (double)(b.tv_nsec - a.tv_nsec)) * 1e-3;
    }
    if (rc != PB_OK) __atomic_store_n((uint32_t*)ping, 0xffffffffu, __ATOMIC_RELEASE);   // lets the kernel run out its poll limit
    cudaStreamSynchronize(st);
    cudaStreamDestroy(st);
    cudaFreeHost((void*)ping);
    cudaFreeHost(status);
    pb_notifier_free_array(nf);
    pb_ring_destroy(ring);
    return rc;
}

// The same one-thread kernel with a ping that never comes: its wait runs out after `max_polls` polls of host
// memory, it records status 2 and returns; the context stays usable.  This is how a device-side wait is
// expected to fail everywhere in this library, and the test of that.
int pb_ring_wait_expiry_probe(int device, uint32_t max_polls, uint32_t* status_out, uint32_t* records_out) {
    PB_REQUIRE(status_out && max_polls >= 1 && max_polls <= (1u << 16), "pb_ring_wait_expiry_probe: max_polls outside 1..65536");
    PB_CUDA(cudaSetDevice(device));
    pb_ring* ring = nullptr;
    void* nf = nullptr;
    int rc = pb_ring_create(device, 1 << 8, &ring);
    if (rc != PB_OK) return rc;
    rc = pb_notifier_create_array(ring, 1, &nf);
    if (rc != PB_OK) { pb_ring_destroy(ring); return rc; }
    volatile uint32_t* ping = nullptr;
    uint32_t* status = nullptr;
    cudaError_t e = cudaHostAlloc((void**)&ping, 64, cudaHostAllocMapped);
    if (e == cudaSuccess) e = cudaHostAlloc((void**)&status, 64, cudaHostAllocMapped);
    if (e == cudaSuccess) {
        *ping = 0;          // the kernel waits for 1
        *status = 0;
        ring_pingpong_kernel<<<1, 32>>>(ping, 1, max_polls, (FinishedBlockNotifier*)nf, status);
        rc = pb::launch_check("ring_pingpong");
        e = cudaDeviceSynchronize();
    }
    if (e != cudaSuccess && rc == PB_OK) rc = pb::cuda_fail(e, "wait-expiry probe", __FILE__, __LINE__);
    if (rc == PB_OK) {
        *status_out = *status;
        uint64_t rec = 0;
        if (records_out) *records_out = pb_ring_poll(ring, &rec, 1) == 1 ? 1u : 0u;
    }
    if (ping) cudaFreeHost((void*)ping);
    if (status) cudaFreeHost(status);
    pb_notifier_free_array(nf);
    pb_ring_destroy(ring);
    return rc;
}

int pb_vec_add_bench(int device, uint64_t n, int iters, size_t flush_bytes, double* us_out) {
    PB_REQUIRE(us_out && n > 0 && iters > 0, "pb_vec_add_bench: bad arguments");
    PB_CUDA(cudaSetDevice(device));
    float *a = nullptr, *b = nullptr;
    void* flush = nullptr;
    cudaStream_t st = nullptr;
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    cudaError_t e = cudaMalloc((void**)&a, n * 4);
    if (e == cudaSuccess) e = cudaMalloc((void**)&b, n * 4);
    if (e == cudaSuccess && flush_bytes) e = cudaMalloc(&flush, flush_bytes);
    if (e == cudaSuccess) e = cudaMemset(a, 0, n * 4);
    if (e == cudaSuccess) e = cudaMemset(b, 0, n * 4);
    if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaEventCreate(&e0);
    if (e == cudaSuccess) e = cudaEventCreate(&e1);
    int rc = e == cudaSuccess ? PB_OK : pb::cuda_fail(e, "vec_add bench set-up", __FILE__, __LINE__);
    double total_ms = 0;
    for (int i = 0; rc == PB_OK && i < iters + 3; ++i) {
        if (flush) cudaMemsetAsync(flush, i, flush_bytes, st);
        cudaEventRecord(e0, st);
        rc = pb_vec_add_launch(a, b, n, st, 0, nullptr);
        cudaEventRecord(e1, st);
        if (cudaEventSynchronize(e1) != cudaSuccess) { rc = PB_ERR_CUDA; break; }
        float ms = 0;
        cudaEventElapsedTime(&ms, e0, e1);
        if (i >= 3) total_ms += ms;
    }
    if (e0) cudaEventDestroy(e0);
    if (e1) cudaEventDestroy(e1);
    if (st) cudaStreamDestroy(st);
    if (a) cudaFree(a);
    if (b) cudaFree(b);
    if (flush) cudaFree(flush);
    if (rc == PB_OK) *us_out = total_ms * 1000.0 / iters;
    return rc;
}

static int kernel_regs(const void* fn) {
    cudaFuncAttributes a;
    if (cudaFuncGetAttributes(&a, fn) != cudaSuccess) { cudaGetLastError(); return 32; }
    return a.numRegs;
}

static uint32_t vec_add_blocks(uint64_t n) {
    // 4 elements per thread per trip; cap the grid at 8 blocks per SM of a 148-SM part.
    uint64_t b = pb::ceil_div<uint64_t>(pb::ceil_div<uint64_t>(n, 4), 256);
    if (b < 1) b = 1;
    if (b > 148 * 8) b = 148 * 8;
    return (uint32_t)b;
}

int pb_vec_add_info(uint64_t n, pb_launch_info* out) {
    PB_REQUIRE(out != nullptr, "pb_vec_add_info: out is NULL");
    memset(out, 0, sizeof(*out));
    out->num_blocks = vec_add_blocks(n);
    out->threads_per_block = 256;
    out->regs_per_thread = kernel_regs((const void*)vec_add_kernel);
    out->bytes = 12ull * n;
    return PB_OK;
}

int pb_vec_add_launch(float* out_dev, const float* in_dev, uint64_t n, void* stream, uint32_t job_id, void* notifier) {
    PB_REQUIRE(out_dev && in_dev, "pb_vec_add_launch: NULL buffer");
    PB_REQUIRE(((uintptr_t)out_dev % 16 == 0) && ((uintptr_t)in_dev % 16 == 0), "pb_vec_add_launch: buffers must be 16-byte aligned");
    vec_add_kernel<<<vec_add_blocks(n), 256, 0, (cudaStream_t)stream>>>(out_dev, in_dev, n, job_id,
                                                                      (FinishedBlockNotifier*)notifier);
    return pb::launch_check("vec_add");
}

int pb_spin_info(uint32_t num_blocks, pb_launch_info* out) {
    PB_REQUIRE(out != nullptr && num_blocks > 0, "pb_spin_info: bad arguments");
    memset(out, 0, sizeof(*out));
    out->num_blocks = num_blocks;
    out->threads_per_block = 256;
    out->regs_per_thread = kernel_regs((const void*)spin_kernel);
    return PB_OK;
}

int pb_spin_launch(uint32_t num_blocks, uint64_t spin_ns, uint32_t* sink_dev, void* stream, uint32_t job_id,
                   void* notifier) {
    PB_REQUIRE(num_blocks > 0, "pb_spin_launch: zero blocks");
    PB_REQUIRE(spin_ns <= 50ull * 1000 * 1000, "pb_spin_launch: spin longer than 50 ms refused");
    spin_kernel<<<num_blocks, 256, 0, (cudaStream_t)stream>>>(spin_ns, sink_dev, job_id, (FinishedBlockNotifier*)notifier);
    return pb::launch_check("spin");
}

}  // extern "C"
