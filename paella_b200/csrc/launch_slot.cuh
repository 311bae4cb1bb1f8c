// Launch slot: per-instance device record through which kernels captured in a CUDA graph learn,
// at run time, what a graph cannot bake in: the job id and notifier of this dispatch and the
// input/output buffers of the request, or of every request of a gang (up to kMaxGang requests of
// one model that run as one batched launch; member i is image i of every activation tensor).  The first node of every stage graph copies the slot from a
// pinned host mirror that the host fills right before cudaGraphLaunch.
//
// Kernel parameter convention (all instrumented kernels end with `uint32_t job_id, Notifier* nf`):
//   job_id == kSlotNotify : `nf` is really a `const LaunchSlot*`; notify with the slot's job id / notifier
//   job_id == kSlotQuiet  : `nf` is a `const LaunchSlot*` used for the I/O pointers only; no records
//   otherwise             : direct arguments (nf may be NULL = no records)
#pragma once

#include <llis/job/finished_block_notifier.h>

#include <cstdint>

namespace pb {

constexpr int kMaxGang = 8;

struct LaunchSlot {
    llis::job::FinishedBlockNotifier* nf;
    uint32_t job_id;
    uint32_t reserved;
    const float* io_in[kMaxGang];   // request inputs, NCHW fp32 (host-mapped pinned or device memory), one per member
    float* io_out[kMaxGang];        // request outputs, fp32, one per member
};
static_assert(sizeof(LaunchSlot) == 16 + 16 * kMaxGang, "launch slot layout");

constexpr uint32_t kSlotNotify = 0xFFFFFFFFu;
constexpr uint32_t kSlotQuiet = 0xFFFFFFFEu;

#ifdef __CUDACC__
// Programmatic dependent launch: a kernel launched with the programmatic-serialization attribute may
// start while its predecessor in the stream (or graph) is still running; griddep_wait() blocks until
// that predecessor has completed and its writes are visible, griddep_launch() lets the successor's
// blocks be scheduled early.  Both are no-ops for an ordinary launch.
__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void griddep_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Returns the slot (or NULL) and rewrites job_id / nf to what the notifier calls need.
__device__ __forceinline__ const LaunchSlot* resolve_slot(uint32_t& job_id, llis::job::FinishedBlockNotifier*& nf) {
    if (job_id < kSlotQuiet) return nullptr;
    const LaunchSlot* s = reinterpret_cast<const LaunchSlot*>(nf);
    if (job_id == kSlotNotify) {
        nf = s->nf;
        job_id = s->job_id;
    } else {
        nf = nullptr;
    }
    return s;
}
#endif

}  // namespace pb
