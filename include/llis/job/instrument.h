// Un-aggregated notifications: one record per thread block per direction, carrying
// the SM id.  Same API as the reference's include/llis/job/instrument.h:9-63, with
// the channel passed by its device view.
#pragma once

#include <llis/ipc/shm_primitive_channel.h>

namespace llis {
namespace job {

#ifdef __CUDACC__
__device__ __forceinline__ unsigned pb_smid() {
    unsigned smid;
    asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
    return smid;
}

__device__ __forceinline__ void kernel_start(JobId job_id, const ipc::Gpu2SchedChannelDev* channel) {
    if (threadIdx.x == 0 && threadIdx.y == 0 && threadIdx.z == 0) {
        channel->write(InstrumentInfo::kStart, (uint8_t)pb_smid(), 1, job_id, false);
    }
}

__device__ __forceinline__ void kernel_end(JobId job_id, const ipc::Gpu2SchedChannelDev* channel) {
    __syncthreads();
    if (threadIdx.x == 0 && threadIdx.y == 0 && threadIdx.z == 0) {
        __threadfence();
        channel->write(InstrumentInfo::kEnd, (uint8_t)pb_smid(), 1, job_id, true);
    }
}
#endif

}  // namespace job
}  // namespace llis
