// FinishedBlockNotifier: per-stream device object through which every thread
// block of an instrumented kernel reports its start and its end.
//
// Same contract as the reference (include/llis/job/finished_block_notifier.h:18-94,
// create_array in src/job/finished_block_notifier.cu:21-42): thread (0,0,0) of each
// block takes a ticket on a per-notifier counter that wraps at the grid size; one
// record is emitted per 16 blocks plus one remainder record by the last block, so a
// grid of G blocks yields floor(G/16) records {num=16} and, if G%16 != 0, one
// {num=G%16}, per direction.  end() starts with a block barrier.
//
// What differs: the end path fences (gpu scope) before its counter ticket and
// publishes with a system-scope release store, so that when the host sees the last
// end record every block's global writes are visible to whatever the scheduler
// launches next, on any stream.  The reference publishes with a plain volatile
// store and no fence.
#pragma once

#include <llis/ipc/shm_primitive_channel.h>
#include <llis/job/instrument_info.h>

namespace llis {
namespace job {

class FinishedBlockNotifier {
  public:
    static constexpr unsigned noti_batch_size_ = 16;

#ifdef __CUDACC__
    __device__ __forceinline__ void start(JobId job_id) {
        if (threadIdx.x == 0 && threadIdx.y == 0 && threadIdx.z == 0) {
            const unsigned g = gridDim.x * gridDim.y * gridDim.z;
            const unsigned total = atomicInc(&agg_counter_start_, g - 1) + 1;
            const unsigned batch = total % noti_batch_size_;
            if (batch == 0) {
                channel_.write(InstrumentInfo::kStart, 0, (uint8_t)noti_batch_size_, job_id, false);
            } else if (total == g) {
                channel_.write(InstrumentInfo::kStart, 0, (uint8_t)batch, job_id, false);
            }
        }
    }

    __device__ __forceinline__ void end(JobId job_id) {
        __syncthreads();
        if (threadIdx.x == 0 && threadIdx.y == 0 && threadIdx.z == 0) {
            const unsigned g = gridDim.x * gridDim.y * gridDim.z;
            __threadfence();
            const unsigned total = atomicInc(&agg_counter_end_, g - 1) + 1;
            const unsigned batch = total % noti_batch_size_;
            if (batch == 0 || total == g) {
                __threadfence();
                channel_.write(InstrumentInfo::kEnd, 0, (uint8_t)(batch == 0 ? noti_batch_size_ : batch), job_id, true);
            }
        }
    }
#endif

    // Host: n notifiers in device memory, all bound to `channel`.
    static FinishedBlockNotifier* create_array(unsigned num, ipc::Gpu2SchedChannel* channel);
    static void free_array(FinishedBlockNotifier* ptr);

    ipc::Gpu2SchedChannelDev channel_;
    unsigned agg_counter_start_ = 0;
    unsigned agg_counter_end_ = 0;
};

}  // namespace job
}  // namespace llis
