// Gpu2SchedChannel: the fixed-record ring that device code writes and the
// scheduler thread reads.
//
// Replaces the reference's ShmPrimitiveChannelGpu<uint64_t>
// (include/llis/ipc/shm_primitive_channel.h:11-68, write/read/can_read in
// include/llis/ipc/shm_primitive_channel_impl.h:18-64, set-up in
// src/ipc/shm_primitive_channel.cu:49-131).  Kept: one ring per scheduler, 8-byte
// records, a ticket counter in DEVICE memory, slots in host-mapped pinned memory,
// no back-pressure on the writer.  Changed: capacity is a power of two, tickets
// are a monotonic 64-bit atomicAdd (slot = ticket & mask), every slot has exactly
// one writer per lap, the record is published with one 8-byte system-scope store
// (release for end records), and the reader never writes to the ring (see
// instrument_info.h for the lap-tagged status byte).
#pragma once

#include <cstddef>
#include <cstdint>

#include <llis/job/instrument_info.h>
#include <llis/utils/gpu.h>

struct pb_ring;  // C-ABI handle, see paella_b200.h

namespace llis {
namespace ipc {

// Device-side view of the ring; trivially copyable, embedded in every notifier.
struct Gpu2SchedChannelDev {
    uint64_t* slots;              // device-visible address of the pinned slots
    unsigned long long* ticket;   // device memory
    uint32_t mask;                // capacity - 1
    uint32_t log2_capacity;

#ifdef __CUDACC__
    // One call = one record.  `release` orders the caller's (and, through the
    // block barrier and the notifier's counter, the kernel's) earlier global
    // writes before the record becomes visible to the host.
    __device__ __forceinline__ void write(uint8_t is_start, uint8_t smid, uint8_t num, JobId job_id, bool release) const {
        const unsigned long long t = atomicAdd(ticket, 1ULL);
        const uint8_t status = job::InstrumentInfo::status_for(t, log2_capacity);
        const uint64_t rec = job::InstrumentInfo::pack(is_start, smid, num, status, job_id);
        uint64_t* p = slots + (t & mask);
        if (release) {
            asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(rec) : "memory");
        } else {
            asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(rec) : "memory");
        }
    }
#endif
};

// Host-side owner.  Thin C++ face over the C ABI (pb_ring_*).
class Gpu2SchedChannel {
  public:
    Gpu2SchedChannel() = default;
    explicit Gpu2SchedChannel(size_t count, int device = 0);
    ~Gpu2SchedChannel();
    Gpu2SchedChannel(const Gpu2SchedChannel&) = delete;
    Gpu2SchedChannel& operator=(const Gpu2SchedChannel&) = delete;

    void connect(size_t count, int device = 0);
    void disconnect();
    bool is_connected() const { return ring_ != nullptr; }

    // Non-blocking: true and *out filled when a record is available.
    // Throws std::runtime_error if the writer lapped the reader.
    bool try_read(job::InstrumentInfo* out);
    // Blocking read with a spin limit (0 = unlimited); returns false on timeout.
    bool read(job::InstrumentInfo* out, uint64_t max_spins = 0);

    pb_ring* handle() const { return ring_; }
    Gpu2SchedChannelDev device_view() const;

  private:
    pb_ring* ring_ = nullptr;
};

}  // namespace ipc
}  // namespace llis
