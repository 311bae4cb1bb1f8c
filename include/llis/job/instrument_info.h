// The 8-byte GPU->host notification record.
//
// Field layout follows the reference record (include/llis/job/instrument_info.h:9-38):
//   byte 0 is_start, byte 1 smid, byte 2 num, byte 3 status, bytes 4..7 job_id.
// Differences, both deliberate:
//  * status is not a full/empty flag that the reader clears.  It carries the lap
//    of the ring the record was written in (1 + lap % 255, never 0), so the host
//    only ever READS the pinned ring and can tell "not written yet" (previous
//    lap's value) from "writer lapped the reader" (any other value).
//  * is_start has a third value, kMemDone, used by the tiny kernel that follows an
//    asynchronous copy stage; the reference signals those through
//    cudaLaunchHostFunc and a second CPU ring (src/server/scheduler_full3.cpp:429-431,465-468).
#pragma once

#include <cstdint>

#include <llis/ipc/defs.h>
#include <llis/utils/gpu.h>

namespace llis {
namespace job {

struct InstrumentInfo {
    static constexpr uint8_t kEnd = 0;
    static constexpr uint8_t kStart = 1;
    static constexpr uint8_t kMemDone = 2;

    uint8_t is_start;
    uint8_t smid;
    uint8_t num;
    uint8_t status;
    JobId job_id;

    CUDA_HOSTDEV static uint64_t pack(uint8_t is_start, uint8_t smid, uint8_t num, uint8_t status, JobId job_id) {
        return (uint64_t)is_start | ((uint64_t)smid << 8) | ((uint64_t)num << 16) | ((uint64_t)status << 24) |
               ((uint64_t)job_id << 32);
    }
    CUDA_HOSTDEV static InstrumentInfo unpack(uint64_t v) {
        InstrumentInfo i;
        i.is_start = (uint8_t)(v & 0xff);
        i.smid = (uint8_t)((v >> 8) & 0xff);
        i.num = (uint8_t)((v >> 16) & 0xff);
        i.status = (uint8_t)((v >> 24) & 0xff);
        i.job_id = (JobId)(v >> 32);
        return i;
    }
    // Status byte a record written with ring ticket `ticket` carries.
    CUDA_HOSTDEV static uint8_t status_for(uint64_t ticket, unsigned log2_capacity) {
        return (uint8_t)(1u + (unsigned)((ticket >> log2_capacity) % 255u));
    }
};

static_assert(sizeof(InstrumentInfo) == 8, "notification record must stay 8 bytes");

}  // namespace job
}  // namespace llis
