// Identifier types and client/server message tags of the serving boundary.
// Same names and numeric values as the reference's include/llis/ipc/defs.h:7-21,
// because they travel on the client<->server wire.
#pragma once

#include <cstdint>

namespace llis {

using ClientId = uint32_t;
using JobRefId = uint32_t;
using JobInstanceRefId = uint32_t;
using JobId = uint32_t;

enum class MsgType : uint32_t {
    REGISTER_CLIENT = 0,
    REGISTER_JOB = 1,
    LAUNCH_JOB = 2,
    GROW_POOL = 3,
    CUDA_PROFILER_START = 4,
    CUDA_PROFILER_STOP = 5,
    PROFILER_CMD = 6,
    EXIT_CMD = 7
};

// Sub-commands that follow MsgType::PROFILER_CMD on the wire (include/llis/ipc/defs.h:23-37 of the
// reference); SAVE is followed by the output path prefix as a string.
enum class ProfilerMsgType : uint32_t {
    SET_RECORD_KERNEL_INFO = 0,
    UNSET_RECORD_KERNEL_INFO = 1,
    SET_RECORD_BLOCK_EXEC_TIME = 2,
    UNSET_RECORD_BLOCK_EXEC_TIME = 3,
    SET_RECORD_KERNEL_BLOCK_MIS_ALLOC = 4,
    UNSET_RECORD_KERNEL_BLOCK_MIS_ALLOC = 5,
    SET_RECORD_RUN_NEXT_TIMES = 6,
    UNSET_RECORD_RUN_NEXT_TIMES = 7,
    SET_RECORD_JOB_EVENTS = 8,
    UNSET_RECORD_JOB_EVENTS = 9,
    SET_RECORD_RESOURCE_EVENTS = 10,
    UNSET_RECORD_RESOURCE_EVENTS = 11,
    SAVE = 12
};

}  // namespace llis
