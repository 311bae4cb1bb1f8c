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

}  // namespace llis
