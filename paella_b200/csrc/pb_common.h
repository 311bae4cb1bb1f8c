// Shared helpers of the CUDA library: error reporting and CUDA call checking.
#pragma once

#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>

#include "paella_b200.h"

namespace pb {

void set_error(const char* fmt, ...);

inline int cuda_fail(cudaError_t e, const char* what, const char* file, int line) {
    set_error("%s failed: %s (%s:%d)", what, cudaGetErrorString(e), file, line);
    return PB_ERR_CUDA;
}

#define PB_CUDA(call)                                                        \
    do {                                                                     \
        cudaError_t pb_e_ = (call);                                          \
        if (pb_e_ != cudaSuccess) return ::pb::cuda_fail(pb_e_, #call, __FILE__, __LINE__); \
    } while (0)

#define PB_REQUIRE(cond, ...)                 \
    do {                                      \
        if (!(cond)) {                        \
            ::pb::set_error(__VA_ARGS__);     \
            return PB_ERR_INVALID;            \
        }                                     \
    } while (0)

inline int launch_check(const char* what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        set_error("launch of %s failed: %s", what, cudaGetErrorString(e));
        return PB_ERR_CUDA;
    }
    return PB_OK;
}

// Device-global error flag raised by kernels whose bounded waits run out.
uint32_t* device_error_flag_ptr(int device);

template <typename T>
constexpr T ceil_div(T a, T b) { return (a + b - 1) / b; }
template <typename T>
constexpr T round_up(T a, T b) { return (a + b - 1) / b * b; }

}  // namespace pb
