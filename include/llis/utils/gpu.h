// Host/device function qualifier usable from both g++ and nvcc translation units.
#pragma once

#ifdef __CUDACC__
#define CUDA_HOSTDEV __host__ __device__
#define PB_DEVICE_INLINE __device__ __forceinline__
#else
#define CUDA_HOSTDEV
#define PB_DEVICE_INLINE inline
#endif
