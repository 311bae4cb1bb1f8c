// Internal operator interface shared by the kernel translation units.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>

#include "paella_b200.h"

namespace pb {

// Kernel-side copy of pb_op_params (passed by value as a kernel argument).
struct OpArgs {
    int C, H, W, Cs;
    int K, P, Q, Ks;
    int out_c_off;
    int R, S, stride_h, stride_w, pad_h, pad_w, groups;
    int act, flags, res_Cs;
    int dil_h, dil_w;      // filter dilation (>= 1)
    const void* x;
    const void* w;
    const float* bias;
    const void* residual;
    void* y;
};

// kernels.cu
int simple_op_info(int kind, const pb_op_params* p, pb_launch_info* out);
int simple_op_launch(int kind, const pb_op_params* p, cudaStream_t st, uint32_t job_id, void* notifier, bool pdl = false);
int64_t simple_pack_weights(int kind, const pb_op_params* p, const float* w_oihw, void* dst_host);
void store_elem(void* dst, size_t i, float v, int dtype);
int mnist_fused_info(pb_launch_info* out);
int mnist_fused_launch(const float* x, const float* w1, const float* b1, const float* w2, const float* b2,
                       const float* wd, const float* bd, float* y, int batch, cudaStream_t st, uint32_t job_id, void* notifier);

// conv_umma.cu: tcgen05 implicit-GEMM convolution (bf16 operands, fp32 accumulation in TMEM)
bool conv_umma_supported(const pb_op_params* p);
int conv_umma_info(const pb_op_params* p, pb_launch_info* out);
int conv_umma_launch(const pb_op_params* p, cudaStream_t st, uint32_t job_id, void* notifier);
int64_t conv_umma_pack_weights(const pb_op_params* p, const float* w_oihw, void* dst_host);
// Per-layer state the tensor-core path needs beyond pb_op_params (the TMA descriptor of the
// packed weights).  Created once per layer at model load; `w_dev` is the packed weight buffer.
struct ConvUmmaPlan;
int conv_umma_plan_create(const pb_op_params* p, const void* w_dev, ConvUmmaPlan** out);
void conv_umma_plan_destroy(ConvUmmaPlan* plan);
// Per-instance state: the im2col TMA descriptor of one layer's INPUT tensor (`p->x`).
struct ConvUmmaXMap;
int conv_umma_xmap_create(const pb_op_params* p, ConvUmmaXMap** out);
void conv_umma_xmap_destroy(ConvUmmaXMap* m);
// xmap may be NULL: the descriptor is then encoded for this one launch.
// err_flag: device word raised when a bounded wait runs out (NULL = the library's per-device flag).
// pdl: launch with the programmatic-serialization attribute (the kernel waits for its predecessor
// itself, after its set-up); only meaningful when the previous operation in `st` is a kernel.
int conv_umma_launch_planned(const ConvUmmaPlan* plan, const ConvUmmaXMap* xmap, const pb_op_params* p, cudaStream_t st,
                             uint32_t job_id, void* notifier, uint32_t* err_flag = nullptr, bool pdl = false);
// Grouped launch: up to 8 independent convolutions (their plans, input descriptors and resolved
// parameters) run as ONE grid; the table of descriptors is copied to device memory here.
struct ConvUmmaMulti;
bool conv_umma_multi_available();
// Model launches of tensor-core convolutions go through ConvUmmaMulti tables (one entry for a lone convolution);
// when the persistent kernel is on (PB_CONV_PERSIST=1 when the model is loaded; off by default) a launch of T tiles runs
// conv_umma_persist_grid(T) CTAs, which is what conv_umma_multi_info reports and what notifies.
bool conv_umma_persist_enabled();
uint32_t conv_umma_persist_grid(uint32_t total_tiles);
// Footprint of a persistent launch over `total_tiles` tiles whose widest accumulator has `max_tmem_cols` columns.
void conv_umma_persist_footprint(uint32_t total_tiles, uint32_t max_tmem_cols, pb_launch_info* out);
// kinds[i] (NULL = all convolutions): PB_STAGE_CONV_UMMA, or PB_STAGE_MAXPOOL / PB_STAGE_AVGPOOL for a 3x3 pooling layer that rides
// along (conv_umma_pool_fusable; its plan and map entries are NULL).  At least one entry is a convolution.
int conv_umma_multi_create(const ConvUmmaPlan* const* plans, const ConvUmmaXMap* const* xmaps, const pb_op_params* const* params, const int* kinds,
                           int n, ConvUmmaMulti** out);
bool conv_umma_pool_fusable(int kind, const pb_op_params* p);
uint32_t conv_umma_pool_blocks(const pb_op_params* p);
void conv_umma_multi_destroy(ConvUmmaMulti* m);
void conv_umma_multi_info(const ConvUmmaMulti* m, pb_launch_info* out);
int conv_umma_multi_launch(const ConvUmmaMulti* m, cudaStream_t st, uint32_t job_id, void* notifier, bool pdl);
int conv_umma_time(const pb_op_params* p, int mode, int iters, size_t flush_bytes, double* us_out);
void conv_umma_set_split_gain_us(double us);   // < 0: back to PB_CONV_SPLIT_GAIN_US / the default
int conv_umma_launch_noalloc(const pb_op_params* p, cudaStream_t st, uint32_t job_id, void* notifier);
uint32_t* noalloc_error_flag_ptr(int device);   // NULL until the no-allocation path ran on the device

}  // namespace pb
