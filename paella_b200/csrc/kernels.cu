// Inference operators other than the tensor-core convolution: channels-last
// ([H][W][Cs]) kernels for layout conversion, direct (SIMT) convolution, depthwise
// convolution, pooling, dense, add and softmax.  These are the memory-bound members
// of the kernel family the reference's TVM adapters launch
// (jobs/tvm_<model>/tvm_<model>.cpp:24-47); every kernel reports block start/end on
// the job's notifier exactly once per block.
//
// Access pattern: the channel dimension is innermost and padded to a 16-byte vector
// (4 fp32 / 8 bf16), so one thread moves one 128-bit vector and a warp reads a
// contiguous 512-byte span whenever Cs >= 32 vectors.
#include <cuda_bf16.h>
#include <llis/job/finished_block_notifier.h>

#include <cstdlib>
#include <cstring>

#include "launch_slot.cuh"
#include "ops.h"
#include "pb_common.h"

using llis::job::FinishedBlockNotifier;

namespace pb {

// ---- 128-bit vectors of activations ---------------------------------------
template <typename T> struct Vec;
template <> struct Vec<float> {
    static constexpr int N = 4;
    float v[4];
    __device__ __forceinline__ static Vec load(const float* p) {
        Vec r; const float4 t = *reinterpret_cast<const float4*>(p);
        r.v[0] = t.x; r.v[1] = t.y; r.v[2] = t.z; r.v[3] = t.w; return r;
    }
    __device__ __forceinline__ void store(float* p) const { *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]); }
};
template <> struct Vec<__nv_bfloat16> {
    static constexpr int N = 8;
    float v[8];
    __device__ __forceinline__ static Vec load(const __nv_bfloat16* p) {
        Vec r; const uint4 t = *reinterpret_cast<const uint4*>(p);
        const uint32_t u[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            r.v[2 * i] = __uint_as_float(u[i] << 16);
            r.v[2 * i + 1] = __uint_as_float(u[i] & 0xffff0000u);
        }
        return r;
    }
    __device__ __forceinline__ void store(__nv_bfloat16* p) const {
        uint32_t u[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
            u[i] = *reinterpret_cast<const uint32_t*>(&h);
        }
        *reinterpret_cast<uint4*>(p) = make_uint4(u[0], u[1], u[2], u[3]);
    }
};

template <typename T> __device__ __forceinline__ float to_f(T x);
template <> __device__ __forceinline__ float to_f<float>(float x) { return x; }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }
template <typename T> __device__ __forceinline__ T from_f(float x);
template <> __device__ __forceinline__ float from_f<float>(float x) { return x; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }

__device__ __forceinline__ float act_fn(float v, int act) {
    if (act == 1) return fmaxf(v, 0.f);
    if (act == 2) return fminf(fmaxf(v, 0.f), 6.f);
    return v;
}

// Every kernel here may be launched as a programmatic dependent of the previous kernel of its stage
// graph: it waits for that kernel on the device before touching memory (a no-op otherwise).
#define PB_NOTIFY_START()                                        \
    pb::griddep_wait();                                           \
    const pb::LaunchSlot* slot_ = pb::resolve_slot(job_id, nf);  \
    (void)slot_;                                                  \
    if (nf) nf->start(job_id)
#define PB_NOTIFY_END() if (nf) nf->end(job_id)

// Batched launches (a gang of requests of one model): blockIdx.y is the image.  Image i of an
// activation tensor follows image i - 1 without padding, so the tensor-core convolution sees the
// images as one [batch * pixels][channels] matrix.
template <typename T> __device__ __forceinline__ const T* x_img(const OpArgs& a) {
    return static_cast<const T*>(a.x) + (size_t)blockIdx.y * a.H * a.W * a.Cs;
}
template <typename T> __device__ __forceinline__ T* y_img(const OpArgs& a) {
    return static_cast<T*>(a.y) + (size_t)blockIdx.y * a.P * a.Q * a.Ks;
}
// fp32 model output of this image (a.flags & 2): the request's own buffer when a.y is NULL
__device__ __forceinline__ float* out_f32_img(const OpArgs& a, const pb::LaunchSlot* slot, int n_out) {
    return (!a.y && slot) ? slot->io_out[blockIdx.y] : static_cast<float*>(a.y) + (size_t)blockIdx.y * n_out;
}

// ---- NCHW fp32 -> channels-last T ------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) input_transform_kernel(const float* x, T* __restrict__ y, int C, int HW,
                                                              int Cs, uint32_t job_id, FinishedBlockNotifier* nf) {
    PB_NOTIFY_START();
    x = (!x && slot_) ? slot_->io_in[blockIdx.y] : x + (size_t)blockIdx.y * C * HW;   // the request's input buffer, known only at dispatch
    y += (size_t)blockIdx.y * HW * Cs;
    const int pix = blockIdx.x * blockDim.x + threadIdx.x;
    if (pix < HW) {
        for (int c0 = 0; c0 < Cs; c0 += Vec<T>::N) {
            Vec<T> o;
#pragma unroll
            for (int j = 0; j < Vec<T>::N; ++j) o.v[j] = (c0 + j < C) ? x[(size_t)(c0 + j) * HW + pix] : 0.f;
            o.store(y + (size_t)pix * Cs + c0);
        }
    }
    PB_NOTIFY_END();
}

// ---- NCHW fp32 -> patch matrix [P*Q][Ks] ------------------------------------------------
// The first convolution of an image model has 3 input channels: as an implicit GEMM every filter tap
// would be padded to a 64-channel k-block (1/21 useful).  This kernel writes the im2col rows themselves,
// y[(p, q)][k] with k = (r*S + s)*C + c (zero for k >= R*S*C and outside the image), so that the
// convolution becomes a pointwise one over R*S*C "channels": 1 k-block instead of 9 for a 3x3 stem,
// 3 instead of 49 for a 7x7 one.  One thread per (output pixel, 8 consecutive k).
template <typename T>
__global__ void __launch_bounds__(256) input_patch_kernel(OpArgs a, uint32_t job_id, FinishedBlockNotifier* nf) {
    PB_NOTIFY_START();
    const float* __restrict__ x = (!a.x && slot_) ? slot_->io_in[blockIdx.y]      // the request's input buffer, known only at dispatch
                                                  : static_cast<const float*>(a.x) + (size_t)blockIdx.y * a.C * a.H * a.W;
    constexpr int N = Vec<T>::N;
    const int kv = a.Ks / N;
    const int total = a.P * a.Q * kv;
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx < total) {
        const int k0 = (idx % kv) * N;
        const int pix = idx / kv;
        const int q = pix % a.Q, p = pix / a.Q;
        const int taps_c = a.R * a.S * a.C;
        Vec<T> o;
#pragma unroll
        for (int j = 0; j < N; ++j) {
            const int k = k0 + j;
            float v = 0.f;
            if (k < taps_c) {
                const int tap = k / a.C, c = k - tap * a.C;
                const int r = tap / a.S, s = tap - r * a.S;
                const int ih = p * a.stride_h + r - a.pad_h, iw = q * a.stride_w + s - a.pad_w;
                if (ih >= 0 && ih < a.H && iw >= 0 && iw < a.W) v = __ldg(x + ((size_t)c * a.H + ih) * a.W + iw);
            }
            o.v[j] = v;
        }
        o.store(y_img<T>(a) + (size_t)pix * a.Ks + k0);
    }
    PB_NOTIFY_END();
}

// The same patch matrix, a tile of output pixels per block.  input_patch_kernel reads every input value through eight
// scattered 4-byte loads per output vector (each value about 2.25 times, with the index arithmetic of its filter tap
// every time) and holds a block slot for 256 output vectors; under serving load that costs more than its share of a
// lone request (6.7 % of the Inception-v3 throughput, measured by leaving it out).  Here a block first copies the
// window of its kPatchTileP x kPatchTileQ output pixels into shared memory with coalesced loads that are all in flight
// together (fp32, zero outside the image), then writes its output vectors from there; the offset of every k in the
// window is looked up in a table (up to 256 values of k) built once per block.  Same values, same rounding: identical bits.
constexpr int kPatchTileP = 8, kPatchTileQ = 32;
__host__ __device__ __forceinline__ int patch_tile_rows(int R, int sh) { return (kPatchTileP - 1) * sh + R; }
__host__ __device__ __forceinline__ int patch_tile_cols(int S, int sw) { return (kPatchTileQ - 1) * sw + S; }

template <typename T>
__global__ void __launch_bounds__(256) input_patch_tile_kernel(OpArgs a, uint32_t job_id, FinishedBlockNotifier* nf) {
    PB_NOTIFY_START();
    extern __shared__ __align__(16) unsigned char s_patch[];
    const float* __restrict__ x = (!a.x && slot_) ? slot_->io_in[blockIdx.y]      // the request's input buffer, known only at dispatch
                                                  : static_cast<const float*>(a.x) + (size_t)blockIdx.y * a.C * a.H * a.W;
    constexpr int N = Vec<T>::N;
    const int rows = patch_tile_rows(a.R, a.stride_h), cols = patch_tile_cols(a.S, a.stride_w);
    int* s_off = reinterpret_cast<int*>(s_patch);                 // [Ks] offset of k in the window, -1 = zero
    float* s_win = reinterpret_cast<float*>(s_patch + 1024);      // [C][rows][cols]
    const int tiles_q = (a.Q + kPatchTileQ - 1) / kPatchTileQ;
    const int p0 = (blockIdx.x / tiles_q) * kPatchTileP, q0 = (blockIdx.x % tiles_q) * kPatchTileQ;
    const int ih0 = p0 * a.stride_h - a.pad_h, iw0 = q0 * a.stride_w - a.pad_w;
    if (threadIdx.x < a.Ks) {
        const int k = threadIdx.x, taps_c = a.R * a.S * a.C;
        int off = -1;
        if (k < taps_c) {
            const int tap = k / a.C, c = k - tap * a.C;
            const int r = tap / a.S, s2 = tap - r * a.S;
            off = (c * rows + r) * cols + s2;
        }
        s_off[k] = off;
    }
    const int n_win = a.C * rows * cols;
    for (int i = threadIdx.x; i < n_win; i += 256) {
        const int col = i % cols, rest = i / cols;
        const int r = rest % rows, c = rest / rows;
        const int ih = ih0 + r, iw = iw0 + col;
        s_win[i] = (ih >= 0 && ih < a.H && iw >= 0 && iw < a.W) ? __ldg(x + ((size_t)c * a.H + ih) * a.W + iw) : 0.f;
    }
    __syncthreads();
    const int kv = a.Ks / N;
    T* __restrict__ y = y_img<T>(a);
    for (int v = threadIdx.x; v < kPatchTileP * kPatchTileQ * kv; v += 256) {
        const int k0 = (v % kv) * N, pl = v / kv;
        const int pr = pl / kPatchTileQ, pc = pl - pr * kPatchTileQ;
        const int p = p0 + pr, q = q0 + pc;
        if (p >= a.P || q >= a.Q) continue;
        const int base = pr * a.stride_h * cols + pc * a.stride_w;
        Vec<T> o;
#pragma unroll
        for (int j = 0; j < N; ++j) {
            const int off = s_off[k0 + j];
            o.v[j] = off >= 0 ? s_win[base + off] : 0.f;
        }
        o.store(y + ((size_t)p * a.Q + q) * a.Ks + k0);
    }
    PB_NOTIFY_END();
}
// Dynamic shared memory of the tiled patch kernel, or 0 when the layer keeps input_patch_kernel (a window that does
// not fit, more than 256 values of k).
static size_t patch_tile_smem(const pb_op_params* p) {
    if (p->Ks > 256 || p->R * p->S <= 1) return 0;
    const size_t n = 1024 + (size_t)p->C * patch_tile_rows(p->R, p->stride_h) * patch_tile_cols(p->S, p->stride_w) * 4;
    return n <= 40 * 1024 ? n : 0;
}
static uint32_t patch_tile_blocks(const pb_op_params* p) {
    return (uint32_t)(((p->P + kPatchTileP - 1) / kPatchTileP) * ((p->Q + kPatchTileQ - 1) / kPatchTileQ));
}

// ---- direct convolution ------------------------------------------------------
// One thread per (output pixel, output channel).  Weights [R][S][C/groups][K]: a warp
// reads consecutive k (coalesced) and shares the input value (broadcast).
template <typename T>
__global__ void __launch_bounds__(256) conv_simt_kernel(OpArgs a, uint32_t job_id, FinishedBlockNotifier* nf) {
    PB_NOTIFY_START();
    const T* __restrict__ x = x_img<T>(a);
    const T* __restrict__ w = static_cast<const T*>(a.w);
    const int total = a.P * a.Q * a.K;
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx < total) {
        const int k = idx % a.K;
        const int pix = idx / a.K;
        const int q = pix % a.Q, p = pix / a.Q;
        const int cg = a.C / a.groups;
        const int g = k / (a.K / a.groups);
        float acc = 0.f;
        for (int r = 0; r < a.R; ++r) {
            const int ih = p * a.stride_h + r * a.dil_h - a.pad_h;
            if (ih < 0 || ih >= a.H) continue;
            for (int s = 0; s < a.S; ++s) {
                const int iw = q * a.stride_w + s * a.dil_w - a.pad_w;
                if (iw < 0 || iw >= a.W) continue;
                const T* xp = x + ((size_t)ih * a.W + iw) * a.Cs + g * cg;
                const T* wp = w + ((size_t)(r * a.S + s) * cg) * a.K + k;
                for (int c = 0; c < cg; ++c) acc = fmaf(to_f<T>(xp[c]), to_f<T>(wp[(size_t)c * a.K]), acc);
            }
        }
        if (a.bias) acc += a.bias[k];
        if (a.residual) acc += to_f<T>(static_cast<const T*>(a.residual)[((size_t)blockIdx.y * a.P * a.Q + pix) * a.res_Cs + k]);
        if (a.act == 3) acc = acc > 0.f ? acc : acc * a.bias[a.K + k];      // PReLU: slopes follow the biases
        else acc = act_fn(acc, a.act);
        y_img<T>(a)[(size_t)pix * a.Ks + a.out_c_off + k] = from_f<T>(acc);
    }
    PB_NOTIFY_END();
}

// ---- depthwise convolution -----------------------------------------------------
// One thread per (output pixel, channel vector); weights [R][S][Cs].
template <typename T>
__global__ void __launch_bounds__(256, 6) dwconv_kernel(OpArgs a, uint32_t job_id, FinishedBlockNotifier* nf) {
    PB_NOTIFY_START();
    constexpr int N = Vec<T>::N;
    const int cv = a.Cs / N;
    const int total = a.P * a.Q * cv;
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx < total) {
        const int c0 = (idx % cv) * N;
        const int pix = idx / cv;
        const int q = pix % a.Q, p = pix / a.Q;
        const T* __restrict__ x = x_img<T>(a);
        const T* __restrict__ w = static_cast<const T*>(a.w);
        float acc[N];
#pragma unroll
        for (int j = 0; j < N; ++j) acc[j] = 0.f;
        for (int r = 0; r < a.R; ++r) {
            const int ih = p * a.stride_h + r - a.pad_h;
            if (ih < 0 || ih >= a.H) continue;
            for (int s = 0; s < a.S; ++s) {
                const int iw = q * a.stride_w + s - a.pad_w;
                if (iw < 0 || iw >= a.W) continue;
                const Vec<T> xv = Vec<T>::load(x + ((size_t)ih * a.W + iw) * a.Cs + c0);
                const Vec<T> wv = Vec<T>::load(w + (size_t)(r * a.S + s) * a.Cs + c0);
#pragma unroll
                for (int j = 0; j < N; ++j) acc[j] = fmaf(xv.v[j], wv.v[j], acc[j]);
            }
        }
        Vec<T> o;
#pragma unroll
        for (int j = 0; j < N; ++j) {
            float v = acc[j] + ((a.bias && c0 + j < a.K) ? a.bias[c0 + j] : 0.f);
            o.v[j] = (c0 + j < a.K) ? act_fn(v, a.act) : 0.f;
        }
        o.store(y_img<T>(a) + (size_t)pix * a.Ks + a.out_c_off + c0);
    }
    PB_NOTIFY_END();
}

// ---- pooling -------------------------------------------------------------------
template <typename T, bool kMax>
__global__ void __launch_bounds__(256, 6) pool_kernel(OpArgs a, uint32_t job_id, FinishedBlockNotifier* nf) {
    PB_NOTIFY_START();
    constexpr int N = Vec<T>::N;
    const int cv = a.Cs / N;
    const int total = a.P * a.Q * cv;
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx < total) {
        const int c0 = (idx % cv) * N;
        const int pix = idx / cv;
        const int q = pix % a.Q, p = pix / a.Q;
        const T* __restrict__ x = x_img<T>(a);
        float acc[N];
#pragma unroll
        for (int j = 0; j < N; ++j) acc[j] = kMax ? -INFINITY : 0.f;
        int cnt = 0;
        for (int r = 0; r < a.R; ++r) {
            const int ih = p * a.stride_h + r - a.pad_h;
            if (ih < 0 || ih >= a.H) continue;
            for (int s = 0; s < a.S; ++s) {
                const int iw = q * a.stride_w + s - a.pad_w;
                if (iw < 0 || iw >= a.W) continue;
                const Vec<T> xv = Vec<T>::load(x + ((size_t)ih * a.W + iw) * a.Cs + c0);
#pragma unroll
                for (int j = 0; j < N; ++j) acc[j] = kMax ? fmaxf(acc[j], xv.v[j]) : acc[j] + xv.v[j];
                ++cnt;
            }
        }
        Vec<T> o;
        const float div = (a.flags & 1) ? (float)(a.R * a.S) : (float)(cnt > 0 ? cnt : 1);
#pragma unroll
        for (int j = 0; j < N; ++j) {
            float v = kMax ? acc[j] : acc[j] / div;
            if (a.bias && c0 + j < a.C) v += a.bias[c0 + j];      // the tail of a convolution that ran before the pooling
            o.v[j] = (c0 + j < a.C) ? act_fn(v, a.act) : 0.f;
        }
        o.store(y_img<T>(a) + (size_t)pix * a.Ks + a.out_c_off + c0);
    }
    PB_NOTIFY_END();
}

// ---- 3x3 windows over large tensors: a strip of output pixels per thread ------------------
// dwconv_kernel and pool_kernel issue one guarded 128-bit load per filter tap and output vector: on a
// tensor that fills the GPU each thread has about one load in flight at a time and every input vector is
// fetched up to nine times through L1, so they run at the latency of the load path, not at HBM speed
// (depthwise 3x3 stride 1 at 128 x 1024 x 1024 bf16: 19 % of the measured copy bandwidth).  Here a thread
// owns one channel vector of kStrip consecutive output pixels of one output row.  Per input row it issues
// ALL loads of the strip's window back to back, unconditionally (addresses clamped into the tensor, the
// taps that fall outside are dropped afterwards), so 6-9 loads per thread are in flight; each loaded
// vector feeds every output it belongs to, and a row of weights is loaded once per thread.
// The order of the additions per output is the one of dwconv_kernel / pool_kernel (rows, then columns),
// so results are bit-identical to theirs.  Used when the strips alone fill the GPU (strip_threads()).
// With kStrip = 1 (every other 3x3 layer of stride 1 or 2, i.e. the batch-1 layers of the served models)
// the thread owns one output vector as in dwconv_kernel / pool_kernel, but its nine loads are
// unconditional and in flight together instead of one guarded load after the other.
constexpr int kStripWide1 = 4, kStripWide2 = 2;   // stride 1: 18 loads per thread; stride 2: 15
enum { kWinDw = 0, kWinMax = 1, kWinAvg = 2 };

template <typename T> struct RawVec;
template <> struct RawVec<float> { typedef float4 type; };
template <> struct RawVec<__nv_bfloat16> { typedef uint4 type; };
__device__ __forceinline__ Vec<float> vec_of(const float4& t) {
    Vec<float> r; r.v[0] = t.x; r.v[1] = t.y; r.v[2] = t.z; r.v[3] = t.w; return r;
}
__device__ __forceinline__ Vec<__nv_bfloat16> vec_of(const uint4& t) {
    Vec<__nv_bfloat16> r;
    const uint32_t u[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        r.v[2 * i] = __uint_as_float(u[i] << 16);
        r.v[2 * i + 1] = __uint_as_float(u[i] & 0xffff0000u);
    }
    return r;
}

// Pairs of fp32 values.  PB_F32X2=1 keeps a pair in one 64-bit register and uses the packed fp32
// instructions of sm_100 (fma.rn.f32x2 / add.rn.f32x2: each half is the IEEE operation of the scalar
// instruction); otherwise the pair is two scalars and the compiler schedules scalar instructions.
#ifndef PB_F32X2
#define PB_F32X2 0
#endif
#if PB_F32X2
typedef uint64_t f2_t;
__device__ __forceinline__ f2_t f2_pack(float lo, float hi) {
    f2_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void f2_unpack(f2_t v, float& lo, float& hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
__device__ __forceinline__ f2_t f2_fma(f2_t a, f2_t b, f2_t c) {
    f2_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ f2_t f2_add(f2_t a, f2_t b) {
    f2_t d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ f2_t f2_max(f2_t a, f2_t b) {
    float a0, a1, b0, b1;
    f2_unpack(a, a0, a1);
    f2_unpack(b, b0, b1);
    return f2_pack(fmaxf(a0, b0), fmaxf(a1, b1));
}
#else
struct f2_t { float lo, hi; };
__device__ __forceinline__ f2_t f2_pack(float lo, float hi) { f2_t r; r.lo = lo; r.hi = hi; return r; }
__device__ __forceinline__ void f2_unpack(f2_t v, float& lo, float& hi) { lo = v.lo; hi = v.hi; }
__device__ __forceinline__ f2_t f2_fma(f2_t a, f2_t b, f2_t c) { return f2_pack(fmaf(a.lo, b.lo, c.lo), fmaf(a.hi, b.hi, c.hi)); }
__device__ __forceinline__ f2_t f2_add(f2_t a, f2_t b) { return f2_pack(a.lo + b.lo, a.hi + b.hi); }
__device__ __forceinline__ f2_t f2_max(f2_t a, f2_t b) { return f2_pack(fmaxf(a.lo, b.lo), fmaxf(a.hi, b.hi)); }
#endif
// A 128-bit vector of activations as fp32 pairs: 2 pairs from float4, 4 pairs from 8 bf16.
__device__ __forceinline__ void unpack_pairs(const float4& t, f2_t (&r)[2]) {
    r[0] = f2_pack(t.x, t.y);
    r[1] = f2_pack(t.z, t.w);
}
__device__ __forceinline__ void unpack_pairs(const uint4& t, f2_t (&r)[4]) {
    const uint32_t u[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) r[i] = f2_pack(__uint_as_float(u[i] << 16), __uint_as_float(u[i] & 0xffff0000u));
}

// Dynamic shared memory of a depthwise launch: filter [3][3][Cs] + fp32 biases [Cs], or 0 when that
// exceeds what a kernel gets without opting in (the kernel then reads the filter from global memory).
__host__ __device__ __forceinline__ int window3_smem_bytes(int Cs, int elem_bytes) {
    const int n = 9 * Cs * elem_bytes + 4 * Cs;
    return n <= 40 * 1024 ? n : 0;
}

template <typename T, int kMode, int kStride, int kStrip>
__global__ void __launch_bounds__(256, 2) window3_strip_kernel(OpArgs a, uint32_t job_id, FinishedBlockNotifier* nf) {
    PB_NOTIFY_START();
    constexpr int N = Vec<T>::N;
    constexpr int NP = N / 2;
    constexpr int kCols = (kStrip - 1) * kStride + 3;
    typedef typename RawVec<T>::type Raw;
    const int cv = a.Cs / N;
    const int strips = (a.Q + kStrip - 1) / kStrip;
    const int total = a.P * strips * cv;
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    // Depthwise: the block's copy of the filter ([3][3][Cs]) and of the biases, in shared memory.  Read
    // through L1 they compete with the streamed activations for cache lines, and a miss sits on every
    // thread's critical path three times; the host passes window3_smem_bytes() of dynamic shared memory
    // (0 = the filter does not fit: read it from global memory).  Wide strips only: on a batch-1 layer the
    // staging round trip would come before the first activation load of a block that lives a few microseconds.
    extern __shared__ __align__(16) unsigned char s_w3[];
    const bool staged = kMode == kWinDw && kStrip > 1 && window3_smem_bytes(a.Cs, (int)sizeof(T)) > 0;
    if (staged) {
        Raw* sw = reinterpret_cast<Raw*>(s_w3);
        const Raw* gw = static_cast<const Raw*>(a.w);
        for (int i = threadIdx.x; i < 9 * cv; i += blockDim.x) sw[i] = __ldg(gw + i);
        float* sb = reinterpret_cast<float*>(s_w3 + (size_t)9 * a.Cs * sizeof(T));
        for (int i = threadIdx.x; i < a.Cs; i += blockDim.x) sb[i] = (a.bias && i < a.K) ? a.bias[i] : 0.f;
        __syncthreads();
    }
    if (idx < total) {
        const int c0 = (idx % cv) * N;
        const int rest = idx / cv;
        const int q0 = (rest % strips) * kStrip, p = rest / strips;
        const T* __restrict__ x = x_img<T>(a) + c0;
        const T* __restrict__ w = (staged ? reinterpret_cast<const T*>(s_w3) : static_cast<const T*>(a.w)) + c0;
        f2_t acc[kStrip][NP];
        const f2_t init = (kMode == kWinMax) ? f2_pack(-INFINITY, -INFINITY) : f2_pack(0.f, 0.f);
#pragma unroll
        for (int t = 0; t < kStrip; ++t)
#pragma unroll
            for (int j = 0; j < NP; ++j) acc[t][j] = init;
        const int iw0 = q0 * kStride - a.pad_w;
        uint32_t col_ok = 0;                    // bit col: input column iw0 + col lies inside the tensor
        int off[kCols];                         // element offset of that column within a row (clamped)
#pragma unroll
        for (int col = 0; col < kCols; ++col) {
            const int iw = iw0 + col;
            if (iw >= 0 && iw < a.W) col_ok |= 1u << col;
            off[col] = min(max(iw, 0), a.W - 1) * a.Cs;
        }
        // every load of the 3 x kCols window first, so that all of them are in flight together
        Raw raw[3][kCols];
        uint32_t ok[3];
        int rows = 0;
#pragma unroll
        for (int r = 0; r < 3; ++r) {
            const int ih = p * kStride + r - a.pad_h;
            const bool row_ok = ih >= 0 && ih < a.H;
            rows += row_ok ? 1 : 0;
            ok[r] = row_ok ? col_ok : 0u;
            const T* xrow = x + (size_t)min(max(ih, 0), a.H - 1) * a.W * a.Cs;
#pragma unroll
            for (int col = 0; col < kCols; ++col) raw[r][col] = *reinterpret_cast<const Raw*>(xrow + off[col]);
        }
#pragma unroll
        for (int r = 0; r < 3; ++r) {
            f2_t wv[3][NP];
            if (kMode == kWinDw) {
#pragma unroll
                for (int s = 0; s < 3; ++s) unpack_pairs(*reinterpret_cast<const Raw*>(w + (r * 3 + s) * a.Cs), wv[s]);
            }
#pragma unroll
            for (int col = 0; col < kCols; ++col) {
                if (!((ok[r] >> col) & 1u)) continue;
                f2_t xv[NP];
                unpack_pairs(raw[r][col], xv);
#pragma unroll
                for (int s = 0; s < 3; ++s) {
                    // input column col is tap s of output t when col == t * kStride + s
                    if (col - s < 0 || (col - s) % kStride != 0 || (col - s) / kStride >= kStrip) continue;
                    const int t = (col - s) / kStride;
#pragma unroll
                    for (int j = 0; j < NP; ++j) {
                        if (kMode == kWinDw) acc[t][j] = f2_fma(xv[j], wv[s][j], acc[t][j]);
                        else if (kMode == kWinMax) acc[t][j] = f2_max(acc[t][j], xv[j]);
                        else acc[t][j] = f2_add(acc[t][j], xv[j]);
                    }
                }
            }
        }
        T* yrow = y_img<T>(a) + ((size_t)p * a.Q + q0) * a.Ks + a.out_c_off + c0;
        float bias[N];
        if (kMode == kWinDw) {
#pragma unroll
            for (int j = 0; j < N; ++j)
                bias[j] = staged ? reinterpret_cast<const float*>(s_w3 + (size_t)9 * a.Cs * sizeof(T))[c0 + j]
                                 : ((a.bias && c0 + j < a.K) ? a.bias[c0 + j] : 0.f);
        }
#pragma unroll
        for (int t = 0; t < kStrip; ++t) {
            const int q = q0 + t;
            if (q >= a.Q) break;
            float v[N];
#pragma unroll
            for (int j = 0; j < NP; ++j) f2_unpack(acc[t][j], v[2 * j], v[2 * j + 1]);
            Vec<T> o;
            if (kMode == kWinDw) {
                // the activation is the same for every element: branch once, not per element
                if (a.act == 2) {
#pragma unroll
                    for (int j = 0; j < N; ++j) o.v[j] = (c0 + j < a.K) ? fminf(fmaxf(v[j] + bias[j], 0.f), 6.f) : 0.f;
                } else if (a.act == 1) {
#pragma unroll
                    for (int j = 0; j < N; ++j) o.v[j] = (c0 + j < a.K) ? fmaxf(v[j] + bias[j], 0.f) : 0.f;
                } else {
#pragma unroll
                    for (int j = 0; j < N; ++j) o.v[j] = (c0 + j < a.K) ? v[j] + bias[j] : 0.f;
                }
            } else if (kMode == kWinMax) {
#pragma unroll
                for (int j = 0; j < N; ++j) {
                    const float pv = (a.bias && c0 + j < a.C) ? v[j] + a.bias[c0 + j] : v[j];
                    o.v[j] = (c0 + j < a.C) ? act_fn(pv, a.act) : 0.f;
                }
            } else {
                float div = 9.f;
                if (!(a.flags & 1)) {
                    const int lo = max(q * kStride - a.pad_w, 0), hi = min(q * kStride - a.pad_w + 3, a.W);
                    const int cnt = rows * max(hi - lo, 0);
                    div = (float)(cnt > 0 ? cnt : 1);
                }
                // v / div, correctly rounded, in three instructions per element instead of the division
                // sequence (which was more than half of this kernel's instructions): with inv the correctly
                // rounded reciprocal, q = v * inv is within an ulp, the fused residual v - div * q is exact
                // and q + r * inv rounds to the quotient (Markstein); non-finite q passes through.  (-0.0
                // would come out as +0.0, but a sum that starts from +0.0 is never -0.0.)
                const float inv = 1.f / div;
#pragma unroll
                for (int j = 0; j < N; ++j) {
                    const float qv = v[j] * inv;
                    const float rv = fmaf(-div, qv, v[j]);
                    float out = fabsf(qv) <= 3.0e38f ? fmaf(rv, inv, qv) : qv;
                    if (a.bias && c0 + j < a.C) out += a.bias[c0 + j];
                    o.v[j] = (c0 + j < a.C) ? act_fn(out, a.act) : 0.f;
                }
            }
            o.store(yrow + (size_t)t * a.Ks);
        }
    }
    PB_NOTIFY_END();
}

// ---- 3x3 windows over tensors that fill the GPU many times over -------------------------------------------
// window3_strip_kernel loads every input row three times (once per output row it belongs to) and converts
// it to fp32 each time: about 300 instructions per output vector of 8 bf16 channels, which is what bounds
// it (28 % of the copy bandwidth for the depthwise case; 70 % of the issue slots busy).  window3_tile_kernel
// below lets a thread own TWO channels (one 32-bit word of bf16) of a strip of output columns and walk down
// the output rows: each input row is read and converted ONCE and feeds the (up to) three output rows it
// belongs to, whose accumulators stay in registers, as do the 18 filter values and the 2 biases of the
// thread's channels.  Max pooling compares the bf16 pairs themselves (a maximum needs no wider type);
// ReLU / ReLU6 clamp the rounded bf16 pair (rounding is monotonic and 0 and 6 are bf16 values, so clamping
// after rounding equals rounding after clamping).  Taps outside the tensor contribute the neutral element
// (0 for sums and products, -inf for max), which leaves every partial result as it is: the additions per
// output happen in the order of dwconv_kernel / pool_kernel (filter rows, then columns), so the results
// are theirs bit for bit (finite filter values assumed).  bf16 only.
constexpr int kTileStrip1 = 4, kTileStrip2 = 2;
__device__ __forceinline__ f2_t pair_of(uint32_t u) { return f2_pack(__uint_as_float(u << 16), __uint_as_float(u & 0xffff0000u)); }
__device__ __forceinline__ uint32_t bits_of(__nv_bfloat162 h) { return *reinterpret_cast<const uint32_t*>(&h); }
__device__ __forceinline__ __nv_bfloat162 bf2_of(uint32_t u) { return *reinterpret_cast<const __nv_bfloat162*>(&u); }

// What a thread keeps per (output, channel pair): fp32 pairs for sums, the bf16 pair itself for a maximum.
template <int kMode> struct WinAcc { typedef f2_t type; };
template <> struct WinAcc<kWinMax> { typedef uint32_t type; };
template <int kMode> __device__ __forceinline__ typename WinAcc<kMode>::type win_neutral() { return f2_pack(0.f, 0.f); }
template <> __device__ __forceinline__ uint32_t win_neutral<kWinMax>() { return 0xff80ff80u; }       // (-inf, -inf)
template <int kMode> __device__ __forceinline__ typename WinAcc<kMode>::type win_value(uint32_t raw) { return pair_of(raw); }
template <> __device__ __forceinline__ uint32_t win_value<kWinMax>(uint32_t raw) { return raw; }
__device__ __forceinline__ f2_t win_step(f2_t acc, f2_t x, f2_t w, bool dw) { return dw ? f2_fma(x, w, acc) : f2_add(acc, x); }
__device__ __forceinline__ uint32_t win_step(uint32_t acc, uint32_t x, f2_t, bool) { return bits_of(__hmax2(bf2_of(acc), bf2_of(x))); }

// One finished output (two channels) -> bf16 pair.  kAct: 0 none, 1 ReLU, 2 ReLU6 (depthwise only).  div / inv: the
// average pool's divisor and its reciprocal.
template <int kMode, int kAct>
__device__ __forceinline__ uint32_t win_finish(f2_t acc, float b0, float b1, float div, float inv) {
    float v0, v1;
    f2_unpack(acc, v0, v1);
    if (kMode == kWinDw) {
        __nv_bfloat162 h = __floats2bfloat162_rn(v0 + b0, v1 + b1);
        if (kAct >= 1) h = __hmax2(h, bf2_of(0u));
        if (kAct == 2) h = __hmin2(h, bf2_of(0x40c040c0u));          // (6, 6)
        return bits_of(h);
    }
    // correctly rounded v / div without the division sequence (see window3_strip_kernel)
    const float q0 = v0 * inv, q1 = v1 * inv;
    const float r0 = fmaf(-div, q0, v0), r1 = fmaf(-div, q1, v1);
    v0 = fabsf(q0) <= 3.0e38f ? fmaf(r0, inv, q0) : q0;
    v1 = fabsf(q1) <= 3.0e38f ? fmaf(r1, inv, q1) : q1;
    return bits_of(__floats2bfloat162_rn(v0, v1));
}
template <int kMode, int kAct>
__device__ __forceinline__ uint32_t win_finish(uint32_t acc, float, float, float, float) { return acc; }

// ---- 3x3 windows over large tensors, staged through shared memory ---------------------------------------
// Reading the rows with 4-byte global loads spends a third of the instructions on addresses (every load needs
// its own 64-bit address; measured on a first version that did so).  Here a block of 8 warps owns a tile of kTileRows x (8 * strip) outputs of ONE slab of
// 64 channels.  It first copies the tile's input window into shared memory with 16-byte cp.async (zero-filled
// outside the tensor; 65 KB in flight per block, three blocks per SM), then every warp walks down its strip of output columns with
// lane l holding channels 2l, 2l+1 of the slab: all its shared-memory loads are at compile-time offsets from
// one pointer that advances once per three rows, and consecutive lanes read consecutive words (no bank
// conflict).  The results are the bits of every other 3x3 kernel here.
constexpr int kTileSlab = 64;                       // channels per block
#ifndef PB_TILE_ROWS1
#define PB_TILE_ROWS1 13
#endif
#ifndef PB_TILE_ROWS2
#define PB_TILE_ROWS2 6
#endif
#ifndef PB_TILE_BLOCKS
#define PB_TILE_BLOCKS 3
#endif
constexpr int kTileRows1 = PB_TILE_ROWS1, kTileRows2 = PB_TILE_ROWS2;      // output rows per block at stride 1 / 2

template <int kStride> struct TileGeom {
    static constexpr int kStrip = kStride == 1 ? kTileStrip1 : kTileStrip2;
    static constexpr int kRows = kStride == 1 ? kTileRows1 : kTileRows2;
    static constexpr int kOutCols = 8 * kStrip;
    static constexpr int kInCols = (kOutCols - 1) * kStride + 3;
    static constexpr int kInRows = (kRows - 1) * kStride + 3;
    static constexpr int kSmemBytes = kInRows * kInCols * kTileSlab * 2;
};

template <int kMode, int kStride>
__global__ void __launch_bounds__(256, PB_TILE_BLOCKS) window3_tile_kernel(OpArgs a, uint32_t job_id, FinishedBlockNotifier* nf) {
    PB_NOTIFY_START();
    typedef __nv_bfloat16 T;
    typedef TileGeom<kStride> G;
    typedef typename WinAcc<kMode>::type Acc;
    constexpr int kStrip = G::kStrip, kCols = (kStrip - 1) * kStride + 3;
    constexpr bool kDw = kMode == kWinDw;
    extern __shared__ __align__(16) unsigned char s_tile[];

    const int slabs = (a.Cs + kTileSlab - 1) / kTileSlab;
    const int col_tiles = (a.Q + G::kOutCols - 1) / G::kOutCols;
    int b = blockIdx.x;
    const int slab = b % slabs; b /= slabs;
    const int q_tile = (b % col_tiles) * G::kOutCols;
    const int p_tile = (b / col_tiles) * G::kRows;
    const int ih0 = p_tile * kStride - a.pad_h, iw0 = q_tile * kStride - a.pad_w;
    const int ch0 = slab * kTileSlab;

    // ---- fill: pixel (r, c) of the window is 8 vectors of 8 channels.  A thread keeps its eighth of the pixel and
    // moves 32 pixels on per turn (the window is at least 32 pixels wide: at most one row wrap per turn). ----
    {
        static_assert(G::kInCols >= 32, "one row wrap per turn of the fill");
        const T* __restrict__ x = x_img<T>(a);
        const int ch = ch0 + (threadIdx.x & 7) * 8;
        const bool ch_ok = ch < a.Cs;
        int pix = threadIdx.x >> 3;
        int r = pix / G::kInCols, c = pix - r * G::kInCols;
        uint32_t dst = (uint32_t)__cvta_generic_to_shared(s_tile) + threadIdx.x * 16u;
        for (; pix < G::kInRows * G::kInCols; pix += 32, dst += 32u * 128u) {
            const int ih = ih0 + r, iw = iw0 + c;
            const bool ok = ch_ok && (unsigned)ih < (unsigned)a.H && (unsigned)iw < (unsigned)a.W;
            if (kMode == kWinMax && !ok) {
                asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(dst), "r"(0xff80ff80u) : "memory");
            } else {
                const T* src = ok ? x + (size_t)(ih * a.W + iw) * a.Cs + ch : x;
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(ok ? 16u : 0u) : "memory");
            }
            c += 32;
            if (c >= G::kInCols) { c -= G::kInCols; ++r; }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();
    }

    // ---- walk: warp = strip of output columns, lane = channel pair ----
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int c0 = ch0 + lane * 2;
    const int q0 = q_tile + warp * kStrip;
    if (c0 < a.Cs && q0 < a.Q) {
        const Acc neutral = win_neutral<kMode>();
        f2_t w[3][3];
        float b0 = 0.f, b1 = 0.f;
#pragma unroll
        for (int r = 0; r < 3; ++r)
#pragma unroll
            for (int s2 = 0; s2 < 3; ++s2) w[r][s2] = f2_pack(0.f, 0.f);
        if (kDw) {
            const T* wp = static_cast<const T*>(a.w) + c0;
#pragma unroll
            for (int r = 0; r < 3; ++r)
#pragma unroll
                for (int s2 = 0; s2 < 3; ++s2) w[r][s2] = pair_of(__ldg(reinterpret_cast<const uint32_t*>(wp + (r * 3 + s2) * a.Cs)));
            if (a.bias) { b0 = c0 < a.K ? a.bias[c0] : 0.f; b1 = c0 + 1 < a.K ? a.bias[c0 + 1] : 0.f; }
        }
        const int nt = min(kStrip, a.Q - q0);
        const int c_lim = kDw ? a.K : a.C;
        const uint32_t keep = c0 + 1 < c_lim ? 0xffffffffu : (c0 < c_lim ? 0x0000ffffu : 0u);
        const int p_end = min(p_tile + G::kRows, a.P);
        const bool count_pad = (a.flags & 1) != 0;
        const float inv9 = 1.f / 9.f;
        T* __restrict__ y = y_img<T>(a) + a.out_c_off + c0;
        // word (r, col) of this thread: s_row[r * kRowWords + col * 32]
        constexpr int kRowWords = G::kInCols * (kTileSlab / 2);
        const uint32_t* s_row = reinterpret_cast<const uint32_t*>(s_tile) + (warp * kStrip * kStride) * (kTileSlab / 2) + lane;

        auto load_row = [&](int r, Acc (&xv)[kCols]) {
#pragma unroll
            for (int col = 0; col < kCols; ++col) xv[col] = win_value<kMode>(s_row[r * kRowWords + col * (kTileSlab / 2)]);
        };
        auto row_into = [&](Acc (&acc)[kStrip], const Acc (&xv)[kCols], int r) {
#pragma unroll
            for (int t = 0; t < kStrip; ++t)
#pragma unroll
                for (int s2 = 0; s2 < 3; ++s2) acc[t] = win_step(acc[t], xv[t * kStride + s2], w[r][s2], kDw);
        };
        const bool full = nt == kStrip && keep == 0xffffffffu;      // every output of the strip and both channels exist
        // one output row of the strip; ACT and FULL are literals so that the loop body carries no test of them
#define PB_TILE_STORE_ROW(ACT, FULL)                                                                                             \
    do {                                                                                                                         \
        _Pragma("unroll") for (int t = 0; t < kStrip; ++t) {                                                                     \
            if (!(FULL) && t >= nt) break;                                                                                       \
            if (kMode == kWinAvg && !count_pad) {                                                                                \
                const int cols_in = max(min((q0 + t) * kStride - a.pad_w + 3, a.W) - max((q0 + t) * kStride - a.pad_w, 0), 0);   \
                const int cnt = rows_in * cols_in;                                                                               \
                if (cnt != 9) { div = (float)(cnt > 0 ? cnt : 1); inv = 1.f / div; }                                             \
                else { div = 9.f; inv = inv9; }                                                                                  \
            }                                                                                                                    \
            const uint32_t o = win_finish<kMode, ACT>(acc[t], b0, b1, div, inv);                                                \
            *reinterpret_cast<uint32_t*>(yrow + (size_t)t * a.Ks) = (FULL) ? o : (o & keep);                                     \
        }                                                                                                                        \
    } while (0)
        auto close_row = [&](Acc (&acc)[kStrip], int p) {
            if (p >= p_tile && p < p_end) {
                int rows_in = 3;
                float div = 9.f, inv = inv9;
                if (kMode == kWinAvg && !count_pad) rows_in = min(p * kStride - a.pad_h + 3, a.H) - max(p * kStride - a.pad_h, 0);
                T* yrow = y + ((size_t)p * a.Q + q0) * a.Ks;
                const int act = kDw ? a.act : 0;
                if (full) {
                    if (act == 2) PB_TILE_STORE_ROW(2, true);
                    else if (act == 1) PB_TILE_STORE_ROW(1, true);
                    else PB_TILE_STORE_ROW(0, true);
                } else {
                    if (act == 2) PB_TILE_STORE_ROW(2, false);
                    else if (act == 1) PB_TILE_STORE_ROW(1, false);
                    else PB_TILE_STORE_ROW(0, false);
                }
            }
#pragma unroll
            for (int t = 0; t < kStrip; ++t) acc[t] = neutral;
        };
#undef PB_TILE_STORE_ROW

        if (kStride == 1) {
            // window row r opens output row p_tile + r (filter row 0), continues p_tile + r - 1, closes p_tile + r - 2
            Acc accA[kStrip], accB[kStrip], accC[kStrip];
#pragma unroll
            for (int t = 0; t < kStrip; ++t) accA[t] = accB[t] = accC[t] = neutral;
            static_assert(kStride != 1 || G::kInRows % 3 == 0, "the stride-1 walk takes three window rows per turn");
#pragma unroll 1
            for (int r = 0; r < G::kInRows; r += 3) {
                Acc xv[kCols];
                load_row(r, xv);     row_into(accB, xv, 2); row_into(accC, xv, 1); row_into(accA, xv, 0); close_row(accB, p_tile + r - 2);
                load_row(r + 1, xv); row_into(accC, xv, 2); row_into(accA, xv, 1); row_into(accB, xv, 0); close_row(accC, p_tile + r - 1);
                load_row(r + 2, xv); row_into(accA, xv, 2); row_into(accB, xv, 1); row_into(accC, xv, 0); close_row(accA, p_tile + r);
            }
        } else {
            // window row r: even r closes output row p_tile + r/2 - 1 (filter row 2) and opens p_tile + r/2 (row 0);
            // odd r is filter row 1 of p_tile + (r - 1)/2
            Acc acc[kStrip];
#pragma unroll
            for (int t = 0; t < kStrip; ++t) acc[t] = neutral;
#pragma unroll 1
            for (int r = 0; r + 1 < G::kInRows; r += 2) {
                Acc xv[kCols];
                load_row(r, xv);     row_into(acc, xv, 2); close_row(acc, p_tile + r / 2 - 1); row_into(acc, xv, 0);
                load_row(r + 1, xv); row_into(acc, xv, 1);
            }
            Acc xv[kCols];
            load_row(G::kInRows - 1, xv);
            row_into(acc, xv, 2);
            close_row(acc, p_tile + (G::kInRows - 1) / 2 - 1);
        }
    }
    PB_NOTIFY_END();
}

// ---- global average pool: [HW][Cs] -> [Cs] ---------------------------------------
// Block = 32 channel vectors x 8 pixel groups; shared-memory reduction over the groups.
template <typename T>
__global__ void __launch_bounds__(256) gap_kernel(OpArgs a, uint32_t job_id, FinishedBlockNotifier* nf) {
    PB_NOTIFY_START();
    constexpr int N = Vec<T>::N;
    __shared__ float red[8][32][N + 1];
    const int cv = a.Cs / N;
    const int lane = threadIdx.x & 31, grp = threadIdx.x >> 5;
    const int v = blockIdx.x * 32 + lane;
    const int HW = a.H * a.W;
    float acc[N];
#pragma unroll
    for (int j = 0; j < N; ++j) acc[j] = 0.f;
    if (v < cv) {
        const T* __restrict__ x = x_img<T>(a);
        for (int pix = grp; pix < HW; pix += 8) {
            const Vec<T> xv = Vec<T>::load(x + (size_t)pix * a.Cs + v * N);
#pragma unroll
            for (int j = 0; j < N; ++j) acc[j] += xv.v[j];
        }
    }
#pragma unroll
    for (int j = 0; j < N; ++j) red[grp][lane][j] = acc[j];
    __syncthreads();
    if (grp == 0 && v < cv) {
        const float inv = 1.f / (float)HW;
        float o[N];
#pragma unroll
        for (int j = 0; j < N; ++j) {
            float s = 0.f;
#pragma unroll
            for (int gI = 0; gI < 8; ++gI) s += red[gI][lane][j];
            o[j] = s * inv;
        }
        if (a.flags & 2) {
            float* y = out_f32_img(a, slot_, a.C);
#pragma unroll
            for (int j = 0; j < N; ++j) if (v * N + j < a.C) y[v * N + j] = o[j];
        } else {
            Vec<T> ov;
#pragma unroll
            for (int j = 0; j < N; ++j) ov.v[j] = (v * N + j < a.C) ? o[j] : 0.f;
            ov.store(y_img<T>(a) + v * N);
        }
    }
    PB_NOTIFY_END();
}

// ---- dense: y[k] = act(w[k,:] . x + b[k]); one warp per output row -----------------
// x has n_in = a.C elements (already in the device's flattened channels-last order, padded
// entries zero); w is [K][C] with C a multiple of the vector width.
template <typename T>
__global__ void __launch_bounds__(256) dense_kernel(OpArgs a, uint32_t job_id, FinishedBlockNotifier* nf) {
    PB_NOTIFY_START();
    constexpr int N = Vec<T>::N;
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (warp < a.K) {
        const T* __restrict__ x = x_img<T>(a);
        const T* __restrict__ w = static_cast<const T*>(a.w) + (size_t)warp * a.C;
        float acc = 0.f;
        // A row of weights is streamed once, from HBM: four raw 128-bit loads per lane are issued before
        // the first is used (cache-streaming, so they do not evict the input vector from L1); the sum keeps
        // the order of the plain loop.
        typedef typename RawVec<T>::type Raw;
        constexpr int kStep = 32 * N;
        int i = lane * N;
        for (; i + 3 * kStep < a.C; i += 4 * kStep) {
            Raw wr[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) wr[u] = __ldcs(reinterpret_cast<const Raw*>(w + i + u * kStep));
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const Vec<T> xv = Vec<T>::load(x + i + u * kStep);
                const Vec<T> wv = vec_of(wr[u]);
#pragma unroll
                for (int j = 0; j < N; ++j) acc = fmaf(xv.v[j], wv.v[j], acc);
            }
        }
        for (; i < a.C; i += kStep) {
            const Vec<T> xv = Vec<T>::load(x + i);
            const Vec<T> wv = vec_of(__ldcs(reinterpret_cast<const Raw*>(w + i)));
#pragma unroll
            for (int j = 0; j < N; ++j) acc = fmaf(xv.v[j], wv.v[j], acc);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
        if (lane == 0) {
            const float v = act_fn(acc + (a.bias ? a.bias[warp] : 0.f), a.act);
            if (a.flags & 2) out_f32_img(a, slot_, a.K)[warp] = v;
            else y_img<T>(a)[warp] = from_f<T>(v);
        }
    }
    PB_NOTIFY_END();
}

// ---- elementwise add (+activation) over [HW][Cs] ----------------------------------
template <typename T>
__global__ void __launch_bounds__(256) add_kernel(OpArgs a, uint32_t job_id, FinishedBlockNotifier* nf) {
    PB_NOTIFY_START();
    constexpr int N = Vec<T>::N;
    const size_t nv = (size_t)a.H * a.W * a.Cs / N;      // the host folds the images into H
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < nv) {
        const Vec<T> u = Vec<T>::load(static_cast<const T*>(a.x) + i * N);
        const Vec<T> v = Vec<T>::load(static_cast<const T*>(a.residual) + i * N);
        Vec<T> o;
#pragma unroll
        for (int j = 0; j < N; ++j) o.v[j] = act_fn(u.v[j] + v.v[j], a.act);
        o.store(static_cast<T*>(a.y) + i * N);
    }
    PB_NOTIFY_END();
}

// ---- per-channel affine (+activation) over [HW][C] of a tensor with channel stride Cs ----------
// y[pix][c] = act(x[pix][c] * scale[c] + bias[c]) for the first a.C channels: the folded batch-norm +
// ReLU that DenseNet applies to the concatenated features BEFORE each convolution.
constexpr int kAffinePer = 4;      // vectors per thread

template <typename T>
__global__ void __launch_bounds__(256) affine_kernel(OpArgs a, uint32_t job_id, FinishedBlockNotifier* nf) {
    PB_NOTIFY_START();
    constexpr int N = Vec<T>::N;
    typedef typename RawVec<T>::type Raw;
    const int cv = (a.C + N - 1) / N;
    const size_t total = (size_t)a.H * a.W * cv;
    // kAffinePer vectors per thread, a quarter of the tensor apart, all loads issued (as raw 128-bit words)
    // before any is used: with one load in flight per thread the kernel ran at 54 % of the copy bandwidth
    // on a tensor larger than L2, which needs about 50 KB in flight per SM.
    const size_t part = (total + kAffinePer - 1) / kAffinePer;
    const size_t i0 = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i0 < part) {
        size_t pix[kAffinePer];
        int c0[kAffinePer];
        Raw raw[kAffinePer];
#pragma unroll
        for (int h = 0; h < kAffinePer; ++h) {
            const size_t i = (i0 + h * part < total) ? i0 + h * part : i0;
            // 32-bit division whenever the index fits (always, short of a 64 GB tensor)
            pix[h] = total <= 0xffffffffull ? (size_t)((uint32_t)i / (uint32_t)cv) : i / cv;
            c0[h] = (int)(i - pix[h] * cv) * N;
            raw[h] = *reinterpret_cast<const Raw*>(static_cast<const T*>(a.x) + pix[h] * a.Cs + c0[h]);
        }
        const float* __restrict__ sc = static_cast<const float*>(a.w);
        const bool aligned = ((reinterpret_cast<uintptr_t>(sc) | reinterpret_cast<uintptr_t>(a.bias)) & 15) == 0;
#pragma unroll
        for (int h = 0; h < kAffinePer; ++h) {
            if (h > 0 && i0 + h * part >= total) break;
            const Vec<T> u = vec_of(raw[h]);
            Vec<T> o;
            if (c0[h] + N <= a.C && aligned) {
                // whole vector inside the tensor: scale and bias as 128-bit loads instead of 2 x N scalar ones
                float scv[N], biv[N];
#pragma unroll
                for (int j = 0; j < N; j += 4) {
                    *reinterpret_cast<float4*>(scv + j) = __ldg(reinterpret_cast<const float4*>(sc + c0[h] + j));
                    *reinterpret_cast<float4*>(biv + j) = __ldg(reinterpret_cast<const float4*>(a.bias + c0[h] + j));
                }
#pragma unroll
                for (int j = 0; j < N; ++j) o.v[j] = act_fn(u.v[j] * scv[j] + biv[j], a.act);
            } else {
#pragma unroll
                for (int j = 0; j < N; ++j)
                    o.v[j] = (c0[h] + j < a.C) ? act_fn(u.v[j] * __ldg(sc + c0[h] + j) + __ldg(a.bias + c0[h] + j), a.act) : 0.f;
            }
            o.store(static_cast<T*>(a.y) + pix[h] * a.Ks + a.out_c_off + c0[h]);
        }
    }
    PB_NOTIFY_END();
}

// ---- softmax over a.C values, one block --------------------------------------------
template <typename T, bool kInF32>
__global__ void __launch_bounds__(256) softmax_kernel(OpArgs a, uint32_t job_id, FinishedBlockNotifier* nf) {
    PB_NOTIFY_START();
    __shared__ float red[8];
    __shared__ float bc;
    const int n = a.C;
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    // flags bit2: a bare fp32 vector per image; otherwise image i is tensor i of [H][W][Cs]
    const float* xf = static_cast<const float*>(a.x) + (size_t)blockIdx.y * ((a.flags & 4) ? (size_t)n : (size_t)a.H * a.W * a.Cs);
    const T* xt = x_img<T>(a);
    auto ld = [&](int i) { return kInF32 ? xf[i] : to_f<T>(xt[i]); };
    float m = -INFINITY;
    for (int i = threadIdx.x; i < n; i += blockDim.x) m = fmaxf(m, ld(i));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if (lane == 0) red[wid] = m;
    __syncthreads();
    if (threadIdx.x == 0) { float t = red[0]; for (int i = 1; i < 8; ++i) t = fmaxf(t, red[i]); bc = t; }
    __syncthreads();
    m = bc;
    float s = 0.f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) s += __expf(ld(i) - m);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    __syncthreads();
    if (lane == 0) red[wid] = s;
    __syncthreads();
    if (threadIdx.x == 0) { float t = 0.f; for (int i = 0; i < 8; ++i) t += red[i]; bc = t; }
    __syncthreads();
    const float inv = 1.f / bc;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const float v = __expf(ld(i) - m) * inv;
        if (a.flags & 2) out_f32_img(a, slot_, n)[i] = v;
        else y_img<T>(a)[i] = from_f<T>(v);
    }
    PB_NOTIFY_END();
}

// ---- detection head over one feature map ----------------------------------------------
// One thread per prior (cell, anchor) of the map.  x is [H][W][Cs] with C = 6A channels: 2A class logits
// (anchor, class), then 4A box regressions (anchor, coordinate).  a.w = fp32 priors [H*W*A][4] = (cx, cy, w, h),
// a.bias = {centre variance, size variance}, a.K = priors of the whole model, a.out_c_off = this map's first
// prior.  The fp32 model output is [K*2 scores | K*4 corner-form boxes].
template <typename T>
__global__ void __launch_bounds__(256) detect_kernel(OpArgs a, uint32_t job_id, FinishedBlockNotifier* nf) {
    PB_NOTIFY_START();
    const int A = a.C / 6;
    const int n = a.H * a.W * A;
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) {
        const int cell = i / A, an = i - cell * A;
        const T* __restrict__ x = x_img<T>(a) + (size_t)cell * a.Cs;
        const float c0 = to_f<T>(x[an * 2]), c1 = to_f<T>(x[an * 2 + 1]);
        const float m = fmaxf(c0, c1);
        const float e0 = expf(c0 - m), e1 = expf(c1 - m);
        const float inv = 1.f / (e0 + e1);
        float* out = out_f32_img(a, slot_, a.K * 6);
        float* sc = out + (size_t)(a.out_c_off + i) * 2;       // scalar stores: a request's buffer need not be 16-byte aligned
        sc[0] = e0 * inv; sc[1] = e1 * inv;
        const float4 pr = __ldg(reinterpret_cast<const float4*>(a.w) + i);
        const float cv = __ldg(a.bias), sv = __ldg(a.bias + 1);
        const T* l = x + 2 * A + an * 4;
        const float cx = to_f<T>(l[0]) * cv * pr.z + pr.x, cy = to_f<T>(l[1]) * cv * pr.w + pr.y;
        const float bw = expf(to_f<T>(l[2]) * sv) * pr.z, bh = expf(to_f<T>(l[3]) * sv) * pr.w;
        float* bo = out + (size_t)a.K * 2 + (size_t)(a.out_c_off + i) * 4;
        bo[0] = cx - bw * 0.5f; bo[1] = cy - bh * 0.5f; bo[2] = cx + bw * 0.5f; bo[3] = cy + bh * 0.5f;
    }
    PB_NOTIFY_END();
}

// ---- whole MNIST-CNN in one launch ---------------------------------------------------
// conv5x5(1->8)+ReLU, maxpool2, conv5x5(8->16)+ReLU, maxpool3, dense 256->10 for one
// 28x28 image, fp32, activations in shared memory.  One block of 256 threads: the network
// is 1.57 MFLOP and 24 KB of weights, so the request is launch-latency bound and one
// kernel (one start and one end record) replaces six.
// Weights: w1 [5][5][1][8], w2 [5][5][8][16], wd [10][4*4*16] (h, w, c order), biases fp32.
struct MnistArgs {
    const float* x;     // [28][28]
    const float* w1; const float* b1;
    const float* w2; const float* b2;
    const float* wd; const float* bd;
    float* y;           // [10]
};

__global__ void __launch_bounds__(256) mnist_fused_kernel(MnistArgs a, uint32_t job_id, FinishedBlockNotifier* nf) {
    PB_NOTIFY_START();
    // one block per image of the gang
    a.x = (!a.x && slot_) ? slot_->io_in[blockIdx.x] : a.x + (size_t)blockIdx.x * 784;
    a.y = (!a.y && slot_) ? slot_->io_out[blockIdx.x] : a.y + (size_t)blockIdx.x * 10;
    __shared__ float s_in[32][33];          // 28x28 image with a 2-pixel zero border
    __shared__ float s_w1[25 * 8];
    __shared__ float s_p1[18][18][8];       // pool1 output 14x14x8 with a 2-pixel zero border
    __shared__ float s_w2[25 * 8 * 16];
    __shared__ float s_c2[14 * 14][17];     // conv2 output (padded row to dodge bank conflicts)
    __shared__ float s_p2[256];
    const int t = threadIdx.x;
    for (int i = t; i < 32 * 33; i += 256) (&s_in[0][0])[i] = 0.f;
    for (int i = t; i < 18 * 18 * 8; i += 256) (&s_p1[0][0][0])[i] = 0.f;
    for (int i = t; i < 200; i += 256) s_w1[i] = a.w1[i];
    for (int i = t; i < 3200; i += 256) s_w2[i] = a.w2[i];
    __syncthreads();
    for (int i = t; i < 784; i += 256) s_in[i / 28 + 2][i % 28 + 2] = a.x[i];
    __syncthreads();
    // conv1 + ReLU + 2x2 max pool: one thread per (pooled pixel, channel): 14*14*8 = 1568
    for (int i = t; i < 1568; i += 256) {
        const int k = i & 7, pp = i >> 3;
        const int py = pp / 14, px = pp % 14;
        float best = 0.f;  // ReLU output is >= 0
        const float b = a.b1[k];
        for (int dy = 0; dy < 2; ++dy)
            for (int dx = 0; dx < 2; ++dx) {
                float acc = b;
                const int oy = 2 * py + dy, ox = 2 * px + dx;
#pragma unroll
                for (int r = 0; r < 5; ++r)
#pragma unroll
                    for (int s = 0; s < 5; ++s) acc = fmaf(s_in[oy + r][ox + s], s_w1[(r * 5 + s) * 8 + k], acc);
                best = fmaxf(best, acc);
            }
        s_p1[py + 2][px + 2][k] = best;
    }
    __syncthreads();
    // conv2 + ReLU: one thread per (pixel, channel): 196*16 = 3136
    for (int i = t; i < 3136; i += 256) {
        const int k = i & 15, pp = i >> 4;
        const int oy = pp / 14, ox = pp % 14;
        float acc = a.b2[k];
        for (int r = 0; r < 5; ++r)
            for (int s = 0; s < 5; ++s) {
                const float* ip = &s_p1[oy + r][ox + s][0];
                const float* wp = &s_w2[((r * 5 + s) * 8) * 16 + k];
#pragma unroll
                for (int c = 0; c < 8; ++c) acc = fmaf(ip[c], wp[c * 16], acc);
            }
        s_c2[pp][k] = fmaxf(acc, 0.f);
    }
    __syncthreads();
    // 3x3/3 max pool (floor: 14 -> 4), output order (h, w, c)
    {
        const int k = t & 15, pp = t >> 4;
        const int py = pp >> 2, px = pp & 3;
        float best = -INFINITY;
        for (int dy = 0; dy < 3; ++dy)
            for (int dx = 0; dx < 3; ++dx) best = fmaxf(best, s_c2[(3 * py + dy) * 14 + 3 * px + dx][k]);
        s_p2[t] = best;
    }
    __syncthreads();
    // dense 256 -> 10: warps 0..7 take rows w, w+8
    {
        const int lane = t & 31, wid = t >> 5;
        for (int o = wid; o < 10; o += 8) {
            float acc = 0.f;
            for (int i = lane; i < 256; i += 32) acc = fmaf(s_p2[i], a.wd[o * 256 + i], acc);
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
            if (lane == 0) a.y[o] = acc + a.bd[o];
        }
    }
    PB_NOTIFY_END();
}

// ---------------------------------------------------------------------------------
// Host: geometry, resources, weight layouts, dispatch
// ---------------------------------------------------------------------------------
static OpArgs to_args(const pb_op_params* p) {
    OpArgs a;
    a.C = p->C; a.H = p->H; a.W = p->W; a.Cs = p->Cs; a.K = p->K; a.P = p->P; a.Q = p->Q; a.Ks = p->Ks;
    a.out_c_off = p->out_c_off; a.R = p->R; a.S = p->S; a.stride_h = p->stride_h; a.stride_w = p->stride_w;
    a.pad_h = p->pad_h; a.pad_w = p->pad_w; a.groups = p->groups > 0 ? p->groups : 1; a.act = p->act; a.flags = p->flags;
    a.res_Cs = p->res_Cs; a.dil_h = p->dil_h > 1 ? p->dil_h : 1; a.dil_w = p->dil_w > 1 ? p->dil_w : 1; a.x = p->x; a.w = p->w; a.bias = p->bias; a.residual = p->residual; a.y = p->y;
    return a;
}

static int vec_n(int dtype) { return dtype == 0 ? 4 : 8; }
static int batch_of(const pb_op_params* p) { return p->batch > 1 ? p->batch : 1; }
static size_t elem_size(int dtype) { return dtype == 0 ? 4 : 2; }

template <typename F>
static uint32_t regs_of(F fn) {
    cudaFuncAttributes at;
    if (cudaFuncGetAttributes(&at, (const void*)fn) != cudaSuccess) { cudaGetLastError(); return 32; }
    return (uint32_t)at.numRegs;
}
template <typename F>
static uint32_t static_smem_of(F fn) {
    cudaFuncAttributes at;
    if (cudaFuncGetAttributes(&at, (const void*)fn) != cudaSuccess) { cudaGetLastError(); return 0; }
    return (uint32_t)at.sharedSizeBytes;
}

// Threads of work -> blocks of 256.
static uint32_t blocks_for(size_t work) { return (uint32_t)((work + 255) / 256 > 0 ? (work + 255) / 256 : 1); }

// Output pixels per thread of window3_strip_kernel for a depthwise convolution or pooling layer: 0 when the
// window is not 3x3 with stride 1 or 2 (the layer keeps dwconv_kernel / pool_kernel); the wide strip when the
// strips (4 pixels at stride 1, 2 at stride 2) alone give each SM 2048 threads; else 1 (all batch-1 layers of the
// served models: there the launch is latency-bound and more, smaller threads finish sooner).
static int strip_of(const pb_op_params* p) {
    if (p->R != 3 || p->S != 3 || p->stride_h != p->stride_w || (p->stride_h != 1 && p->stride_h != 2)) return 0;
    static thread_local int sms = 0;      // of the device current at the first call of this thread (replicas: one GPU per thread)
    if (sms == 0) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) {
            cudaGetLastError();
            sms = 148;
        }
    }
    const int wide = p->stride_h == 1 ? kStripWide1 : kStripWide2;
    const size_t n = (size_t)batch_of(p) * p->P * ((p->Q + wide - 1) / wide) * (p->Cs / vec_n(p->dtype));
    // Below that size the one-pixel variant still pays: its nine loads are in flight together.  (Tried for the sake of
    // a busy GPU: the plain kernels, 40 registers instead of 100-126, so that their blocks fit beside resident
    // tensor-core CTAs.  Serving throughput FELL, 26.9k -> 24.8k Inception-v3 req/s with 96 in flight: under load these
    // launches cost what they take in time, not in registers.)
    return n >= (size_t)sms * 2048 ? wide : 1;
}
static size_t strip_threads(const pb_op_params* p, int strip) {
    return (size_t)p->P * ((p->Q + strip - 1) / strip) * (p->Cs / vec_n(p->dtype));
}

// Blocks of window3_tile_kernel for one image, or 0 when the layer keeps the strip kernels: bf16, a 3x3 window of stride 1
// or 2, and at least 100 blocks in the launch (all images).  Measured on Inception-v3 served in gangs of 8: thresholds of
// 30, 100 and 300 blocks give the same +2 % requests/s over 592 (its two stem max pools then run here); below 100 a lone
// request's pooling layers are a few dozen blocks and keep the strip kernels, which finish sooner on an idle GPU.
// PB_WINDOW_TILE=0 switches it off; PB_WINDOW_TILE_MIN_BLOCKS sets another threshold (tests use 1).  Read at every call:
// this runs when a launch is built (graph capture, direct operator calls), never on the replay path.
static uint32_t tile_blocks(const pb_op_params* p) {
    if (p->groups <= 1 && (p->bias != nullptr || p->act != 0)) return 0;      // pooling with a bias / activation tail: strip kernels
    if (p->dtype != 1 || (p->Cs & 7) || (p->Ks & 1) || (p->out_c_off & 1) || strip_of(p) == 0) return 0;
    const char* e = getenv("PB_WINDOW_TILE");
    if (e && e[0] == '0') return 0;
    size_t least = 100;
    if (const char* m = getenv("PB_WINDOW_TILE_MIN_BLOCKS")) least = (size_t)strtoull(m, nullptr, 10);
    const int rows = p->stride_h == 1 ? TileGeom<1>::kRows : TileGeom<2>::kRows;
    const int cols = p->stride_h == 1 ? TileGeom<1>::kOutCols : TileGeom<2>::kOutCols;
    const size_t n = (size_t)((p->Cs + kTileSlab - 1) / kTileSlab) * ((p->Q + cols - 1) / cols) * ((p->P + rows - 1) / rows);
    return n * (size_t)batch_of(p) >= least ? (uint32_t)n : 0;
}
static const void* tile_fn(int kind, int stride) {
#define PB_TILE(M) (stride == 1 ? (const void*)window3_tile_kernel<M, 1> : (const void*)window3_tile_kernel<M, 2>)
    return kind == PB_STAGE_DWCONV ? PB_TILE(kWinDw) : kind == PB_STAGE_MAXPOOL ? PB_TILE(kWinMax) : PB_TILE(kWinAvg);
#undef PB_TILE
}
static uint32_t tile_smem(int stride) { return stride == 1 ? TileGeom<1>::kSmemBytes : TileGeom<2>::kSmemBytes; }

template <int kMode>
static const void* window3_fn(bool f32, int stride, int strip) {
#define PB_W3(T) (stride == 1 ? (strip == 1 ? (const void*)window3_strip_kernel<T, kMode, 1, 1> : (const void*)window3_strip_kernel<T, kMode, 1, kStripWide1>) \
                              : (strip == 1 ? (const void*)window3_strip_kernel<T, kMode, 2, 1> : (const void*)window3_strip_kernel<T, kMode, 2, kStripWide2>))
    return f32 ? PB_W3(float) : PB_W3(__nv_bfloat16);
#undef PB_W3
}
static const void* window3_fn(int kind, bool f32, int stride, int strip) {
    return kind == PB_STAGE_DWCONV ? window3_fn<kWinDw>(f32, stride, strip)
         : kind == PB_STAGE_MAXPOOL ? window3_fn<kWinMax>(f32, stride, strip) : window3_fn<kWinAvg>(f32, stride, strip);
}

// Geometry of ONE image of the launch (blocks, algorithmic work); strip_of() alone looks at the batch.
static int info_one_image(int kind, const pb_op_params* p, pb_launch_info* out) {
    memset(out, 0, sizeof(*out));
    out->kind = (uint32_t)kind;
    out->threads_per_block = 256;
    const int N = vec_n(p->dtype);
    const size_t es = elem_size(p->dtype);
    const bool f32 = p->dtype == 0;
    const size_t in_elems = (size_t)p->C * p->H * p->W;
    const size_t out_elems = (size_t)p->K * p->P * p->Q;
    switch (kind) {
        case PB_STAGE_INPUT:
            if (p->R * p->S > 1) {      // patch-matrix form (see input_patch_kernel)
                out->num_blocks = blocks_for((size_t)p->P * p->Q * (p->Ks / N));
                out->regs_per_thread = f32 ? regs_of(input_patch_kernel<float>) : regs_of(input_patch_kernel<__nv_bfloat16>);
                if (const size_t sm = patch_tile_smem(p)) {
                    out->num_blocks = patch_tile_blocks(p);
                    out->regs_per_thread = f32 ? regs_of(input_patch_tile_kernel<float>) : regs_of(input_patch_tile_kernel<__nv_bfloat16>);
                    out->smem_per_block = (uint32_t)sm;
                }
                out->bytes = in_elems * 4 + (size_t)p->P * p->Q * p->Ks * es;
                break;
            }
            out->num_blocks = blocks_for((size_t)p->H * p->W);
            out->regs_per_thread = f32 ? regs_of(input_transform_kernel<float>) : regs_of(input_transform_kernel<__nv_bfloat16>);
            // the output is counted as laid out, Ks channels per pixel: the zero padding up to the vector width is part
            // of the format the convolutions read
            out->bytes = in_elems * 4 + (size_t)p->H * p->W * p->Ks * es;
            break;
        case PB_STAGE_CONV_SIMT:
            out->num_blocks = blocks_for((size_t)p->P * p->Q * p->K);
            out->regs_per_thread = f32 ? regs_of(conv_simt_kernel<float>) : regs_of(conv_simt_kernel<__nv_bfloat16>);
            out->flops = 2ull * out_elems * (p->C / (p->groups > 0 ? p->groups : 1)) * p->R * p->S;
            out->bytes = es * (in_elems + (size_t)p->K * (p->C / (p->groups > 0 ? p->groups : 1)) * p->R * p->S + out_elems +
                               (p->residual ? out_elems : 0)) + 4ull * p->K;
            break;
        case PB_STAGE_DWCONV:
            out->num_blocks = blocks_for((size_t)p->P * p->Q * (p->Cs / N));
            out->regs_per_thread = f32 ? regs_of(dwconv_kernel<float>) : regs_of(dwconv_kernel<__nv_bfloat16>);
            if (const int strip = strip_of(p)) {
                out->num_blocks = blocks_for(strip_threads(p, strip));
                out->regs_per_thread = regs_of(window3_fn(kind, f32, p->stride_h, strip));
                out->smem_per_block = strip > 1 ? (uint32_t)window3_smem_bytes(p->Cs, f32 ? 4 : 2) : 0;
            }
            if (const uint32_t nblk = tile_blocks(p)) {
                out->num_blocks = nblk;
                out->regs_per_thread = regs_of(tile_fn(kind, p->stride_h));
                out->smem_per_block = tile_smem(p->stride_h);
            }
            out->flops = 2ull * out_elems * p->R * p->S;
            out->bytes = es * (in_elems + (size_t)p->K * p->R * p->S + out_elems) + 4ull * p->K;
            break;
        case PB_STAGE_MAXPOOL:
        case PB_STAGE_AVGPOOL:
            out->num_blocks = blocks_for((size_t)p->P * p->Q * (p->Cs / N));
            if (kind == PB_STAGE_MAXPOOL)
                out->regs_per_thread = f32 ? regs_of(pool_kernel<float, true>) : regs_of(pool_kernel<__nv_bfloat16, true>);
            else
                out->regs_per_thread = f32 ? regs_of(pool_kernel<float, false>) : regs_of(pool_kernel<__nv_bfloat16, false>);
            if (const int strip = strip_of(p)) {
                out->num_blocks = blocks_for(strip_threads(p, strip));
                out->regs_per_thread = regs_of(window3_fn(kind, f32, p->stride_h, strip));
            }
            if (const uint32_t nblk = tile_blocks(p)) {
                out->num_blocks = nblk;
                out->regs_per_thread = regs_of(tile_fn(kind, p->stride_h));
                out->smem_per_block = tile_smem(p->stride_h);
            }
            out->bytes = es * (in_elems + out_elems) + (p->bias ? 4ull * p->K : 0);
            break;
        case PB_STAGE_GAP:
            out->num_blocks = (uint32_t)pb::ceil_div(p->Cs / N, 32);
            out->regs_per_thread = f32 ? regs_of(gap_kernel<float>) : regs_of(gap_kernel<__nv_bfloat16>);
            out->smem_per_block = f32 ? static_smem_of(gap_kernel<float>) : static_smem_of(gap_kernel<__nv_bfloat16>);
            out->bytes = es * in_elems + ((p->flags & 2) ? 4 : es) * (size_t)p->C;
            break;
        case PB_STAGE_DENSE:
            out->num_blocks = (uint32_t)pb::ceil_div(p->K, 8);
            out->regs_per_thread = f32 ? regs_of(dense_kernel<float>) : regs_of(dense_kernel<__nv_bfloat16>);
            out->flops = 2ull * p->C * p->K;
            out->bytes = es * ((size_t)p->C + (size_t)p->C * p->K) + 4ull * p->K + ((p->flags & 2) ? 4 : es) * (size_t)p->K;
            break;
        case PB_STAGE_ADD:
            out->num_blocks = blocks_for((size_t)p->H * p->W * p->Cs / N);
            out->regs_per_thread = f32 ? regs_of(add_kernel<float>) : regs_of(add_kernel<__nv_bfloat16>);
            out->bytes = es * 3 * in_elems;
            break;
        case PB_STAGE_AFFINE:
            out->num_blocks = blocks_for(((size_t)p->H * p->W * pb::ceil_div(p->C, N) + kAffinePer - 1) / kAffinePer);
            out->regs_per_thread = f32 ? regs_of(affine_kernel<float>) : regs_of(affine_kernel<__nv_bfloat16>);
            out->flops = 2ull * p->C * p->H * p->W;
            out->bytes = es * 2ull * p->C * p->H * p->W + 8ull * p->C;
            break;
        case PB_STAGE_SOFTMAX:
            out->num_blocks = 1;
            out->regs_per_thread = regs_of(softmax_kernel<float, true>);
            out->smem_per_block = static_smem_of(softmax_kernel<float, true>);
            out->bytes = 8ull * p->C;
            break;
        case PB_STAGE_DETECT:
            out->num_blocks = blocks_for((size_t)p->H * p->W * (p->C / 6));
            out->regs_per_thread = f32 ? regs_of(detect_kernel<float>) : regs_of(detect_kernel<__nv_bfloat16>);
            out->flops = 20ull * p->H * p->W * (p->C / 6);
            out->bytes = es * (uint64_t)p->H * p->W * p->C + (16ull + 24ull) * p->H * p->W * (p->C / 6);
            break;
        default:
            set_error("pb_op_info: unknown stage kind %d", kind);
            return PB_ERR_INVALID;
    }
    return PB_OK;
}

// Elementwise kernels see a batch as one taller tensor (images are contiguous).
static bool folds_batch(int kind) { return kind == PB_STAGE_ADD || kind == PB_STAGE_AFFINE; }

int simple_op_info(int kind, const pb_op_params* p, pb_launch_info* out) {
    const int nb = batch_of(p);
    const int rc = info_one_image(kind, p, out);
    if (rc != PB_OK || nb == 1) return rc;
    if (folds_batch(kind)) {
        pb_op_params q = *p;
        q.H *= nb;
        return info_one_image(kind, &q, out);
    }
    out->num_blocks *= (uint32_t)nb;
    out->flops *= (uint64_t)nb;
    // the weights are read once per launch whatever the batch
    const uint64_t es = p->dtype == 0 ? 4 : 2;
    const uint64_t wbytes = kind == PB_STAGE_DENSE ? es * (uint64_t)p->C * p->K
                          : kind == PB_STAGE_DWCONV ? es * (uint64_t)p->K * p->R * p->S : 0;
    out->bytes = wbytes + (out->bytes - wbytes) * (uint64_t)nb;
    return PB_OK;
}

static thread_local size_t t_launch_smem = 0;      // dynamic shared memory of the next launch_k (reset by it)

template <typename... KArgs, typename... Args>
static void launch_k(void (*kern)(KArgs...), dim3 grid, dim3 block, cudaStream_t st, bool pdl, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.stream = st;
    cfg.dynamicSmemBytes = t_launch_smem;
    t_launch_smem = 0;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

int simple_op_launch(int kind, const pb_op_params* p, cudaStream_t st, uint32_t job_id, void* notifier, bool pdl) {
    FinishedBlockNotifier* nf = static_cast<FinishedBlockNotifier*>(notifier);
    pb_launch_info li;
    pb_op_params folded;
    int nb = batch_of(p);
    if (nb > 1 && folds_batch(kind)) {
        folded = *p;
        folded.H *= nb;
        folded.batch = 1;
        p = &folded;
        nb = 1;
    }
    int rc = info_one_image(kind, p, &li);
    if (rc != PB_OK) return rc;
    const OpArgs a = to_args(p);
    const bool f32 = p->dtype == 0;
    const int N = vec_n(p->dtype);
    if (kind == PB_STAGE_INPUT) PB_REQUIRE(p->Ks % N == 0, "output channel stride %d is not a multiple of the %d-element vector", p->Ks, N);
    else PB_REQUIRE(p->Cs % N == 0, "channel stride %d is not a multiple of the %d-element vector", p->Cs, N);
    const dim3 grid(li.num_blocks, (unsigned)nb), block(256);      // blockIdx.y = image
#ifdef PB_DEBUG_SKIP
    // development builds only: PB_DEBUG_SKIP_MEMBOUND=1 leaves out the pooling / layout kernels that never notify
    // (wrong results; shows what they cost the tensor-core kernels under load)
    if (job_id != kSlotNotify && nf == nullptr || job_id == kSlotQuiet) {
        const char* e = getenv("PB_DEBUG_SKIP_MEMBOUND");
        const int mask = e ? atoi(e) : 0;      // 1 layout, 2 max pooling, 4 average pooling
        if ((kind == PB_STAGE_INPUT && (mask & 1)) || (kind == PB_STAGE_MAXPOOL && (mask & 2)) || (kind == PB_STAGE_AVGPOOL && (mask & 4))) return PB_OK;
    }
#endif
#define PB_DISPATCH(kern_f32, kern_bf16, ...)                                           \
    do {                                                                                \
        if (f32) launch_k(kern_f32, grid, block, st, pdl, __VA_ARGS__);                 \
        else launch_k(kern_bf16, grid, block, st, pdl, __VA_ARGS__);                    \
    } while (0)
    switch (kind) {
        case PB_STAGE_INPUT:
            if (p->R * p->S > 1) {
                PB_REQUIRE(p->Ks >= p->R * p->S * p->C, "input patches: row stride %d is shorter than R*S*C = %d", p->Ks, p->R * p->S * p->C);
                if (const size_t sm = patch_tile_smem(p)) {
                    t_launch_smem = sm;
                    if (f32) launch_k(input_patch_tile_kernel<float>, grid, block, st, pdl, a, job_id, nf);
                    else launch_k(input_patch_tile_kernel<__nv_bfloat16>, grid, block, st, pdl, a, job_id, nf);
                    break;
                }
                PB_DISPATCH(input_patch_kernel<float>, input_patch_kernel<__nv_bfloat16>, a, job_id, nf);
                break;
            }
            if (f32) launch_k(input_transform_kernel<float>, grid, block, st, pdl, (const float*)p->x, (float*)p->y, p->C, p->H * p->W, p->Ks, job_id, nf);
            else launch_k(input_transform_kernel<__nv_bfloat16>, grid, block, st, pdl, (const float*)p->x, (__nv_bfloat16*)p->y, p->C, p->H * p->W, p->Ks, job_id, nf);
            break;
        case PB_STAGE_CONV_SIMT:
            PB_REQUIRE(a.C % a.groups == 0 && a.K % a.groups == 0, "conv: groups must divide channels");
            PB_DISPATCH(conv_simt_kernel<float>, conv_simt_kernel<__nv_bfloat16>, a, job_id, nf);
            break;
        case PB_STAGE_DWCONV:
            PB_REQUIRE(a.groups == a.C && a.K == a.C, "dwconv: needs groups == C == K");
            PB_REQUIRE((a.Ks % N) == 0 && (a.out_c_off % N) == 0, "dwconv: output slice must be vector aligned");
            if (tile_blocks(p)) {
                const void* fn = tile_fn(kind, p->stride_h);
                PB_CUDA(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)tile_smem(p->stride_h)));
                t_launch_smem = tile_smem(p->stride_h);
                launch_k((void (*)(OpArgs, uint32_t, FinishedBlockNotifier*))fn, grid, block, st, pdl, a, job_id, nf);
                break;
            }
            if (const int strip = strip_of(p)) {
                t_launch_smem = strip > 1 ? (size_t)window3_smem_bytes(p->Cs, f32 ? 4 : 2) : 0;
                launch_k((void (*)(OpArgs, uint32_t, FinishedBlockNotifier*))window3_fn(kind, f32, p->stride_h, strip), grid, block, st, pdl, a, job_id, nf);
                break;
            }
            PB_DISPATCH(dwconv_kernel<float>, dwconv_kernel<__nv_bfloat16>, a, job_id, nf);
            break;
        case PB_STAGE_MAXPOOL:
            PB_REQUIRE((a.Ks % N) == 0 && (a.out_c_off % N) == 0, "pool: output slice must be vector aligned");
            if (tile_blocks(p)) {
                const void* fn = tile_fn(kind, p->stride_h);
                PB_CUDA(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)tile_smem(p->stride_h)));
                t_launch_smem = tile_smem(p->stride_h);
                launch_k((void (*)(OpArgs, uint32_t, FinishedBlockNotifier*))fn, grid, block, st, pdl, a, job_id, nf);
                break;
            }
            if (const int strip = strip_of(p)) {
                launch_k((void (*)(OpArgs, uint32_t, FinishedBlockNotifier*))window3_fn(kind, f32, p->stride_h, strip), grid, block, st, pdl, a, job_id, nf);
                break;
            }
            PB_DISPATCH((pool_kernel<float, true>), (pool_kernel<__nv_bfloat16, true>), a, job_id, nf);
            break;
        case PB_STAGE_AVGPOOL:
            PB_REQUIRE((a.Ks % N) == 0 && (a.out_c_off % N) == 0, "pool: output slice must be vector aligned");
            if (tile_blocks(p)) {
                const void* fn = tile_fn(kind, p->stride_h);
                PB_CUDA(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)tile_smem(p->stride_h)));
                t_launch_smem = tile_smem(p->stride_h);
                launch_k((void (*)(OpArgs, uint32_t, FinishedBlockNotifier*))fn, grid, block, st, pdl, a, job_id, nf);
                break;
            }
            if (const int strip = strip_of(p)) {
                launch_k((void (*)(OpArgs, uint32_t, FinishedBlockNotifier*))window3_fn(kind, f32, p->stride_h, strip), grid, block, st, pdl, a, job_id, nf);
                break;
            }
            PB_DISPATCH((pool_kernel<float, false>), (pool_kernel<__nv_bfloat16, false>), a, job_id, nf);
            break;
        case PB_STAGE_GAP:
            PB_DISPATCH(gap_kernel<float>, gap_kernel<__nv_bfloat16>, a, job_id, nf);
            break;
        case PB_STAGE_DENSE:
            PB_REQUIRE(a.C % N == 0, "dense: input length %d is not a multiple of %d", a.C, N);
            PB_DISPATCH(dense_kernel<float>, dense_kernel<__nv_bfloat16>, a, job_id, nf);
            break;
        case PB_STAGE_ADD:
            PB_REQUIRE(a.residual != nullptr, "add: second operand missing");
            PB_DISPATCH(add_kernel<float>, add_kernel<__nv_bfloat16>, a, job_id, nf);
            break;
        case PB_STAGE_AFFINE:
            PB_REQUIRE(a.w != nullptr && a.bias != nullptr, "affine: scale and bias are required");
            PB_REQUIRE((a.Ks % N) == 0 && (a.out_c_off % N) == 0, "affine: output slice must be vector aligned");
            PB_DISPATCH(affine_kernel<float>, affine_kernel<__nv_bfloat16>, a, job_id, nf);
            break;
        case PB_STAGE_SOFTMAX:
            // flags bit2: the input is fp32 regardless of dtype
            if (f32 || (p->flags & 4)) launch_k(softmax_kernel<float, true>, grid, block, st, pdl, a, job_id, nf);
            else launch_k(softmax_kernel<__nv_bfloat16, false>, grid, block, st, pdl, a, job_id, nf);
            break;
        case PB_STAGE_DETECT:
            PB_REQUIRE(a.w != nullptr && a.bias != nullptr && a.C % 6 == 0 && a.C > 0, "detect: priors, variances and 6 channels per anchor are required");
            PB_REQUIRE((p->flags & 2) != 0, "detect: writes the fp32 model output only");
            PB_REQUIRE((size_t)a.out_c_off + (size_t)a.H * a.W * (a.C / 6) <= (size_t)a.K, "detect: priors of this map exceed the model's count");
            PB_DISPATCH(detect_kernel<float>, detect_kernel<__nv_bfloat16>, a, job_id, nf);
            break;
        default:
            set_error("pb_op_launch: unknown stage kind %d", kind);
            return PB_ERR_INVALID;
    }
#undef PB_DISPATCH
    return launch_check("operator kernel");
}

// Weight layouts (host side).  Source: OIHW fp32.
//  conv_simt: [R][S][C/groups][K]      dwconv: [R][S][Cs]      dense: see graph loader
static uint16_t f32_to_bf16_bits(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40);
    u += 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}

void store_elem(void* dst, size_t i, float v, int dtype) {
    if (dtype == 0) static_cast<float*>(dst)[i] = v;
    else static_cast<uint16_t*>(dst)[i] = f32_to_bf16_bits(v);
}

int64_t simple_pack_weights(int kind, const pb_op_params* p, const float* w, void* dst) {
    const size_t es = elem_size(p->dtype);
    const int groups = p->groups > 0 ? p->groups : 1;
    if (kind == PB_STAGE_CONV_SIMT) {
        const int cg = p->C / groups;
        const size_t n = (size_t)p->R * p->S * cg * p->K;
        if (dst) {
            for (int k = 0; k < p->K; ++k)
                for (int c = 0; c < cg; ++c)
                    for (int r = 0; r < p->R; ++r)
                        for (int s = 0; s < p->S; ++s)
                            store_elem(dst, ((size_t)(r * p->S + s) * cg + c) * p->K + k,
                                       w[(((size_t)k * cg + c) * p->R + r) * p->S + s], p->dtype);
        }
        return (int64_t)(n * es);
    }
    if (kind == PB_STAGE_DWCONV) {
        const size_t n = (size_t)p->R * p->S * p->Cs;
        if (dst) {
            memset(dst, 0, n * es);
            for (int c = 0; c < p->C; ++c)
                for (int r = 0; r < p->R; ++r)
                    for (int s = 0; s < p->S; ++s)
                        store_elem(dst, (size_t)(r * p->S + s) * p->Cs + c, w[((size_t)c * p->R + r) * p->S + s], p->dtype);
        }
        return (int64_t)(n * es);
    }
    set_error("pb_op_pack_weights: stage kind %d has no packed weights here", kind);
    return PB_ERR_INVALID;
}

int mnist_fused_info(pb_launch_info* out) {
    memset(out, 0, sizeof(*out));
    out->kind = PB_STAGE_MNIST_FUSED;
    out->num_blocks = 1;
    out->threads_per_block = 256;
    out->regs_per_thread = regs_of(mnist_fused_kernel);
    out->smem_per_block = static_smem_of(mnist_fused_kernel);
    out->flops = 2ull * (156800 + 627200 + 2560);
    out->bytes = 4ull * (784 + 200 + 8 + 3200 + 16 + 2560 + 10 + 10);
    return PB_OK;
}

int mnist_fused_launch(const float* x, const float* w1, const float* b1, const float* w2, const float* b2,
                       const float* wd, const float* bd, float* y, int batch, cudaStream_t st, uint32_t job_id, void* notifier) {
    MnistArgs a{x, w1, b1, w2, b2, wd, bd, y};
    mnist_fused_kernel<<<batch > 1 ? batch : 1, 256, 0, st>>>(a, job_id, static_cast<FinishedBlockNotifier*>(notifier));
    return launch_check("mnist_fused");
}

}  // namespace pb
