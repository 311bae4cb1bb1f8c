// Dense convolution as an implicit GEMM on the 5th-generation tensor cores (sm_100a).
//
//   D[m, n] = sum_k A[m, k] * B[n, k]     m = output pixel (p*Q + q), n = output channel,
//                                          k = (r*S + s)*Cs + c   (filter tap, input channel)
//
// A is never materialised.  One thread per CTA issues, per 64-deep k-block, an im2col-mode TMA
// (cp.async.bulk.tensor.4d...im2col: 128 consecutive output pixels x 64 channels of one filter tap,
// padding and the ragged last tile zero-filled by the hardware; a plain tiled TMA when the layer is
// pointwise) that lands A in the 128-byte-swizzled K-major shared-memory layout tcgen05.mma reads,
// and a tiled TMA for B (packed weights [Kout_pad][Kdim_pad], no multicast).  One elected thread
// issues tcgen05.mma (M=128, N=BN, K=16, bf16 x bf16 -> fp32) with the accumulator in tensor
// memory; tcgen05.commit releases pipeline stages and signals the epilogue, which reads TMEM with
// tcgen05.ld, adds bias and residual, applies the activation and stores bf16 into the channel
// slice of the output tensor.
//
// CTA = 6 warps: warps 0-3 run the epilogue (thread t owns accumulator lane t), warp 4 is the TMA
// producer, warp 5 allocates TMEM and issues the MMAs.  Sized for three CTAs per SM.
// Two entry points share the body (conv_tile_tma): conv_umma_tma_kernel runs one convolution,
// conv_umma_multi_kernel runs several independent ones as one grid from a descriptor table in
// device memory.  conv_umma_gather_kernel (PB_CONV_GATHER=1) is the earlier design, kept for
// comparison: 128 producer threads gather A with 16-byte cp.async copies.
//
// Every wait is bounded: when a wait runs out the CTA raises a device-global error flag,
// sets a shared abort flag that releases all other waits of the CTA, skips the epilogue,
// lets in-flight copies land, frees its TMEM and still reports block end.
//
// This is the tensor-core member of the kernel family the reference's TVM adapters launch
// (jobs/tvm_<model>/tvm_<model>.cpp:24-47; generated SIMT fp32 kernels there).
#include <cuda.h>
#include <cuda_bf16.h>
#include <llis/job/finished_block_notifier.h>

#include <cstdlib>
#include <cstring>
#include <algorithm>
#include <atomic>
#include <mutex>
#include <vector>

#include "launch_slot.cuh"
#include "ops.h"
#include "pb_common.h"

using llis::job::FinishedBlockNotifier;

namespace pb {

namespace {

constexpr int kBM = 128;            // tile rows (output pixels) = TMEM lanes
constexpr int kBK = 64;             // bf16 elements per k-block = one 128-byte swizzle row
// Pipeline depth is a template parameter: kStages shared-memory stages.  Each producer thread keeps
// kLag = kStages/2 cp.async groups in flight (it arrives on a stage's barrier kLag iterations after
// issuing its copies).  The other half of the stages is slack for the hand-off round trip
// (producer arrive -> MMA issue -> tcgen05.commit -> producer may refill), which the probe measured
// at well over a microsecond: with only two stages of slack that round trip paced the whole loop.
#ifndef PB_LAG_OF
#define PB_LAG_OF(stages) ((stages) / 2)
#endif
constexpr int kMaxStages = 8;
constexpr int kMaxBN = 256;          // output channels per CTA tile at most (tcgen05.mma N <= 256)
constexpr uint32_t kSmemBudget = 200u * 1024u;   // one CTA per SM (gather kernel)
// The TMA kernel is sized for THREE CTAs per SM (73 KB of pipeline + ~2 KB static and reserved each
// out of 228 KB; <= 112 registers; <= 128 of 512 TMEM columns).  One CTA cannot pull more than about
// 60 bytes per clock through its SM and spends a third of its life in fixed latencies (set-up, first
// operand arrival, epilogue), so with many requests in flight residency, not pipeline depth, sets the
// GPU's convolution throughput: the co-resident CTAs keep the SM's load path busy between them.
#ifndef PB_CONV_SMEM_KB
#define PB_CONV_SMEM_KB 73
#endif
constexpr uint32_t kSmemBudgetTma = PB_CONV_SMEM_KB * 1024u;
constexpr uint32_t kCounterBytes = 4096;        // split-K tile counters at the head of the scratch buffer
#ifndef PB_NOALLOC_SCRATCH_BYTES
#define PB_NOALLOC_SCRATCH_BYTES (4u << 20)      // built-in scratch of pb_conv2d_umma_noalloc: 4 MiB per GPU
#endif
constexpr int kATileBytes = kBM * kBK * 2;   // 16 KiB
constexpr uint32_t kWaitLimit = 4u * 1000u * 1000u;  // polls of mbarrier.try_wait before giving up
constexpr int kThreads = 160;

struct ConvArgs {
    const __nv_bfloat16* x;
    const __nv_bfloat16* residual;
    const float* bias;
    __nv_bfloat16* y;
    uint32_t* err_flag;
    int H, W, Cs;
    int P, Q, M;          // M = batch * P*Q: the images of a batch are consecutive rows of the GEMM
    int PQ;               // output pixels per image
    int dh, dw;           // filter dilation
    int K, Ks, out_c_off, res_Cs;
    int R, S, sh, sw, ph, pw;
    int act;
    int a_tiled;          // 1: pointwise convolution, operand A is the plain [M][Cs] matrix (tiled TMA, no im2col)
    int nkb;              // k-blocks of 64 = taps * chunks per tap
    int taps;             // R*S
    int Cp;               // channels per tap rounded up to 64: k = tap*Cp + c
    int BN;               // output channels per CTA (multiple of 16, <= 256)
    uint32_t idesc;       // tcgen05 instruction descriptor
    uint32_t tmem_cols;   // power of two >= max(32, BN)
    uint32_t b_stage_bytes;
    // split-K: blockIdx.z handles k-blocks [z*kb_per_split, ...); partial tiles meet in `ws`
    int splits, kb_per_split;
    float* ws;              // [tile][split][128][BN] fp32 partial accumulators
    unsigned* counters;     // [tile] arrival counters, zero between launches
};

// ---- PTX wrappers -----------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.shared::cta.b64 st, [%0];\n\t}" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.expect_tx.relaxed.cta.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Non-blocking probe of a phase (never suspends the thread).
__device__ __forceinline__ bool mbar_test_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait.  Returns false if the CTA is aborting (this wait or another ran out).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile uint32_t* s_abort, uint32_t* err_flag,
                                          uint32_t code) {
    for (uint32_t i = 0; i < kWaitLimit; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 63u) == 63u && *s_abort) return false;
    }
    *s_abort = 1;
    atomicExch(err_flag, code);
    return false;
}

__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src, uint32_t src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar)
        : "memory");
}

// im2col-mode TMA: 128 consecutive output pixels (traversed W, then H, then N inside the bounding
// box of filter-window origins) x 64 channels, at filter offset (w_off, h_off); elements outside
// the tensor arrive as zeros.
__device__ __forceinline__ void tma_load_im2col_4d(uint32_t dst, const CUtensorMap* map, int c, int w, int h, int n,
                                                   uint16_t w_off, uint16_t h_off, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.im2col.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4, %5, %6}], [%2], {%7, %8};"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c), "r"(w), "r"(h), "r"(n), "h"(w_off), "h"(h_off)
        : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1;\n\t}" ::"r"(bar), "r"(bytes) : "memory");
}

__device__ __forceinline__ void tcgen05_alloc(uint32_t slot_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot_smem), "r"(cols) : "memory");
}
__device__ __forceinline__ void tcgen05_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tcgen05_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tcgen05_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcgen05_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcgen05_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tcgen05_mma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                                 uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void tcgen05_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tcgen05_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor: K-major operand, 128-byte swizzle, rows of 128 bytes,
// 8-row groups 1024 bytes apart.  Bits: [0,14) address>>4, [16,30) leading offset>>4 (unused
// for swizzled K-major, set to 1), [32,46) stride offset>>4, [46,48) version 1, [61,64) swizzle mode 2.
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr) {
    return (uint64_t)((smem_addr & 0x3ffffu) >> 4) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) |
           (2ull << 61);
}

__device__ __forceinline__ unsigned long long globaltimer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// Optional phase stamps for development builds (-DPB_CONV_TIMING): %globaltimer at eight points of
// the first 64 CTAs, written to a device array the probe program reads back.
#ifdef PB_CONV_TIMING
__device__ unsigned long long g_conv_t[64 * 8];
#define PB_T(i)                                                                                         \
    do {                                                                                                \
        const unsigned b_ = blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z);             \
        if (b_ < 64) g_conv_t[b_ * 8 + (i)] = globaltimer_ns();                                         \
    } while (0)
// per-k-block SM-clock stamps of the first 8 CTAs: [cta][kb][0 = loads issued, 1 = operands landed, 2 = MMAs issued]
__device__ unsigned long long g_conv_kb[8 * 64 * 3];
#define PB_TK(kb, i)                                                                                    \
    do {                                                                                                \
        const unsigned b_ = blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z);             \
        if (b_ < 8 && (kb) < 64) g_conv_kb[(b_ * 64 + (kb)) * 3 + (i)] = (unsigned long long)clock64();              \
    } while (0)
#else
#define PB_T(i) do {} while (0)
#define PB_TK(kb, i) do {} while (0)
#endif

// Optional per-phase cycle sums over every CTA of the TMA kernels (-DPB_CONV_STATS, development builds):
// [0] CTAs, [1] k-blocks, then clock64 differences: [2] set-up, [3] wait for the previous kernel, [4] first
// operands, [5] main loop (first operands landed -> last MMA issued), [6] accumulator drain, [7] epilogue,
// [8] tear-down, [9] whole CTA.
#ifdef PB_CONV_STATS
__device__ unsigned long long g_conv_stats[16];      // [10..15]: CTAs that found 0..5+ other conv CTAs resident on their SM
__device__ unsigned int g_conv_resident[256];        // conv CTAs resident per SM right now
__device__ long long g_persist_kb[64 * 6];          // CTA 0, its first tile: per k-block clock64 stamps (see PB_PK)
#define PB_PK(kb, i) do { if (blockIdx.x == 0 && first_tile && (kb) < 64) g_persist_kb[(kb) * 6 + (i)] = clock64(); } while (0)
__device__ unsigned int g_persist_resident;          // persistent CTAs resident GPU-wide right now
__device__ unsigned long long g_persist_hist[16];     // [b]: CTAs that found 32*b .. 32*b+31 others resident when they started; [15]: sum of lifetimes (clk)
__device__ long long g_persist_tile[16 * 6];        // CTA 0: per tile clock64 stamps (see PB_PT)
#define PB_PT(ti, i) do { if (blockIdx.x == 0 && (ti) < 16) g_persist_tile[(ti) * 6 + (i)] = clock64(); } while (0)
__device__ unsigned long long g_conv_ns;             // sum of the CTAs' lifetimes by %globaltimer (ns): cycles / ns = the SM clock
#define PB_S(i) do { s_clk[(i)] = clock64(); } while (0)
#else
#define PB_S(i) do {} while (0)
#define PB_PK(kb, i) do {} while (0)
#define PB_PT(ti, i) do {} while (0)
#endif

// ---- the kernel -----------------------------------------------------------------------
// Packed fp32 pairs (sm_100 has two-wide fp32 adds) and the bf16 pair conversion with the activation
// folded in: cvt's .relu clamps negatives to zero, ReLU6 is one more packed min against 6.0.
// Rounding is monotonic and 0 and 6 are bf16 values, so activation-after-rounding equals
// rounding-after-activation.
__device__ __forceinline__ uint64_t pack_f32x2(uint32_t lo, uint32_t hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(lo), "r"(hi));
    return r;
}
__device__ __forceinline__ uint64_t add_f32x2(uint64_t x, uint64_t y) {
    uint64_t r;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(x), "l"(y));
    return r;
}
template <int ACT>
__device__ __forceinline__ uint32_t to_bf16x2_act(uint64_t v, float slope_lo = 0.f, float slope_hi = 0.f) {
    uint32_t lo, hi, d;
    asm("mov.b64 {%0, %1}, %2;" : "=r"(lo), "=r"(hi) : "l"(v));
    if constexpr (ACT == 3) {       // PReLU: v > 0 ? v : slope * v, per channel
        const float a = __uint_as_float(lo), b = __uint_as_float(hi);
        lo = __float_as_uint(a > 0.f ? a : a * slope_lo);
        hi = __float_as_uint(b > 0.f ? b : b * slope_hi);
    }
    if constexpr (ACT == 0 || ACT == 3) {
        asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(__uint_as_float(hi)), "f"(__uint_as_float(lo)));
    } else {
        asm("cvt.rn.relu.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(__uint_as_float(hi)), "f"(__uint_as_float(lo)));
        if constexpr (ACT == 2) asm("min.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(d), "r"(0x40C040C0u));
    }
    return d;
}

// One group of NC (= 16) accumulator columns of this thread's row: TMEM -> registers, (+ split-K
// partial tiles), + bias (+ residual), activation, bf16, 16-byte stores.  Everything that does not
// depend on the accumulator is fetched before the TMEM wait.  The four epilogue warps run one per
// scheduler with nothing to hide instruction latency behind, so the column loop is kept to one
// packed add and one convert per two columns.
template <int NC, int ACT>
__device__ __forceinline__ void epilogue_chunk(const ConvArgs& a, uint32_t lane_addr, int cb, int n0, bool row_valid,
                                               __nv_bfloat16* yrow, const __nv_bfloat16* rrow, const float* part, size_t tile_floats,
                                               const float* s_bias) {
    uint32_t v[NC];
    static_assert(NC == 16, "16 accumulator columns per step keep the kernel within 112 registers (three CTAs per SM)");
    tcgen05_ld16(lane_addr + (uint32_t)cb, v);   // warp-collective: all lanes take part
    const int k0 = n0 + cb;
    const bool live = row_valid && k0 < a.K;
    uint4 rv[NC / 8];
#pragma unroll
    for (int h = 0; h < NC / 8; ++h) rv[h] = make_uint4(0, 0, 0, 0);
    if (live && rrow) {
#pragma unroll
        for (int h = 0; h < NC / 8; ++h)
            if (k0 + h * 8 + 8 <= a.K) rv[h] = *reinterpret_cast<const uint4*>(rrow + k0 + h * 8);
    }
    uint64_t bias2[NC / 2];
#pragma unroll
    for (int j = 0; j < NC; j += 4) {
        const uint4 b4 = *reinterpret_cast<const uint4*>(s_bias + cb + j);
        bias2[j / 2] = pack_f32x2(b4.x, b4.y);
        bias2[j / 2 + 1] = pack_f32x2(b4.z, b4.w);
    }
    if (live && part) {
        // every partial tile, this CTA's own included, is read from the workspace in split order, so
        // the fp32 sum does not depend on which CTA arrived last; it starts from the bias
        for (int z = 0; z < a.splits; ++z) {
            const uint4* other = reinterpret_cast<const uint4*>(part + (size_t)z * tile_floats) + threadIdx.x;
#pragma unroll
            for (int j = 0; j < NC / 4; ++j) {
                const uint4 o = __ldcg(other + (size_t)(cb / 4 + j) * kBM);
                bias2[2 * j] = add_f32x2(bias2[2 * j], pack_f32x2(o.x, o.y));
                bias2[2 * j + 1] = add_f32x2(bias2[2 * j + 1], pack_f32x2(o.z, o.w));
            }
        }
    }
    tcgen05_wait_ld();
    if (!live) return;
#pragma unroll
    for (int h = 0; h < NC / 8; ++h) {
        const int kk = k0 + h * 8;
        if (kk + 8 <= a.K) {
            const uint32_t ru[4] = {rv[h].x, rv[h].y, rv[h].z, rv[h].w};
            uint32_t o[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                uint64_t f = bias2[h * 4 + j];
                if (!part) f = add_f32x2(pack_f32x2(v[h * 8 + 2 * j], v[h * 8 + 2 * j + 1]), f);
                if (rrow) f = add_f32x2(f, pack_f32x2(ru[j] << 16, ru[j] & 0xffff0000u));
                if constexpr (ACT == 3) {
                    const float2 sl = __ldg(reinterpret_cast<const float2*>(a.bias + a.K + kk) + j);   // slopes follow the biases
                    o[j] = to_bf16x2_act<ACT>(f, sl.x, sl.y);
                } else {
                    o[j] = to_bf16x2_act<ACT>(f);
                }
            }
            *reinterpret_cast<uint4*>(yrow + kk) = make_uint4(o[0], o[1], o[2], o[3]);
        }
    }
}

template <int ACT>
__device__ __forceinline__ void epilogue_columns(const ConvArgs& a, uint32_t lane_addr, int n0, bool row_valid, __nv_bfloat16* yrow,
                                                 const __nv_bfloat16* rrow, const float* part, size_t tile_floats,
                                                 const float* s_bias) {
    int cb = 0;
    for (; cb < a.BN; cb += 16)
        epilogue_chunk<16, ACT>(a, lane_addr, cb, n0, row_valid, yrow, rrow, part, tile_floats, s_bias);
}

// Epilogue, run by warps 0-3 (thread t owns accumulator lane t = tile row t): wait for the
// accumulator, optionally meet the other split-K CTAs of the tile in the workspace, then
// bias + residual + activation and bf16 stores into the output channel slice.  (Staging the bf16
// tile in shared memory for row-contiguous stores was measured slower: the epilogue is bound by its
// instruction count, not by the scattered 16-byte stores.)
__device__ __forceinline__ void epilogue(const ConvArgs& a, uint32_t tmem_base, bool ok, int m0, int n0, uint32_t tile, uint32_t split,
                                     const float* s_bias, uint64_t* s_accum_p, volatile uint32_t* s_abort_p, uint32_t* s_is_last_p,
                                     uint32_t accum_parity = 0u) {
    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int m = m0 + tid;
    const bool row_valid = m < a.M;
    if (ok) ok = mbar_wait(smem_u32(s_accum_p), accum_parity, s_abort_p, a.err_flag, 3u);
    ok = __all_sync(0xffffffffu, ok);   // tcgen05.ld below is warp-collective
    if (tid == 0) PB_T(5);
    tcgen05_fence_after();
    const uint32_t lane_addr = tmem_base + ((uint32_t)(warp * 32) << 16);
    // Partial tiles in the workspace are stored [BN/4][128 rows] x float4, so consecutive lanes
    // (= rows) touch consecutive 16-byte words.
    const size_t tile_floats = (size_t)kBM * a.BN;
    bool finalize = ok;
    if (a.splits > 1) {
        // Park this CTA's partial tile; the CTA that arrives last on the tile's counter adds the
        // others to its own accumulators and runs the epilogue.
        float4* mine = reinterpret_cast<float4*>(a.ws + ((size_t)tile * a.splits + split) * tile_floats) + tid;
        if (ok) {
            for (int cb = 0; cb < a.BN; cb += 16) {
                uint32_t v[16];
                tcgen05_ld16(lane_addr + (uint32_t)cb, v);
                tcgen05_wait_ld();
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    mine[(size_t)(cb / 4 + j) * kBM] = make_float4(__uint_as_float(v[4 * j]), __uint_as_float(v[4 * j + 1]),
                                                                    __uint_as_float(v[4 * j + 2]), __uint_as_float(v[4 * j + 3]));
            }
        }
        __threadfence();
        asm volatile("bar.sync 1, 128;" ::: "memory");          // the four epilogue warps only
        if (tid == 0) {
            const unsigned prev = atomicAdd(a.counters + tile, 1u);
            const bool last = prev == (unsigned)a.splits - 1u;
            if (last) a.counters[tile] = 0;                      // ready for the next launch
            __threadfence();
            *s_is_last_p = last ? 1u : 0u;
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        finalize = ok && *s_is_last_p != 0;
    }
    if (finalize) {
        __nv_bfloat16* yrow = a.y + (size_t)m * a.Ks + a.out_c_off;
        const __nv_bfloat16* rrow = a.residual ? a.residual + (size_t)m * a.res_Cs : nullptr;
        const float* part = a.splits > 1 ? a.ws + (size_t)tile * a.splits * tile_floats : nullptr;
        if (a.act == 3) epilogue_columns<3>(a, lane_addr, n0, row_valid, yrow, rrow, part, tile_floats, s_bias);
        else if (a.act == 1) epilogue_columns<1>(a, lane_addr, n0, row_valid, yrow, rrow, part, tile_floats, s_bias);
        else if (a.act == 2) epilogue_columns<2>(a, lane_addr, n0, row_valid, yrow, rrow, part, tile_floats, s_bias);
        else epilogue_columns<0>(a, lane_addr, n0, row_valid, yrow, rrow, part, tile_floats, s_bias);
    }
}

template <int kStages>
__global__ void __launch_bounds__(kThreads, 1)
conv_umma_gather_kernel(const __grid_constant__ CUtensorMap tmap_w, const ConvArgs a, uint32_t job_id, FinishedBlockNotifier* nf) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t s_full[kStages];
    __shared__ __align__(8) uint64_t s_empty[kStages];
    __shared__ __align__(8) uint64_t s_accum;
    __shared__ uint32_t s_tmem_base;
    __shared__ volatile uint32_t s_abort;
    __shared__ uint32_t s_is_last;
    __shared__ __align__(16) float s_bias[128];
    constexpr int kLag = PB_LAG_OF(kStages);

    resolve_slot(job_id, nf);
    if (nf) nf->start(job_id);
    if (threadIdx.x == 0) PB_T(0);

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t stage_bytes = (uint32_t)kATileBytes + a.b_stage_bytes;

    const int m0 = blockIdx.x * kBM;
    const int n0 = blockIdx.y * a.BN;
    const int kb_begin = blockIdx.z * a.kb_per_split;
    const int kb_end = min(a.nkb, kb_begin + a.kb_per_split);
    const int nkb = kb_end - kb_begin;          // >= 1 by construction of the grid

    if (tid == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(smem_u32(&s_full[s]), 4);      // one arrival per producer warp
            mbar_init(smem_u32(&s_empty[s]), 1);
        }
        mbar_init(smem_u32(&s_accum), 1);
        s_abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (tid < 128) {
        const int k = n0 + tid;
        s_bias[tid] = (a.bias && tid < a.BN && k < a.K) ? __ldg(a.bias + k) : 0.f;
    }
    if (warp == 4) {
        tcgen05_alloc(smem_u32(&s_tmem_base), a.tmem_cols);
        tcgen05_relinquish();
    }

    // A-gather geometry.  Eight consecutive lanes cover the eight 16-byte chunks of one 128-byte tile
    // row, so one warp-wide cp.async touches 4 rows = 4 full 128-byte lines of the activation tensor
    // (when a row's chunks share a filter tap) instead of 32 partial ones.  Thread t copies chunk
    // t%8 of rows t/8 + 16*i, i = 0..7.
    const int chunk = tid & 7;
    const int rbase = (tid >> 3) & 15;
    int ih0[8], iw0[8];
    if (warp < 4) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int m = m0 + rbase + 16 * i;
            if (m < a.M) {
                const int p = m / a.Q, q = m - p * a.Q;
                ih0[i] = p * a.sh - a.ph;
                iw0[i] = q * a.sw - a.pw;
            } else {
                ih0[i] = -(1 << 28);      // fails every bounds check: the row is zero-filled
                iw0[i] = 0;
            }
        }
    }

    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = s_tmem_base;
    if (threadIdx.x == 0) PB_T(1);

    if (warp < 4) {
        // ===== A producer =====
        // position of this thread's chunk in k: filter tap (r, s) and first channel c
        const int kk0 = kb_begin * kBK + chunk * 8;
        int tap = kk0 / a.Cp;
        int c = kk0 - tap * a.Cp;
        int r = tap / a.S, s = tap - r * a.S;
        const uint32_t dst_off = (uint32_t)rbase * 128u + (((uint32_t)chunk ^ (uint32_t)(rbase & 7)) << 4);
        bool ok = true;
        for (int kb = 0; kb < nkb; ++kb) {
            const int st = kb % kStages;
            const uint32_t use = (uint32_t)(kb / kStages);
            if (ok) ok = mbar_wait(smem_u32(&s_empty[st]), (use & 1u) ^ 1u, &s_abort, a.err_flag, 1u);
            const uint32_t a_tile = smem_base + (uint32_t)st * stage_bytes;
            if (ok) {
                if (tid == 0) {
                    mbar_expect_tx(smem_u32(&s_full[st]), a.b_stage_bytes);
                    tma_load_2d(a_tile + kATileBytes, &tmap_w, (kb_begin + kb) * kBK, n0, smem_u32(&s_full[st]));
                }
                const bool tap_ok = tap < a.taps && c < a.Cs;
                const __nv_bfloat16* xc = a.x + c;
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const int ih = ih0[i] + r * a.dh, iw = iw0[i] + s * a.dw;
                    const bool inb = tap_ok && ih >= 0 && ih < a.H && iw >= 0 && iw < a.W;
                    const __nv_bfloat16* src = inb ? xc + ((size_t)ih * a.W + iw) * a.Cs : a.x;
                    cp_async_16(a_tile + dst_off + (uint32_t)i * 2048u, src, inb ? 16u : 0u);
                }
                c += kBK;
                while (c >= a.Cp) {
                    c -= a.Cp; ++tap; ++s;
                    if (s == a.S) { s = 0; ++r; }
                }
            }
            cp_async_commit();
            if (kb == 0 && tid == 0) PB_T(2);
            // One arrival per warp: 128 threads arriving on the same shared-memory word serialise
            // (measured: ~0.2 us per k-block); every lane first makes its own copies visible to the
            // async proxy, the warp converges, one lane arrives.
            if (kb >= kLag) {
                cp_async_wait<kLag>();
                fence_proxy_async();
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&s_full[(kb - kLag) % kStages]));
            }
        }
        // drain: the last kLag k-blocks
        cp_async_wait<0>();
        fence_proxy_async();
        __syncwarp();
        if (lane == 0)
            for (int kb = (nkb > kLag ? nkb - kLag : 0); kb < nkb; ++kb) mbar_arrive(smem_u32(&s_full[kb % kStages]));

        // ===== epilogue: accumulator lane `tid` = tile row `tid` =====
        epilogue(a, tmem_base, ok, m0, n0, blockIdx.y * gridDim.x + blockIdx.x, blockIdx.z, s_bias, &s_accum, &s_abort, &s_is_last);
        if (tid == 0) PB_T(6);
    } else {
        // ===== MMA issuer: one thread =====
        if (lane == 0) {
            bool ok = true;
            for (int kb = 0; kb < nkb && ok; ++kb) {
                const int st = kb % kStages;
                const uint32_t use = (uint32_t)(kb / kStages);
                ok = mbar_wait(smem_u32(&s_full[st]), use & 1u, &s_abort, a.err_flag, 2u);
                if (!ok) break;
                if (kb == 0) PB_T(3);
                tcgen05_fence_after();
                const uint32_t a_tile = smem_base + (uint32_t)st * stage_bytes;
                const uint32_t b_tile = a_tile + kATileBytes;
#pragma unroll
                for (int k = 0; k < kBK / 16; ++k) {
                    tcgen05_mma_bf16(tmem_base, umma_desc_sw128(a_tile + k * 32), umma_desc_sw128(b_tile + k * 32), a.idesc,
                                     (kb > 0 || k > 0) ? 1u : 0u);
                }
                tcgen05_commit(smem_u32(&s_empty[st]));   // frees the stage once these MMAs have read it
            }
            if (ok) tcgen05_commit(smem_u32(&s_accum));   // accumulator complete
            PB_T(4);
        }
        __syncwarp();
    }

    tcgen05_fence_before();
    __syncthreads();
    if (s_abort) {
        // Let copies that may still be in flight land before shared memory is released.
        const unsigned long long t0 = globaltimer_ns();
        for (uint32_t i = 0; i < (1u << 20); ++i) {
            if (globaltimer_ns() - t0 > 50000ull) break;
        }
        __syncthreads();
    }
    if (warp == 4) {
        tcgen05_fence_after();
        tcgen05_dealloc(tmem_base, a.tmem_cols);
    }
    if (threadIdx.x == 0) PB_T(7);
    if (nf) nf->end(job_id);
}

// ---- the kernel, operand A by im2col TMA ---------------------------------------------------------
// CTA = 6 warps.  Warp 4: one thread issues, per k-block, one im2col TMA for A (128 output pixels x
// 64 channels of one filter tap) and one tiled TMA for B.  Warp 5: allocates TMEM, one thread issues
// the MMAs.  Warps 0-3 only run the epilogue.  No thread computes an address in the main loop.
constexpr int kThreadsTma = 192;

// One CTA's share of one convolution: output tile (bx, by) of a grid gx tiles wide, reduction
// slice bz, `stages` pipeline buffers.  Shared by the single-convolution kernel and the grouped one.
__device__ __forceinline__ void conv_tile_tma(const CUtensorMap* tmap_w, const CUtensorMap* tmap_x, const ConvArgs& a, const int stages,
                                              const int bx, const int by, const int bz, const int gx, uint8_t* smem_raw,
                                              uint64_t* s_full, uint64_t* s_empty, uint64_t* s_accum, uint32_t* s_tmem_base,
                                              volatile uint32_t* s_abort, uint32_t* s_is_last, float* s_bias) {
    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;
#ifdef PB_CONV_STATS
    __shared__ long long s_clk[8];
    __shared__ unsigned s_smid;
    __shared__ unsigned long long s_ns0;
    if (tid == 0) {
        PB_S(0);
        s_ns0 = globaltimer_ns();
        unsigned smid;
        asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
        s_smid = smid & 255u;
        const unsigned others = atomicAdd(&g_conv_resident[s_smid], 1u);
        atomicAdd(&g_conv_stats[10 + (others < 5 ? others : 5)], 1ull);
    }
#endif
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t stage_bytes = (uint32_t)kATileBytes + a.b_stage_bytes;

    const int m0 = bx * kBM;
    const int n0 = by * a.BN;
    const int kb_begin = bz * a.kb_per_split;
    const int kb_end = min(a.nkb, kb_begin + a.kb_per_split);
    const int nkb = kb_end - kb_begin;

    // the first copy of each descriptor otherwise pays its fetch into the descriptor cache
    if (tid == 32) asm volatile("prefetch.tensormap [%0];" ::"l"(tmap_w) : "memory");
    if (tid == 64) asm volatile("prefetch.tensormap [%0];" ::"l"(tmap_x) : "memory");
    if (tid == 0) {
        for (int s = 0; s < stages; ++s) {
            mbar_init(smem_u32(&s_full[s]), 1);      // the producer's arrive.expect_tx
            mbar_init(smem_u32(&s_empty[s]), 1);     // tcgen05.commit
        }
        mbar_init(smem_u32(s_accum), 1);
        *s_abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    for (int j = tid; j < a.BN; j += kThreadsTma) {
        const int k = n0 + j;
        s_bias[j] = (a.bias && k < a.K) ? __ldg(a.bias + k) : 0.f;
    }
    if (warp == 5) {
        tcgen05_alloc(smem_u32(s_tmem_base), a.tmem_cols);
        tcgen05_relinquish();
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *s_tmem_base;
    if (threadIdx.x == 0) { PB_T(1); PB_S(1); }
    // Everything above touched only this CTA's shared/tensor memory and constant weights (bias), so it
    // may overlap the previous kernel's tail.  Activations, the residual, the output and the split-K
    // workspace may only be touched once the previous kernel has completed.
    griddep_wait();
    if (threadIdx.x == 0) PB_S(2);

    // ===== producers: lane 0 of warp 4 and of the four epilogue warps =====
    // A thread that issues tensor copies one after the other is slow however small the copies: measured with a
    // copy-only kernel on tiles like these, one thread sustains one 16 KB copy per ~650 clocks (25 B/clk) at any
    // pipeline depth, four issuing warps of the same CTA 100 B/clk, and the whole GPU saturates near 60 B/clk per
    // SM.  The tensor cores need a k-block (two copies) every ~270 clocks, so a lone producer thread paced the
    // whole CTA.  The epilogue warps have nothing to do until the accumulator is complete, so lane 0 of each
    // joins warp 4: the 2 x stages (stage, operand) pairs are dealt round-robin to the kProducers threads, and a
    // pair is always refilled by the same thread, in k order.  The thread that loads operand A also arms the
    // stage's barrier with the byte count of both copies; operand B's bytes may land before that (the
    // transaction count goes negative for a moment; the phase cannot complete before the arrival).
    // (Several lanes of ONE warp would not do: they reconverge after each wait, so no copy could be issued
    // before every stage had been drained.)
    constexpr int kProducers = 5;
    const int prod = warp == 4 ? 0 : warp + 1;              // producer index of this warp's lane 0
    if (warp <= 4 && lane == 0) {
        const int img = m0 / a.PQ, rem = m0 - img * a.PQ;      // the tile may run on into the next image
        const int p0 = rem / a.Q, q0 = rem - p0 * a.Q;
        const int w0 = q0 * a.sw - a.pw;          // filter-window origin of the tile's first pixel
        const int h0 = p0 * a.sh - a.ph;
        const int cpt = a.Cp / kBK;               // k-blocks per filter tap
        bool ok = true;
        int st = 0;
        uint32_t parity = 1u;                     // a fresh barrier passes a wait on the "previous" phase
        // which (stage, operand) pairs are this thread's (bit st), and the filter tap / channel chunk of the k-block,
        // carried along: a division per k-block is a tenth of what the thread has per copy
        uint32_t mask_a = 0, mask_b = 0;
        for (int q = 0; q < stages; ++q) {
            if ((q * 2) % kProducers == prod) mask_a |= 1u << q;
            if ((q * 2 + 1) % kProducers == prod) mask_b |= 1u << q;
        }
        int tap = kb_begin / cpt, chunk = kb_begin - tap * cpt;
        int r = tap / a.S, s = tap - r * a.S;
        uint32_t* const err_flag = a.err_flag;
        for (int kb = 0; kb < nkb && ok; ++kb) {
            const bool mine_a = (mask_a >> st) & 1u, mine_b = (mask_b >> st) & 1u;
            if (mine_a || mine_b) {
                ok = mbar_wait(smem_u32(&s_empty[st]), parity, s_abort, err_flag, 1u);
                if (!ok) break;
                const uint32_t a_tile = smem_base + (uint32_t)st * stage_bytes;
                const uint32_t bar = smem_u32(&s_full[st]);
                const int kbg = kb_begin + kb;
                if (mine_a) {
                    mbar_arrive_expect_tx(bar, (uint32_t)kATileBytes + a.b_stage_bytes);
                    if (a.a_tiled) tma_load_2d(a_tile, tmap_x, chunk * kBK, m0, bar);
                    else tma_load_im2col_4d(a_tile, tmap_x, chunk * kBK, w0, h0, img, (uint16_t)(s * a.dw), (uint16_t)(r * a.dh), bar);
                    if (kb == 0) PB_T(2);
                    PB_TK(kb, 0);
                }
                if (mine_b) tma_load_2d(a_tile + kATileBytes, tmap_w, kbg * kBK, n0, bar);
            }
            if (++chunk == cpt) {
                chunk = 0;
                if (++s == a.S) { s = 0; ++r; }
            }
            if (++st == stages) { st = 0; parity ^= 1u; }
        }
    }
    if (warp <= 4) __syncwarp();

    if (warp < 4) {
        griddep_launch();      // the next kernel's blocks may be scheduled as SM resources free up
        epilogue(a, tmem_base, true, m0, n0, (uint32_t)(by * gx + bx), (uint32_t)bz, s_bias, s_accum, s_abort, s_is_last);
        if (tid == 0) { PB_T(6); PB_S(6); }
    } else if (warp == 4) {
        __syncwarp();
        griddep_launch();
    } else {
        // ===== MMA issuer: one thread =====
        // This thread's own instruction chain per k-block paces the CTA (measured: four MMA issues + commit ~320
        // clocks, most of it the tensor cores taking the instructions, then ~400 clocks until the next k-block's
        // barrier had been looked at; an mbarrier wait costs ~170 clocks even when its phase is long complete).
        // So the NEXT k-block's barrier is probed (test_wait, never blocks) before this k-block's MMAs are issued:
        // the probe's latency runs under them; and the descriptors are stage 0's plus a stride.
        if (lane == 0) {
            uint32_t st = 0, parity = 0u;
            bool ok = true, have_next = false;
            uint32_t* const err_flag = a.err_flag;
            const uint32_t idesc = a.idesc;
            const uint64_t desc_a0 = umma_desc_sw128(smem_base), desc_b0 = umma_desc_sw128(smem_base + kATileBytes);
            const uint64_t desc_step = (uint64_t)(stage_bytes >> 4);      // address field counts 16-byte units; no carry out of its 14 bits
            for (int kb = 0; kb < nkb; ++kb) {
                if (!have_next) {
                    ok = mbar_wait(smem_u32(&s_full[st]), parity, s_abort, err_flag, 2u);
                    if (!ok) break;
                }
                if (kb == 0) { PB_T(3); PB_S(3); }
                PB_TK(kb, 1);
                tcgen05_fence_after();
                uint32_t st_n = st + 1, parity_n = parity;
                if (st_n == (uint32_t)stages) { st_n = 0; parity_n ^= 1u; }
                have_next = kb + 1 < nkb && mbar_test_wait(smem_u32(&s_full[st_n]), parity_n);
                const uint64_t da = desc_a0 + (uint64_t)st * desc_step, db = desc_b0 + (uint64_t)st * desc_step;
#pragma unroll
                for (int k = 0; k < kBK / 16; ++k)
                    tcgen05_mma_bf16(tmem_base, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, (kb > 0 || k > 0) ? 1u : 0u);   // +32 bytes per K=16 slice
                tcgen05_commit(smem_u32(&s_empty[st]));
                PB_TK(kb, 2);
                st = st_n;
                parity = parity_n;
            }
            PB_S(4);
            if (ok) tcgen05_commit(smem_u32(s_accum));
            PB_T(4);
#ifdef PB_CONV_STATS
            if (ok) mbar_wait(smem_u32(s_accum), 0u, s_abort, a.err_flag, 3u);
            PB_S(5);
#endif
        }
        __syncwarp();
        griddep_launch();
    }

    tcgen05_fence_before();
    __syncthreads();
    if (*s_abort) {
        const unsigned long long t0 = globaltimer_ns();
        for (uint32_t i = 0; i < (1u << 20); ++i) {
            if (globaltimer_ns() - t0 > 50000ull) break;
        }
        __syncthreads();
    }
    if (warp == 5) {
        tcgen05_fence_after();
        tcgen05_dealloc(tmem_base, a.tmem_cols);
    }
    if (threadIdx.x == 0) PB_T(7);
#ifdef PB_CONV_STATS
    __syncthreads();
    if (threadIdx.x == 0) {
        const long long c7 = clock64();
        atomicAdd(&g_conv_stats[0], 1ull);
        atomicAdd(&g_conv_stats[1], (unsigned long long)nkb);
        for (int i = 0; i < 6; ++i) atomicAdd(&g_conv_stats[2 + i], (unsigned long long)(s_clk[i + 1] - s_clk[i]));
        atomicAdd(&g_conv_stats[8], (unsigned long long)(c7 - s_clk[6]));
        atomicAdd(&g_conv_stats[9], (unsigned long long)(c7 - s_clk[0]));
        atomicSub(&g_conv_resident[s_smid], 1u);
        atomicAdd(&g_conv_ns, globaltimer_ns() - s_ns0);
    }
#endif
}

__global__ void __launch_bounds__(kThreadsTma, 3)
conv_umma_tma_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x, const ConvArgs a,
                     int stages, uint32_t job_id, FinishedBlockNotifier* nf) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t s_full[kMaxStages];
    __shared__ __align__(8) uint64_t s_empty[kMaxStages];
    __shared__ __align__(8) uint64_t s_accum;
    __shared__ uint32_t s_tmem_base;
    __shared__ volatile uint32_t s_abort;
    __shared__ uint32_t s_is_last;
    __shared__ __align__(16) float s_bias[kMaxBN];

    resolve_slot(job_id, nf);
    if (nf) nf->start(job_id);
    if (threadIdx.x == 0) PB_T(0);
    conv_tile_tma(&tmap_w, &tmap_x, a, stages, (int)blockIdx.x, (int)blockIdx.y, (int)blockIdx.z, (int)gridDim.x, smem_raw, s_full,
                  s_empty, &s_accum, &s_tmem_base, &s_abort, &s_is_last, s_bias);
    if (nf) nf->end(job_id);
}

// Grouped launch: several independent convolutions (the parallel branches of an Inception block at the
// same depth, a ResNet block's shortcut beside its first convolution) in ONE grid.  Kernel-level
// concurrency on a GPU is capped by its hardware queues, and a batch-1 convolution rarely has more
// than a dozen tiles, so running the branches side by side in one launch is what fills the SMs.
// Block b belongs to the sub-problem i with first_block[i] <= b < first_block[i + 1]; the table with
// each sub-problem's tensor maps and arguments lives in device memory, written once per instance.
// A 3x3 pooling layer of the same dependence depth can ride along as one more entry (stages == kSubPool): its blocks
// run pool_sub_block() instead of a convolution tile.  Why it was tried: under serving load every launch of a request's
// chain waits about 45 us for SM resources behind the other requests' CTAs, whatever its own size, so the 13 pooling
// launches of an Inception-v3 request cost 20 % of the throughput although they are 6 % of a lone request's time.
// What came of it: see PB_FUSE_POOLS where the launches are planned (off by default).
struct PoolSubArgs {
    const __nv_bfloat16* x;
    __nv_bfloat16* y;
    int C, H, W, Cs, P, Q, Ks, out_c_off;
    int sh, sw, ph, pw;
    int is_max, count_pad, batch, reserved;
};
struct alignas(128) SubConv {
    CUtensorMap tmap_w;
    CUtensorMap tmap_x;
    union {
        ConvArgs a;
        PoolSubArgs pool;
    };
    uint32_t first_block, gx, gy, stages;
};
static_assert(sizeof(PoolSubArgs) <= sizeof(ConvArgs), "a pooling entry fits where a convolution's arguments are");
constexpr int kMaxSubConvs = 8;
constexpr uint32_t kSubPool = 0xffffffffu;
constexpr int kPoolVecsPerThread = 2;                 // output vectors (8 channels) per thread of a pooling block

// One block's share of a 3x3 pooling layer: thread t takes output vectors base + t and base + 192 + t.  All nine
// loads of a window are issued before the first use (addresses clamped into the tensor, taps outside dropped
// afterwards).  Arithmetic and its order are those of pool_kernel / window3_strip_kernel (rows, then columns, fp32
// sums from +0, IEEE division; fmaxf from -inf), so the bits are theirs.
__device__ __forceinline__ void pool_sub_block(const PoolSubArgs& a, uint32_t local_block) {
    const int cv = a.Cs >> 3;
    const long long total = (long long)a.batch * a.P * a.Q * cv;
    const long long base = (long long)local_block * (kThreadsTma * kPoolVecsPerThread) + threadIdx.x;
#pragma unroll 1
    for (int u = 0; u < kPoolVecsPerThread; ++u) {
        const long long idx = base + (long long)u * kThreadsTma;
        if (idx >= total) break;
        const int c0 = (int)(idx % cv) * 8;
        long long pix = idx / cv;
        const int q = (int)(pix % a.Q);
        pix /= a.Q;
        const int p = (int)(pix % a.P), img = (int)(pix / a.P);
        const __nv_bfloat16* x = a.x + (size_t)img * a.H * a.W * a.Cs + c0;
        uint4 raw[3][3];
        uint32_t ok = 0;
#pragma unroll
        for (int r = 0; r < 3; ++r) {
            const int ih = p * a.sh + r - a.ph;
            const bool row_ok = ih >= 0 && ih < a.H;
            const __nv_bfloat16* xrow = x + (size_t)min(max(ih, 0), a.H - 1) * a.W * a.Cs;
#pragma unroll
            for (int s2 = 0; s2 < 3; ++s2) {
                const int iw = q * a.sw + s2 - a.pw;
                if (row_ok && iw >= 0 && iw < a.W) ok |= 1u << (r * 3 + s2);
                raw[r][s2] = *reinterpret_cast<const uint4*>(xrow + (size_t)min(max(iw, 0), a.W - 1) * a.Cs);
            }
        }
        float acc[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = a.is_max ? -INFINITY : 0.f;
        int cnt = 0;
#pragma unroll
        for (int r = 0; r < 3; ++r)
#pragma unroll
            for (int s2 = 0; s2 < 3; ++s2) {
                if (!((ok >> (r * 3 + s2)) & 1u)) continue;
                const uint32_t w[4] = {raw[r][s2].x, raw[r][s2].y, raw[r][s2].z, raw[r][s2].w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float lo = __uint_as_float(w[j] << 16), hi = __uint_as_float(w[j] & 0xffff0000u);
                    acc[2 * j] = a.is_max ? fmaxf(acc[2 * j], lo) : acc[2 * j] + lo;
                    acc[2 * j + 1] = a.is_max ? fmaxf(acc[2 * j + 1], hi) : acc[2 * j + 1] + hi;
                }
                ++cnt;
            }
        const float div = a.count_pad ? 9.f : (float)(cnt > 0 ? cnt : 1);
        uint32_t o[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            float v0 = a.is_max ? acc[2 * j] : acc[2 * j] / div, v1 = a.is_max ? acc[2 * j + 1] : acc[2 * j + 1] / div;
            if (c0 + 2 * j >= a.C) v0 = 0.f;
            if (c0 + 2 * j + 1 >= a.C) v1 = 0.f;
            const __nv_bfloat162 h = __floats2bfloat162_rn(v0, v1);
            o[j] = *reinterpret_cast<const uint32_t*>(&h);
        }
        __nv_bfloat16* y = a.y + (((size_t)img * a.P + p) * a.Q + q) * a.Ks + a.out_c_off + c0;
        *reinterpret_cast<uint4*>(y) = make_uint4(o[0], o[1], o[2], o[3]);
    }
}

__global__ void __launch_bounds__(kThreadsTma, 3)
conv_umma_multi_kernel(const SubConv* __restrict__ table, int n_sub, uint32_t job_id, FinishedBlockNotifier* nf) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t s_full[kMaxStages];
    __shared__ __align__(8) uint64_t s_empty[kMaxStages];
    __shared__ __align__(8) uint64_t s_accum;
    __shared__ uint32_t s_tmem_base;
    __shared__ volatile uint32_t s_abort;
    __shared__ uint32_t s_is_last;
    __shared__ __align__(16) float s_bias[kMaxBN];
    __shared__ __align__(16) ConvArgs s_args;

    resolve_slot(job_id, nf);
    if (nf) nf->start(job_id);
    if (threadIdx.x == 0) PB_T(0);

    int sub = 0;
    while (sub + 1 < n_sub && blockIdx.x >= table[sub + 1].first_block) ++sub;
    const SubConv* sc = table + sub;
    // the table is constant for the life of the instance: it may be read before griddepcontrol.wait
    static_assert(sizeof(ConvArgs) % 4 == 0, "ConvArgs is copied word by word");
    if (threadIdx.x < sizeof(ConvArgs) / 4)
        reinterpret_cast<uint32_t*>(&s_args)[threadIdx.x] = reinterpret_cast<const uint32_t*>(&sc->a)[threadIdx.x];
    __syncthreads();
    const uint32_t local = blockIdx.x - sc->first_block;
    if (sc->stages == kSubPool) {        // a pooling layer riding along: no tensor memory, no pipeline
        griddep_wait();
        griddep_launch();
        pool_sub_block(*reinterpret_cast<const PoolSubArgs*>(&s_args), local);
        if (nf) nf->end(job_id);
        return;
    }
    const uint32_t gx = sc->gx, gy = sc->gy;
    const uint32_t bx = local % gx, rest = local / gx;
    const uint32_t by = rest % gy, bz = rest / gy;
    conv_tile_tma(&sc->tmap_w, &sc->tmap_x, s_args, (int)sc->stages, (int)bx, (int)by, (int)bz, (int)gx, smem_raw, s_full, s_empty,
                  &s_accum, &s_tmem_base, &s_abort, &s_is_last, s_bias);
    if (nf) nf->end(job_id);
}


// ---- persistent form: a CTA walks several tiles ------------------------------------------------------------
// What a one-tile CTA costs besides its main loop was measured under serving load (cycle stamps summed over all
// CTAs): 1.0 us of set-up, 1.4 us until the first operands land, 0.2 us of accumulator drain, 1.4 us of epilogue,
// 0.35 us of tear-down and about 1 us before the SM slot holds the next CTA, against 4.7 us of main loop; and the
// GPU's throughput on these layers is what its CTA slots turn over.  Here a CTA is given several tiles of the
// launch (tile t = blockIdx.x, + gridDim.x, ...) and pays set-up and tear-down once; the producers run on
// into the next tile's k-blocks while the current tile finishes, so operand latency is paid once per CTA; and
// there are TWO accumulators in tensor memory, so the epilogue of tile i (warps 0-3) runs under the MMAs of tile
// i + 1 (warp 4).  9 warps: 0-3 epilogue, 4 TMEM allocation + MMA issue, 5-8 producers (a thread that issues
// tensor copies back to back sustains only one copy per ~500 clocks - ~170 for the wait on the stage's barrier,
// ~250 for the copy instruction itself - so the 2 x stages (stage, operand) pairs are dealt to four threads; a
// pair is always refilled by the same thread).  Sized for two CTAs per SM: <= 108 KB of pipeline, 288 threads
// of <= 112 registers, 2 x 128 tensor-memory columns.
// Every tile comes from the launch's table of sub-problems (one entry for a lone convolution, several for the
// independent convolutions of a grouped launch): tile index -> entry by first_block, then (m tile, n tile,
// k split) inside it.
constexpr int kPersistProducers = 4;
constexpr int kThreadsPersist = 32 * (5 + kPersistProducers);
#ifndef PB_CONV_PERSIST_SMEM_KB
#define PB_CONV_PERSIST_SMEM_KB 108
#endif
constexpr uint32_t kSmemBudgetPersist = PB_CONV_PERSIST_SMEM_KB * 1024u;

// A sub-problem's arguments as the CTA keeps them in shared memory (the tensor maps stay in global memory,
// where the TMA unit reads them): decoding a tile and reading its arguments from the global table cost every
// role a chain of dependent loads at each tile boundary, about 5 us per tile.
struct SubArgs {
    ConvArgs a;
    uint32_t first_block, gx, gy, pad;
};
struct TileRef {
    const SubArgs* sa;
    const SubConv* sc;
    int bx, by, bz;
};
__device__ __forceinline__ TileRef tile_ref(const SubConv* __restrict__ table, const SubArgs* s_sub, int n_sub, uint32_t t) {
    int sub = 0;
    while (sub + 1 < n_sub && t >= s_sub[sub + 1].first_block) ++sub;
    TileRef r;
    r.sa = s_sub + sub;
    r.sc = table + sub;
    const uint32_t local = t - r.sa->first_block;
    const uint32_t gx = r.sa->gx, gy = r.sa->gy;
    r.bx = (int)(local % gx);
    const uint32_t rest = local / gx;
    r.by = (int)(rest % gy);
    r.bz = (int)(rest / gy);
    return r;
}

__global__ void __launch_bounds__(kThreadsPersist, 2)
conv_umma_persist_kernel(const SubConv* __restrict__ table, int n_sub, uint32_t total_tiles, int stages, uint32_t stage_bytes,
                         uint32_t acc_cols, uint32_t job_id, FinishedBlockNotifier* nf) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t s_full[kMaxStages];
    __shared__ __align__(8) uint64_t s_empty[kMaxStages];
    __shared__ __align__(8) uint64_t s_tfull[2];       // accumulator complete (tcgen05.commit)
    __shared__ __align__(8) uint64_t s_tempty[2];      // accumulator read out (one arrival per epilogue warp)
    __shared__ uint32_t s_tmem_base;
    __shared__ volatile uint32_t s_abort;
    __shared__ uint32_t s_is_last;
    __shared__ __align__(16) float s_bias[2][kMaxBN];
    __shared__ __align__(16) SubArgs s_sub[kMaxSubConvs];

    resolve_slot(job_id, nf);
    if (nf) nf->start(job_id);

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
#ifdef PB_CONV_STATS
    __shared__ long long s_cta_t0;
    if (tid == 0) {
        const unsigned others = atomicAdd(&g_persist_resident, 1u);
        atomicAdd(&g_persist_hist[others / 32u < 14u ? others / 32u : 14u], 1ull);
        s_cta_t0 = clock64();
    }
#endif

    // the table is constant for the life of the instance: it may be read before griddepcontrol.wait
    {
        static_assert(sizeof(ConvArgs) % 4 == 0 && sizeof(SubArgs) % 4 == 0, "copied word by word");
        constexpr int kWords = (int)(sizeof(ConvArgs) / 4);
        for (int j = tid; j < n_sub * (kWords + 3); j += kThreadsPersist) {
            const int sub = j / (kWords + 3), w = j - sub * (kWords + 3);
            if (w < kWords) reinterpret_cast<uint32_t*>(&s_sub[sub].a)[w] = reinterpret_cast<const uint32_t*>(&table[sub].a)[w];
            else (&s_sub[sub].first_block)[w - kWords] = (&table[sub].first_block)[w - kWords];
        }
    }

    if (tid == 0) {
        for (int s = 0; s < stages; ++s) {
            mbar_init(smem_u32(&s_full[s]), 1);
            mbar_init(smem_u32(&s_empty[s]), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(smem_u32(&s_tfull[b]), 1);
            mbar_init(smem_u32(&s_tempty[b]), 4);
        }
        s_abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 4) {
        tcgen05_alloc(smem_u32(&s_tmem_base), 2u * acc_cols);
        tcgen05_relinquish();
    }
    // the first tile's descriptors: their fetch into the descriptor cache overlaps the rest of the set-up
    if (warp >= 5 && warp <= 6 && lane == 0) {
        int sub = 0;
        while (sub + 1 < n_sub && blockIdx.x >= table[sub + 1].first_block) ++sub;
        asm volatile("prefetch.tensormap [%0];" ::"l"(warp == 5 ? &table[sub].tmap_x : &table[sub].tmap_w) : "memory");
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = s_tmem_base;
    // Nothing above touched activations, the output or the split-K workspace: it may overlap the previous
    // kernel's tail.  From here on this kernel reads what the previous one wrote.
    griddep_wait();

    if (warp < 4) {
        // ===== epilogue warps: thread t owns accumulator lane t = tile row t =====
        uint32_t i = 0;
        for (uint32_t t = blockIdx.x; t < total_tiles; t += gridDim.x, ++i) {
            const uint32_t acc = i & 1u, use = i >> 1;
            const TileRef tr = tile_ref(table, s_sub, n_sub, t);
            const ConvArgs& a = tr.sa->a;
            // the tile's biases, staged by these four warps for themselves
            asm volatile("bar.sync 1, 128;" ::: "memory");      // the tile that used this buffer before is done with it
            const int n0 = tr.by * a.BN;
            for (int j = tid; j < a.BN; j += 128) {
                const int k = n0 + j;
                s_bias[acc][j] = (a.bias && k < a.K) ? __ldg(a.bias + k) : 0.f;
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (tid == 0) PB_PT(i, 2);
            epilogue(a, tmem_base + acc * acc_cols, true, tr.bx * kBM, n0, (uint32_t)(tr.by * (int)tr.sa->gx + tr.bx), (uint32_t)tr.bz,
                     s_bias[acc], &s_tfull[acc], &s_abort, &s_is_last, use & 1u);
            if (tid == 0) PB_PT(i, 3);
            // this accumulator may be overwritten: every tcgen05.ld of the warp has completed (wait::ld)
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&s_tempty[acc]));
        }
    } else if (warp == 4) {
        // ===== MMA issuer: one thread =====
        // The thread's own instruction chain per k-block decides the pace of the CTA (measured: four MMA issues +
        // commit 360 clocks, most of it the tensor cores taking the instructions; then 415 clocks until the next
        // k-block's barrier had been looked at: a division for the stage index, a load of the error-flag pointer, and
        // an mbarrier wait that costs ~170 clocks even when the phase is long complete).  So: stage and parity are
        // carried, not divided; and the NEXT k-block's barrier is probed (test_wait, never blocks) before this
        // k-block's MMAs are issued, so the probe's latency runs under them.
        if (lane == 0) {
            uint32_t i = 0;                         // tiles of this CTA so far
            uint32_t st = 0, parity = 0;            // pipeline stage and phase of the next k-block
            bool ok = true;
            uint32_t* const err_flag = s_sub[0].a.err_flag;
            // descriptors of stage 0; stage q is stage_bytes further on (the address field counts 16-byte units and
            // cannot carry out of its 14 bits: shared memory ends below 256 KB)
            const uint64_t desc_a0 = umma_desc_sw128(smem_base), desc_b0 = umma_desc_sw128(smem_base + kATileBytes);
            const uint64_t desc_step = (uint64_t)(stage_bytes >> 4);
            bool have_next = false;                 // the barrier of (st, parity) is already known to be complete
            for (uint32_t t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, ++i) {
                const uint32_t acc = i & 1u, use = i >> 1;
                const TileRef tr = tile_ref(table, s_sub, n_sub, t);
                const ConvArgs& a = tr.sa->a;
                const int kb_begin = tr.bz * a.kb_per_split;
                const int nkb = min(a.nkb, kb_begin + a.kb_per_split) - kb_begin;
                const uint32_t idesc = a.idesc;
#ifdef PB_CONV_STATS
                const bool first_tile = i == 0;
#endif
                ok = mbar_wait(smem_u32(&s_tempty[acc]), (use & 1u) ^ 1u, &s_abort, err_flag, 4u);
                if (!ok) break;
                PB_PT(i, 0);
                tcgen05_fence_after();
                const uint32_t d_tmem = tmem_base + acc * acc_cols;
                for (int kb = 0; kb < nkb; ++kb) {
                    if (!have_next) {
                        ok = mbar_wait(smem_u32(&s_full[st]), parity, &s_abort, err_flag, 2u);
                        if (!ok) break;
                    }
                    PB_PK(kb, 4);
                    tcgen05_fence_after();
                    // stage of the k-block after this one (of this tile or of the CTA's next tile: the pipeline runs on)
                    uint32_t st_n = st + 1, parity_n = parity;
                    if (st_n == (uint32_t)stages) { st_n = 0; parity_n ^= 1u; }
                    have_next = mbar_test_wait(smem_u32(&s_full[st_n]), parity_n);
                    const uint64_t da = desc_a0 + (uint64_t)st * desc_step, db = desc_b0 + (uint64_t)st * desc_step;
#pragma unroll
                    for (int k = 0; k < kBK / 16; ++k)
                        tcgen05_mma_bf16(d_tmem, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, (kb > 0 || k > 0) ? 1u : 0u);   // +32 bytes per K=16 slice
                    tcgen05_commit(smem_u32(&s_empty[st]));
                    PB_PK(kb, 5);
                    st = st_n;
                    parity = parity_n;
                }
                if (ok) tcgen05_commit(smem_u32(&s_tfull[acc]));
                PB_PT(i, 1);
            }
        }
        __syncwarp();
    } else {
        // ===== producers: lane 0 of warps 5-8 =====
        if (lane == 0) {
            const uint32_t prod = (uint32_t)(warp - 5);
            // which (stage, operand) pairs are this thread's: bit st of mask_a / mask_b (no division in the loop)
            uint32_t mask_a = 0, mask_b = 0;
            for (int q = 0; q < stages; ++q) {
                if ((uint32_t)(q * 2) % kPersistProducers == prod) mask_a |= 1u << q;
                if ((uint32_t)(q * 2 + 1) % kPersistProducers == prod) mask_b |= 1u << q;
            }
            uint32_t st = 0, parity = 1u;           // a fresh barrier passes a wait on the "previous" phase
            bool ok = true;
            uint32_t* const err_flag = s_sub[0].a.err_flag;
            for (uint32_t t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
#ifdef PB_CONV_STATS
                const bool first_tile = t == blockIdx.x;
#endif
                const TileRef tr = tile_ref(table, s_sub, n_sub, t);
                const ConvArgs& a = tr.sa->a;
                const CUtensorMap* tmap_w = &tr.sc->tmap_w;
                const CUtensorMap* tmap_x = &tr.sc->tmap_x;
                const int kb_begin = tr.bz * a.kb_per_split;
                const int nkb = min(a.nkb, kb_begin + a.kb_per_split) - kb_begin;
                const int m0 = tr.bx * kBM, n0 = tr.by * a.BN;
                const int PQ = a.PQ, Q = a.Q;
                const int img = m0 / PQ, rem = m0 - img * PQ;
                const int p0 = rem / Q, q0 = rem - p0 * Q;
                const int w0 = q0 * a.sw - a.pw, h0 = p0 * a.sh - a.ph;
                const int cpt = a.Cp / kBK, S = a.S, dw = a.dw, dh = a.dh, a_tiled = a.a_tiled;
                const uint32_t tx_bytes = (uint32_t)kATileBytes + a.b_stage_bytes;
                // filter tap (r, s2) and channel chunk of the k-block, carried along
                int tap = kb_begin / cpt, chunk = kb_begin - tap * cpt;
                int r = tap / S, s2 = tap - r * S;
                if (prod == 0) PB_PT((t - blockIdx.x) / gridDim.x, 4);
                for (int kb = 0; kb < nkb; ++kb) {
                    const bool mine_a = (mask_a >> st) & 1u, mine_b = (mask_b >> st) & 1u;
                    if (mine_a || mine_b) {
                        if (mine_a) PB_PK(kb, 0);
                        if (mine_b) PB_PK(kb, 2);
                        ok = mbar_wait(smem_u32(&s_empty[st]), parity, &s_abort, err_flag, 1u);
                        if (!ok) break;
                        const uint32_t a_tile = smem_base + st * stage_bytes;
                        const uint32_t bar = smem_u32(&s_full[st]);
                        if (mine_a) {
                            mbar_arrive_expect_tx(bar, tx_bytes);
                            if (a_tiled) tma_load_2d(a_tile, tmap_x, chunk * kBK, m0, bar);
                            else tma_load_im2col_4d(a_tile, tmap_x, chunk * kBK, w0, h0, img, (uint16_t)(s2 * dw), (uint16_t)(r * dh), bar);
                            PB_PK(kb, 1);
                        }
                        if (mine_b) { tma_load_2d(a_tile + kATileBytes, tmap_w, (kb_begin + kb) * kBK, n0, bar); PB_PK(kb, 3); }
                    }
                    if (++chunk == cpt) {
                        chunk = 0;
                        if (++s2 == S) { s2 = 0; ++r; }
                    }
                    if (++st == (uint32_t)stages) { st = 0; parity ^= 1u; }
                }
            }
        }
        __syncwarp();
    }

    // the next kernel's blocks may take SM slots from here on: this CTA is about to leave
    griddep_launch();
    tcgen05_fence_before();
    __syncthreads();
    if (s_abort) {
        const unsigned long long t0 = globaltimer_ns();
        for (uint32_t i = 0; i < (1u << 20); ++i) {
            if (globaltimer_ns() - t0 > 50000ull) break;
        }
        __syncthreads();
    }
    if (warp == 4) {
        tcgen05_fence_after();
        tcgen05_dealloc(tmem_base, 2u * acc_cols);
    }
#ifdef PB_CONV_STATS
    if (tid == 0) {
        atomicSub(&g_persist_resident, 1u);
        atomicAdd(&g_persist_hist[15], (unsigned long long)(clock64() - s_cta_t0));
    }
#endif
    if (nf) nf->end(job_id);
}

// ---- host side ----------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
        else
            cudaGetLastError();
    });
    return fn;
}

typedef CUresult (*EncodeIm2colFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                   const int*, const int*, cuuint32_t, cuuint32_t, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeIm2colFn encode_im2col_fn() {
    static EncodeIm2colFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeIm2col", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeIm2colFn)p;
        else
            cudaGetLastError();
    });
    return fn;
}

// Operand A by im2col TMA unless PB_CONV_GATHER=1 asks for the cp.async gather kernel.
bool use_tma_a() {
    static const bool v = [] {
        const char* e = getenv("PB_CONV_GATHER");
        return !(e && e[0] == '1');
    }();
    return v;
}

// Widest output-channel tile of the TMA kernel.  A tile of N channels re-reads operand A once per tile,
// so wide tiles cut the bytes an SM pulls; they also take 2 x 48 KB of pipeline and 256 TMEM columns
// (two CTAs per SM instead of three) and halve the CTAs of a launch.  Measured (GPU us per request, 1 / 32 /
// 64 requests in flight, one image per launch): Inception-v3 696 / 46.0 / 43.4 at 128 against 750 / 46.3 / 40.3 at
// 256; ResNet-50 583 / 39.0 / 34.9 against 737 / 43.1 / 37.5; with 8 images per launch (gangs) and 96 requests in
// flight 256 gives +3.7 % requests/s.  So the width follows the launch: 128 for a lone image, 256 for launches of at
// least PB_CONV_WIDE_MIN_BATCH images (default 2: under Poisson arrivals near capacity, where gangs average 3-4
// requests, the mix met its latency bound at 290k offered requests/s with 2 and not with 4; 0 = never wide).
// PB_CONV_MAX_BN=128 / 256 fixes the width for every launch.
int bn_limit(const pb_op_params* p) {
    static const int fixed = [] {
        const char* e = getenv("PB_CONV_MAX_BN");
        return e ? (atoi(e) >= 256 ? 256 : 128) : 0;
    }();
    static const int wide_from = [] {
        const char* e = getenv("PB_CONV_WIDE_MIN_BATCH");
        return e ? atoi(e) : 2;
    }();
    if (!use_tma_a()) return 128;
    if (fixed) return fixed;
    return (wide_from > 0 && (p->batch > 1 ? p->batch : 1) >= wide_from) ? 256 : 128;
}

// PB_CONV_PERSIST=1: model launches run the persistent kernel (a CTA walks several tiles).  Off by default.
// Measured on B200: a lone Inception-v3 request 723 -> 604 us (3 tiles per CTA: 868 us), Inception-v3 alone with 96
// requests in flight 26.5k -> 27.4k req/s, but the headline mix (MNIST : Inception-v3 = 9 : 1, 96 clients, gangs of 4)
// 242k -> 221k req/s: its 108 KB CTAs leave an SM no room for anything else, and fewer, longer CTAs per launch lengthen
// every request's chain of launches, which is what the mix runs out of first.
bool persist_enabled() {
    const char* e = getenv("PB_CONV_PERSIST");      // read at every use: a model keeps what it was loaded with
    return e && e[0] == '1' && use_tma_a();
}
// Tiles a persistent CTA is given (PB_CONV_TILES_PER_CTA): more tiles per CTA spread the per-CTA costs thinner
// and leave SM slots to the other requests in flight; fewer tiles per CTA finish a lone launch sooner.
int tiles_per_cta() {
    const char* e = getenv("PB_CONV_TILES_PER_CTA");      // read at every use: a model instance keeps what it was built with
    const int n = e ? atoi(e) : 3;
    return n < 1 ? 1 : (n > 64 ? 64 : n);
}

// A split of the reduction must save at least this much (us) of a lone launch's modelled time.
// Measured on Inception-v3 (us per request alone / GPU time per request with 32 / 64 in flight):
// threshold 0 -> 727 / 52.7 / 52.6, 0.5 -> 709 / 46.8 / 45.0, 2 -> 706 / 45.7 / 43.3, never split ->
// 721 / 45.4 / 42.0: the partial tiles cost load bandwidth that a busy GPU does not have to spare.
// On the serving mix (MNIST : Inception-v3 = 9 : 1, 48 Inception requests in flight): 2 -> 224k req/s,
// 6 -> 229k, never -> 230k.  At 6 only the reductions that gain most still split (the 448 -> 384 3x3
// convolutions on 8x8 maps of Inception-v3, the 512-channel 3x3 ones of a ResNet's last stage).
// PB_CONV_SPLIT_GAIN_US or pb_set_conv_split_gain_us() overrides it (a large value disables splitting).
std::atomic<double> g_split_gain_us{-1.0};      // < 0: not set yet, take PB_CONV_SPLIT_GAIN_US or the default
double split_gain_us() {
    double v = g_split_gain_us.load(std::memory_order_relaxed);
    if (v < 0) {
        const char* e = getenv("PB_CONV_SPLIT_GAIN_US");
        v = e ? atof(e) : 6.0;
        if (v < 0) v = 0;
        g_split_gain_us.store(v, std::memory_order_relaxed);
    }
    return v;
}

int batch_of(const pb_op_params* p) { return p->batch > 1 ? p->batch : 1; }
int dil_h(const pb_op_params* p) { return p->dil_h > 1 ? p->dil_h : 1; }
int dil_w(const pb_op_params* p) { return p->dil_w > 1 ? p->dil_w : 1; }

struct Geometry {
    int cpt, Cp;                // 64-channel k-blocks per filter tap; Cp = cpt * 64
    int Kdim_pad, nkb;          // k = tap * Cp + c
    int Kp16, n_tiles, BN, Kout_pad;
    int m_tiles;
    int stages;                 // 4, 6 or 8
    int splits, kb_per_split;   // split-K factor the kernel uses when scratch memory is supplied
    uint64_t scratch_bytes;     // counters + partial tiles for that factor
    uint32_t tmem_cols, b_stage_bytes, smem_bytes, idesc;
};

Geometry geometry(const pb_op_params* p, int bn_max = 0) {
    Geometry g;
    if (bn_max <= 0) bn_max = bn_limit(p);
    g.cpt = ceil_div(p->Cs, kBK);
    g.Cp = g.cpt * kBK;
    g.nkb = p->R * p->S * g.cpt;
    g.Kdim_pad = g.nkb * kBK;
    g.Kp16 = round_up(p->K, 16);
    g.n_tiles = ceil_div(g.Kp16, bn_max);
    g.BN = round_up(ceil_div(g.Kp16, g.n_tiles), 16);
    g.Kout_pad = g.n_tiles * g.BN;
    g.m_tiles = ceil_div(batch_of(p) * p->P * p->Q, kBM);
    g.tmem_cols = 32;
    while ((int)g.tmem_cols < g.BN) g.tmem_cols <<= 1;
    g.b_stage_bytes = (uint32_t)g.BN * 128u;
    // Split the reduction over blockIdx.z when that shortens the launch.  Cost model fitted to phase
    // timings on B200 (microseconds): a k-block costs 0.2 + 0.001*BN in the main loop; a split launch
    // pays 1.5 for parking the partial tiles plus 0.0088*BN per partial tile the last CTA adds up.
    const int tiles = g.m_tiles * g.n_tiles;
    const double per_kb = 0.2 + 0.001 * g.BN, per_partial = 0.0088 * g.BN;
    int want = 1;
    double best = g.nkb * per_kb;
    for (int sp = 2; sp <= 16 && tiles * sp <= 296 && sp * 4 <= g.nkb; ++sp) {
        const double t = ceil_div(g.nkb, sp) * per_kb + 1.5 + sp * per_partial;
        if (t < best - split_gain_us()) { best = t; want = sp; }
    }
    g.kb_per_split = ceil_div(g.nkb, want);
    g.splits = ceil_div(g.nkb, g.kb_per_split);
    g.scratch_bytes = g.splits > 1 ? (uint64_t)kCounterBytes + (uint64_t)tiles * g.splits * kBM * g.BN * 4ull : 0;
    if ((uint64_t)tiles * 4 > kCounterBytes) { g.splits = 1; g.kb_per_split = g.nkb; g.scratch_bytes = 0; }
    // Pipeline depth: as many stages as the k-loop can use and the shared-memory budget holds.
    const uint32_t stage_bytes = (uint32_t)kATileBytes + g.b_stage_bytes;
    const uint32_t budget = use_tma_a() ? kSmemBudgetTma : kSmemBudget;
    static const int kDepths[] = {8, 6, 4, 3, 2};
    g.stages = 2;
    for (int d : kDepths) {
        if (!use_tma_a() && d < 4) break;                       // the gather kernel exists for 4, 6, 8
        if ((uint32_t)d * stage_bytes + 1024u <= budget && d <= g.kb_per_split + 1) { g.stages = d; break; }
        if (d == (use_tma_a() ? 2 : 4)) g.stages = d;
    }
    g.smem_bytes = (uint32_t)g.stages * stage_bytes + 1024u;
    // c_format f32 (1 << 4), a/b format bf16 (1 << 7, 1 << 10), K-major both, N >> 3 at bit 17, M >> 4 at bit 24
    g.idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(g.BN >> 3) << 17) | ((uint32_t)(kBM >> 4) << 24);
    return g;
}

// Without (enough) scratch memory the kernel runs the whole reduction in one CTA per tile.
void drop_split(Geometry* g) {
    g->splits = 1;
    g->kb_per_split = g->nkb;
}

const void* kernel_for(int stages, bool tma) {
    if (tma) return (const void*)conv_umma_tma_kernel;
    switch (stages) {
        case 4: return (const void*)conv_umma_gather_kernel<4>;
        case 6: return (const void*)conv_umma_gather_kernel<6>;
        default: return (const void*)conv_umma_gather_kernel<8>;
    }
}

// Raises the dynamic shared-memory limit of every kernel of this file on the current device.
cudaError_t raise_smem_limits() {
    const void* kernels[] = {(const void*)conv_umma_tma_kernel, (const void*)conv_umma_multi_kernel, (const void*)conv_umma_persist_kernel,
                             (const void*)conv_umma_gather_kernel<4>, (const void*)conv_umma_gather_kernel<6>,
                             (const void*)conv_umma_gather_kernel<8>};
    for (const void* k : kernels) {
        cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBudget + 2048);
        if (e != cudaSuccess) return e;
        // An SM's split between shared memory and L1 is fixed while blocks are resident.  Left to the default, the
        // first block to land on an idle SM sizes the split for itself alone and the SM then holds one or two blocks
        // instead of three until it has drained (measured under load: 14 % of the blocks started alone on their SM,
        // 40 % with one other, 45 % with two).  Ask for the largest shared-memory split whenever these kernels run.
        e = cudaFuncSetAttribute(k, cudaFuncAttributePreferredSharedMemoryCarveout, (int)cudaSharedmemCarveoutMaxShared);
        if (e != cudaSuccess) return e;
    }
    return cudaSuccess;
}

}  // namespace

struct ConvUmmaPlan {
    CUtensorMap tmap;        // weights [Kout_pad][Kdim_pad], boxes of g.BN rows (the width a launch of one image uses)
    CUtensorMap tmap_wide;   // the same weights in boxes of BN_wide rows (launches of a gang)
    Geometry g;
    int BN_wide;             // = g.BN when the layer has one column tile either way
    int device;
    const CUtensorMap* map_for(int BN) const { return BN == g.BN ? &tmap : (BN == BN_wide ? &tmap_wide : nullptr); }
};

#ifdef PB_CONV_STATS
extern "C" __attribute__((visibility("default"))) int pb_debug_persist_hist(unsigned long long* out16, int reset) {
    if (cudaMemcpyFromSymbol(out16, g_persist_hist, sizeof(unsigned long long) * 16) != cudaSuccess) return -1;
    if (reset) { unsigned long long z[16] = {0}; cudaMemcpyToSymbol(g_persist_hist, z, sizeof(z)); }
    return 0;
}
extern "C" __attribute__((visibility("default"))) int pb_debug_persist_tile(long long* out96) {
    return cudaMemcpyFromSymbol(out96, g_persist_tile, sizeof(long long) * 16 * 6) == cudaSuccess ? 0 : -1;
}
extern "C" __attribute__((visibility("default"))) int pb_debug_persist_kb(long long* out384) {
    return cudaMemcpyFromSymbol(out384, g_persist_kb, sizeof(long long) * 64 * 6) == cudaSuccess ? 0 : -1;
}
extern "C" __attribute__((visibility("default"))) int pb_debug_conv_stats(unsigned long long* out16, int reset) {
    if (cudaMemcpyFromSymbol(out16, g_conv_stats, sizeof(unsigned long long) * 16) != cudaSuccess) return -1;
    unsigned long long ns = 0;
    if (cudaMemcpyFromSymbol(&ns, g_conv_ns, sizeof(ns)) != cudaSuccess) return -1;
    out16[15] = ns;          // replaces the 5+ bucket of the residency histogram
    if (reset) { const unsigned long long z1 = 0; cudaMemcpyToSymbol(g_conv_ns, &z1, sizeof(z1)); }
    if (reset) {
        unsigned long long z[16] = {0};
        if (cudaMemcpyToSymbol(g_conv_stats, z, sizeof(z)) != cudaSuccess) return -1;
    }
    return 0;
}
#endif

void conv_umma_set_split_gain_us(double us) { g_split_gain_us.store(us, std::memory_order_relaxed); }

bool conv_umma_supported(const pb_op_params* p) {
    const int groups = p->groups > 0 ? p->groups : 1;
    return p->dtype == 1 && groups == 1 && p->Cs % 8 == 0 && p->Ks % 8 == 0 && p->out_c_off % 8 == 0 && p->K % 8 == 0 &&
           (p->residual == nullptr || p->res_Cs % 8 == 0) && p->R >= 1 && p->S >= 1 && p->P * p->Q >= 1 &&
           !(p->flags & 2);
}

int conv_umma_info(const pb_op_params* p, pb_launch_info* out) {
    PB_REQUIRE(conv_umma_supported(p), "conv_umma: unsupported convolution");
    Geometry g = geometry(p);
    memset(out, 0, sizeof(*out));
    out->scratch_bytes = g.scratch_bytes;       // what a split launch needs
    if (g.splits > 1 && (p->scratch == nullptr || p->scratch_bytes < g.scratch_bytes)) drop_split(&g);
    out->kind = PB_STAGE_CONV_UMMA;
    out->num_blocks = (uint32_t)(g.m_tiles * g.n_tiles * g.splits);
    out->threads_per_block = use_tma_a() ? kThreadsTma : kThreads;
    cudaFuncAttributes at;
    uint32_t regs = 64, sstatic = 128;
    if (cudaFuncGetAttributes(&at, kernel_for(g.stages, use_tma_a())) == cudaSuccess) {
        regs = (uint32_t)at.numRegs;
        sstatic = (uint32_t)at.sharedSizeBytes;
    } else {
        cudaGetLastError();
    }
    out->regs_per_thread = regs;
    out->smem_per_block = g.smem_bytes + sstatic;
    out->tmem_cols_per_block = g.tmem_cols;
    const uint64_t nb = (uint64_t)batch_of(p);
    const uint64_t out_elems = nb * p->K * p->P * p->Q;
    out->flops = 2ull * out_elems * p->C * p->R * p->S;
    out->bytes = 2ull * (nb * p->C * p->H * p->W + (uint64_t)p->K * p->C * p->R * p->S + out_elems +
                         (p->residual ? out_elems : 0)) + 4ull * p->K;
    return PB_OK;
}

int64_t conv_umma_pack_weights(const pb_op_params* p, const float* w, void* dst) {
    if (!conv_umma_supported(p)) { set_error("conv_umma: unsupported convolution"); return PB_ERR_INVALID; }
    pb_op_params one = *p;      // the layout does not depend on how many images a launch will carry
    one.batch = 1;
    const Geometry g = geometry(&one);
    const size_t n = (size_t)g.Kout_pad * g.Kdim_pad;
    if (dst) {
        memset(dst, 0, n * 2);
        for (int k = 0; k < p->K; ++k)
            for (int c = 0; c < p->C; ++c)
                for (int r = 0; r < p->R; ++r)
                    for (int s = 0; s < p->S; ++s)
                        store_elem(dst, (size_t)k * g.Kdim_pad + (size_t)(r * p->S + s) * g.Cp + c,
                                   w[(((size_t)k * p->C + c) * p->R + r) * p->S + s], 1);
    }
    return (int64_t)(n * 2);
}

static int make_tmap(const Geometry& g, const void* w_dev, CUtensorMap* out) {
    EncodeTiledFn enc = encode_fn();
    PB_REQUIRE(enc != nullptr, "cuTensorMapEncodeTiled is not available from this driver");
    PB_REQUIRE(((uintptr_t)w_dev & 15) == 0, "conv_umma: packed weights must be 16-byte aligned");
    const cuuint64_t dims[2] = {(cuuint64_t)g.Kdim_pad, (cuuint64_t)g.Kout_pad};
    const cuuint64_t strides[1] = {(cuuint64_t)g.Kdim_pad * 2};
    const cuuint32_t box[2] = {(cuuint32_t)kBK, (cuuint32_t)g.BN};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(w_dev), dims, strides, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_error("cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
        return PB_ERR_CUDA;
    }
    return PB_OK;
}

// im2col tensor map over the channels-last activation tensor [N=1][H][W][Cs] (dims listed innermost
// first).  The bounding box of filter-window origins is [-pad, dim + pad - (filter-1)); traversal
// strides are the convolution strides; each load brings 128 pixels x 64 channels.
// A 1x1, stride-1, unpadded convolution reads its input as the matrix [pixels][channels]: a tiled
// load moves the same 128 x 64 tile with far fewer requests than the im2col mode's per-pixel walk.
static bool pointwise(const pb_op_params* p) {
    return p->R == 1 && p->S == 1 && p->stride_h == 1 && p->stride_w == 1 && p->pad_h == 0 && p->pad_w == 0;      // any batch: images are contiguous
}

static int make_xmap(const pb_op_params* p, CUtensorMap* out) {
    if (pointwise(p)) {
        EncodeTiledFn enc2 = encode_fn();
        PB_REQUIRE(enc2 != nullptr, "cuTensorMapEncodeTiled is not available from this driver");
        PB_REQUIRE(((uintptr_t)p->x & 15) == 0, "conv_umma: activations must be 16-byte aligned");
        const cuuint64_t dims2[2] = {(cuuint64_t)p->Cs, (cuuint64_t)batch_of(p) * p->H * p->W};
        const cuuint64_t strides2[1] = {(cuuint64_t)p->Cs * 2};
        const cuuint32_t box2[2] = {(cuuint32_t)kBK, (cuuint32_t)kBM};
        const cuuint32_t estr2[2] = {1, 1};
        const CUresult r2 = enc2(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(p->x), dims2, strides2, box2, estr2,
                                 CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                                 CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r2 != CUDA_SUCCESS) {
            set_error("cuTensorMapEncodeTiled (activations) failed with CUresult %d (C %d, %d pixels)", (int)r2, p->Cs, p->H * p->W);
            return PB_ERR_CUDA;
        }
        return PB_OK;
    }
    EncodeIm2colFn enc = encode_im2col_fn();
    PB_REQUIRE(enc != nullptr, "cuTensorMapEncodeIm2col is not available from this driver");
    PB_REQUIRE(((uintptr_t)p->x & 15) == 0, "conv_umma: activations must be 16-byte aligned");
    const cuuint64_t dims[4] = {(cuuint64_t)p->Cs, (cuuint64_t)p->W, (cuuint64_t)p->H, (cuuint64_t)batch_of(p)};
    const cuuint64_t strides[3] = {(cuuint64_t)p->Cs * 2, (cuuint64_t)p->W * p->Cs * 2, (cuuint64_t)p->H * p->W * p->Cs * 2};
    const int lower[2] = {-p->pad_w, -p->pad_h};
    const int upper[2] = {p->pad_w - (p->S - 1) * dil_w(p), p->pad_h - (p->R - 1) * dil_h(p)};
    const cuuint32_t estr[4] = {1, (cuuint32_t)p->stride_w, (cuuint32_t)p->stride_h, 1};
    const CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(p->x), dims, strides, lower, upper,
                           (cuuint32_t)kBK, (cuuint32_t)kBM, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                           CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_error("cuTensorMapEncodeIm2col failed with CUresult %d (C %d W %d H %d pad %d,%d filter %dx%d stride %d,%d)", (int)r, p->Cs,
                  p->W, p->H, p->pad_h, p->pad_w, p->R, p->S, p->stride_h, p->stride_w);
        return PB_ERR_CUDA;
    }
    return PB_OK;
}

struct alignas(64) ConvUmmaXMap {
    CUtensorMap map;
};

int conv_umma_xmap_create(const pb_op_params* p, ConvUmmaXMap** out) {
    if (!use_tma_a()) { *out = nullptr; return PB_OK; }
    ConvUmmaXMap* m = new ConvUmmaXMap();
    const int rc = make_xmap(p, &m->map);
    if (rc != PB_OK) { delete m; return rc; }
    *out = m;
    return PB_OK;
}

void conv_umma_xmap_destroy(ConvUmmaXMap* m) { delete m; }

int conv_umma_plan_create(const pb_op_params* p, const void* w_dev, ConvUmmaPlan** out) {
    PB_REQUIRE(conv_umma_supported(p), "conv_umma: unsupported convolution");
    ConvUmmaPlan* plan = new ConvUmmaPlan();
    pb_op_params one = *p;
    one.batch = 1;
    plan->g = geometry(&one);
    cudaGetDevice(&plan->device);
    int rc = make_tmap(plan->g, w_dev, &plan->tmap);
    if (rc != PB_OK) { delete plan; return rc; }
    // The weights were packed for plan->g (rows padded to its column tiles); a wider tiling needs at most as many rows.
    const Geometry gw = geometry(&one, 256);
    plan->BN_wide = gw.BN;
    plan->tmap_wide = plan->tmap;
    if (gw.BN != plan->g.BN) {
        if (gw.Kout_pad > plan->g.Kout_pad) { delete plan; set_error("conv_umma: wide tiling needs more weight rows than were packed"); return PB_ERR_INVALID; }
        rc = make_tmap(gw, w_dev, &plan->tmap_wide);
        if (rc != PB_OK) { delete plan; return rc; }
    }
    // The shared-memory limit is a per-device function attribute: raise it once on every device used.
    static std::once_flag once[16];
    static cudaError_t attr_errs[16] = {};
    if (plan->device < 0 || plan->device >= 16) {
        const int bad = plan->device;
        delete plan;
        set_error("conv_umma: device index %d outside 0..15 (the per-device kernel attributes are kept for 16 devices)", bad);
        return PB_ERR_INVALID;
    }
    const int dev = plan->device;
    std::call_once(once[dev], [dev] { attr_errs[dev] = raise_smem_limits(); });
    const cudaError_t attr_err = attr_errs[dev];
    if (attr_err != cudaSuccess) { delete plan; return cuda_fail(attr_err, "cudaFuncSetAttribute(conv_umma)", __FILE__, __LINE__); }
    *out = plan;
    return PB_OK;
}

void conv_umma_plan_destroy(ConvUmmaPlan* plan) { delete plan; }

// Kernel arguments of one convolution; `g` may have had its split dropped for lack of scratch.
static int fill_args(const ConvUmmaPlan* plan, const Geometry& g, const pb_op_params* p, uint32_t* err_flag, ConvArgs* out) {
    ConvArgs& a = *out;
    memset(&a, 0, sizeof(a));
    a.x = static_cast<const __nv_bfloat16*>(p->x);
    a.residual = static_cast<const __nv_bfloat16*>(p->residual);
    a.bias = p->bias;
    a.y = static_cast<__nv_bfloat16*>(p->y);
    a.err_flag = err_flag ? err_flag : device_error_flag_ptr(plan->device);
    PB_REQUIRE(a.err_flag != nullptr, "conv_umma: no device error flag");
    a.H = p->H; a.W = p->W; a.Cs = p->Cs; a.P = p->P; a.Q = p->Q; a.PQ = p->P * p->Q; a.M = batch_of(p) * a.PQ;
    a.dh = dil_h(p); a.dw = dil_w(p);
    a.K = p->K; a.Ks = p->Ks; a.out_c_off = p->out_c_off; a.res_Cs = p->res_Cs;
    a.R = p->R; a.S = p->S; a.sh = p->stride_h; a.sw = p->stride_w; a.ph = p->pad_h; a.pw = p->pad_w;
    a.act = p->act; a.a_tiled = pointwise(p) ? 1 : 0; a.nkb = g.nkb; a.taps = p->R * p->S; a.Cp = g.Cp; a.BN = g.BN; a.idesc = g.idesc; a.tmem_cols = g.tmem_cols;
    a.b_stage_bytes = g.b_stage_bytes;
    a.splits = g.splits;
    a.kb_per_split = g.kb_per_split;
    a.counters = g.splits > 1 ? static_cast<unsigned*>(p->scratch) : nullptr;
    a.ws = g.splits > 1 ? reinterpret_cast<float*>(static_cast<char*>(p->scratch) + kCounterBytes) : nullptr;
    return PB_OK;
}

template <typename... Args>
static cudaError_t launch_pdl(void (*kern)(Args...), dim3 grid, uint32_t smem, cudaStream_t st, bool pdl, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(kThreadsTma);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, args...);
}

int conv_umma_launch_planned(const ConvUmmaPlan* plan, const ConvUmmaXMap* xmap, const pb_op_params* p, cudaStream_t st,
                             uint32_t job_id, void* notifier, uint32_t* err_flag, bool pdl) {
    Geometry g = geometry(p);       // the plan's own geometry is that of one image; tiles and split follow the batch
    if (g.splits > 1 && (p->scratch == nullptr || p->scratch_bytes < g.scratch_bytes)) drop_split(&g);
    if (!use_tma_a()) PB_REQUIRE(batch_of(p) == 1, "conv_umma: the cp.async gather kernel (PB_CONV_GATHER=1) runs one image per launch");
    ConvArgs a;
    const int frc = fill_args(plan, g, p, err_flag, &a);
    if (frc != PB_OK) return frc;
    const dim3 grid((unsigned)g.m_tiles, (unsigned)g.n_tiles, (unsigned)g.splits);
    FinishedBlockNotifier* nf = static_cast<FinishedBlockNotifier*>(notifier);
    if (use_tma_a()) {
        ConvUmmaXMap local;
        if (!xmap) {
            const int rc = make_xmap(p, &local.map);
            if (rc != PB_OK) return rc;
            xmap = &local;
        }
        const CUtensorMap* wmap = plan->map_for(g.BN);
        PB_REQUIRE(wmap != nullptr, "conv_umma: no weight map for a tile of %d channels", g.BN);
        const cudaError_t e = launch_pdl(conv_umma_tma_kernel, grid, g.smem_bytes, st, pdl, *wmap, xmap->map, a, g.stages, job_id, nf);
        if (e != cudaSuccess) return cuda_fail(e, "launch of conv_umma_tma_kernel", __FILE__, __LINE__);
        return PB_OK;
    } else {
        switch (g.stages) {
            case 4: conv_umma_gather_kernel<4><<<grid, kThreads, g.smem_bytes, st>>>(plan->tmap, a, job_id, nf); break;
            case 6: conv_umma_gather_kernel<6><<<grid, kThreads, g.smem_bytes, st>>>(plan->tmap, a, job_id, nf); break;
            default: conv_umma_gather_kernel<8><<<grid, kThreads, g.smem_bytes, st>>>(plan->tmap, a, job_id, nf); break;
        }
    }
    return launch_check("conv_umma");
}

// ---- grouped launch ----------------------------------------------------------------------------
struct ConvUmmaMulti {
    SubConv* table_dev = nullptr;
    int n = 0;
    unsigned total_blocks = 0;      // tiles of all sub-problems (= CTAs of the one-tile-per-CTA kernel)
    uint32_t smem = 0;
    uint32_t tmem_cols = 0;
    bool has_pool = false;          // pooling layers ride along (one-tile kernel only)
    // persistent kernel
    bool persist = false;
    unsigned grid = 0;
    int stages = 0;
    uint32_t stage_bytes = 0, persist_smem = 0;
};

bool conv_umma_multi_available() { return use_tma_a(); }
bool conv_umma_persist_enabled() { return persist_enabled(); }
uint32_t conv_umma_persist_grid(uint32_t total_tiles) {
    const uint32_t g = ceil_div<uint32_t>(total_tiles, (uint32_t)tiles_per_cta());
    return g < 1 ? 1 : g;
}

// A 3x3 max / average pooling layer (bf16, vector-aligned slice) can ride along in a grouped launch.
bool conv_umma_pool_fusable(int kind, const pb_op_params* p) {
    return (kind == PB_STAGE_MAXPOOL || kind == PB_STAGE_AVGPOOL) && p->dtype == 1 && p->R == 3 && p->S == 3 && p->Cs % 8 == 0 &&
           p->Ks % 8 == 0 && p->out_c_off % 8 == 0 && !(p->flags & 2) && p->H >= 1 && p->W >= 1 && p->bias == nullptr && p->act == 0;
}
uint32_t conv_umma_pool_blocks(const pb_op_params* p) {
    const uint64_t vecs = (uint64_t)batch_of(p) * p->P * p->Q * (p->Cs / 8);
    return (uint32_t)ceil_div<uint64_t>(vecs, (uint64_t)kThreadsTma * kPoolVecsPerThread);
}

int conv_umma_multi_create(const ConvUmmaPlan* const* plans, const ConvUmmaXMap* const* xmaps, const pb_op_params* const* params, const int* kinds,
                           int n, ConvUmmaMulti** out) {
    PB_REQUIRE(out && plans && xmaps && params && n >= 1 && n <= kMaxSubConvs, "conv_umma_multi_create: 1..%d entries", kMaxSubConvs);
    PB_REQUIRE(use_tma_a(), "conv_umma_multi_create: needs the TMA operand path");
    std::vector<SubConv> table((size_t)n);
    memset(table.data(), 0, sizeof(SubConv) * (size_t)n);
    ConvUmmaMulti* m = new ConvUmmaMulti();
    m->n = n;
    for (int i = 0; i < n; ++i) {
        if (kinds && kinds[i] != PB_STAGE_CONV_UMMA) {
            const pb_op_params* p = params[i];
            if (!p || !conv_umma_pool_fusable(kinds[i], p)) { delete m; set_error("conv_umma_multi_create: entry %d cannot ride along", i); return PB_ERR_INVALID; }
            SubConv& sc = table[(size_t)i];
            PoolSubArgs& a = sc.pool;
            a.x = static_cast<const __nv_bfloat16*>(p->x);
            a.y = static_cast<__nv_bfloat16*>(p->y);
            a.C = p->C; a.H = p->H; a.W = p->W; a.Cs = p->Cs; a.P = p->P; a.Q = p->Q; a.Ks = p->Ks; a.out_c_off = p->out_c_off;
            a.sh = p->stride_h; a.sw = p->stride_w; a.ph = p->pad_h; a.pw = p->pad_w;
            a.is_max = kinds[i] == PB_STAGE_MAXPOOL; a.count_pad = p->flags & 1; a.batch = batch_of(p);
            sc.first_block = m->total_blocks;
            sc.gx = sc.gy = 1;
            sc.stages = kSubPool;
            m->total_blocks += conv_umma_pool_blocks(p);
            m->has_pool = true;
            continue;
        }
        PB_REQUIRE(plans[i] && xmaps[i] && params[i], "conv_umma_multi_create: NULL entry %d", i);
        Geometry g = geometry(params[i]);
        if (g.splits > 1 && (params[i]->scratch == nullptr || params[i]->scratch_bytes < g.scratch_bytes)) drop_split(&g);
        SubConv& sc = table[(size_t)i];
        const CUtensorMap* wmap = plans[i]->map_for(g.BN);
        if (!wmap) { delete m; set_error("conv_umma_multi_create: no weight map for a tile of %d channels", g.BN); return PB_ERR_INVALID; }
        sc.tmap_w = *wmap;
        sc.tmap_x = xmaps[i]->map;
        const int rc = fill_args(plans[i], g, params[i], nullptr, &sc.a);
        if (rc != PB_OK) { delete m; return rc; }
        sc.first_block = m->total_blocks;
        sc.gx = (uint32_t)g.m_tiles;
        sc.gy = (uint32_t)g.n_tiles;
        sc.stages = (uint32_t)g.stages;
        m->total_blocks += (unsigned)(g.m_tiles * g.n_tiles * g.splits);
        m->smem = std::max(m->smem, g.smem_bytes);
        m->tmem_cols = std::max(m->tmem_cols, g.tmem_cols);
        m->stage_bytes = std::max(m->stage_bytes, (uint32_t)kATileBytes + g.b_stage_bytes);
    }
    if (m->stage_bytes == 0) { delete m; set_error("conv_umma_multi_create: no convolution among the entries"); return PB_ERR_INVALID; }
    // persistent kernel: one pipeline for every sub-problem (stages of the widest), two accumulators
    m->stages = (int)std::min<uint32_t>(kMaxStages, (kSmemBudgetPersist - 1024u) / m->stage_bytes);
    m->persist_smem = (uint32_t)m->stages * m->stage_bytes + 1024u;
    m->grid = conv_umma_persist_grid(m->total_blocks);
    m->persist = persist_enabled() && m->stages >= 2 && 2u * m->tmem_cols <= 512u && !m->has_pool;
    cudaError_t e = cudaMalloc((void**)&m->table_dev, sizeof(SubConv) * (size_t)n);
    if (e == cudaSuccess) e = cudaMemcpy(m->table_dev, table.data(), sizeof(SubConv) * (size_t)n, cudaMemcpyHostToDevice);
    if (e != cudaSuccess) { conv_umma_multi_destroy(m); return cuda_fail(e, "conv_umma_multi_create", __FILE__, __LINE__); }
    *out = m;
    return PB_OK;
}

void conv_umma_multi_destroy(ConvUmmaMulti* m) {
    if (!m) return;
    if (m->table_dev) cudaFree(m->table_dev);
    delete m;
}

void conv_umma_persist_footprint(uint32_t total_tiles, uint32_t max_tmem_cols, pb_launch_info* out) {
    memset(out, 0, sizeof(*out));
    out->num_blocks = conv_umma_persist_grid(total_tiles);
    out->threads_per_block = kThreadsPersist;
    out->smem_per_block = kSmemBudgetPersist;
    cudaFuncAttributes at;
    out->regs_per_thread = 128;
    if (cudaFuncGetAttributes(&at, (const void*)conv_umma_persist_kernel) == cudaSuccess) out->regs_per_thread = (uint32_t)at.numRegs;
    else cudaGetLastError();
    out->tmem_cols_per_block = 2u * max_tmem_cols;
    out->kind = PB_STAGE_CONV_UMMA;
}

void conv_umma_multi_info(const ConvUmmaMulti* m, pb_launch_info* out) {
    memset(out, 0, sizeof(*out));
    out->num_blocks = m->persist ? m->grid : m->total_blocks;
    out->threads_per_block = m->persist ? kThreadsPersist : kThreadsTma;
    out->smem_per_block = m->persist ? m->persist_smem : m->smem;
    cudaFuncAttributes at;
    out->regs_per_thread = 112;
    if (cudaFuncGetAttributes(&at, m->persist ? (const void*)conv_umma_persist_kernel : (const void*)conv_umma_multi_kernel) == cudaSuccess)
        out->regs_per_thread = (uint32_t)at.numRegs;
    else cudaGetLastError();
    out->tmem_cols_per_block = m->persist ? 2u * m->tmem_cols : m->tmem_cols;
    out->kind = PB_STAGE_CONV_UMMA;
}

int conv_umma_multi_launch(const ConvUmmaMulti* m, cudaStream_t st, uint32_t job_id, void* notifier, bool pdl) {
    if (m->persist) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(m->grid);
        cfg.blockDim = dim3(kThreadsPersist);
        cfg.dynamicSmemBytes = m->persist_smem;
        cfg.stream = st;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = pdl ? 1 : 0;
        const cudaError_t e = cudaLaunchKernelEx(&cfg, conv_umma_persist_kernel, (const SubConv*)m->table_dev, m->n, (uint32_t)m->total_blocks, m->stages,
                                                 m->stage_bytes, m->tmem_cols, job_id, static_cast<FinishedBlockNotifier*>(notifier));
        if (e != cudaSuccess) return cuda_fail(e, "launch of conv_umma_persist_kernel", __FILE__, __LINE__);
        return PB_OK;
    }
    const cudaError_t e = launch_pdl(conv_umma_multi_kernel, dim3(m->total_blocks), m->smem, st, pdl, (const SubConv*)m->table_dev, m->n,
                                     job_id, static_cast<FinishedBlockNotifier*>(notifier));
    if (e != cudaSuccess) return cuda_fail(e, "launch of conv_umma_multi_kernel", __FILE__, __LINE__);
    return PB_OK;
}

int conv_umma_launch(const pb_op_params* p, cudaStream_t st, uint32_t job_id, void* notifier) {
    ConvUmmaPlan* plan = nullptr;
    int rc = conv_umma_plan_create(p, p->w, &plan);
    if (rc != PB_OK) return rc;
    // PB_CONV_PERSIST_OPS=1 (read at every call; for tests): a lone operator launch also runs the persistent kernel
    // the model launches use, through a one-entry table that lives for this call only (allocates and synchronises).
    const char* po = getenv("PB_CONV_PERSIST_OPS");
    if (po && po[0] == '1' && persist_enabled()) {
        ConvUmmaXMap* xm = nullptr;
        ConvUmmaMulti* mu = nullptr;
        rc = conv_umma_xmap_create(p, &xm);
        if (rc == PB_OK) {
            const ConvUmmaPlan* plans[1] = {plan};
            const ConvUmmaXMap* xms[1] = {xm};
            const pb_op_params* pp[1] = {p};
            rc = conv_umma_multi_create(plans, xms, pp, nullptr, 1, &mu);
        }
        if (rc == PB_OK && !mu->persist) { set_error("conv_umma: this shape does not fit the persistent kernel"); rc = PB_ERR_INVALID; }
        if (rc == PB_OK) rc = conv_umma_multi_launch(mu, st, job_id, notifier, false);
        if (rc == PB_OK && cudaStreamSynchronize(st) != cudaSuccess) rc = cuda_fail(cudaGetLastError(), "persistent convolution", __FILE__, __LINE__);
        conv_umma_multi_destroy(mu);
        conv_umma_xmap_destroy(xm);
        conv_umma_plan_destroy(plan);
        return rc;
    }
    rc = conv_umma_launch_planned(plan, nullptr, p, st, job_id, notifier, nullptr);
    conv_umma_plan_destroy(plan);   // the tensor maps were copied into the launch parameters
    return rc;
}

// Times `iters` launches of one convolution between CUDA events (after 3 warm-up launches), an L2 flush (a write
// of flush_bytes) before each when asked: mode 0 = the one-tile-per-CTA kernel, 1 = the persistent kernel.
int conv_umma_time(const pb_op_params* p, int mode, int iters, size_t flush_bytes, double* us_out) {
    PB_REQUIRE(p && us_out && iters > 0, "pb_conv_umma_time: bad arguments");
    ConvUmmaPlan* plan = nullptr;
    ConvUmmaXMap* xm = nullptr;
    ConvUmmaMulti* mu = nullptr;
    void* flush = nullptr;
    cudaStream_t st = nullptr;
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    int rc = conv_umma_plan_create(p, p->w, &plan);
    if (rc == PB_OK) rc = conv_umma_xmap_create(p, &xm);
    if (rc == PB_OK && mode == 1) {
        const ConvUmmaPlan* plans[1] = {plan};
        const ConvUmmaXMap* xms[1] = {xm};
        const pb_op_params* pp[1] = {p};
        rc = conv_umma_multi_create(plans, xms, pp, nullptr, 1, &mu);
        if (rc == PB_OK && !mu->persist) { set_error("pb_conv_umma_time: the persistent kernel is off or does not fit this shape"); rc = PB_ERR_INVALID; }
    }
    cudaError_t e = cudaSuccess;
    if (rc == PB_OK) e = cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking);
    if (rc == PB_OK && e == cudaSuccess && flush_bytes) e = cudaMalloc(&flush, flush_bytes);
    if (rc == PB_OK && e == cudaSuccess) e = cudaEventCreate(&e0);
    if (rc == PB_OK && e == cudaSuccess) e = cudaEventCreate(&e1);
    double total_ms = 0;
    auto launch = [&]() { return mode == 1 ? conv_umma_multi_launch(mu, st, 0, nullptr, false) : conv_umma_launch_planned(plan, xm, p, st, 0, nullptr, nullptr, false); };
    for (int i = 0; rc == PB_OK && e == cudaSuccess && i < 3; ++i) rc = launch();
    for (int i = 0; rc == PB_OK && e == cudaSuccess && i < iters; ++i) {
        if (flush) cudaMemsetAsync(flush, i & 0xff, flush_bytes, st);
        cudaEventRecord(e0, st);
        rc = launch();
        cudaEventRecord(e1, st);
        e = cudaEventSynchronize(e1);
        float ms = 0;
        if (e == cudaSuccess) { cudaEventElapsedTime(&ms, e0, e1); total_ms += ms; }
    }
    if (e0) cudaEventDestroy(e0);
    if (e1) cudaEventDestroy(e1);
    if (flush) cudaFree(flush);
    if (st) cudaStreamDestroy(st);
    conv_umma_multi_destroy(mu);
    conv_umma_xmap_destroy(xm);
    conv_umma_plan_destroy(plan);
    if (rc != PB_OK) return rc;
    if (e != cudaSuccess) return cuda_fail(e, "pb_conv_umma_time", __FILE__, __LINE__);
    *us_out = total_ms * 1000.0 / iters;
    return PB_OK;
}

// ---- launch without any allocation -----------------------------------------------------------------
// Scratch for pb_conv2d_umma_noalloc: split-K tile counters (first kCounterBytes) and partial tiles.
// It lives in the library image, so every GPU that loads the library holds these bytes until exit.
constexpr size_t kStaticScratchBytes = PB_NOALLOC_SCRATCH_BYTES;
static __device__ __align__(256) unsigned char g_noalloc_scratch[kStaticScratchBytes];
static __device__ uint32_t g_noalloc_err_flag;

namespace {
struct NoAllocDevice {
    bool ready = false;
    void* scratch = nullptr;      // device address of g_noalloc_scratch on this device
    uint32_t* err_flag = nullptr;
};
NoAllocDevice g_noalloc_dev[16];
std::mutex g_noalloc_mu;
}  // namespace

uint32_t* noalloc_error_flag_ptr(int device) {
    if (device < 0 || device >= 16) return nullptr;
    std::lock_guard<std::mutex> lk(g_noalloc_mu);
    return g_noalloc_dev[device].ready ? g_noalloc_dev[device].err_flag : nullptr;
}

int conv_umma_launch_noalloc(const pb_op_params* p, cudaStream_t st, uint32_t job_id, void* notifier) {
    PB_REQUIRE(p != nullptr && conv_umma_supported(p), "pb_conv2d_umma_noalloc: unsupported convolution");
    int device = -1;
    PB_CUDA(cudaGetDevice(&device));
    PB_REQUIRE(device >= 0 && device < 16, "pb_conv2d_umma_noalloc: device %d out of range", device);
    NoAllocDevice& nd = g_noalloc_dev[device];
    {
        // First call on this device: resolve the device addresses of the file-scope arrays.  In host
        // code their names are only stand-ins, not device addresses; the kernel must be given what
        // cudaGetSymbolAddress returns, with this device current.
        std::lock_guard<std::mutex> lk(g_noalloc_mu);
        if (!nd.ready) {
            void* sp = nullptr;
            void* fp = nullptr;
            PB_CUDA(cudaGetSymbolAddress(&sp, g_noalloc_scratch));
            PB_CUDA(cudaGetSymbolAddress(&fp, g_noalloc_err_flag));
            PB_CUDA(raise_smem_limits());
            nd.scratch = sp;
            nd.err_flag = static_cast<uint32_t*>(fp);
            nd.ready = true;
        }
    }
    ConvUmmaPlan plan;            // on the stack: no host allocation either
    plan.g = geometry(p);
    plan.device = device;
    if (plan.g.scratch_bytes > kStaticScratchBytes) {
        set_error("pb_conv2d_umma_noalloc: this convolution wants %llu bytes of scratch, the built-in buffer holds %llu "
                  "(use pb_op_launch with caller-provided scratch instead)",
                  (unsigned long long)plan.g.scratch_bytes, (unsigned long long)kStaticScratchBytes);
        return PB_ERR_INVALID;
    }
    int rc = make_tmap(plan.g, p->w, &plan.tmap);
    if (rc != PB_OK) return rc;
    pb_op_params q = *p;
    q.scratch = plan.g.scratch_bytes ? nd.scratch : nullptr;
    q.scratch_bytes = plan.g.scratch_bytes ? kStaticScratchBytes : 0;
    // The buffer keeps whatever the previous call left; only the tile counters have to start at zero.
    if (plan.g.scratch_bytes) PB_CUDA(cudaMemsetAsync(nd.scratch, 0, kCounterBytes, st));
    return conv_umma_launch_planned(&plan, nullptr, &q, st, job_id, notifier, nd.err_flag);
}

}  // namespace pb
