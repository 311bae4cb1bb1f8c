// Dense convolution as an implicit GEMM on the 5th-generation tensor cores (sm_100a).
//
//   D[m, n] = sum_k A[m, k] * B[n, k]     m = output pixel (p*Q + q), n = output channel,
//                                          k = (r*S + s)*Cs + c   (filter tap, input channel)
//
// A is never materialised: 128 producer threads gather it from the channels-last bf16
// activation tensor with 16-byte cp.async copies (zero fill for padding and for the k tail)
// straight into the 128-byte-swizzled K-major shared-memory layout that tcgen05.mma reads.
// B (packed weights [Kout_pad][Kdim_pad]) arrives by TMA (cp.async.bulk.tensor.2d, 128B
// swizzle, no multicast).  One elected thread issues tcgen05.mma (M=128, N=BN, K=16, bf16 x
// bf16 -> fp32) with the accumulator in tensor memory; tcgen05.commit releases pipeline
// stages and signals the epilogue, which reads TMEM with tcgen05.ld, adds bias and residual,
// applies the activation and stores bf16 into the channel slice of the output tensor.
//
// CTA = 5 warps: warps 0-3 produce A (one tile row per thread) and then run the epilogue
// (thread t owns accumulator lane t); warp 4 allocates TMEM and issues the MMAs.
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

#include <cstring>
#include <mutex>

#include "ops.h"
#include "pb_common.h"

using llis::job::FinishedBlockNotifier;

namespace pb {

namespace {

constexpr int kBM = 128;            // tile rows (output pixels) = TMEM lanes
constexpr int kBK = 64;             // bf16 elements per k-block = one 128-byte swizzle row
constexpr int kStages = 4;
constexpr int kLag = 2;             // cp.async groups kept in flight per producer thread
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
    int P, Q, M;          // M = P*Q
    int K, Ks, out_c_off, res_Cs;
    int R, S, sh, sw, ph, pw;
    int act;
    int nkb;              // k-blocks of 64
    int taps;             // R*S
    int BN;               // output channels per CTA (multiple of 16, <= 256)
    uint32_t idesc;       // tcgen05 instruction descriptor
    uint32_t tmem_cols;   // power of two >= max(32, BN)
    uint32_t b_stage_bytes;
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

__device__ __forceinline__ float act_fn(float v, int act) {
    if (act == 1) return fmaxf(v, 0.f);
    if (act == 2) return fminf(fmaxf(v, 0.f), 6.f);
    return v;
}

// ---- the kernel -----------------------------------------------------------------------
__global__ void __launch_bounds__(kThreads, 1)
conv_umma_kernel(const __grid_constant__ CUtensorMap tmap_w, const ConvArgs a, uint32_t job_id, FinishedBlockNotifier* nf) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t s_full[kStages];
    __shared__ __align__(8) uint64_t s_empty[kStages];
    __shared__ __align__(8) uint64_t s_accum;
    __shared__ uint32_t s_tmem_base;
    __shared__ volatile uint32_t s_abort;

    if (nf) nf->start(job_id);

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t stage_bytes = (uint32_t)kATileBytes + a.b_stage_bytes;

    if (tid == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(smem_u32(&s_full[s]), 128);
            mbar_init(smem_u32(&s_empty[s]), 1);
        }
        mbar_init(smem_u32(&s_accum), 1);
        s_abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 4) {
        tcgen05_alloc(smem_u32(&s_tmem_base), a.tmem_cols);
        tcgen05_relinquish();
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = s_tmem_base;

    const int m0 = blockIdx.x * kBM;
    const int n0 = blockIdx.y * a.BN;

    if (warp < 4) {
        // ===== A producer: thread `tid` owns tile row `tid` =====
        const int m = m0 + tid;
        const bool row_valid = m < a.M;
        const int p = row_valid ? m / a.Q : 0;
        const int q = row_valid ? m % a.Q : 0;
        const int ih0 = p * a.sh - a.ph;
        const int iw0 = q * a.sw - a.pw;
        const uint32_t row_off = (uint32_t)tid * 128u;
        const uint32_t sw = (uint32_t)(tid & 7);
        // running position in k: filter tap (r, s) and channel c
        int r = 0, s = 0, c = 0, tap = 0;
        bool ok = true;
        for (int kb = 0; kb < a.nkb; ++kb) {
            const int st = kb % kStages;
            const uint32_t use = (uint32_t)(kb / kStages);
            if (ok) ok = mbar_wait(smem_u32(&s_empty[st]), (use & 1u) ^ 1u, &s_abort, a.err_flag, 1u);
            const uint32_t a_tile = smem_base + (uint32_t)st * stage_bytes;
            if (ok) {
                if (tid == 0) {
                    mbar_expect_tx(smem_u32(&s_full[st]), a.b_stage_bytes);
                    tma_load_2d(a_tile + kATileBytes, &tmap_w, kb * kBK, n0, smem_u32(&s_full[st]));
                }
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const int ih = ih0 + r, iw = iw0 + s;
                    const bool inb = row_valid && tap < a.taps && ih >= 0 && ih < a.H && iw >= 0 && iw < a.W;
                    const __nv_bfloat16* src = inb ? a.x + ((size_t)ih * a.W + iw) * a.Cs + c : a.x;
                    cp_async_16(a_tile + row_off + (((uint32_t)j ^ sw) << 4), src, inb ? 16u : 0u);
                    c += 8;
                    if (c >= a.Cs) {
                        c = 0; ++tap; ++s;
                        if (s == a.S) { s = 0; ++r; }
                    }
                }
            }
            cp_async_commit();
            if (kb >= kLag) {
                cp_async_wait<kLag>();
                fence_proxy_async();
                mbar_arrive(smem_u32(&s_full[(kb - kLag) % kStages]));
            }
        }
        // drain: the last kLag k-blocks
        cp_async_wait<0>();
        fence_proxy_async();
        for (int kb = (a.nkb > kLag ? a.nkb - kLag : 0); kb < a.nkb; ++kb) mbar_arrive(smem_u32(&s_full[kb % kStages]));

        // ===== epilogue: accumulator lane `tid` = tile row `tid` =====
        if (ok) ok = mbar_wait(smem_u32(&s_accum), 0u, &s_abort, a.err_flag, 3u);
        ok = __all_sync(0xffffffffu, ok);   // tcgen05.ld below is warp-collective
        tcgen05_fence_after();
        if (ok) {
            const uint32_t lane_addr = tmem_base + ((uint32_t)(warp * 32) << 16);
            __nv_bfloat16* yrow = a.y + (size_t)m * a.Ks + a.out_c_off;
            const __nv_bfloat16* rrow = a.residual ? a.residual + (size_t)m * a.res_Cs : nullptr;
            for (int cb = 0; cb < a.BN; cb += 16) {
                uint32_t v[16];
                tcgen05_ld16(lane_addr + (uint32_t)cb, v);   // warp-collective: all lanes take part
                tcgen05_wait_ld();
                const int k0 = n0 + cb;
                if (row_valid && k0 < a.K) {
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const int kk = k0 + h * 8;
                        if (kk + 8 <= a.K) {
                            float f[8];
#pragma unroll
                            for (int j = 0; j < 8; ++j) f[j] = __uint_as_float(v[h * 8 + j]) + (a.bias ? __ldg(a.bias + kk + j) : 0.f);
                            if (rrow) {
                                const uint4 rv = *reinterpret_cast<const uint4*>(rrow + kk);
                                const uint32_t ru[4] = {rv.x, rv.y, rv.z, rv.w};
#pragma unroll
                                for (int j = 0; j < 4; ++j) {
                                    f[2 * j] += __uint_as_float(ru[j] << 16);
                                    f[2 * j + 1] += __uint_as_float(ru[j] & 0xffff0000u);
                                }
                            }
                            uint32_t o[4];
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                const __nv_bfloat162 hv = __floats2bfloat162_rn(act_fn(f[2 * j], a.act), act_fn(f[2 * j + 1], a.act));
                                o[j] = *reinterpret_cast<const uint32_t*>(&hv);
                            }
                            *reinterpret_cast<uint4*>(yrow + kk) = make_uint4(o[0], o[1], o[2], o[3]);
                        }
                    }
                }
            }
        }
    } else {
        // ===== MMA issuer: one thread =====
        if (lane == 0) {
            bool ok = true;
            for (int kb = 0; kb < a.nkb && ok; ++kb) {
                const int st = kb % kStages;
                const uint32_t use = (uint32_t)(kb / kStages);
                ok = mbar_wait(smem_u32(&s_full[st]), use & 1u, &s_abort, a.err_flag, 2u);
                if (!ok) break;
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

struct Geometry {
    int Kdim, Kdim_pad, nkb;
    int Kp16, n_tiles, BN, Kout_pad;
    int m_tiles;
    uint32_t tmem_cols, b_stage_bytes, smem_bytes, idesc;
};

Geometry geometry(const pb_op_params* p) {
    Geometry g;
    g.Kdim = p->R * p->S * p->Cs;
    g.Kdim_pad = round_up(g.Kdim, kBK);
    g.nkb = g.Kdim_pad / kBK;
    g.Kp16 = round_up(p->K, 16);
    g.n_tiles = ceil_div(g.Kp16, 128);
    g.BN = round_up(ceil_div(g.Kp16, g.n_tiles), 16);
    g.Kout_pad = g.n_tiles * g.BN;
    g.m_tiles = ceil_div(p->P * p->Q, kBM);
    g.tmem_cols = 32;
    while ((int)g.tmem_cols < g.BN) g.tmem_cols <<= 1;
    g.b_stage_bytes = (uint32_t)g.BN * 128u;
    g.smem_bytes = kStages * ((uint32_t)kATileBytes + g.b_stage_bytes) + 1024u;
    // c_format f32 (1 << 4), a/b format bf16 (1 << 7, 1 << 10), K-major both, N >> 3 at bit 17, M >> 4 at bit 24
    g.idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(g.BN >> 3) << 17) | ((uint32_t)(kBM >> 4) << 24);
    return g;
}

}  // namespace

struct ConvUmmaPlan {
    CUtensorMap tmap;
    Geometry g;
    int device;
};

bool conv_umma_supported(const pb_op_params* p) {
    const int groups = p->groups > 0 ? p->groups : 1;
    return p->dtype == 1 && groups == 1 && p->Cs % 8 == 0 && p->Ks % 8 == 0 && p->out_c_off % 8 == 0 && p->K % 8 == 0 &&
           (p->residual == nullptr || p->res_Cs % 8 == 0) && p->R >= 1 && p->S >= 1 && p->P * p->Q >= 1 &&
           !(p->flags & 2);
}

int conv_umma_info(const pb_op_params* p, pb_launch_info* out) {
    PB_REQUIRE(conv_umma_supported(p), "conv_umma: unsupported convolution");
    const Geometry g = geometry(p);
    memset(out, 0, sizeof(*out));
    out->kind = PB_STAGE_CONV_UMMA;
    out->num_blocks = (uint32_t)(g.m_tiles * g.n_tiles);
    out->threads_per_block = kThreads;
    cudaFuncAttributes at;
    uint32_t regs = 64, sstatic = 128;
    if (cudaFuncGetAttributes(&at, (const void*)conv_umma_kernel) == cudaSuccess) {
        regs = (uint32_t)at.numRegs;
        sstatic = (uint32_t)at.sharedSizeBytes;
    } else {
        cudaGetLastError();
    }
    out->regs_per_thread = regs;
    out->smem_per_block = g.smem_bytes + sstatic;
    out->tmem_cols_per_block = g.tmem_cols;
    const uint64_t out_elems = (uint64_t)p->K * p->P * p->Q;
    out->flops = 2ull * out_elems * p->C * p->R * p->S;
    out->bytes = 2ull * ((uint64_t)p->C * p->H * p->W + (uint64_t)p->K * p->C * p->R * p->S + out_elems +
                         (p->residual ? out_elems : 0)) + 4ull * p->K;
    return PB_OK;
}

int64_t conv_umma_pack_weights(const pb_op_params* p, const float* w, void* dst) {
    if (!conv_umma_supported(p)) { set_error("conv_umma: unsupported convolution"); return PB_ERR_INVALID; }
    const Geometry g = geometry(p);
    const size_t n = (size_t)g.Kout_pad * g.Kdim_pad;
    if (dst) {
        memset(dst, 0, n * 2);
        for (int k = 0; k < p->K; ++k)
            for (int c = 0; c < p->C; ++c)
                for (int r = 0; r < p->R; ++r)
                    for (int s = 0; s < p->S; ++s)
                        store_elem(dst, (size_t)k * g.Kdim_pad + (size_t)(r * p->S + s) * p->Cs + c,
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

int conv_umma_plan_create(const pb_op_params* p, const void* w_dev, ConvUmmaPlan** out) {
    PB_REQUIRE(conv_umma_supported(p), "conv_umma: unsupported convolution");
    ConvUmmaPlan* plan = new ConvUmmaPlan();
    plan->g = geometry(p);
    cudaGetDevice(&plan->device);
    int rc = make_tmap(plan->g, w_dev, &plan->tmap);
    if (rc != PB_OK) { delete plan; return rc; }
    static std::once_flag once;
    static cudaError_t attr_err = cudaSuccess;
    std::call_once(once, [] {
        attr_err = cudaFuncSetAttribute((const void*)conv_umma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024 - 1024);
    });
    if (attr_err != cudaSuccess) { delete plan; return cuda_fail(attr_err, "cudaFuncSetAttribute(conv_umma)", __FILE__, __LINE__); }
    *out = plan;
    return PB_OK;
}

void conv_umma_plan_destroy(ConvUmmaPlan* plan) { delete plan; }

int conv_umma_launch_planned(const ConvUmmaPlan* plan, const pb_op_params* p, cudaStream_t st, uint32_t job_id, void* notifier) {
    const Geometry& g = plan->g;
    ConvArgs a;
    a.x = static_cast<const __nv_bfloat16*>(p->x);
    a.residual = static_cast<const __nv_bfloat16*>(p->residual);
    a.bias = p->bias;
    a.y = static_cast<__nv_bfloat16*>(p->y);
    a.err_flag = device_error_flag_ptr(plan->device);
    PB_REQUIRE(a.err_flag != nullptr, "conv_umma: no device error flag");
    a.H = p->H; a.W = p->W; a.Cs = p->Cs; a.P = p->P; a.Q = p->Q; a.M = p->P * p->Q;
    a.K = p->K; a.Ks = p->Ks; a.out_c_off = p->out_c_off; a.res_Cs = p->res_Cs;
    a.R = p->R; a.S = p->S; a.sh = p->stride_h; a.sw = p->stride_w; a.ph = p->pad_h; a.pw = p->pad_w;
    a.act = p->act; a.nkb = g.nkb; a.taps = p->R * p->S; a.BN = g.BN; a.idesc = g.idesc; a.tmem_cols = g.tmem_cols;
    a.b_stage_bytes = g.b_stage_bytes;
    const dim3 grid((unsigned)g.m_tiles, (unsigned)g.n_tiles);
    conv_umma_kernel<<<grid, kThreads, g.smem_bytes, st>>>(plan->tmap, a, job_id, static_cast<FinishedBlockNotifier*>(notifier));
    return launch_check("conv_umma");
}

int conv_umma_launch(const pb_op_params* p, cudaStream_t st, uint32_t job_id, void* notifier) {
    ConvUmmaPlan* plan = nullptr;
    int rc = conv_umma_plan_create(p, p->w, &plan);
    if (rc != PB_OK) return rc;
    rc = conv_umma_launch_planned(plan, p, st, job_id, notifier);
    conv_umma_plan_destroy(plan);   // the tensor map was copied into the launch parameters
    return rc;
}

}  // namespace pb
