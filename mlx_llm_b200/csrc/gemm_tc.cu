// Large-M projection GEMM on the 5th-generation tensor cores (tcgen05 + TMEM), sm_100a only.
//
//   y[M, N] = x[M, K] . W[N, K]^T,   W dense bf16 or MLX-format group-64 affine Q4 / Q8
//
// Same contract as the warp-level tile kernel in gemm.cu (it replaces primitives::nn::linear,
// src/primitives/nn.rs:26-33, and QuantizedLinear::forward, src/primitives/quant.rs:56-70); this one
// takes over once a step carries enough tokens for the tensor pipe to be the bound (prefill chunks
// packed with decode tokens).
//
// CTA tile: 128 output features (UMMA M, operand A = W) x 256 tokens (UMMA N, operand B = x) x
// K/splits.  Both operands sit in shared memory K-major with the 128-byte swizzle of the canonical
// UMMA layout (row = 64 bf16 = 128 B, 8-row groups 1024 B apart, 16-byte chunk c of row r stored
// at c ^ (r & 7)).
//   warps 0-7  producers: x tile by cp.async; W tile dequantised in registers
//              (w = bf16(code*scale+bias), one rounding) and stored with st.shared; then a
//              generic->async proxy fence and an mbarrier arrive per stage (4-stage ring)
//   warp  8    one elected thread issues tcgen05.mma (4 x K=16 per stage) into a 128-lane x
//              256-column f32 accumulator in TMEM and releases stages with tcgen05.commit
//   warps 0-3  epilogue: tcgen05.ld 32 lanes x 32 columns at a time, then bf16 / residual-add /
//              f32 split-K partial stores
// Every mbarrier wait is bounded: on expiry the kernel raises an error word, drains and frees its
// TMEM columns instead of spinning forever.
#include "common.cuh"
#include "kernels.h"

namespace {

constexpr int TM = 128;         // features per CTA (UMMA M)
constexpr int TN = 256;         // tokens per CTA (UMMA N)
constexpr int TK = 64;          // K per stage (one 128-byte swizzled row, one quant group)
constexpr int STAGES = 4;
constexpr int A_BYTES = TM * TK * 2, B_BYTES = TN * TK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int kProducerThreads = 256, kThreads = kProducerThreads + 32;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;
constexpr uint32_t kSpinLimit = 64;  // try_wait attempts between two looks at the clock

__device__ __forceinline__ void mbar_init(uint32_t addr, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(addr), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint32_t addr) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(addr) : "memory");
}
// Bounded wait; returns false when the limit ran out.
__device__ __forceinline__ bool mbar_wait(uint32_t addr, uint32_t parity) {
    for (uint32_t i = 0; i < kSpinLimit; i++) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}\n"
            : "=r"(ok)
            : "r"(addr), "r"(parity)
            : "memory");
        if (ok) return true;
    }
    return false;
}
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t mbar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(mbar) : "memory");
}
__device__ __forceinline__ void tc_mma(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n" ::"r"(tmem_d),
        "l"(da), "l"(db), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]),
          "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]),
          "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]),
          "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
}

// K-major, 128-byte swizzle, rows of 128 B, 8-row groups 1024 B apart (SBO = 64 x 16 B), LBO unused (1),
// descriptor version 1 (bit 46), layout type 2 = SWIZZLE_128B (bits 61-63).
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr) {
    return (uint64_t)((smem_addr >> 4) & 0x3fff) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
// f32 accumulate, bf16 x bf16, both K-major, N = 256 (>>3 at bit 17), M = 128 (>>4 at bit 24)
constexpr uint32_t kIdesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(TN >> 3) << 17) | ((uint32_t)(TM >> 4) << 24);

__device__ __forceinline__ uint32_t sub_bf2(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("sub.rn.bf16x2 %0, %1, %2;\n" : "=r"(d) : "r"(a), "r"(b));
    return d;
}
__device__ __forceinline__ uint32_t fma_bf2(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("fma.rn.bf16x2 %0, %1, %2, %3;\n" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;\n" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}
__device__ __forceinline__ void sts128(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};\n" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
// 8 nibbles -> 8 bf16 in natural order (see gemm.cu for the derivation; bit-identical result)
__device__ __forceinline__ void dequant8_q4(uint32_t w, uint32_t s2, uint32_t b2, uint32_t (&out)[4]) {
    const uint32_t magic = 0x43004300u;
    uint32_t r0 = (w & 0x000f000fu) | magic, r1 = ((w >> 4) & 0x000f000fu) | magic;
    uint32_t r2 = ((w >> 8) & 0x000f000fu) | magic, r3 = ((w >> 12) & 0x000f000fu) | magic;
    r0 = fma_bf2(sub_bf2(r0, magic), s2, b2);
    r1 = fma_bf2(sub_bf2(r1, magic), s2, b2);
    r2 = fma_bf2(sub_bf2(r2, magic), s2, b2);
    r3 = fma_bf2(sub_bf2(r3, magic), s2, b2);
    out[0] = prmt(r0, r1, 0x5410u);
    out[1] = prmt(r2, r3, 0x5410u);
    out[2] = prmt(r0, r1, 0x7632u);
    out[3] = prmt(r2, r3, 0x7632u);
}
__device__ __forceinline__ void dequant4_q8(uint32_t w, float s, float b, uint32_t (&out)[2]) {
    const float c0 = (float)(w & 0xffu), c1 = (float)((w >> 8) & 0xffu), c2 = (float)((w >> 16) & 0xffu), c3 = (float)(w >> 24);
    out[0] = pack_bf2(__fmaf_rn(c0, s, b), __fmaf_rn(c1, s, b));
    out[1] = pack_bf2(__fmaf_rn(c2, s, b), __fmaf_rn(c3, s, b));
}

struct TcExtra {
    int splits;
    float* partial;  // [splits, M, N] f32 when splits > 1
    int* err;        // device error word
};

__device__ __forceinline__ bool mbar_wait_timed(uint32_t addr, uint32_t parity) {
    const long long start = clock64();
    while (true) {
        if (mbar_wait(addr, parity)) return true;
        if (clock64() - start > 4000000000ll) return false;  // ~2 s: give up instead of hanging
    }
}

template <int WK, int EPI>
__global__ void __launch_bounds__(kThreads, 1) gemm_tc_kernel(const GemmParams p, const TcExtra ex) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    const uint32_t bar = base + STAGES * STAGE_BYTES;
    auto full = [&](int s) { return bar + 8u * s; };
    auto empty = [&](int s) { return bar + 8u * (STAGES + s); };
    const uint32_t accum = bar + 8u * (2 * STAGES);
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem_raw + (accum + 8 - raw));
    volatile uint32_t* abort_flag = tmem_slot + 1;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n0 = blockIdx.x * TM, t0 = blockIdx.y * TN, split = blockIdx.z;
    const int M = p.M, N = p.N, K = p.K;
    const int KT = K / TK;
    const int kb_begin = (int)((long)split * KT / ex.splits), kb_end = (int)((long)(split + 1) * KT / ex.splits);

    if (tid == 0) {
        for (int s = 0; s < STAGES; s++) {
            mbar_init(full(s), kProducerThreads);
            mbar_init(empty(s), 1);
        }
        mbar_init(accum, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 8) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(accum + 8), "r"(TN) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp < 8) {
        // ---------------- producers ----------------
        const int row = tid >> 1, half = tid & 1;
        const int gn = n0 + row;
        const int groups = K / 64;
        const uint32_t* wq = nullptr;
        if (WK != 0) wq = reinterpret_cast<const uint32_t*>(p.w) + (size_t)gn * (K * WK / 32);
        int it = 0;
        for (int kb = kb_begin; kb < kb_end; kb++, it++) {
            const int s = it % STAGES;
            const uint32_t ph = (uint32_t)(it / STAGES) & 1u;
            // weight codes and group parameters first: their latency overlaps the wait below
            uint4 q0 = make_uint4(0, 0, 0, 0), q1 = make_uint4(0, 0, 0, 0);
            uint32_t sc = 0, bi = 0;
            if (WK == 4) {
                q0 = __ldg(reinterpret_cast<const uint4*>(wq + kb * 8 + half * 4));
            } else if (WK == 8) {
                q0 = __ldg(reinterpret_cast<const uint4*>(wq + kb * 16 + half * 8));
                q1 = __ldg(reinterpret_cast<const uint4*>(wq + kb * 16 + half * 8 + 4));
            }
            if (WK != 0) {
                sc = __ldg(p.scales + (size_t)gn * groups + kb);
                bi = __ldg(p.biases + (size_t)gn * groups + kb);
            }
            if (!mbar_wait_timed(empty(s), ph ^ 1u)) {
                *abort_flag = 1;
                atomicExch(ex.err, 1);
                break;
            }
            const uint32_t sA = base + s * STAGE_BYTES, sB = sA + A_BYTES;
#pragma unroll
            for (int j = 0; j < TN * 8 / kProducerThreads; j++) {
                const int c = tid + kProducerThreads * j;
                const int r = c >> 3, cc = c & 7;
                const int gm = t0 + r;
                const bool ok = gm < M;
                const uint16_t* src = p.x + (size_t)(ok ? gm : 0) * p.ldx + kb * TK + cc * 8;
                cp_async16_zfill(sB + r * 128 + ((cc ^ (r & 7)) << 4), src, ok);
            }
            if (WK == 0) {
                const uint16_t* wd = reinterpret_cast<const uint16_t*>(p.w);
#pragma unroll
                for (int j = 0; j < TM * 8 / kProducerThreads; j++) {
                    const int c = tid + kProducerThreads * j;
                    const int r = c >> 3, cc = c & 7;
                    cp_async16(sA + r * 128 + ((cc ^ (r & 7)) << 4), wd + (size_t)(n0 + r) * K + kb * TK + cc * 8);
                }
            }
            cp_async_commit();
            if (WK == 4) {
                const uint32_t s2 = sc * 0x10001u, b2 = bi * 0x10001u;
                const uint32_t wds[4] = {q0.x, q0.y, q0.z, q0.w};
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    uint32_t o[4];
                    dequant8_q4(wds[i], s2, b2, o);
                    const int cc = half * 4 + i;
                    sts128(sA + row * 128 + ((cc ^ (row & 7)) << 4), o[0], o[1], o[2], o[3]);
                }
            } else if (WK == 8) {
                const float sf = __uint_as_float(sc << 16), bf = __uint_as_float(bi << 16);
                const uint32_t wds[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    uint32_t lo[2], hi[2];
                    dequant4_q8(wds[2 * i], sf, bf, lo);
                    dequant4_q8(wds[2 * i + 1], sf, bf, hi);
                    const int cc = half * 4 + i;
                    sts128(sA + row * 128 + ((cc ^ (row & 7)) << 4), lo[0], lo[1], hi[0], hi[1]);
                }
            }
            cp_async_wait<0>();
            fence_proxy_async();
            mbar_arrive(full(s));
        }
    } else {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            int it = 0;
            for (int kb = kb_begin; kb < kb_end; kb++, it++) {
                const int s = it % STAGES;
                const uint32_t ph = (uint32_t)(it / STAGES) & 1u;
                if (!mbar_wait_timed(full(s), ph)) {
                    *abort_flag = 1;
                    atomicExch(ex.err, 1);
                    break;
                }
                tc_fence_after();
                const uint32_t sA = base + s * STAGE_BYTES, sB = sA + A_BYTES;
#pragma unroll
                for (int k = 0; k < TK / 16; k++)
                    tc_mma(tmem_base, umma_desc(sA + k * 32), umma_desc(sB + k * 32), kIdesc, (it > 0 || k > 0) ? 1u : 0u);
                tc_commit(empty(s));
            }
            tc_commit(accum);
        }
        __syncwarp();
    }

    if (warp < 4) {
        // ---------------- epilogue ----------------
        bool ok = mbar_wait_timed(accum, 0);
        if (!ok) {
            *abort_flag = 1;
            atomicExch(ex.err, 1);
        }
        tc_fence_after();
        ok = ok && (*abort_flag == 0) && kb_end > kb_begin;
        const int f = n0 + warp * 32 + lane;
        if (ok) {
#pragma unroll 1
            for (int j = 0; j < TN / 32; j++) {
                if (t0 + j * 32 >= M) break;
                uint32_t v[32];
                tc_ld32(tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)(j * 32), v);
#pragma unroll
                for (int i = 0; i < 32; i++) {
                    const int t = t0 + j * 32 + i;
                    if (t >= M) break;
                    const float a = __uint_as_float(v[i]);
                    if (ex.splits > 1) {
                        ex.partial[((size_t)split * M + t) * N + f] = a;
                    } else if (EPI == EPI_F32) {
                        p.out_f32[(size_t)t * p.ldo + f] = a;
                    } else if (EPI == EPI_BF16) {
                        p.out[(size_t)t * p.ldo + f] = f2bf(a);
                    } else {
                        p.out[(size_t)t * p.ldo + f] = f2bf(bf2f(p.res[(size_t)t * p.ldres + f]) + rbf(a));
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 8) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(TN) : "memory");
    }
}

// out = epilogue(sum over splits of partial)
template <int EPI>
__global__ void splitk_reduce_kernel(const GemmParams p, const float* __restrict__ partial, int splits) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t total = (size_t)p.M * p.N;
    if (i >= total) return;
    float a = 0.f;
    for (int z = 0; z < splits; z++) a += partial[(size_t)z * total + i];
    const int t = (int)(i / p.N), f = (int)(i % p.N);
    if (EPI == EPI_F32)
        p.out_f32[(size_t)t * p.ldo + f] = a;
    else if (EPI == EPI_BF16)
        p.out[(size_t)t * p.ldo + f] = f2bf(a);
    else
        p.out[(size_t)t * p.ldo + f] = f2bf(bf2f(p.res[(size_t)t * p.ldres + f]) + rbf(a));
}

template <int WK, int EPI>
int32_t launch_tc(b2_ctx* ctx, const GemmParams& p, int splits, float* partial, int* err) {
    B2_SMEM_ONCE(ctx, (gemm_tc_kernel<WK, EPI>), SMEM_BYTES);
    TcExtra ex{splits, partial, err};
    dim3 grid(p.N / TM, (p.M + TN - 1) / TN, splits);
    gemm_tc_kernel<WK, EPI><<<grid, kThreads, SMEM_BYTES, ctx->stream>>>(p, ex);
    B2_LAUNCHED(ctx);
    if (splits > 1) {
        const size_t total = (size_t)p.M * p.N;
        splitk_reduce_kernel<EPI><<<(unsigned)((total + 255) / 256), 256, 0, ctx->stream>>>(p, partial, splits);
        B2_LAUNCHED(ctx);
    }
    B2_CUDA(cudaGetLastError());
    return B2_OK;
}

template <int WK>
int32_t dispatch_tc(b2_ctx* ctx, const GemmParams& p, int splits, float* partial, int* err) {
    switch (p.epilogue) {
        case EPI_BF16: return launch_tc<WK, EPI_BF16>(ctx, p, splits, partial, err);
        case EPI_BF16_RESADD: return launch_tc<WK, EPI_BF16_RESADD>(ctx, p, splits, partial, err);
        case EPI_F32: return launch_tc<WK, EPI_F32>(ctx, p, splits, partial, err);
    }
    return b2_fail(B2_ERR_MSG, "gemm: bad epilogue");
}

}  // namespace

bool b2_gemm_tc_eligible(const GemmParams& p) {
    return p.M > 64 && p.N % TM == 0 && p.K % TK == 0 && p.ldx % 8 == 0 && (p.bits == 0 || p.bits == 4 || p.bits == 8);
}

int32_t b2_gemm_tc_launch(b2_ctx* ctx, const GemmParams& p) {
    // split K when the (feature, token) tiles alone leave SMs idle: pick the split count with the
    // best wave efficiency, smallest first
    const int tiles = (p.N / TM) * ((p.M + TN - 1) / TN);
    const int KT = p.K / TK;
    int best = 1;
    double best_eff = 0;
    for (int s = 1; s <= 4 && s * 8 <= KT; s++) {
        const int ctas = tiles * s;
        const double eff = (double)ctas / (((ctas + ctx->sm_count - 1) / ctx->sm_count) * ctx->sm_count);
        if (eff > best_eff + 0.05) {
            best_eff = eff;
            best = s;
        }
    }
    float* partial = nullptr;
    if (best > 1) {
        const size_t bytes = (size_t)best * p.M * p.N * sizeof(float);
        if (bytes > ctx->tc_partial_bytes) {
            B2_CUDA(cudaStreamSynchronize(ctx->stream));
            if (ctx->tc_partial) B2_CUDA(cudaFree(ctx->tc_partial));
            ctx->tc_partial = nullptr;
            B2_CUDA(cudaMalloc((void**)&ctx->tc_partial, bytes + (bytes >> 2)));
            ctx->tc_partial_bytes = bytes + (bytes >> 2);
        }
        partial = ctx->tc_partial;
    }
    if (!ctx->dev_err) {
        B2_CUDA(cudaMalloc((void**)&ctx->dev_err, 16));
        B2_CUDA(cudaMemsetAsync(ctx->dev_err, 0, 16, ctx->stream));
    }
    if (p.bits == 0) return dispatch_tc<0>(ctx, p, best, partial, ctx->dev_err);
    if (p.bits == 4) return dispatch_tc<4>(ctx, p, best, partial, ctx->dev_err);
    return dispatch_tc<8>(ctx, p, best, partial, ctx->dev_err);
}
