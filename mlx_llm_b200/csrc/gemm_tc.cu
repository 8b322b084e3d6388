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
//   warps 0-15 weight producers: packed codes prefetched four stages ahead into registers,
//              dequantised (w = bf16(code*scale+bias), one rounding) and stored with st.shared in
//              the swizzled layout; then a generic->async proxy fence and an mbarrier arrive
//   warp  16   one thread drives TMA (cp.async.bulk.tensor, 128B swizzle, no multicast): the x
//              tile of every stage, and the W tile too when the weights are dense bf16
//   warp  17   one thread issues tcgen05.mma (4 x K=16 per stage) into a 128-lane x 256-column
//              f32 accumulator in TMEM and releases stages with tcgen05.commit (4-stage ring)
//   warps 0-15 epilogue: tcgen05.ld 32 lanes x 32 columns at a time (warp w owns TMEM lanes
//              32*(w%4).. and every 4th column block), then bf16 / residual-add / f32 split-K stores
// Every mbarrier wait is bounded: on expiry the kernel raises an error word, drains and frees its
// TMEM columns instead of spinning forever.
#include <cuda.h>

#include "common.cuh"
#include "kernels.h"

namespace {

constexpr int TM = 128;         // features per CTA (UMMA M)
constexpr int TN = 256;         // tokens per CTA (UMMA N)
constexpr int TK = 64;          // K per stage (one 128-byte swizzled row, one quant group)
constexpr int STAGES = 4;
constexpr int A_BYTES = TM * TK * 2, B_BYTES = TN * TK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int kProducerWarps = 16, kProducerThreads = kProducerWarps * 32;
constexpr int kTmaWarp = kProducerWarps, kMmaWarp = kProducerWarps + 1, kThreads = kProducerThreads + 64;
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
// instruction descriptor: f32 accumulate (bit 4), bf16 x bf16 (bits 7, 10), both K-major, N >> 3 at bit 17, M >> 4 at bit 24

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
    int tile_tokens;  // tokens per CTA (UMMA N), a multiple of 16, <= 256
    float* partial;   // [splits, M, N] f32 when splits > 1
    int* err;         // device error word
};

__device__ __forceinline__ bool mbar_wait_timed(uint32_t addr, uint32_t parity) {
    const long long start = clock64();
    while (true) {
        if (mbar_wait(addr, parity)) return true;
        if (clock64() - start > 4000000000ll) return false;  // ~2 s: give up instead of hanging
    }
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t addr, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(addr), "r"(bytes) : "memory");
}
// 2-D tiled TMA load (no multicast): box lands at `dst`, completion bytes on `mbar`.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t mbar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n" ::"r"(dst),
        "l"(map), "r"(x), "r"(y), "r"(mbar)
        : "memory");
}

template <int WK, int EPI>
__global__ void __launch_bounds__(kThreads, 1)
    gemm_tc_kernel(const GemmParams p, const TcExtra ex, const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w) {
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
    const int tn = ex.tile_tokens;
    const int n0 = blockIdx.x * TM, t0 = blockIdx.y * tn, split = blockIdx.z;
    const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(tn >> 3) << 17) | ((uint32_t)(TM >> 4) << 24);
    const int M = p.M, N = p.N, K = p.K;
    const int KT = K / TK;
    const int kb_begin = (int)((long)split * KT / ex.splits), kb_end = (int)((long)(split + 1) * KT / ex.splits);
    const int n_it = kb_end - kb_begin;
    // arrivals per stage: every dequantising thread, plus the TMA thread's expect_tx arrive
    constexpr uint32_t kFullCount = (WK != 0 ? kProducerThreads : 0) + 1;

    if (tid == 0) {
        for (int s = 0; s < STAGES; s++) {
            mbar_init(full(s), kFullCount);
            mbar_init(empty(s), 1);
        }
        mbar_init(accum, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == kMmaWarp) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(accum + 8), "r"(TN) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp < kProducerWarps) {
        if (WK != 0) {
            // ---------------- weight producers: thread = (feature row, quarter of the 64-wide K slab) ----------------
            constexpr int PREFETCH = 4;
            const int row = tid >> 2, quarter = tid & 3;
            const int gn = n0 + row;
            const int groups = K / 64;
            const uint32_t* wq = reinterpret_cast<const uint32_t*>(p.w) + (size_t)gn * (K * WK / 32);
            uint4 qa[PREFETCH];
            uint32_t sb[PREFETCH];
            auto load_codes = [&](int it, uint4& a, uint32_t& scale_bias) {
                const int kb = kb_begin + it;
                if (WK == 4) {  // 16 codes = 8 bytes
                    const uint2 v = __ldg(reinterpret_cast<const uint2*>(wq + kb * 8 + quarter * 2));
                    a = make_uint4(v.x, v.y, 0, 0);
                } else {        // 16 codes = 16 bytes
                    a = __ldg(reinterpret_cast<const uint4*>(wq + kb * 16 + quarter * 4));
                }
                scale_bias = (uint32_t)__ldg(p.scales + (size_t)gn * groups + kb) | ((uint32_t)__ldg(p.biases + (size_t)gn * groups + kb) << 16);
            };
#pragma unroll
            for (int j = 0; j < PREFETCH; j++) {
                qa[j] = make_uint4(0, 0, 0, 0);
                sb[j] = 0;
                if (j < n_it) load_codes(j, qa[j], sb[j]);
            }
            bool alive = true;
            for (int it0 = 0; it0 < n_it && alive; it0 += PREFETCH) {
#pragma unroll
                for (int jj = 0; jj < PREFETCH; jj++) {
                    const int it = it0 + jj;
                    if (it >= n_it || !alive) break;
                    const int s = it % STAGES;
                    const uint32_t ph = (uint32_t)(it / STAGES) & 1u;
                    const uint32_t sA = base + s * STAGE_BYTES + row * 128;
                    const uint4 c = qa[jj];
                    const uint32_t csc = sb[jj] & 0xffffu, cbi = sb[jj] >> 16;
                    if (it + PREFETCH < n_it) load_codes(it + PREFETCH, qa[jj], sb[jj]);
                    if (!mbar_wait_timed(empty(s), ph ^ 1u)) {
                        alive = false;
                        break;
                    }
                    if (WK == 4) {
                        const uint32_t s2 = csc * 0x10001u, b2 = cbi * 0x10001u;
                        uint32_t o[4];
                        dequant8_q4(c.x, s2, b2, o);
                        sts128(sA + (((quarter * 2) ^ (row & 7)) << 4), o[0], o[1], o[2], o[3]);
                        dequant8_q4(c.y, s2, b2, o);
                        sts128(sA + (((quarter * 2 + 1) ^ (row & 7)) << 4), o[0], o[1], o[2], o[3]);
                    } else {
                        const float sf = __uint_as_float(csc << 16), bf = __uint_as_float(cbi << 16);
                        uint32_t lo[2], hi[2];
                        dequant4_q8(c.x, sf, bf, lo);
                        dequant4_q8(c.y, sf, bf, hi);
                        sts128(sA + (((quarter * 2) ^ (row & 7)) << 4), lo[0], lo[1], hi[0], hi[1]);
                        dequant4_q8(c.z, sf, bf, lo);
                        dequant4_q8(c.w, sf, bf, hi);
                        sts128(sA + (((quarter * 2 + 1) ^ (row & 7)) << 4), lo[0], lo[1], hi[0], hi[1]);
                    }
                    fence_proxy_async();
                    mbar_arrive(full(s));
                }
            }
            if (!alive) {
                *abort_flag = 1;
                atomicExch(ex.err, 1);
            }
        }
    } else if (warp == kTmaWarp) {
        // ---------------- TMA: x tile (and the W tile of dense weights) ----------------
        if (lane == 0) {
            for (int it = 0; it < n_it; it++) {
                const int s = it % STAGES;
                const uint32_t ph = (uint32_t)(it / STAGES) & 1u;
                if (!mbar_wait_timed(empty(s), ph ^ 1u)) {
                    *abort_flag = 1;
                    atomicExch(ex.err, 1);
                    break;
                }
                const uint32_t sA = base + s * STAGE_BYTES, sB = sA + A_BYTES;
                const int kx = (kb_begin + it) * TK;
                mbar_expect_tx(full(s), (uint32_t)(B_BYTES + (WK == 0 ? A_BYTES : 0)));
                tma_load_2d(sB, &map_x, kx, t0, full(s));
                if (WK == 0) tma_load_2d(sA, &map_w, kx, n0, full(s));
            }
        }
        __syncwarp();
    } else {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            for (int it = 0; it < n_it; it++) {
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
                    tc_mma(tmem_base, umma_desc(sA + k * 32), umma_desc(sB + k * 32), idesc, (it > 0 || k > 0) ? 1u : 0u);
                tc_commit(empty(s));
            }
            tc_commit(accum);
        }
        __syncwarp();
    }

    if (warp < kProducerWarps) {
        // ---------------- epilogue ----------------
        bool ok = mbar_wait_timed(accum, 0);
        if (!ok) {
            *abort_flag = 1;
            atomicExch(ex.err, 1);
        }
        tc_fence_after();
        ok = ok && (*abort_flag == 0) && n_it > 0;
        const int lane_grp = warp & 3, col_grp = warp >> 2;
        const int f = n0 + lane_grp * 32 + lane;
        if (ok) {
#pragma unroll 1
            for (int j = col_grp; j * 32 < tn; j += kProducerWarps / 4) {
                if (t0 + j * 32 >= M) break;
                uint32_t v[32];
                tc_ld32(tmem_base + ((uint32_t)(lane_grp * 32) << 16) + (uint32_t)(j * 32), v);
#pragma unroll
                for (int i = 0; i < 32; i++) {
                    const int t = t0 + j * 32 + i;
                    if (t >= M || j * 32 + i >= tn) break;
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
    if (warp == kMmaWarp) {
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

// ---- TMA tensor maps (encoded on the host through the driver entry point; cached) -------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(ptr);
    }
    return fn;
}
struct MapEntry {
    const void* ptr;
    uint64_t rows, k, ld, box_rows;
    int device;
    CUtensorMap map;
};
// bf16 matrix [rows, k] with row stride ld elements; box = 64 (k) x box_rows, 128-byte swizzle, zero fill
int32_t get_map(b2_ctx* ctx, const void* ptr, uint64_t rows, uint64_t k, uint64_t ld, uint32_t box_rows, const CUtensorMap** out) {
    static thread_local std::vector<MapEntry> cache;
    for (auto& e : cache)
        if (e.ptr == ptr && e.rows == rows && e.k == k && e.ld == ld && e.box_rows == box_rows && e.device == ctx->device) {
            *out = &e.map;
            return B2_OK;
        }
    EncodeTiledFn fn = encode_fn();
    B2_REQUIRE(fn != nullptr, B2_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    B2_REQUIRE(((uintptr_t)ptr & 15) == 0 && (ld * 2) % 16 == 0, B2_ERR_UNSUPPORTED, "tcgen05 gemm: operand must be 16-byte aligned");
    if (cache.size() >= 256) cache.clear();
    MapEntry e{ptr, rows, k, ld, box_rows, ctx->device, {}};
    const cuuint64_t dims[2] = {k, rows};
    const cuuint64_t strides[1] = {ld * 2};
    const cuuint32_t box[2] = {(cuuint32_t)TK, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = fn(&e.map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    B2_REQUIRE(r == CUDA_SUCCESS, B2_ERR_CUDA, "cuTensorMapEncodeTiled failed with code " + std::to_string((int)r));
    cache.push_back(e);
    *out = &cache.back().map;
    return B2_OK;
}

template <int WK, int EPI>
int32_t launch_tc(b2_ctx* ctx, const GemmParams& p, int splits, float* partial, int* err) {
    B2_SMEM_ONCE(ctx, (gemm_tc_kernel<WK, EPI>), SMEM_BYTES);
    // token tiles of equal size (a multiple of 16, at most 256) so no CTA runs a mostly empty tile
    const int n_tiles = (p.M + TN - 1) / TN;
    const int tile_tokens = (((p.M + n_tiles - 1) / n_tiles) + 15) / 16 * 16;
    TcExtra ex{splits, tile_tokens, partial, err};
    const CUtensorMap *mx = nullptr, *mw = nullptr;
    const uint64_t x_rows = p.x_rows_cap > p.M ? (uint64_t)p.x_rows_cap : (uint64_t)p.M;
    B2_CHECK(get_map(ctx, p.x, x_rows, (uint64_t)p.K, (uint64_t)p.ldx, TN, &mx));
    CUtensorMap map_x = *mx, map_w = *mx;
    if (WK == 0) {
        B2_CHECK(get_map(ctx, p.w, (uint64_t)p.N, (uint64_t)p.K, (uint64_t)p.K, TM, &mw));
        map_w = *mw;
    }
    dim3 grid(p.N / TM, n_tiles, splits);
    gemm_tc_kernel<WK, EPI><<<grid, kThreads, SMEM_BYTES, ctx->stream>>>(p, ex, map_x, map_w);
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
    return p.M > 64 && p.N % TM == 0 && p.K % TK == 0 && p.ldx % 8 == 0 && ((uintptr_t)p.x & 15) == 0 &&
           (p.bits == 4 || p.bits == 8 || (p.bits == 0 && ((uintptr_t)p.w & 15) == 0));
}

int32_t b2_gemm_tc_launch(b2_ctx* ctx, const GemmParams& p) {
    // Split K only when the (feature, token) tiles cannot even fill one wave of SMs (o_proj / down_proj
    // at a few hundred tokens): the f32 partial sums cost a write and a read of splits*M*N*4 bytes, which
    // wipes out the gain as soon as the plain grid already covers the machine.
    const int tiles = (p.N / TM) * ((p.M + TN - 1) / TN);
    const int KT = p.K / TK;
    int best = 1;
    if (tiles * 10 <= ctx->sm_count * 7) {
        double best_eff = (double)tiles / ctx->sm_count;
        for (int s = 2; s <= 4 && s * 16 <= KT; s++) {
            const int ctas = tiles * s;
            const double eff = (double)ctas / (((ctas + ctx->sm_count - 1) / ctx->sm_count) * ctx->sm_count);
            if (eff > best_eff + 0.1) {
                best_eff = eff;
                best = s;
            }
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
