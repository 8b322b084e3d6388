// y[M,N] = x[M,K] . W[N,K]^T for dense bf16 and MLX-format group-64 affine Q4/Q8 weights.
//
// Replaces primitives::nn::linear (src/primitives/nn.rs:26-33) and QuantizedLinear::forward
// (src/primitives/quant.rs:56-70 -> mlx quantized_matmul(transpose=true)).
//
// Weight format (MLX affine): row-major [N, K*bits/32] u32, codes along K lowest bits first
// (8 nibbles or 4 bytes per word); scales/biases [N, K/64] bf16.  The dequantised weight is
//     w = bf16_rne(code * scale + bias)      (one rounding: fma.rn.bf16x2 / fmaf + cvt.rn)
// which is bit-identical to the standalone dequantize entry point.
//
// This file holds the general tile kernel: CTA tile BM x 128 x 64 (BM = 64 or 128 tokens), 8 warps,
// mma.sync m16n8k16 bf16 with f32 accumulation, x tiles by cp.async, quantised weight tiles
// dequantised from registers into XOR-swizzled shared memory (one K tile == one quant group).
#include "common.cuh"
#include "kernels.h"

namespace {

constexpr int BN = 128, BK = 64, kThreads = 256;

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

// 8 nibbles of `w` -> 8 dequantised bf16 in natural order, as 4 packed pairs.
__device__ __forceinline__ void dequant8_q4(uint32_t w, uint32_t s2, uint32_t b2, uint32_t (&out)[4]) {
    const uint32_t magic = 0x43004300u;  // bf16 128.0 in both halves; 128 + c is exact for c < 128
    uint32_t r0 = (w & 0x000f000fu) | magic;          // (c0, c4)
    uint32_t r1 = ((w >> 4) & 0x000f000fu) | magic;   // (c1, c5)
    uint32_t r2 = ((w >> 8) & 0x000f000fu) | magic;   // (c2, c6)
    uint32_t r3 = ((w >> 12) & 0x000f000fu) | magic;  // (c3, c7)
    r0 = fma_bf2(sub_bf2(r0, magic), s2, b2);
    r1 = fma_bf2(sub_bf2(r1, magic), s2, b2);
    r2 = fma_bf2(sub_bf2(r2, magic), s2, b2);
    r3 = fma_bf2(sub_bf2(r3, magic), s2, b2);
    out[0] = prmt(r0, r1, 0x5410u);  // (c0, c1)
    out[1] = prmt(r2, r3, 0x5410u);  // (c2, c3)
    out[2] = prmt(r0, r1, 0x7632u);  // (c4, c5)
    out[3] = prmt(r2, r3, 0x7632u);  // (c6, c7)
}
// 4 bytes of `w` -> 4 dequantised bf16 as 2 packed pairs (f32 fma, one rounding).
__device__ __forceinline__ void dequant4_q8(uint32_t w, float s, float b, uint32_t (&out)[2]) {
    float c0 = (float)(w & 0xffu), c1 = (float)((w >> 8) & 0xffu), c2 = (float)((w >> 16) & 0xffu), c3 = (float)(w >> 24);
    out[0] = pack_bf2(__fmaf_rn(c0, s, b), __fmaf_rn(c1, s, b));
    out[1] = pack_bf2(__fmaf_rn(c2, s, b), __fmaf_rn(c3, s, b));
}

template <int WK /*0 dense, 4, 8*/, int BM, int EPI>
__global__ void __launch_bounds__(kThreads) gemm_tile_kernel(const GemmParams p) {
    constexpr int WM = BM / 2;       // warp tile rows (tokens)
    constexpr int MT = WM / 16;      // m16 tiles per warp
    constexpr int NT = 4;            // n8 tiles per warp (warp tile 32 outputs)
    constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2;
    extern __shared__ __align__(128) uint8_t smem[];
    const uint32_t sA = smem_u32(smem), sB = sA + 2 * A_BYTES;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int warp_m = warp >> 2, warp_n = warp & 3;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int M = p.M, N = p.N, K = p.K;
    const int KT = (K + BK - 1) / BK;
    const uint16_t* x = p.x;

    float acc[MT][NT][4];
#pragma unroll
    for (int i = 0; i < MT; i++)
#pragma unroll
        for (int j = 0; j < NT; j++) acc[i][j][0] = acc[i][j][1] = acc[i][j][2] = acc[i][j][3] = 0.f;

    auto load_a = [&](int kt, int stage) {
#pragma unroll
        for (int c = tid; c < BM * 8; c += kThreads) {
            const int r = c >> 3, cc = c & 7;
            const int gm = m0 + r, gk = kt * BK + cc * 8;
            const bool ok = gm < M && gk < K;
            const uint16_t* src = x + (size_t)(ok ? gm : 0) * p.ldx + (ok ? gk : 0);
            cp_async16_zfill(sA + stage * A_BYTES + r * 128 + ((cc ^ (r & 7)) << 4), src, ok);
        }
    };
    auto load_b_dense = [&](int kt, int stage) {
        const uint16_t* w = reinterpret_cast<const uint16_t*>(p.w);
#pragma unroll
        for (int c = tid; c < BN * 8; c += kThreads) {
            const int r = c >> 3, cc = c & 7;
            const int gn = n0 + r, gk = kt * BK + cc * 8;
            const bool ok = gn < N && gk < K;
            const uint16_t* src = w + (size_t)(ok ? gn : 0) * K + (ok ? gk : 0);
            cp_async16_zfill(sB + stage * B_BYTES + r * 128 + ((cc ^ (r & 7)) << 4), src, ok);
        }
    };
    // quantised weights: thread -> (row = tid/2, half = tid%2) = 32 codes of one group
    const int qrow = tid >> 1, qhalf = tid & 1;
    const int gnq = n0 + qrow;
    const bool qok = gnq < N;
    uint4 qreg[WK == 8 ? 2 : 1];
    uint32_t qsb = 0;  // packed (scale, bias) bf16
    auto ldg_b_quant = [&](int kt) {
        if (WK == 0) return;
        const int words_per_row = K * WK / 32;
        const uint32_t* wrow = reinterpret_cast<const uint32_t*>(p.w) + (size_t)(qok ? gnq : 0) * words_per_row;
        const int groups = K / 64;
        if (WK == 4) {
            qreg[0] = qok ? *reinterpret_cast<const uint4*>(wrow + kt * 8 + qhalf * 4) : make_uint4(0, 0, 0, 0);
        } else {
            qreg[0] = qok ? *reinterpret_cast<const uint4*>(wrow + kt * 16 + qhalf * 8) : make_uint4(0, 0, 0, 0);
            qreg[WK == 8 ? 1 : 0] = qok ? *reinterpret_cast<const uint4*>(wrow + kt * 16 + qhalf * 8 + 4) : make_uint4(0, 0, 0, 0);
        }
        const uint32_t s = qok ? p.scales[(size_t)gnq * groups + kt] : 0, b = qok ? p.biases[(size_t)gnq * groups + kt] : 0;
        qsb = s | (b << 16);
    };
    auto sts_b_quant = [&](int stage) {
        if (WK == 0) return;
        const uint32_t base = sB + stage * B_BYTES + qrow * 128;
        if (WK == 4) {
            const uint32_t s2 = (qsb & 0xffffu) * 0x10001u, b2 = (qsb >> 16) * 0x10001u;
            const uint32_t wds[4] = {qreg[0].x, qreg[0].y, qreg[0].z, qreg[0].w};
#pragma unroll
            for (int i = 0; i < 4; i++) {
                uint32_t o[4];
                dequant8_q4(wds[i], s2, b2, o);
                const int cc = qhalf * 4 + i;  // 16-byte chunk (8 elements) within the 64-wide K tile
                asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};\n" ::"r"(base + ((cc ^ (qrow & 7)) << 4)), "r"(o[0]), "r"(o[1]),
                             "r"(o[2]), "r"(o[3]));
            }
        } else {
            const float s = bflo(qsb), b = bfhi(qsb);
            const uint32_t wds[8] = {qreg[0].x, qreg[0].y, qreg[0].z, qreg[0].w, qreg[WK == 8 ? 1 : 0].x, qreg[WK == 8 ? 1 : 0].y,
                                     qreg[WK == 8 ? 1 : 0].z, qreg[WK == 8 ? 1 : 0].w};
#pragma unroll
            for (int i = 0; i < 4; i++) {
                uint32_t lo[2], hi[2];
                dequant4_q8(wds[2 * i], s, b, lo);
                dequant4_q8(wds[2 * i + 1], s, b, hi);
                const int cc = qhalf * 4 + i;
                asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};\n" ::"r"(base + ((cc ^ (qrow & 7)) << 4)), "r"(lo[0]), "r"(lo[1]),
                             "r"(hi[0]), "r"(hi[1]));
            }
        }
    };

    // prologue
    load_a(0, 0);
    if (WK == 0) load_b_dense(0, 0);
    cp_async_commit();
    if (WK != 0) {
        ldg_b_quant(0);
        sts_b_quant(0);
    }

    const int mi = lane >> 3, lr = lane & 7;
    for (int kt = 0; kt < KT; kt++) {
        const int stage = kt & 1;
        if (kt + 1 < KT) {
            load_a(kt + 1, stage ^ 1);
            if (WK == 0) load_b_dense(kt + 1, stage ^ 1);
            if (WK != 0) ldg_b_quant(kt + 1);
        }
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();

        const uint32_t a_base = sA + stage * A_BYTES, b_base = sB + stage * B_BYTES;
#pragma unroll
        for (int ks = 0; ks < BK / 16; ks++) {
            uint32_t bf[NT][2];
#pragma unroll
            for (int np = 0; np < NT / 2; np++) {
                // matrices: (n 0-7, k lo), (n 0-7, k hi), (n 8-15, k lo), (n 8-15, k hi)
                const int r = warp_n * 32 + np * 16 + lr + (mi >> 1) * 8;
                const int ch = 2 * ks + (mi & 1);
                ldmatrix_x4(bf[2 * np][0], bf[2 * np][1], bf[2 * np + 1][0], bf[2 * np + 1][1], b_base + r * 128 + ((ch ^ (r & 7)) << 4));
            }
#pragma unroll
            for (int mt = 0; mt < MT; mt++) {
                // matrices: (m 0-7, k lo), (m 8-15, k lo), (m 0-7, k hi), (m 8-15, k hi)
                const int r = warp_m * WM + mt * 16 + lr + (mi & 1) * 8;
                const int ch = 2 * ks + (mi >> 1);
                uint32_t af[4];
                ldmatrix_x4(af[0], af[1], af[2], af[3], a_base + r * 128 + ((ch ^ (r & 7)) << 4));
#pragma unroll
                for (int nt = 0; nt < NT; nt++) mma_bf16_16816(acc[mt][nt], af, bf[nt]);
            }
        }
        if (WK != 0 && kt + 1 < KT) sts_b_quant(stage ^ 1);
        __syncthreads();
    }

    // epilogue
    const int g = lane >> 2, t = lane & 3;
#pragma unroll
    for (int mt = 0; mt < MT; mt++)
#pragma unroll
        for (int nt = 0; nt < NT; nt++)
#pragma unroll
            for (int hh = 0; hh < 2; hh++) {
                const int gm = m0 + warp_m * WM + mt * 16 + g + hh * 8;
                const int gn = n0 + warp_n * 32 + nt * 8 + 2 * t;
                if (gm >= M || gn >= N) continue;
                const float v0 = acc[mt][nt][2 * hh], v1 = acc[mt][nt][2 * hh + 1];
                const size_t o = (size_t)gm * p.ldo + gn;
                if (EPI == EPI_F32) {
                    float* dst = gemm_f32_dst(p, gm, gn);  // gn is even and the chunk a multiple of 4: both columns in one chunk
                    dst[0] = v0;
                    if (gn + 1 < N) dst[1] = v1;
                } else if (EPI == EPI_BF16) {
                    if (gn + 1 < N)
                        *reinterpret_cast<uint32_t*>(p.out + o) = pack_bf2(v0, v1);
                    else
                        p.out[o] = f2bf(v0);
                } else {  // EPI_BF16_RESADD: residual stream h = bf16(res + bf16(y))
                    const size_t ro = (size_t)gm * p.ldres + gn;
                    if (gn + 1 < N) {
                        const uint32_t r = *reinterpret_cast<const uint32_t*>(p.res + ro);
                        *reinterpret_cast<uint32_t*>(p.out + o) = pack_bf2(bflo(r) + rbf(v0), bfhi(r) + rbf(v1));
                    } else {
                        p.out[o] = f2bf(bf2f(p.res[ro]) + rbf(v0));
                    }
                }
            }
}

template <int WK, int BM, int EPI>
int32_t launch_tile(b2_ctx* ctx, const GemmParams& p) {
    const int smem = 2 * (BM * BK * 2) + 2 * (BN * BK * 2);
    B2_SMEM_ONCE(ctx, (gemm_tile_kernel<WK, BM, EPI>), smem);
    dim3 grid((p.N + BN - 1) / BN, (p.M + BM - 1) / BM);
    gemm_tile_kernel<WK, BM, EPI><<<grid, kThreads, smem, ctx->stream>>>(p);
    B2_LAUNCHED(ctx);
    B2_CUDA(cudaGetLastError());
    return B2_OK;
}

template <int WK, int BM>
int32_t dispatch_epi(b2_ctx* ctx, const GemmParams& p) {
    switch (p.epilogue) {
        case EPI_BF16: return launch_tile<WK, BM, EPI_BF16>(ctx, p);
        case EPI_BF16_RESADD: return launch_tile<WK, BM, EPI_BF16_RESADD>(ctx, p);
        case EPI_F32: return launch_tile<WK, BM, EPI_F32>(ctx, p);
    }
    return b2_fail(B2_ERR_MSG, "gemm: bad epilogue");
}

template <int WK>
int32_t dispatch_bm(b2_ctx* ctx, const GemmParams& p) {
    if (p.M <= 64) return dispatch_epi<WK, 64>(ctx, p);
    return dispatch_epi<WK, 128>(ctx, p);
}

}  // namespace

int32_t b2_gemm_launch(b2_ctx* ctx, const GemmParams& p) {
    B2_REQUIRE(p.M >= 0 && p.N > 0 && p.K > 0, B2_ERR_MSG, "gemm: bad shape");
    if (p.M == 0) return B2_OK;
    ctx->gemm_flops += 2.0 * p.M * (double)p.N * p.K;
    ctx->gemm_weight_bytes += p.bits ? (double)p.N * p.K * p.bits / 8 + (double)p.N * (p.K / 64) * 4 : (double)p.N * p.K * 2;
    B2_REQUIRE(p.K % 8 == 0, B2_ERR_UNSUPPORTED, "gemm: K must be a multiple of 8");
    B2_REQUIRE(p.ldx % 8 == 0, B2_ERR_UNSUPPORTED, "gemm: activation row stride must be a multiple of 8 elements");
    if (p.bits != 0) {
        B2_REQUIRE(p.group == 64, B2_ERR_UNSUPPORTED, "gemm: only group size 64 is supported for quantized weights");
        B2_REQUIRE(p.K % 64 == 0, B2_ERR_UNSUPPORTED, "gemm: K must be a multiple of the group size");
        B2_REQUIRE(p.bits == 4 || p.bits == 8, B2_ERR_UNSUPPORTED, "gemm: bits must be 4 or 8");
    }
    // Up to 32 tokens the weight-streaming kernel wins; from 33 on the tcgen05 kernel does where its tiling fits (one
    // 16-token-granular block costs it the same as a full one, while the streaming kernel's cost grows with the tokens);
    // the streaming kernel keeps 33..64 tokens for the shapes the tcgen05 tiling does not take.
    const bool tc_ok = ctx->use_tc && b2_gemm_tc_eligible(p);
    if (ctx->use_tc && b2_gemm_stream_eligible(p) && !tc_ok) return b2_gemm_stream_launch(ctx, p);
    if (tc_ok) return b2_gemm_tc_launch(ctx, p);
    if (p.bits == 0) return dispatch_bm<0>(ctx, p);
    B2_REQUIRE(p.group == 64, B2_ERR_UNSUPPORTED, "gemm: only group size 64 is supported for quantized weights");
    B2_REQUIRE(p.K % 64 == 0, B2_ERR_UNSUPPORTED, "gemm: K must be a multiple of the group size");
    if (p.bits == 4) return dispatch_bm<4>(ctx, p);
    if (p.bits == 8) return dispatch_bm<8>(ctx, p);
    return b2_fail(B2_ERR_UNSUPPORTED, "gemm: bits must be 4 or 8");
}
