// Small-M projection (decode steps, up to 64 tokens): a weight-streaming kernel bound by HBM.
//
//   y[M, N] = x[M, K] . W[N, K]^T,   W dense bf16 or MLX-format group-64 affine Q4 / Q8,   M <= 64
//
// Same contract as the tile kernel in gemm.cu (it replaces primitives::nn::linear, src/primitives/nn.rs:26-33,
// and QuantizedLinear::forward, src/primitives/quant.rs:56-70).  With a handful of tokens every weight byte is
// used once, so the only thing that matters is to keep enough 16-byte weight loads in flight on every SM and
// to touch nothing else in HBM.
//
// Orientation: the weights are the A operand of mma.sync m16n8k16 (16 feature rows x 16 K), the tokens the
// 8-wide N side, so a feature row's packed codes go from global memory to registers to the tensor core with
// no shared-memory round trip: a thread loads 16 bytes of one row (32 Q4 codes, 16 Q8 codes or 8 bf16),
// dequantises them (w = bf16(code*scale+bias), one rounding, as everywhere in this library) and holds exactly
// the A-fragment elements of its (row, K) positions.  The K order inside an MMA is free as long as both
// operands agree, so the activations are stored in shared memory in the permuted order that makes a thread's
// B-fragment for K step s one 8-byte load (see `perm` below).
//
// CTA = 4 warps x 32 feature rows (two 16-row MMA tiles per warp, sharing every B fragment) = 128 rows, over
// one K range; the activations of the range pass through a double-buffered shared-memory chunk of 256 K.
// K is split over CTAs (grid.y) until the grid fills every CTA slot of the machine; with more than one range the
// f32 partial sums go to scratch; up to 16 tokens the CTA of a row tile that finishes last adds them (in range
// order) and applies the epilogue, so a projection is one launch; beyond that a second kernel does it with the
// whole machine.
#include "common.cuh"
#include "kernels.h"

namespace {

constexpr int ROWS_PER_CTA = 128, KC = 256, kThreads = 128;
constexpr int XS_STRIDE = KC * 2 + 32;  // bytes per token row of a chunk: 8 rows x 32 B of skew cover all banks

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
// 8 nibbles -> 8 bf16 in natural order as 4 packed pairs (same arithmetic as gemm.cu / gemm_tc.cu)
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
// The same eight values in the order the nibble masks produce them: (c0,c4) (c1,c5) (c2,c6) (c3,c7).  Used when
// there are few token tiles: the four interleaving permutes per word and ROW are saved, and the activation
// fragments (per word and TOKEN TILE) are permuted to match instead.
__device__ __forceinline__ void dequant8_q4_paired(uint32_t w, uint32_t s2, uint32_t b2, uint32_t (&out)[4]) {
    const uint32_t magic = 0x43004300u;
    const uint32_t r0 = (w & 0x000f000fu) | magic, r1 = ((w >> 4) & 0x000f000fu) | magic;
    const uint32_t r2 = ((w >> 8) & 0x000f000fu) | magic, r3 = ((w >> 12) & 0x000f000fu) | magic;
    out[0] = fma_bf2(sub_bf2(r0, magic), s2, b2);
    out[1] = fma_bf2(sub_bf2(r1, magic), s2, b2);
    out[2] = fma_bf2(sub_bf2(r2, magic), s2, b2);
    out[3] = fma_bf2(sub_bf2(r3, magic), s2, b2);
}
__device__ __forceinline__ void dequant4_q8(uint32_t w, float s, float b, uint32_t (&out)[2]) {
    const float c0 = (float)(w & 0xffu), c1 = (float)((w >> 8) & 0xffu), c2 = (float)((w >> 16) & 0xffu), c3 = (float)(w >> 24);
    out[0] = pack_bf2(__fmaf_rn(c0, s, b), __fmaf_rn(c1, s, b));
    out[1] = pack_bf2(__fmaf_rn(c2, s, b), __fmaf_rn(c3, s, b));
}
__device__ __forceinline__ void cp_async8(uint32_t dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;\n" ::"r"(dst), "l"(src) : "memory");
}

// A "span" is the K extent one 16-byte weight load of a row covers, times the 4 threads that share the row:
//   Q4 : 32 codes per load -> span 128,   Q8 : 16 codes -> span 64,   bf16 : 8 values -> span 32.
// Thread t (= lane & 3) owns K positions [E*t, E*t + E) of the span (E = span / 4) and feeds them to the MMA
// four at a time: step s uses its positions 4s .. 4s+3 (a0/a1 = the first two for rows g / g+8, a2/a3 = the
// last two).  The matching B fragment of token n is x[n][E*t + 4s .. + 3]; the chunk in shared memory stores
// position E*t + 4s + j of a span at 16*s + 4*t + j, so that the four threads of a row group read 32
// contiguous bytes.
template <int WK>
struct Span {
    static constexpr int E = WK == 4 ? 32 : WK == 8 ? 16 : 8;  // K positions per thread per span
    static constexpr int LEN = 4 * E;                            // K positions per span
    static constexpr int STEPS = E / 4;                          // MMA K steps per span
};

struct StreamExtra {
    int splits;          // K ranges (grid.y)
    int k_per_split;     // a multiple of KC
    float* partial;      // [splits, M, N] f32 when splits > 1
    int* counters;       // [row tiles], zero between launches: the CTA that arrives last adds the ranges up
};

template <int WK, int NT, int EPI>
__global__ void __launch_bounds__(kThreads) gemm_stream_kernel(const GemmParams p, const StreamExtra ex) {
    using SP = Span<WK>;
    constexpr bool kPaired = WK == 4 && NT <= 2;  // see dequant8_q4_paired
    extern __shared__ __align__(16) uint8_t smem[];  // two chunks of [NT*8 tokens][XS_STRIDE]
    const uint32_t xs = smem_u32(smem);
    constexpr int CHUNK_BYTES = NT * 8 * XS_STRIDE;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int M = p.M, N = p.N, K = p.K;
    const int n0 = blockIdx.x * ROWS_PER_CTA + warp * 32;  // this warp's 32 feature rows
    const int k_begin = blockIdx.y * ex.k_per_split;
    const int k_end = min(K, k_begin + ex.k_per_split);
    const int n_chunks = (k_end - k_begin) / KC;
    const int groups = K / 64;

    // rows of this thread: tile r in {0,1}: n0 + 16 r + g and + 8
    const uint8_t* wrow[4];
    const uint16_t *srow[4], *brow[4];
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int row = n0 + (i >> 1) * 16 + (i & 1) * 8 + g;
        const size_t row_bytes = WK ? (size_t)K * WK / 8 : (size_t)K * 2;
        wrow[i] = reinterpret_cast<const uint8_t*>(p.w) + (size_t)row * row_bytes;
        srow[i] = WK ? p.scales + (size_t)row * groups : nullptr;
        brow[i] = WK ? p.biases + (size_t)row * groups : nullptr;
    }

    // activations of chunk c (256 K of every token) into buffer `buf`, permuted span by span
    auto load_x = [&](int c, int buf) {
        const int kc0 = k_begin + c * KC;
        constexpr int PIECES = KC / 4;  // 8-byte pieces per token row
        for (int i = tid; i < M * PIECES; i += kThreads) {
            const int m = i / PIECES, q = i % PIECES;       // q: destination piece index within the row
            const int span = (q * 4) / SP::LEN, off = (q * 4) % SP::LEN;  // destination offset inside the span
            const int s = off / 16, tt = (off % 16) / 4;    // destination = 16 s + 4 tt
            const int src_k = kc0 + span * SP::LEN + SP::E * tt + 4 * s;
            cp_async8(xs + buf * CHUNK_BYTES + m * XS_STRIDE + q * 8, p.x + (size_t)m * p.ldx + src_k);
        }
        cp_async_commit();
    };

    float acc[2][NT][4];
#pragma unroll
    for (int r = 0; r < 2; r++)
#pragma unroll
        for (int nt = 0; nt < NT; nt++) acc[r][nt][0] = acc[r][nt][1] = acc[r][nt][2] = acc[r][nt][3] = 0.f;

    // weight registers of the four rows, loaded PF spans ahead of their use.  PF divides the spans of a chunk,
    // so the ring slot of span sp of any chunk is sp % PF, a compile-time constant of the unrolled span loop.
    constexpr int SPANS_PER_CHUNK = KC / SP::LEN;
    constexpr int PF = (SPANS_PER_CHUNK >= 4 && NT <= 2) ? 4 : 2;
    static_assert(SPANS_PER_CHUNK % PF == 0, "ring slots must be static");
    uint4 wq[PF][4];
    uint32_t sb[PF][4];
    auto load_w = [&](int slot, int k0) {  // k0: first K position of the span
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const size_t byte_off = WK ? ((size_t)(k0 + SP::E * t) * WK / 8) : ((size_t)(k0 + SP::E * t) * 2);
            wq[slot][i] = __ldg(reinterpret_cast<const uint4*>(wrow[i] + byte_off));
            if (WK) {
                const int grp = (k0 + SP::E * t) / 64;
                sb[slot][i] = (uint32_t)__ldg(srow[i] + grp) | ((uint32_t)__ldg(brow[i] + grp) << 16);
            }
        }
    };

    // The weights do not depend on the kernel before this one: their first loads go out at once.  Everything else
    // (activations, residual, the shared partial-sum scratch) waits for the previous grid to complete — this kernel
    // is launched with programmatic stream serialisation, so its CTAs may start while that grid's last CTAs finish.
    if (n_chunks > 0) {
#pragma unroll
        for (int j = 0; j < PF; j++)
            if (k_begin + j * SP::LEN < k_end) load_w(j, k_begin + j * SP::LEN);
    }
    asm volatile("griddepcontrol.wait;\n" ::: "memory");
    if (n_chunks > 0) load_x(0, 0);
    for (int c = 0; c < n_chunks; c++) {
        const int buf = c & 1;
        if (c + 1 < n_chunks) load_x(c + 1, buf ^ 1);
        if (c + 1 < n_chunks)
            cp_async_wait<1>();
        else
            cp_async_wait<0>();
        __syncthreads();
        const uint32_t xb = xs + buf * CHUNK_BYTES;
#pragma unroll
        for (int sp = 0; sp < SPANS_PER_CHUNK; sp++) {
            // this span's weights out of the ring, the loads of the span PF ahead into the freed slot
            constexpr int dummy = 0;
            (void)dummy;
            const int slot = sp % PF;  // static after unrolling
            uint4 cw[4];
            uint32_t csb[4];
#pragma unroll
            for (int i = 0; i < 4; i++) {
                cw[i] = wq[slot][i];
                csb[i] = sb[slot][i];
            }
            const int k_next = k_begin + (c * SPANS_PER_CHUNK + sp + PF) * SP::LEN;
            if (k_next < k_end) load_w(slot, k_next);
            const uint32_t xspan = xb + sp * SP::LEN * 2;
            // Eight K positions of every row at a time (one Q4 word, two Q8 words, one bf16 load half): dequantised
            // once, then fed to two MMA K steps.
            uint32_t s2[4], b2[4];
            float sf[4], bf[4];
#pragma unroll
            for (int i = 0; i < 4; i++) {
                if (WK == 4) {
                    s2[i] = (csb[i] & 0xffffu) * 0x10001u;
                    b2[i] = (csb[i] >> 16) * 0x10001u;
                } else if (WK == 8) {
                    sf[i] = __uint_as_float((csb[i] & 0xffffu) << 16);
                    bf[i] = __uint_as_float(csb[i] & 0xffff0000u);
                }
            }
#pragma unroll
            for (int e8 = 0; e8 < SP::E / 8; e8++) {
                uint32_t o[4][4];  // [row][pair]: positions 8 e8 + (0,1) (2,3) (4,5) (6,7)
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    if (WK == 4 && kPaired) {
                        dequant8_q4_paired((&cw[i].x)[e8], s2[i], b2[i], o[i]);
                    } else if (WK == 4) {
                        dequant8_q4((&cw[i].x)[e8], s2[i], b2[i], o[i]);
                    } else if (WK == 8) {
                        uint32_t lo2[2], hi2[2];
                        dequant4_q8((&cw[i].x)[2 * e8], sf[i], bf[i], lo2);
                        dequant4_q8((&cw[i].x)[2 * e8 + 1], sf[i], bf[i], hi2);
                        o[i][0] = lo2[0], o[i][1] = lo2[1], o[i][2] = hi2[0], o[i][3] = hi2[1];
                    } else {
                        o[i][0] = cw[i].x, o[i][1] = cw[i].y, o[i][2] = cw[i].z, o[i][3] = cw[i].w;
                    }
                }
                if (kPaired) {
                    // MMA step h of this word takes positions (2h, 2h+4) and (2h+1, 2h+5): the activation pairs are
                    // built from the two 8-byte pieces that hold positions 0-3 and 4-7
#pragma unroll
                    for (int nt = 0; nt < NT; nt++) {
                        uint32_t x0[2], x1[2];
                        const uint32_t xa = xspan + (uint32_t)(nt * 8 + g) * XS_STRIDE + (uint32_t)(32 * e8 + 4 * t) * 2;
                        asm volatile("ld.shared.v2.b32 {%0, %1}, [%2];\n" : "=r"(x0[0]), "=r"(x0[1]) : "r"(xa));
                        asm volatile("ld.shared.v2.b32 {%0, %1}, [%2];\n" : "=r"(x1[0]), "=r"(x1[1]) : "r"(xa + 32u));
#pragma unroll
                        for (int h = 0; h < 2; h++) {
                            const uint32_t b[2] = {prmt(x0[h], x1[h], 0x5410u), prmt(x0[h], x1[h], 0x7632u)};
                            const uint32_t a0[4] = {o[0][2 * h], o[1][2 * h], o[0][2 * h + 1], o[1][2 * h + 1]};
                            const uint32_t a1[4] = {o[2][2 * h], o[3][2 * h], o[2][2 * h + 1], o[3][2 * h + 1]};
                            mma_bf16_16816(acc[0][nt], a0, b);
                            mma_bf16_16816(acc[1][nt], a1, b);
                        }
                    }
                    continue;
                }
#pragma unroll
                for (int h = 0; h < 2; h++) {
                    const int s = 2 * e8 + h;  // MMA K step: this thread's positions 4s .. 4s+3
                    // rows: i = 0: tile 0 row g, 1: tile 0 row g+8, 2: tile 1 row g, 3: tile 1 row g+8
                    const uint32_t a0[4] = {o[0][2 * h], o[1][2 * h], o[0][2 * h + 1], o[1][2 * h + 1]};
                    const uint32_t a1[4] = {o[2][2 * h], o[3][2 * h], o[2][2 * h + 1], o[3][2 * h + 1]};
#pragma unroll
                    for (int nt = 0; nt < NT; nt++) {
                        uint32_t b[2];
                        asm volatile("ld.shared.v2.b32 {%0, %1}, [%2];\n"
                                     : "=r"(b[0]), "=r"(b[1])
                                     : "r"(xspan + (uint32_t)(nt * 8 + g) * XS_STRIDE + (uint32_t)(16 * s + 4 * t) * 2));
                        mma_bf16_16816(acc[0][nt], a0, b);
                        mma_bf16_16816(acc[1][nt], a1, b);
                    }
                }
            }
        }
        __syncthreads();
    }

    // epilogue: c0,c1 = (row g, tokens 2t, 2t+1); c2,c3 = (row g+8, same tokens)
#pragma unroll
    for (int r = 0; r < 2; r++)
#pragma unroll
        for (int nt = 0; nt < NT; nt++)
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const int row = n0 + r * 16 + (e >> 1) * 8 + g;
                const int tok = nt * 8 + 2 * t + (e & 1);
                if (tok >= M || row >= N) continue;
                const float v = acc[r][nt][e];
                if (ex.splits > 1) {
                    ex.partial[((size_t)blockIdx.y * M + tok) * N + row] = v;
                } else if (EPI == EPI_F32) {
                    *gemm_f32_dst(p, tok, row) = v;
                } else if (EPI == EPI_BF16) {
                    p.out[(size_t)tok * p.ldo + row] = f2bf(v);
                } else {
                    p.out[(size_t)tok * p.ldo + row] = f2bf(bf2f(p.res[(size_t)tok * p.ldres + row]) + rbf(v));
                }
            }
    if (ex.splits == 1 || ex.counters == nullptr) return;  // one range, or a separate pass adds the ranges up

    // Several K ranges: the CTA of this row tile that finishes last adds the ranges up in index order (so the
    // sum does not depend on who is last) and applies the epilogue.  No CTA waits for another.
    __shared__ int s_last;
    __threadfence();  // this CTA's partial sums are visible before its arrival is counted
    __syncthreads();
    if (tid == 0) {
        const int arrived = atomicAdd(ex.counters + blockIdx.x, 1);
        s_last = arrived == ex.splits - 1;
        if (s_last) ex.counters[blockIdx.x] = 0;  // ready for the next launch
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    const int row0 = blockIdx.x * ROWS_PER_CTA;
    const size_t plane = (size_t)M * N;
    // four consecutive rows per thread and iteration; the ranges are added in index order, four loads in flight
    for (int e = tid; e < M * (ROWS_PER_CTA / 4); e += kThreads) {
        const int tok = e / (ROWS_PER_CTA / 4), row = row0 + (e % (ROWS_PER_CTA / 4)) * 4;
        const float* src = ex.partial + (size_t)tok * N + row;
        float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
        int z = 0;
        for (; z + 4 <= ex.splits; z += 4) {
            const float4 v0 = __ldcg(reinterpret_cast<const float4*>(src + (size_t)z * plane));
            const float4 v1 = __ldcg(reinterpret_cast<const float4*>(src + (size_t)(z + 1) * plane));
            const float4 v2 = __ldcg(reinterpret_cast<const float4*>(src + (size_t)(z + 2) * plane));
            const float4 v3 = __ldcg(reinterpret_cast<const float4*>(src + (size_t)(z + 3) * plane));
            a.x = (((a.x + v0.x) + v1.x) + v2.x) + v3.x;
            a.y = (((a.y + v0.y) + v1.y) + v2.y) + v3.y;
            a.z = (((a.z + v0.z) + v1.z) + v2.z) + v3.z;
            a.w = (((a.w + v0.w) + v1.w) + v2.w) + v3.w;
        }
        for (; z < ex.splits; z++) {
            const float4 v = __ldcg(reinterpret_cast<const float4*>(src + (size_t)z * plane));
            a.x += v.x, a.y += v.y, a.z += v.z, a.w += v.w;
        }
        const float av[4] = {a.x, a.y, a.z, a.w};
        if (EPI == EPI_F32) {
            *reinterpret_cast<float4*>(gemm_f32_dst(p, tok, row)) = a;
        } else if (EPI == EPI_BF16) {
            uint2 o;
            o.x = pack_bf2(av[0], av[1]);
            o.y = pack_bf2(av[2], av[3]);
            *reinterpret_cast<uint2*>(p.out + (size_t)tok * p.ldo + row) = o;
        } else {
            const uint2 r = *reinterpret_cast<const uint2*>(p.res + (size_t)tok * p.ldres + row);
            uint2 o;
            o.x = pack_bf2(bflo(r.x) + rbf(av[0]), bfhi(r.x) + rbf(av[1]));
            o.y = pack_bf2(bflo(r.y) + rbf(av[2]), bfhi(r.y) + rbf(av[3]));
            *reinterpret_cast<uint2*>(p.out + (size_t)tok * p.ldo + row) = o;
        }
    }
}

// out = epilogue(sum over K ranges of partial): the separate pass used from 17 tokens on, where one CTA per row
// tile would be too little parallelism for the sums
template <int EPI>
__global__ void stream_reduce_kernel(const GemmParams p, const float* __restrict__ partial, int splits) {
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
    pdl_wait();  // (launched with programmatic stream serialisation behind the kernel that writes the partial sums)
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t total = (size_t)p.M * p.N;
    if (i >= total) return;
    float a = 0.f;
    for (int z = 0; z < splits; z++) a += partial[(size_t)z * total + i];
    const int t = (int)(i / p.N), f = (int)(i % p.N);
    if (EPI == EPI_F32)
        *gemm_f32_dst(p, t, f) = a;
    else if (EPI == EPI_BF16)
        p.out[(size_t)t * p.ldo + f] = f2bf(a);
    else
        p.out[(size_t)t * p.ldo + f] = f2bf(bf2f(p.res[(size_t)t * p.ldres + f]) + rbf(a));
}

template <int WK, int NT, int EPI>
int32_t launch_stream(b2_ctx* ctx, const GemmParams& p) {
    const int smem = 2 * NT * 8 * XS_STRIDE;
    B2_SMEM_ONCE(ctx, (gemm_stream_kernel<WK, NT, EPI>), smem);
    const int row_tiles = p.N / ROWS_PER_CTA;
    const int chunks = p.K / KC;
    // K ranges: enough CTAs for every slot of the machine, at least two chunks per range
    int splits = (4 * ctx->sm_count + row_tiles - 1) / row_tiles;  // four CTAs fit an SM (registers): fill them all
    if (splits > chunks / 2) splits = chunks / 2;
    if (splits < 1) splits = 1;
    const int chunks_per = (chunks + splits - 1) / splits;
    splits = (chunks + chunks_per - 1) / chunks_per;
    StreamExtra ex{splits, chunks_per * KC, nullptr, nullptr};
    if (splits > 1) {
        const size_t bytes = (size_t)splits * p.M * p.N * sizeof(float);
        if (bytes > ctx->tc_partial_bytes) {
            B2_CUDA(cudaStreamSynchronize(ctx->stream));
            if (ctx->tc_partial) B2_CUDA(cudaFree(ctx->tc_partial));
            ctx->tc_partial = nullptr;
            B2_CUDA(cudaMalloc((void**)&ctx->tc_partial, bytes + (bytes >> 2)));
            ctx->tc_partial_bytes = bytes + (bytes >> 2);
        }
        ex.partial = ctx->tc_partial;
        constexpr int kMaxTiles = 8192;  // row tiles of 128: up to N = 1 M features
        B2_REQUIRE(row_tiles <= kMaxTiles, B2_ERR_UNSUPPORTED, "gemm: output too wide for the split-K streaming kernel");
        if (!ctx->tile_counters) {
            B2_CUDA(cudaMalloc((void**)&ctx->tile_counters, kMaxTiles * sizeof(int)));
            B2_CUDA(cudaMemsetAsync(ctx->tile_counters, 0, kMaxTiles * sizeof(int), ctx->stream));
        }
        if (p.M <= 16) ex.counters = ctx->tile_counters;  // the last CTA of a row tile adds the ranges up
    }
    {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(row_tiles, splits);
        cfg.blockDim = dim3(kThreads);
        cfg.dynamicSmemBytes = smem;
        cfg.stream = ctx->stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        B2_CUDA(cudaLaunchKernelEx(&cfg, gemm_stream_kernel<WK, NT, EPI>, p, ex));
    }
    B2_LAUNCHED(ctx);
    if (splits > 1 && !ex.counters) {
        const size_t total = (size_t)p.M * p.N;
        B2_CUDA(b2_launch_pdl(ctx->pdl_consumers, stream_reduce_kernel<EPI>, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, ctx->stream, p, (const float*)ex.partial, splits));
        B2_LAUNCHED(ctx);
    }
    B2_CUDA(cudaGetLastError());
    return B2_OK;
}

template <int WK, int NT>
int32_t dispatch_epi(b2_ctx* ctx, const GemmParams& p) {
    switch (p.epilogue) {
        case EPI_BF16: return launch_stream<WK, NT, EPI_BF16>(ctx, p);
        case EPI_BF16_RESADD: return launch_stream<WK, NT, EPI_BF16_RESADD>(ctx, p);
        case EPI_F32: return launch_stream<WK, NT, EPI_F32>(ctx, p);
    }
    return b2_fail(B2_ERR_MSG, "gemm: bad epilogue");
}

template <int WK>
int32_t dispatch_nt(b2_ctx* ctx, const GemmParams& p) {
    if (p.M <= 8) return dispatch_epi<WK, 1>(ctx, p);
    if (p.M <= 16) return dispatch_epi<WK, 2>(ctx, p);
    if (p.M <= 32) return dispatch_epi<WK, 4>(ctx, p);
    return dispatch_epi<WK, 8>(ctx, p);
}

}  // namespace

bool b2_gemm_stream_eligible(const GemmParams& p) {
    return p.M >= 1 && p.M <= 64 && p.N % ROWS_PER_CTA == 0 && p.K % KC == 0 && p.ldx % 4 == 0 && ((uintptr_t)p.x & 7) == 0 &&
           ((uintptr_t)p.w & 15) == 0 && (p.bits == 0 || p.bits == 4 || p.bits == 8) &&
           // the reduction of several K ranges stores four rows at a time
           p.ldo % 4 == 0 && ((uintptr_t)p.out & 7) == 0 && ((uintptr_t)p.out_f32 & 15) == 0 &&
           (p.epilogue != EPI_BF16_RESADD || (p.ldres % 4 == 0 && ((uintptr_t)p.res & 7) == 0));
}

int32_t b2_gemm_stream_launch(b2_ctx* ctx, const GemmParams& p) {
    if (p.bits == 0) return dispatch_nt<0>(ctx, p);
    if (p.bits == 4) return dispatch_nt<4>(ctx, p);
    return dispatch_nt<8>(ctx, p);
}
