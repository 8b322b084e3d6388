// Bandwidth-bound leaves of the decoder step: RMSNorm, embedding gather, SwiGLU, residual add,
// greedy argmax, and the standalone MLX-format quantize / dequantize / unpack entry points.
//
// Rounding points follow the reference, where every MLX op materialises a bf16 tensor
// (src/models/llama.rs:718-735, :1040-1045): reductions run in f32, each op's result is rounded to
// bf16 once.
#include <cfloat>

#include "common.cuh"
#include "kernels.h"

namespace {

constexpr unsigned kFull = 0xffffffffu;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(kFull, v, o);
    return v;
}

// fast::rms_norm (src/primitives/nn.rs:35-37): y = bf16(x * (1/sqrt(mean(x^2)+eps)) * w).
// One CTA per row, 8 bf16 (16 bytes) per thread per iteration.
__global__ void rms_norm_kernel(const uint16_t* __restrict__ x, const uint16_t* __restrict__ w, float eps, int dim, int ldx,
                                const int32_t* __restrict__ row_idx, uint16_t* __restrict__ out) {
    // lets a dependent launch (the projection that consumes this kernel's output, launched with programmatic
    // stream serialisation) begin its weight prefetch now; it still waits for this grid to complete before it reads
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
    pdl_wait();
    const int row = blockIdx.x;
    const int src = row_idx ? row_idx[row] : row;
    const uint16_t* xr = x + (size_t)src * ldx;
    __shared__ float red[32];
    float ss = 0.f;
    const bool vec = (dim % 8 == 0) && (ldx % 8 == 0);
    if (vec) {
        for (int i = threadIdx.x * 8; i < dim; i += blockDim.x * 8) {
            const uint4 v = *reinterpret_cast<const uint4*>(xr + i);
            const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const float a = bflo(u[j]), b = bfhi(u[j]);
                ss += a * a + b * b;
            }
        }
    } else {
        for (int i = threadIdx.x; i < dim; i += blockDim.x) {
            const float a = bf2f(xr[i]);
            ss += a * a;
        }
    }
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x < 32) {
        float v = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
        v = warp_sum(v);
        if (threadIdx.x == 0) red[0] = v;
    }
    __syncthreads();
    const float inv = 1.0f / sqrtf(red[0] / (float)dim + eps);
    uint16_t* orow = out + (size_t)row * dim;
    if (vec) {
        for (int i = threadIdx.x * 8; i < dim; i += blockDim.x * 8) {
            const uint4 v = *reinterpret_cast<const uint4*>(xr + i);
            const uint4 g = *reinterpret_cast<const uint4*>(w + i);
            const uint32_t u[4] = {v.x, v.y, v.z, v.w}, gw[4] = {g.x, g.y, g.z, g.w};
            uint32_t r[4];
#pragma unroll
            for (int j = 0; j < 4; j++) r[j] = pack_bf2(bflo(u[j]) * inv * bflo(gw[j]), bfhi(u[j]) * inv * bfhi(gw[j]));
            *reinterpret_cast<uint4*>(orow + i) = make_uint4(r[0], r[1], r[2], r[3]);
        }
    } else {
        for (int i = threadIdx.x; i < dim; i += blockDim.x) orow[i] = f2bf(bf2f(xr[i]) * inv * bf2f(w[i]));
    }
}

// Embedding row gather (src/primitives/nn.rs:86-93).
__global__ void embed_kernel(const uint16_t* __restrict__ table, const int32_t* __restrict__ ids, int dim, int vocab,
                             uint16_t* __restrict__ out) {
    const int t = blockIdx.x;
    int id = ids[t];
    id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
    const uint16_t* src = table + (size_t)id * dim;
    uint16_t* dst = out + (size_t)t * dim;
    if (dim % 8 == 0) {
        for (int i = threadIdx.x * 8; i < dim; i += blockDim.x * 8)
            *reinterpret_cast<uint4*>(dst + i) = *reinterpret_cast<const uint4*>(src + i);
    } else {
        for (int i = threadIdx.x; i < dim; i += blockDim.x) dst[i] = src[i];
    }
}

__device__ __forceinline__ float swiglu_one(float g, float u) {
    const float s = rbf(1.0f / (1.0f + expf(-g)));  // sigmoid, rounded
    const float a = rbf(g * s);                     // silu, rounded
    return a * u;                                   // caller rounds
}
// LlamaMlp::forward (src/models/llama.rs:1040-1045) on a fused [rows, 2*inter] gate|up buffer.
__global__ void swiglu_kernel(const uint16_t* __restrict__ gu, int inter, uint16_t* __restrict__ out) {
    // lets a dependent launch (the projection that consumes this kernel's output, launched with programmatic
    // stream serialisation) begin its weight prefetch now; it still waits for this grid to complete before it reads
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
    pdl_wait();
    const int row = blockIdx.y;
    const uint16_t* g = gu + (size_t)row * 2 * inter;
    const uint16_t* u = g + inter;
    uint16_t* o = out + (size_t)row * inter;
    const int i = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
    if (i >= inter) return;
    if (inter % 8 == 0) {  // rows and the gate | up boundary are then 16-byte aligned: eight values per thread
        const uint4 gv = *reinterpret_cast<const uint4*>(g + i), uv = *reinterpret_cast<const uint4*>(u + i);
        const uint32_t ga[4] = {gv.x, gv.y, gv.z, gv.w}, ua[4] = {uv.x, uv.y, uv.z, uv.w};
        uint32_t r[4];
#pragma unroll
        for (int j = 0; j < 4; j++) r[j] = pack_bf2(swiglu_one(bflo(ga[j]), bflo(ua[j])), swiglu_one(bfhi(ga[j]), bfhi(ua[j])));
        *reinterpret_cast<uint4*>(o + i) = make_uint4(r[0], r[1], r[2], r[3]);
    } else {
        for (int j = i; j < inter && j < i + 8; j++) o[j] = f2bf(swiglu_one(bf2f(g[j]), bf2f(u[j])));
    }
}
__global__ void swiglu2_kernel(const uint16_t* __restrict__ g, const uint16_t* __restrict__ u, int64_t n, uint16_t* __restrict__ out) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = f2bf(swiglu_one(bf2f(g[i]), bf2f(u[i])));
}
__global__ void add_kernel(const uint16_t* __restrict__ a, const uint16_t* __restrict__ b, int64_t n, uint16_t* __restrict__ out) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = f2bf(bf2f(a[i]) + bf2f(b[i]));
}

// x = bf16(x + bf16(y)): the residual add of a projection whose f32 result arrives from a reduction
// over tensor-parallel ranks (same two roundings as the fused GEMM epilogue).
__global__ void residual_add_f32_kernel(const float* __restrict__ y, int64_t n, uint16_t* __restrict__ x) {
    const int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (i + 3 < n) {
        const float4 v = *reinterpret_cast<const float4*>(y + i);
        uint2 xv = *reinterpret_cast<const uint2*>(x + i);
        const float a0 = bf2f((uint16_t)(xv.x & 0xffff)) + rbf(v.x), a1 = bf2f((uint16_t)(xv.x >> 16)) + rbf(v.y);
        const float a2 = bf2f((uint16_t)(xv.y & 0xffff)) + rbf(v.z), a3 = bf2f((uint16_t)(xv.y >> 16)) + rbf(v.w);
        xv.x = pack_bf2(a0, a1);
        xv.y = pack_bf2(a2, a3);
        *reinterpret_cast<uint2*>(x + i) = xv;
    } else {
        for (int64_t j = i; j < n; j++) x[j] = f2bf(bf2f(x[j]) + rbf(y[j]));
    }
}

// Greedy argmax over bf16 logits, first maximum wins (src/primitives/sampler.rs:221-241).
__global__ void argmax_kernel(const uint16_t* __restrict__ logits, int vocab, int32_t* __restrict__ out) {
    const uint16_t* row = logits + (size_t)blockIdx.x * vocab;
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
        const float v = bf2f(row[i]);
        if (v > best) {  // strictly greater: within a thread indices ascend, so the first max is kept
            best = v;
            bi = i;
        }
    }
    __shared__ float sv[32];
    __shared__ int si[32];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(kFull, best, o);
        const int oi = __shfl_xor_sync(kFull, bi, o);
        if (ov > best || (ov == best && oi < bi)) {
            best = ov;
            bi = oi;
        }
    }
    if ((threadIdx.x & 31) == 0) {
        sv[threadIdx.x >> 5] = best;
        si[threadIdx.x >> 5] = bi;
    }
    __syncthreads();
    if (threadIdx.x < 32) {
        const int nw = blockDim.x >> 5;
        best = threadIdx.x < nw ? sv[threadIdx.x] : -INFINITY;
        bi = threadIdx.x < nw ? si[threadIdx.x] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(kFull, best, o);
            const int oi = __shfl_xor_sync(kFull, bi, o);
            if (ov > best || (ov == best && oi < bi)) {
                best = ov;
                bi = oi;
            }
        }
        // all logits -inf or NaN: index 0, as a host scan starting from best = -inf, index 0 gives
        if (threadIdx.x == 0) out[blockIdx.x] = bi == 0x7fffffff ? 0 : bi;
    }
}

// Standalone dequantize / unpack of the MLX affine format (src/primitives/quant.rs:73-82).
__global__ void dequantize_kernel(const uint32_t* __restrict__ packed, const uint16_t* __restrict__ scales,
                                  const uint16_t* __restrict__ biases, int64_t total_words, int64_t words_per_row, int64_t groups,
                                  int bits, uint16_t* __restrict__ out) {
    const int64_t wi = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (wi >= total_words) return;
    const int per = 32 / bits;
    const int64_t row = wi / words_per_row, wcol = wi % words_per_row;
    const int64_t col0 = wcol * per;
    const int64_t gi = row * groups + col0 / 64;
    const float s = bf2f(scales[gi]), b = bf2f(biases[gi]);
    const uint32_t w = packed[wi];
    const uint32_t mask = (1u << bits) - 1;
    uint16_t* o = out + row * (words_per_row * per) + col0;
    for (int j = 0; j < per; j++) o[j] = f2bf(__fmaf_rn((float)((w >> (j * bits)) & mask), s, b));
}
__global__ void unpack_kernel(const uint32_t* __restrict__ packed, int64_t total_words, int bits, uint8_t* __restrict__ out) {
    const int64_t wi = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (wi >= total_words) return;
    const int per = 32 / bits;
    const uint32_t w = packed[wi], mask = (1u << bits) - 1;
    for (int j = 0; j < per; j++) out[wi * per + j] = (uint8_t)((w >> (j * bits)) & mask);
}

// Quantize-on-load encoder (QuantizedLinear::quantize, src/primitives/quant.rs:38-54 -> mlx
// ops::quantize, affine mode).  One warp per group of 64 inputs; two values per lane.
__global__ void quantize_kernel(const uint16_t* __restrict__ w, int64_t n_groups, int64_t groups_per_row, int bits,
                                uint32_t* __restrict__ packed, uint16_t* __restrict__ scales, uint16_t* __restrict__ biases) {
    const int64_t gi = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (gi >= n_groups) return;
    const int lane = threadIdx.x & 31;
    const uint32_t v = *reinterpret_cast<const uint32_t*>(w + gi * 64 + lane * 2);
    const float a = bflo(v), b = bfhi(v);
    float wmin = fminf(a, b), wmax = fmaxf(a, b);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        wmin = fminf(wmin, __shfl_xor_sync(kFull, wmin, o));
        wmax = fmaxf(wmax, __shfl_xor_sync(kFull, wmax, o));
    }
    const float n_bins = (float)((1 << bits) - 1);
    float scale = fmaxf((wmax - wmin) / n_bins, 1e-7f);
    const bool side = fabsf(wmin) > fabsf(wmax);
    scale = side ? scale : -scale;
    const float edge = side ? wmin : wmax;
    const float q0 = roundf(edge / scale);
    float bias = 0.f;
    if (q0 != 0.f) {
        scale = edge / q0;
        bias = edge;
    }
    const uint32_t qa = (uint32_t)fminf(fmaxf(roundf((a - bias) / scale), 0.f), n_bins);
    const uint32_t qb = (uint32_t)fminf(fmaxf(roundf((b - bias) / scale), 0.f), n_bins);
    // lane holds codes 2*lane, 2*lane+1; a u32 holds 32/bits codes
    const int per = 32 / bits;
    uint32_t word = (qa << (((2 * lane) % per) * bits)) | (qb << (((2 * lane + 1) % per) * bits));
    const int lanes_per_word = per / 2;  // 4 (Q4) or 2 (Q8)
    for (int o = 1; o < lanes_per_word; o <<= 1) word |= __shfl_xor_sync(kFull, word, o);
    const int64_t row = gi / groups_per_row, g = gi % groups_per_row;
    const int64_t words_per_row = groups_per_row * 64 / per;
    if (lane % lanes_per_word == 0) packed[row * words_per_row + g * (64 / per) + lane / lanes_per_word] = word;
    if (lane == 0) {
        scales[gi] = f2bf(scale);
        biases[gi] = f2bf(bias);
    }
}

}  // namespace

int32_t b2_rms_norm_launch(b2_ctx* ctx, const uint16_t* x, const uint16_t* w, float eps, int rows, int dim, int ldx,
                           const int32_t* row_idx, uint16_t* out) {
    if (rows <= 0) return B2_OK;
    int threads = dim / 8;
    threads = threads < 32 ? 32 : (threads > 1024 ? 1024 : ((threads + 31) / 32) * 32);
    B2_CUDA(b2_launch_pdl(ctx->pdl_consumers, rms_norm_kernel, dim3(rows), dim3(threads), 0, ctx->stream, x, w, eps, dim, ldx, row_idx, out));
    B2_LAUNCHED(ctx);
    B2_CUDA(cudaGetLastError());
    return B2_OK;
}
int32_t b2_embed_launch(b2_ctx* ctx, const uint16_t* table, const int32_t* ids, int n, int dim, int vocab, uint16_t* out) {
    if (n <= 0) return B2_OK;
    int threads = dim / 8;
    threads = threads < 32 ? 32 : (threads > 512 ? 512 : ((threads + 31) / 32) * 32);
    embed_kernel<<<n, threads, 0, ctx->stream>>>(table, ids, dim, vocab, out);
    B2_LAUNCHED(ctx);
    B2_CUDA(cudaGetLastError());
    return B2_OK;
}
int32_t b2_swiglu_launch(b2_ctx* ctx, const uint16_t* gate_up, int rows, int inter, uint16_t* out) {
    if (rows <= 0) return B2_OK;
    dim3 grid(((inter + 7) / 8 + 255) / 256, rows);
    B2_CUDA(b2_launch_pdl(ctx->pdl_consumers, swiglu_kernel, grid, dim3(256), 0, ctx->stream, gate_up, inter, out));
    B2_LAUNCHED(ctx);
    B2_CUDA(cudaGetLastError());
    return B2_OK;
}
int32_t b2_swiglu2_launch(b2_ctx* ctx, const uint16_t* gate, const uint16_t* up, int64_t n, uint16_t* out) {
    if (n <= 0) return B2_OK;
    swiglu2_kernel<<<(unsigned)((n + 255) / 256), 256, 0, ctx->stream>>>(gate, up, n, out);
    B2_LAUNCHED(ctx);
    B2_CUDA(cudaGetLastError());
    return B2_OK;
}
int32_t b2_add_launch(b2_ctx* ctx, const uint16_t* a, const uint16_t* b, int64_t n, uint16_t* out) {
    if (n <= 0) return B2_OK;
    add_kernel<<<(unsigned)((n + 255) / 256), 256, 0, ctx->stream>>>(a, b, n, out);
    B2_LAUNCHED(ctx);
    B2_CUDA(cudaGetLastError());
    return B2_OK;
}
int32_t b2_residual_add_f32_launch(b2_ctx* ctx, const float* y, int64_t n, uint16_t* x) {
    if (n <= 0) return B2_OK;
    const int64_t quads = (n + 3) / 4;
    residual_add_f32_kernel<<<(unsigned)((quads + 255) / 256), 256, 0, ctx->stream>>>(y, n, x);
    B2_LAUNCHED(ctx);
    B2_CUDA(cudaGetLastError());
    return B2_OK;
}
int32_t b2_argmax_launch(b2_ctx* ctx, const uint16_t* logits, int rows, int vocab, int32_t* out) {
    if (rows <= 0) return B2_OK;
    argmax_kernel<<<rows, 1024, 0, ctx->stream>>>(logits, vocab, out);
    B2_LAUNCHED(ctx);
    B2_CUDA(cudaGetLastError());
    return B2_OK;
}
int32_t b2_dequantize_launch(b2_ctx* ctx, const uint32_t* packed, const uint16_t* scales, const uint16_t* biases, int64_t rows,
                             int64_t in_dim, int bits, uint16_t* out) {
    const int64_t wpr = in_dim * bits / 32, total = rows * wpr;
    if (total <= 0) return B2_OK;
    dequantize_kernel<<<(unsigned)((total + 255) / 256), 256, 0, ctx->stream>>>(packed, scales, biases, total, wpr, in_dim / 64, bits, out);
    B2_LAUNCHED(ctx);
    B2_CUDA(cudaGetLastError());
    return B2_OK;
}
int32_t b2_unpack_launch(b2_ctx* ctx, const uint32_t* packed, int64_t rows, int64_t in_dim, int bits, uint8_t* out) {
    const int64_t total = rows * in_dim * bits / 32;
    if (total <= 0) return B2_OK;
    unpack_kernel<<<(unsigned)((total + 255) / 256), 256, 0, ctx->stream>>>(packed, total, bits, out);
    B2_LAUNCHED(ctx);
    B2_CUDA(cudaGetLastError());
    return B2_OK;
}
int32_t b2_quantize_launch(b2_ctx* ctx, const uint16_t* w, int64_t rows, int64_t in_dim, int bits, uint32_t* packed, uint16_t* scales,
                           uint16_t* biases) {
    const int64_t gpr = in_dim / 64, n_groups = rows * gpr;
    if (n_groups <= 0) return B2_OK;
    quantize_kernel<<<(unsigned)((n_groups + 7) / 8), 256, 0, ctx->stream>>>(w, n_groups, gpr, bits, packed, scales, biases);
    B2_LAUNCHED(ctx);
    B2_CUDA(cudaGetLastError());
    return B2_OK;
}
