// Fused (optional per-head q/k RMSNorm) -> NeoX RoPE -> KV append into 16-token pages.
//
// Replaces LlamaAttention::project (src/models/llama.rs:806-825: q_norm/k_norm, apply_rope) plus
// PagedKvCache::update's tail concat (src/primitives/paged_kv_cache.rs:294-304): the rotated key
// and the raw value of every new token are scattered straight to their page slot; queries are
// rotated in place.  cos/sin come from a host-built bf16 table (angle = pos*inv_freq in f32,
// src/primitives/rope.rs:183-208), and the rotation rounds like the reference's op chain
// (rope.rs:381-386):  out = bf16( bf16(x*cos) + bf16(rot*sin) ),  rot = cat(-x2, x1).
//
// One warp per (token, head); a lane owns HD/64 adjacent elements of each half.
#include "common.cuh"
#include "kernels.h"

namespace {

constexpr unsigned kFull = 0xffffffffu;

template <int HD>
__global__ void rope_kv_kernel(const RopeKvParams p) {
    constexpr int V = HD / 64;  // elements per lane per half (1 or 2)
    // the attention kernel after this one may be scheduled as soon as every CTA of this grid has started; it waits for the
    // grid's completion itself
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
    pdl_wait();  // (launched with programmatic stream serialisation: the projection before it may still be finishing)
    const int heads_total = p.hq + 2 * p.hkv;
    const int wid = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (wid >= p.T * heads_total) return;
    const int lane = threadIdx.x & 31;
    const int tok = wid / heads_total, head = wid % heads_total;
    uint16_t* src = p.qkv + (size_t)tok * p.ld + (size_t)head * HD;
    const int slot = p.slot_mapping[tok];

    const bool is_q = head < p.hq, is_k = !is_q && head < p.hq + p.hkv;
    const int kvh = is_q ? 0 : (is_k ? head - p.hq : head - p.hq - p.hkv);
    size_t dst_off = 0;
    if (!is_q) {
        const int page = slot / p.page_size, off = slot % p.page_size;
        dst_off = (((size_t)page * p.hkv + kvh) * p.page_size + off) * HD;
    }
    if (!is_q && !is_k) {  // value: raw copy
        if (slot < 0) return;
        uint16_t* dst = p.v_pool + dst_off;
        if (V == 2) {
            reinterpret_cast<uint32_t*>(dst)[lane] = reinterpret_cast<const uint32_t*>(src)[lane];
            reinterpret_cast<uint32_t*>(dst)[32 + lane] = reinterpret_cast<const uint32_t*>(src)[32 + lane];
        } else {
            reinterpret_cast<uint32_t*>(dst)[lane] = reinterpret_cast<const uint32_t*>(src)[lane];
        }
        return;
    }
    // first-half and second-half elements of this lane
    float x1[V], x2[V];
    if (V == 2) {
        const uint32_t a = reinterpret_cast<const uint32_t*>(src)[lane], b = reinterpret_cast<const uint32_t*>(src)[32 + lane];
        x1[0] = bflo(a);
        x1[V - 1] = bfhi(a);
        x2[0] = bflo(b);
        x2[V - 1] = bfhi(b);
    } else {
        x1[0] = bf2f(src[lane]);
        x2[0] = bf2f(src[32 + lane]);
    }
    const uint16_t* nw = is_q ? p.q_norm : p.k_norm;
    if (nw) {  // per-head RMSNorm before RoPE (Qwen3, llama.rs:814-819)
        float ss = 0.f;
#pragma unroll
        for (int j = 0; j < V; j++) ss += x1[j] * x1[j] + x2[j] * x2[j];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(kFull, ss, o);
        const float inv = 1.0f / sqrtf(ss / (float)HD + p.eps);
#pragma unroll
        for (int j = 0; j < V; j++) {
            x1[j] = rbf(x1[j] * inv * bf2f(nw[lane * V + j]));
            x2[j] = rbf(x2[j] * inv * bf2f(nw[HD / 2 + lane * V + j]));
        }
    }
    const int pos = p.positions[tok];
    const uint16_t* ct = p.cos_table + (size_t)pos * (HD / 2);
    const uint16_t* st = p.sin_table + (size_t)pos * (HD / 2);
    float y1[V], y2[V];
#pragma unroll
    for (int j = 0; j < V; j++) {
        const float c = bf2f(ct[lane * V + j]), s = bf2f(st[lane * V + j]);
        // first half: x1*cos + (-x2)*sin ; second half: x2*cos + x1*sin
        y1[j] = rbf(x1[j] * c) + rbf(-x2[j] * s);
        y2[j] = rbf(x2[j] * c) + rbf(x1[j] * s);
    }
    uint16_t* dst;
    if (is_q) {
        dst = p.q_out + ((size_t)tok * p.hq + head) * HD;
    } else {
        if (slot < 0) return;
        dst = p.k_pool + dst_off;
    }
    if (V == 2) {
        reinterpret_cast<uint32_t*>(dst)[lane] = pack_bf2(y1[0], y1[V - 1]);
        reinterpret_cast<uint32_t*>(dst)[32 + lane] = pack_bf2(y2[0], y2[V - 1]);
    } else {
        dst[lane] = f2bf(y1[0]);
        dst[32 + lane] = f2bf(y2[0]);
    }
}

}  // namespace

int32_t b2_rope_kv_launch(b2_ctx* ctx, const RopeKvParams& p) {
    if (p.T <= 0) return B2_OK;
    B2_REQUIRE(p.hd == 64 || p.hd == 128, B2_ERR_UNSUPPORTED, "rope_kv: head_dim must be 64 or 128");
    B2_REQUIRE(p.ld % 2 == 0, B2_ERR_UNSUPPORTED, "rope_kv: row stride must be even");
    const long warps = (long)p.T * (p.hq + 2 * p.hkv);
    const int wpb = 8;
    const unsigned grid = (unsigned)((warps + wpb - 1) / wpb);
    if (p.hd == 128)
        B2_CUDA(b2_launch_pdl(ctx->pdl_consumers, rope_kv_kernel<128>, dim3(grid), dim3(wpb * 32), 0, ctx->stream, p));
    else
        B2_CUDA(b2_launch_pdl(ctx->pdl_consumers, rope_kv_kernel<64>, dim3(grid), dim3(wpb * 32), 0, ctx->stream, p));
    B2_LAUNCHED(ctx);
    B2_CUDA(cudaGetLastError());
    return B2_OK;
}
