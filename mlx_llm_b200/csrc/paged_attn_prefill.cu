// Chunked-prefill paged attention: the new tokens of a sequence (a chunk of its prompt) attend to
// everything cached so far plus themselves, causally, with K/V read in place from 16-token pages.
//
// Replaces the whole-prompt prefill attention of the reference (admit_lane ->
// CausalLm::decode_logits -> sdpa over the freshly concatenated cache: src/decode/continuous.rs:255,
// src/models/llama.rs:837-852, src/primitives/attention.rs:68-102) and its bottom-right aligned
// causal mask (attention.rs:31-39): query r of a chunk of n new tokens sees keys 0..=ctx-n+r.
//
// CTA = (64-query tile of one sequence, one q head); 4 warps x 16 queries.  K/V tiles of 64 keys
// are staged by cp.async (double buffered, XOR-swizzled) and consumed with ldmatrix + mma.sync
// m16n8k16, flash-attention style online softmax in the log2 domain, f32 accumulation.
// Prefill attention is ~1-2 % of a step's FLOPs for the target workloads, so it stays on the
// warp-level tensor path; the tcgen05 budget goes to the projections.
#include "common.cuh"
#include "kernels.h"

namespace {

constexpr int QT = 64, KT = 64, kThreads = 128;
constexpr unsigned kFull = 0xffffffffu;

template <int HD>
__global__ void __launch_bounds__(kThreads) paged_attn_prefill_kernel(const PrefillAttnParams p) {
    constexpr int ROWB = HD * 2, CHUNKS = ROWB / 16, KS = HD / 16, NT_O = HD / 8;
    constexpr int TILE_B = KT * ROWB;
    extern __shared__ __align__(128) uint8_t smem[];
    const uint32_t sQ = smem_u32(smem), sK = sQ + QT * ROWB, sV = sK + 2 * TILE_B;

    // lets a dependent launch (the o_proj kernel, launched with programmatic stream serialisation) set itself up and
    // fetch its first weights now; it still waits for this grid to complete before it reads the attention output
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
    const int w = blockIdx.x;
    if (w >= *p.n_work) return;
    const int head = blockIdx.y, kvh = head / (p.hq / p.hkv);
    const int b = p.pf_seq[w], q_start = p.pf_qstart[w];
    const int tok0 = p.cu_seqlens[b], qn = p.cu_seqlens[b + 1] - tok0;
    const int ctx = p.context_lens[b], ctx_before = ctx - qn;
    const int rows = min(QT, qn - q_start);
    const int32_t* bt = p.block_tables + (size_t)p.seq_slot[b] * p.max_blocks;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int mi = lane >> 3, lr = lane & 7;
    const int page_size = p.page_tiles * 16;

    // Q tile -> smem (rows beyond the chunk are zero)
    for (int c = tid; c < QT * CHUNKS; c += kThreads) {
        const int r = c / CHUNKS, cc = c % CHUNKS;
        const bool ok = r < rows;
        const uint16_t* src = p.q + ((size_t)(tok0 + q_start + (ok ? r : 0)) * p.hq + head) * HD + cc * 8;
        cp_async16_zfill(sQ + r * ROWB + ((cc ^ (r & 7)) << 4), src, ok);
    }
    auto load_kv = [&](int j, int stage) {
        for (int c = tid; c < KT * CHUNKS; c += kThreads) {
            const int r = c / CHUNKS, cc = c % CHUNKS;
            const int key = j * KT + r;
            const bool ok = key < ctx;
            size_t off = 0;
            if (ok) {
                const int page = bt[key / page_size];
                off = (((size_t)page * p.hkv + kvh) * page_size + key % page_size) * HD + cc * 8;
            }
            const uint32_t o = stage * TILE_B + r * ROWB + ((cc ^ (r & 7)) << 4);
            cp_async16_zfill(sK + o, p.k_pool + off, ok);
            cp_async16_zfill(sV + o, p.v_pool + off, ok);
        }
    };
    // keys needed by this tile: up to the position of its last valid query
    const int last_q_pos = ctx_before + q_start + rows - 1;
    const int n_kv_tiles = last_q_pos / KT + 1;
    load_kv(0, 0);
    cp_async_commit();
    cp_async_wait<0>();
    __syncthreads();

    uint32_t qf[KS][4];
    {
        const int r = warp * 16 + lr + (mi & 1) * 8;
#pragma unroll
        for (int ks = 0; ks < KS; ks++) {
            const int ch = 2 * ks + (mi >> 1);
            ldmatrix_x4(qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3], sQ + r * ROWB + ((ch ^ (r & 7)) << 4));
        }
    }
    // absolute positions of this thread's two query rows; rows past the chunk see everything
    const int r0 = warp * 16 + g, r1 = r0 + 8;
    const int pq0 = r0 < rows ? ctx_before + q_start + r0 : 0x3fffffff;
    const int pq1 = r1 < rows ? ctx_before + q_start + r1 : 0x3fffffff;

    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
    float o[NT_O][4];
#pragma unroll
    for (int i = 0; i < NT_O; i++) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;

    for (int j = 0; j < n_kv_tiles; j++) {
        const int stage = j & 1;
        if (j + 1 < n_kv_tiles) load_kv(j + 1, stage ^ 1);
        cp_async_commit();
        if (j > 0) {
            cp_async_wait<1>();
            __syncthreads();
        }
        const uint32_t kb = sK + stage * TILE_B, vb = sV + stage * TILE_B;
        float s[KT / 8][4];
#pragma unroll
        for (int nt = 0; nt < KT / 8; nt++) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
#pragma unroll
        for (int ks = 0; ks < KS; ks++) {
#pragma unroll
            for (int np = 0; np < KT / 16; np++) {
                const int r = np * 16 + lr + (mi >> 1) * 8;
                const int ch = 2 * ks + (mi & 1);
                uint32_t bk[4];
                ldmatrix_x4(bk[0], bk[1], bk[2], bk[3], kb + r * ROWB + ((ch ^ (r & 7)) << 4));
                const uint32_t b0[2] = {bk[0], bk[1]}, b1[2] = {bk[2], bk[3]};
                mma_bf16_16816(s[2 * np], qf[ks], b0);
                mma_bf16_16816(s[2 * np + 1], qf[ks], b1);
            }
        }
        // scale + causal mask (key position must not exceed the query position)
        const int k_base = j * KT;
        const bool need_mask = k_base + KT - 1 > ctx_before + q_start + warp * 16;
        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int nt = 0; nt < KT / 8; nt++) {
#pragma unroll
            for (int e = 0; e < 4; e++) s[nt][e] *= p.scale_log2;
            if (need_mask) {
                const int kp = k_base + nt * 8 + 2 * t;
                if (kp > pq0) s[nt][0] = -INFINITY;
                if (kp + 1 > pq0) s[nt][1] = -INFINITY;
                if (kp > pq1) s[nt][2] = -INFINITY;
                if (kp + 1 > pq1) s[nt][3] = -INFINITY;
            }
            mx0 = fmaxf(mx0, fmaxf(s[nt][0], s[nt][1]));
            mx1 = fmaxf(mx1, fmaxf(s[nt][2], s[nt][3]));
        }
#pragma unroll
        for (int sh = 1; sh <= 2; sh <<= 1) {
            mx0 = fmaxf(mx0, __shfl_xor_sync(kFull, mx0, sh));
            mx1 = fmaxf(mx1, __shfl_xor_sync(kFull, mx1, sh));
        }
        const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
        // a row whose keys in this tile are all masked keeps its previous (finite) maximum, except
        // when it has seen nothing yet, which cannot happen: key 0 is visible to every query
        const float a0 = fast_exp2(m0 - mn0), a1 = fast_exp2(m1 - mn1);
        m0 = mn0;
        m1 = mn1;
        l0 *= a0;
        l1 *= a1;
#pragma unroll
        for (int i = 0; i < NT_O; i++) {
            o[i][0] *= a0;
            o[i][1] *= a0;
            o[i][2] *= a1;
            o[i][3] *= a1;
        }
        // P as the A operand, split into a bf16 head and a bf16 remainder (~16 mantissa bits)
        uint32_t pa[KT / 16][4], pr[KT / 16][4];
#pragma unroll
        for (int nt = 0; nt < KT / 8; nt++) {
            const float p0 = fast_exp2(s[nt][0] - mn0), p1 = fast_exp2(s[nt][1] - mn0);
            const float p2 = fast_exp2(s[nt][2] - mn1), p3 = fast_exp2(s[nt][3] - mn1);
            l0 += p0 + p1;
            l1 += p2 + p3;
            const uint32_t h01 = pack_bf2(p0, p1), h23 = pack_bf2(p2, p3);
            pa[nt >> 1][(nt & 1) * 2] = h01;
            pa[nt >> 1][(nt & 1) * 2 + 1] = h23;
            pr[nt >> 1][(nt & 1) * 2] = pack_bf2(p0 - bflo(h01), p1 - bfhi(h01));
            pr[nt >> 1][(nt & 1) * 2 + 1] = pack_bf2(p2 - bflo(h23), p3 - bfhi(h23));
        }
        // O += P V
#pragma unroll
        for (int kk = 0; kk < KT / 16; kk++) {
#pragma unroll
            for (int np = 0; np < NT_O / 2; np++) {
                const int r = kk * 16 + lr + (mi & 1) * 8;
                const int ch = 2 * np + (mi >> 1);
                uint32_t bv[4];
                ldmatrix_x4_trans(bv[0], bv[1], bv[2], bv[3], vb + r * ROWB + ((ch ^ (r & 7)) << 4));
                const uint32_t b0[2] = {bv[0], bv[1]}, b1[2] = {bv[2], bv[3]};
                mma_bf16_16816(o[2 * np], pa[kk], b0);
                mma_bf16_16816(o[2 * np + 1], pa[kk], b1);
                mma_bf16_16816(o[2 * np], pr[kk], b0);
                mma_bf16_16816(o[2 * np + 1], pr[kk], b1);
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int sh = 1; sh <= 2; sh <<= 1) {
        l0 += __shfl_xor_sync(kFull, l0, sh);
        l1 += __shfl_xor_sync(kFull, l1, sh);
    }
    const float i0 = 1.0f / l0, i1 = 1.0f / l1;
#pragma unroll
    for (int i = 0; i < NT_O; i++) {
        const int d = i * 8 + 2 * t;
        if (r0 < rows)
            *reinterpret_cast<uint32_t*>(p.out + ((size_t)(tok0 + q_start + r0) * p.hq + head) * HD + d) = pack_bf2(o[i][0] * i0, o[i][1] * i0);
        if (r1 < rows)
            *reinterpret_cast<uint32_t*>(p.out + ((size_t)(tok0 + q_start + r1) * p.hq + head) * HD + d) = pack_bf2(o[i][2] * i1, o[i][3] * i1);
    }
}

}  // namespace

int b2_prefill_q_tile(const b2_ctx* ctx, int head_dim) { return ctx->use_tc && head_dim == 128 ? 128 : QT; }

int32_t b2_prefill_attn_launch(b2_ctx* ctx, const PrefillAttnParams& p, int head_dim, int grid_work) {
    if (grid_work <= 0) return B2_OK;
    B2_REQUIRE(p.hkv > 0 && p.hq % p.hkv == 0, B2_ERR_MSG, "paged_attn_prefill: hq must be a multiple of hkv");
    if (p.q_tile == 128) {
        B2_REQUIRE(b2_prefill_attn_tc_eligible(p, head_dim), B2_ERR_UNSUPPORTED, "paged_attn_prefill: 128-query work items need head_dim 128 and 16-byte aligned operands");
        return b2_prefill_attn_tc_launch(ctx, p, grid_work);
    }
    B2_REQUIRE(p.q_tile == QT, B2_ERR_MSG, "paged_attn_prefill: the work list was built for another tile size");
    dim3 grid(grid_work, p.hq);
    if (head_dim == 128) {
        const int smem = QT * 256 + 4 * KT * 256;
        B2_SMEM_ONCE(ctx, paged_attn_prefill_kernel<128>, smem);
        paged_attn_prefill_kernel<128><<<grid, kThreads, smem, ctx->stream>>>(p);
    } else if (head_dim == 64) {
        const int smem = QT * 128 + 4 * KT * 128;
        B2_SMEM_ONCE(ctx, paged_attn_prefill_kernel<64>, smem);
        paged_attn_prefill_kernel<64><<<grid, kThreads, smem, ctx->stream>>>(p);
    } else {
        return b2_fail(B2_ERR_UNSUPPORTED, "paged_attn_prefill: head_dim must be 64 or 128");
    }
    B2_LAUNCHED(ctx);
    B2_CUDA(cudaGetLastError());
    return B2_OK;
}
