// Paged-attention decode for sm_100a: one query token per sequence over a paged bf16 KV pool.
//
// Replaces the reference's gather-then-SDPA decode (src/primitives/paged_kv_cache.rs:342-354
// concatenates the whole sequence every layer every step, then src/primitives/attention.rs:87-102
// runs the stock fused SDPA on the copy): here K/V pages are read in place, once.
//
// Work decomposition
//   CTA        = (split-K work item, kv head): a chunk of `chunk_tiles` 16-token tiles of one
//                sequence, all q heads of the GQA group at once (K/V bytes are read once per group).
//   warp       = every 4th tile of the chunk, with a private 3-stage cp.async pipeline
//                (16-byte coalesced copies, XOR-swizzled rows so ldmatrix is conflict free);
//                no CTA-wide barrier inside the main loop.
//   tensor op  = mma.sync m16n8k16 with the 16 TOKENS of a tile on M and the (<= 8) q heads of
//                the group on N:  S^T = K Q^T, then O^T += V^T P^T.  P^T reaches the B-operand
//                layout with one movmatrix per 8 tokens.  Softmax statistics are per column,
//                reduced with three xor-shuffles.
//   merge      = per-CTA cross-warp log-sum-exp merge in shared memory; chunks of a sequence are
//                merged by a second small kernel (skipped for single-chunk sequences).
// This is HBM-bound byte streaming: the tensor cores are used only to keep the CUDA cores off the
// critical path, so no tcgen05/TMEM here.
#include <cfloat>

#include "common.cuh"
#include "kernels.h"

namespace {

constexpr int kWarps = 4;
constexpr int kStages = 3;
constexpr unsigned kFull = 0xffffffffu;

// One work item: chunk `chunk` of sequence `seq` (work index w; the sequence's items are w0 .. w0 + n_chunks - 1) for
// kv head `kvh`.  Every thread of the CTA calls it; on return the shared memory may be reused.
template <int HD>
__device__ __forceinline__ void decode_item(const DecodeAttnParams& p, uint8_t* smem, int w, int kvh, int seq, int chunk, int w0,
                                            int n_chunks) {
    constexpr int ROWB = HD * 2;        // bytes per token row of one head
    constexpr int CHUNKS = ROWB / 16;   // 16-byte chunks per row
    constexpr int TILE_B = 16 * ROWB;   // bytes of a 16-token tile
    constexpr int KSTEPS = HD / 16;
    constexpr int MT = HD / 16;
    __shared__ int s_last;
    const int ctx = min(p.ctx_lens[seq], p.max_blocks * p.page_tiles * 16);  // never past the block-table row
    const int tiles_total = (ctx + 15) >> 4;
    const int tile0 = chunk * p.chunk_tiles;
    const int n_tiles = min(p.chunk_tiles, tiles_total - tile0);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int group = p.hq / p.hkv;
    const int qrow = p.q_rows ? p.q_rows[seq] : seq;

    // Q^T as the B operand: thread (g,t) holds Q[head g][16*ks + 2t, +1] and [.. + 8, + 9].
    uint32_t qf[KSTEPS][2];
    {
        const uint16_t* qh = p.q + ((size_t)qrow * p.hq + (size_t)kvh * group + g) * HD;
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ks++) {
            qf[ks][0] = g < group ? *reinterpret_cast<const uint32_t*>(qh + ks * 16 + 2 * t) : 0u;
            qf[ks][1] = g < group ? *reinterpret_cast<const uint32_t*>(qh + ks * 16 + 2 * t + 8) : 0u;
        }
    }

    const int n_my = n_tiles > warp ? (n_tiles - warp + kWarps - 1) / kWarps : 0;
    const int32_t* bt = p.block_tables + (size_t)(p.bt_rows ? p.bt_rows[seq] : seq) * p.max_blocks;
    // lane i keeps the physical page of this warp's i-th tile
    int my_page = 0;
    if (lane < n_my) my_page = bt[(tile0 + warp + lane * kWarps) / p.page_tiles];

    const uint32_t wsm = smem_u32(smem) + warp * (kStages * 2 * TILE_B);

    auto issue = [&](int i) {
        const int tile = tile0 + warp + i * kWarps;
        const int page = __shfl_sync(kFull, my_page, i);
        const size_t off = (((size_t)page * p.hkv + kvh) * p.page_tiles + (tile % p.page_tiles)) * (size_t)(16 * HD);
        const uint8_t* ks = reinterpret_cast<const uint8_t*>(p.k_pool + off);
        const uint8_t* vs = reinterpret_cast<const uint8_t*>(p.v_pool + off);
        const uint32_t dst = wsm + (i % kStages) * 2 * TILE_B;
#pragma unroll
        for (int c = lane; c < 16 * CHUNKS; c += 32) {
            const int r = c / CHUNKS, cc = c % CHUNKS;
            const uint32_t o = r * ROWB + ((cc ^ (r & 7)) << 4);
            cp_async16(dst + o, ks + (size_t)c * 16);
            cp_async16(dst + TILE_B + o, vs + (size_t)c * 16);
        }
    };

    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
    float o[MT][4];
#pragma unroll
    for (int mt = 0; mt < MT; mt++) o[mt][0] = o[mt][1] = o[mt][2] = o[mt][3] = 0.f;

#pragma unroll
    for (int i = 0; i < kStages - 1; i++) {
        if (i < n_my) issue(i);
        cp_async_commit();
    }
    const int mi = lane >> 3, lr = lane & 7;
    for (int i = 0; i < n_my; i++) {
        if (i + kStages - 1 < n_my) issue(i + kStages - 1);
        cp_async_commit();
        cp_async_wait<kStages - 1>();
        __syncwarp();
        const uint32_t kb = wsm + (i % kStages) * 2 * TILE_B, vb = kb + TILE_B;

        // S^T[token, head] = K[token, :] . Q[head, :]
        float s[4] = {0.f, 0.f, 0.f, 0.f};
        {
            const int r = lr + (mi & 1) * 8;
#pragma unroll
            for (int ks = 0; ks < KSTEPS; ks++) {
                const int ch = 2 * ks + (mi >> 1);
                uint32_t a[4];
                ldmatrix_x4(a[0], a[1], a[2], a[3], kb + r * ROWB + ((ch ^ (r & 7)) << 4));
                mma_bf16_16816(s, a, qf[ks]);
            }
        }
        const int tok0 = (tile0 + warp + i * kWarps) * 16;
#pragma unroll
        for (int j = 0; j < 4; j++) s[j] *= p.scale_log2;
        if (tok0 + 16 > ctx) {
            if (tok0 + g >= ctx) s[0] = s[1] = -INFINITY;
            if (tok0 + g + 8 >= ctx) s[2] = s[3] = -INFINITY;
        }
        float mx0 = fmaxf(s[0], s[2]), mx1 = fmaxf(s[1], s[3]);
#pragma unroll
        for (int sh = 4; sh <= 16; sh <<= 1) {
            mx0 = fmaxf(mx0, __shfl_xor_sync(kFull, mx0, sh));
            mx1 = fmaxf(mx1, __shfl_xor_sync(kFull, mx1, sh));
        }
        const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
        const float a0 = fast_exp2(m0 - mn0), a1 = fast_exp2(m1 - mn1);
        const float p0 = fast_exp2(s[0] - mn0), p1 = fast_exp2(s[1] - mn1);
        const float p2 = fast_exp2(s[2] - mn0), p3 = fast_exp2(s[3] - mn1);
        l0 = l0 * a0 + p0 + p2;
        l1 = l1 * a1 + p1 + p3;
        m0 = mn0;
        m1 = mn1;
#pragma unroll
        for (int mt = 0; mt < MT; mt++) {
            o[mt][0] *= a0;
            o[mt][1] *= a1;
            o[mt][2] *= a0;
            o[mt][3] *= a1;
        }
        // P^T as the B operand (tokens on K, heads on N).  P is split into a bf16 head and a bf16
        // remainder so the product with V carries ~16 mantissa bits instead of 8.
        uint32_t pb[2], pl[2];
        {
            const uint32_t h01 = pack_bf2(p0, p1), h23 = pack_bf2(p2, p3);
            const uint32_t l01 = pack_bf2(p0 - bflo(h01), p1 - bfhi(h01)), l23 = pack_bf2(p2 - bflo(h23), p3 - bfhi(h23));
            pb[0] = movmatrix_trans(h01);
            pb[1] = movmatrix_trans(h23);
            pl[0] = movmatrix_trans(l01);
            pl[1] = movmatrix_trans(l23);
        }
        // O^T[d, head] += V^T[d, token] P^T[token, head]
        {
            const int r = lr + (mi >> 1) * 8;
#pragma unroll
            for (int mt = 0; mt < MT; mt++) {
                const int ch = 2 * mt + (mi & 1);
                uint32_t a[4];
                ldmatrix_x4_trans(a[0], a[1], a[2], a[3], vb + r * ROWB + ((ch ^ (r & 7)) << 4));
                mma_bf16_16816(o[mt], a, pb);
                mma_bf16_16816(o[mt], a, pl);
            }
        }
        __syncwarp();
    }
#pragma unroll
    for (int sh = 4; sh <= 16; sh <<= 1) {
        l0 += __shfl_xor_sync(kFull, l0, sh);
        l1 += __shfl_xor_sync(kFull, l1, sh);
    }
    cp_async_wait<0>();
    __syncthreads();

    // cross-warp merge through shared memory (pipeline buffers are free now)
    float* so = reinterpret_cast<float*>(smem);      // [kWarps][HD][8]
    float* sm_m = so + kWarps * HD * 8;              // [kWarps][8]
    float* sm_l = sm_m + kWarps * 8;                 // [kWarps][8]
#pragma unroll
    for (int mt = 0; mt < MT; mt++) {
        float* base = so + ((size_t)warp * HD + 16 * mt + g) * 8 + 2 * t;
        base[0] = o[mt][0];
        base[1] = o[mt][1];
        base[64] = o[mt][2];  // row g + 8
        base[65] = o[mt][3];
    }
    if (g == 0) {
        sm_m[warp * 8 + 2 * t] = m0;
        sm_m[warp * 8 + 2 * t + 1] = m1;
        sm_l[warp * 8 + 2 * t] = l0;
        sm_l[warp * 8 + 2 * t + 1] = l1;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < group * HD; e += kWarps * 32) {
        const int h = e / HD, d = e % HD;
        float M = -INFINITY;
#pragma unroll
        for (int ww = 0; ww < kWarps; ww++) M = fmaxf(M, sm_m[ww * 8 + h]);
        float L = 0.f, O = 0.f;
#pragma unroll
        for (int ww = 0; ww < kWarps; ww++) {
            const float f = fast_exp2(sm_m[ww * 8 + h] - M);
            L += sm_l[ww * 8 + h] * f;
            O += so[((size_t)ww * HD + d) * 8 + h] * f;
        }
        if (n_chunks == 1) {
            p.out[((size_t)qrow * p.hq + (size_t)kvh * group + h) * HD + d] = f2bf(O / L);
        } else {
            const size_t slot = ((size_t)w * p.hkv + kvh) * group + h;
            p.part_o[slot * HD + d] = O;
            if (d == 0) {
                p.part_ml[slot * 2] = M;
                p.part_ml[slot * 2 + 1] = L;
            }
        }
    }
    if (n_chunks == 1) return;
    // Several chunks: the CTA of this (sequence, kv head) that finishes last merges them, in chunk order, so the
    // result does not depend on who is last.  No CTA waits for another; the counter returns to zero for the next call.
    __threadfence();  // this CTA's partial result is visible before its arrival is counted
    __syncthreads();
    if (threadIdx.x == 0) {
        int* counter = p.merge_counters + (size_t)seq * p.hkv + kvh;
        const int arrived = atomicAdd(counter, 1);
        s_last = arrived == n_chunks - 1;
        if (s_last) *counter = 0;
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    // out = sum_c O_c 2^(m_c-M) / sum_c l_c 2^(m_c-M), the sums taken in chunk order.  The merging CTA is on its own here,
    // so its loads are kept independent of one another: every chunk's (max, sum) pair goes to shared memory in one
    // sweep, one thread per head forms the weights in chunk order, then each output adds up its chunks with eight
    // loads in flight.  Batches of kMergeBatch chunks keep the shared-memory use fixed whatever the chunk count.
    constexpr int kMergeBatch = 512;
    float* s_m = reinterpret_cast<float*>(smem);   // [kMergeBatch][8]: a chunk's maximum, then its weight f_c
    float* s_l = s_m + kMergeBatch * 8;            // [kMergeBatch][8]: a chunk's sum
    float* s_M = s_l + kMergeBatch * 8;            // [8]: overall maximum of a head
    float* s_L = s_M + 8;                          // [8]: overall sum of a head
    constexpr int PER = (8 * HD) / (kWarps * 32);  // outputs per thread when the group has 8 heads
    float o_acc[PER];
#pragma unroll
    for (int k = 0; k < PER; k++) o_acc[k] = 0.f;
    // overall maximum per head: taken from shared memory below when all chunks fit one batch (the usual case), else
    // by a first sweep over the chunks (chunk order is irrelevant for a maximum)
    const bool one_batch = n_chunks <= kMergeBatch;
    if (threadIdx.x < group) {
        float mx = -INFINITY;
        if (!one_batch) {
            int c = 0;
            for (; c + 8 <= n_chunks; c += 8) {
                float v[8];
#pragma unroll
                for (int j = 0; j < 8; j++) v[j] = __ldcg(p.part_ml + ((((size_t)(w0 + c + j)) * p.hkv + kvh) * group + threadIdx.x) * 2);
#pragma unroll
                for (int j = 0; j < 8; j++) mx = fmaxf(mx, v[j]);
            }
            for (; c < n_chunks; c++) mx = fmaxf(mx, __ldcg(p.part_ml + ((((size_t)(w0 + c)) * p.hkv + kvh) * group + threadIdx.x) * 2));
        }
        s_M[threadIdx.x] = mx;
        s_L[threadIdx.x] = 0.f;
    }
    __syncthreads();
    for (int c0 = 0; c0 < n_chunks; c0 += kMergeBatch) {
        const int nb = min(kMergeBatch, n_chunks - c0);
        for (int i = threadIdx.x; i < nb * group; i += kWarps * 32) {
            const int c = i / group, h = i - c * group;
            const float2 ml = __ldcg(reinterpret_cast<const float2*>(p.part_ml + ((((size_t)(w0 + c0 + c)) * p.hkv + kvh) * group + h) * 2));
            s_m[c * 8 + h] = ml.x;
            s_l[c * 8 + h] = ml.y;
        }
        __syncthreads();
        if (threadIdx.x < group) {  // weights and the running sum of this head, in chunk order
            float M = s_M[threadIdx.x];
            if (one_batch) {
                for (int c = 0; c < nb; c++) M = fmaxf(M, s_m[c * 8 + threadIdx.x]);
                s_M[threadIdx.x] = M;
            }
            float L = s_L[threadIdx.x];
            for (int c = 0; c < nb; c++) {
                const float f = fast_exp2(s_m[c * 8 + threadIdx.x] - M);
                L += s_l[c * 8 + threadIdx.x] * f;
                s_m[c * 8 + threadIdx.x] = f;
            }
            s_L[threadIdx.x] = L;
        }
        __syncthreads();
        // partial outputs: eight chunks of every output of this thread in flight at a time
        const size_t stride = (size_t)p.hkv * group * HD;  // from one chunk's partial output to the next
        for (int c = 0; c < nb; c += 8) {
            float v[PER][8];
#pragma unroll
            for (int k = 0; k < PER; k++) {
                const int e = threadIdx.x + k * kWarps * 32;
                const float* src = p.part_o + (((size_t)(w0 + c0 + c) * p.hkv + kvh) * group) * HD + e;  // e = h * HD + d
#pragma unroll
                for (int j = 0; j < 8; j++) v[k][j] = (e < group * HD && c + j < nb) ? __ldcg(src + (size_t)j * stride) : 0.f;
            }
#pragma unroll
            for (int k = 0; k < PER; k++) {
                const int e = threadIdx.x + k * kWarps * 32;
                const int h = min(e / HD, 7);
#pragma unroll
                for (int j = 0; j < 8; j++)
                    if (c + j < nb) o_acc[k] += v[k][j] * s_m[(c + j) * 8 + h];
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int k = 0; k < PER; k++) {
        const int e = threadIdx.x + k * kWarps * 32;
        if (e >= group * HD) break;
        const int h = e / HD, d = e % HD;
        p.out[((size_t)qrow * p.hq + (size_t)kvh * group + h) * HD + d] = f2bf(o_acc[k] / s_L[h]);
    }
}

// Two ways to find the work items.  With a work list (the engine's packer builds it with the rest of the step's
// metadata) the grid is (items, kv heads), one item per CTA.  Without one, every CTA of a persistent grid derives the
// list itself from the context lengths (a block-wide scan, up to kInlineSeqs sequences) and takes every gridDim.x-th
// (item, kv head) pair: the whole operation is one launch.
constexpr int kInlineSeqs = 1024;

template <int HD>
__global__ void __launch_bounds__(kWarps * 32) paged_attn_decode_kernel(const DecodeAttnParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    // lets a dependent launch (the projection that consumes this kernel's output, launched with programmatic stream
    // serialisation) begin its weight prefetch now; it still waits for this grid to complete before it reads
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
    pdl_wait();
    if (p.work_seq) {
        const int w = blockIdx.x;
        if (w >= *p.n_work) return;
        const int seq = p.work_seq[w];
        const int w0 = p.seq_work_off[seq];
        decode_item<HD>(p, smem, w, blockIdx.y, seq, p.work_chunk[w], w0, p.seq_work_off[seq + 1] - w0);
        return;
    }
    __shared__ int s_off[kInlineSeqs + 1];  // first work item of every sequence
    __shared__ int s_warp[kWarps];
    {
        const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
        const int per_seq = (p.max_blocks * p.page_tiles + p.chunk_tiles - 1) / p.chunk_tiles;
        int carry = 0;
        for (int base = 0; base < p.num_seqs; base += kWarps * 32) {
            const int i = base + threadIdx.x;
            int n = 0;
            if (i < p.num_seqs) {
                const int tiles = (max(p.ctx_lens[i], 0) + 15) >> 4;
                n = min((tiles + p.chunk_tiles - 1) / p.chunk_tiles, per_seq);
            }
            int incl = n;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int v = __shfl_up_sync(kFull, incl, o);
                if (lane >= o) incl += v;
            }
            if (lane == 31) s_warp[warp] = incl;
            __syncthreads();
            int before = carry;
            for (int ww = 0; ww < warp; ww++) before += s_warp[ww];
            if (i < p.num_seqs) s_off[i] = before + incl - n;
            int total = carry;
            for (int ww = 0; ww < kWarps; ww++) total += s_warp[ww];
            carry = total;
            __syncthreads();
        }
        if (threadIdx.x == 0) s_off[p.num_seqs] = carry;
        __syncthreads();
    }
    const int n_work = s_off[p.num_seqs];
    for (int i = blockIdx.x; i < p.num_seqs; i += gridDim.x)  // an empty context attends to nothing: rows of zeros
        if (s_off[i + 1] == s_off[i]) {
            const int qrow = p.q_rows ? p.q_rows[i] : i;
            for (int e = threadIdx.x; e < p.hq * HD; e += kWarps * 32) p.out[(size_t)qrow * p.hq * HD + e] = 0;
        }
    for (int item = blockIdx.x; item < n_work * p.hkv; item += gridDim.x) {
        const int w = item / p.hkv, kvh = item - w * p.hkv;
        int lo = 0, hi = p.num_seqs - 1;  // the sequence whose items contain w: the last one with s_off <= w among those with items
        while (lo < hi) {
            const int mid = (lo + hi + 1) >> 1;
            if (s_off[mid] <= w)
                lo = mid;
            else
                hi = mid - 1;
        }
        const int seq = lo;  // s_off[seq] <= w < s_off[seq + 1]: sequences without items are never the largest such index
        decode_item<HD>(p, smem, w, kvh, seq, w - s_off[seq], s_off[seq], s_off[seq + 1] - s_off[seq]);
        __syncthreads();  // the pipeline buffers are reused by the next item
    }
}

// Split-K work list for a plain [num_seqs] batch (the engine's packer builds the same list
// together with the rest of the step metadata).
// A context length beyond what the block-table row can address is clamped to `per_seq` chunks (the lists and
// the partial sums are sized for per_seq chunks per sequence; the decode kernel clamps the same way).
__global__ void decode_worklist_kernel(const int32_t* ctx_lens, int num_seqs, int chunk_tiles, int per_seq, int32_t* work_seq,
                                       int32_t* work_chunk, int32_t* seq_work_off, int32_t* n_work) {
    __shared__ int sh[1024];
    __shared__ int carry;
    if (threadIdx.x == 0) carry = 0;
    __syncthreads();
    for (int base = 0; base < num_seqs; base += 1024) {
        const int i = base + threadIdx.x;
        int n = 0;
        if (i < num_seqs) {
            const int tiles = (max(ctx_lens[i], 0) + 15) >> 4;
            n = min((tiles + chunk_tiles - 1) / chunk_tiles, per_seq);
        }
        sh[threadIdx.x] = n;
        __syncthreads();
        for (int d = 1; d < 1024; d <<= 1) {
            int v = threadIdx.x >= d ? sh[threadIdx.x - d] : 0;
            __syncthreads();
            sh[threadIdx.x] += v;
            __syncthreads();
        }
        const int incl = sh[threadIdx.x] + carry, excl = incl - n;
        if (i < num_seqs) {
            seq_work_off[i] = excl;
            for (int c = 0; c < n; c++) {
                work_seq[excl + c] = i;
                work_chunk[excl + c] = c;
            }
        }
        __syncthreads();
        if (threadIdx.x == 1023) carry = incl;
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        seq_work_off[num_seqs] = carry;
        *n_work = carry;
    }
}

template <int HD>
int32_t launch_decode(b2_ctx* ctx, const DecodeAttnParams& p, int grid_work, int num_seqs) {
    const int smem = kWarps * kStages * 2 * 16 * HD * 2;
    B2_SMEM_ONCE(ctx, paged_attn_decode_kernel<HD>, smem);
    dim3 grid(grid_work, p.hkv);
    // in-kernel work list: a fixed grid of sixteen CTAs per SM, each taking every gridDim.x-th item.  Two are resident
    // per SM at a time and none waits for another, so the rest simply queue; the fine grain lets the hardware's block
    // scheduler even out items of different cost (measured: 4 / 8 / 16 CTAs per SM -> 174 / 150 / 137 us on 64 sequences)
    if (!p.work_seq) grid = dim3(16 * ctx->sm_count);
    B2_CUDA(b2_launch_pdl(ctx->pdl_consumers, paged_attn_decode_kernel<HD>, grid, dim3(kWarps * 32), (size_t)smem, ctx->stream, p));
    B2_LAUNCHED(ctx);
    B2_CUDA(cudaGetLastError());
    (void)num_seqs;
    return B2_OK;
}

}  // namespace

size_t b2_decode_attn_scratch_bytes(int max_work, int hq, int head_dim) {
    // part_o [work, hq, hd] f32 + part_ml [work, hq, 2] f32
    return (size_t)max_work * hq * (head_dim + 2) * sizeof(float);
}

// Arrival counters of the fused merge: one int per (sequence, kv head), zero between calls (the kernel resets them).
int32_t b2_decode_attn_counters(b2_ctx* ctx, int num_seqs, int hkv, int** out) {
    const size_t need = (size_t)num_seqs * hkv;
    if (need > ctx->attn_counters_cap) {
        B2_CUDA(cudaStreamSynchronize(ctx->stream));
        if (ctx->attn_counters) B2_CUDA(cudaFree(ctx->attn_counters));
        ctx->attn_counters = nullptr;
        const size_t cap = need + need / 4 + 1024;
        B2_CUDA(cudaMalloc((void**)&ctx->attn_counters, cap * sizeof(int)));
        B2_CUDA(cudaMemsetAsync(ctx->attn_counters, 0, cap * sizeof(int), ctx->stream));
        ctx->attn_counters_cap = cap;
    }
    *out = ctx->attn_counters;
    return B2_OK;
}

int32_t b2_decode_attn_launch(b2_ctx* ctx, const DecodeAttnParams& p, int head_dim, int grid_work, int num_seqs) {
    const int group = p.hq / p.hkv;
    B2_REQUIRE(p.hq % p.hkv == 0 && (group == 1 || group == 2 || group == 4 || group == 8), B2_ERR_UNSUPPORTED,
               "paged_attn_decode: q heads per kv head must be 1, 2, 4 or 8");
    B2_REQUIRE(p.chunk_tiles >= 1 && p.chunk_tiles <= 32 * kWarps, B2_ERR_MSG, "paged_attn_decode: chunk must be 16..2048 tokens");
    B2_REQUIRE(p.merge_counters, B2_ERR_MSG, "paged_attn_decode: no arrival counters for the merge");
    B2_REQUIRE(p.work_seq || (p.num_seqs >= 1 && p.num_seqs <= kInlineSeqs), B2_ERR_MSG, "paged_attn_decode: no work list and too many sequences to derive one in the kernel");
    if (grid_work <= 0 || num_seqs <= 0) return B2_OK;
    if (head_dim == 128) return launch_decode<128>(ctx, p, grid_work, num_seqs);
    if (head_dim == 64) return launch_decode<64>(ctx, p, grid_work, num_seqs);
    return b2_fail(B2_ERR_UNSUPPORTED, "paged_attn_decode: head_dim must be 64 or 128");
}

extern "C" int32_t b2_paged_attn_decode(b2_ctx* ctx, const uint16_t* q_dev, const uint16_t* k_pool_dev,
                                        const uint16_t* v_pool_dev, const int32_t* block_tables_dev, int32_t max_blocks,
                                        const int32_t* ctx_lens_dev, int32_t num_seqs, int32_t hq, int32_t hkv,
                                        int32_t head_dim, int32_t page_size, float scale, int32_t chunk_tokens,
                                        uint16_t* out_dev) {
    B2_REQUIRE(ctx && q_dev && k_pool_dev && v_pool_dev && block_tables_dev && ctx_lens_dev && out_dev, B2_ERR_MSG,
               "b2_paged_attn_decode: null argument");
    B2_REQUIRE(num_seqs >= 0 && max_blocks > 0, B2_ERR_MSG, "b2_paged_attn_decode: bad sizes");
    B2_REQUIRE(page_size > 0 && page_size % 16 == 0, B2_ERR_UNSUPPORTED, "b2_paged_attn_decode: page_size must be a multiple of 16");
    B2_REQUIRE(hkv > 0 && hq % hkv == 0, B2_ERR_MSG, "b2_paged_attn_decode: hq must be a multiple of hkv");
    if (num_seqs == 0) return B2_OK;
    if (chunk_tokens <= 0) {
        // Enough (chunk, kv head) items for ~8 per SM, chunks between 128 and 1024 tokens; the contexts live on the
        // device, so the batch is taken to be half full (half of what its block tables can hold).  Longer chunks mean
        // fewer partial results to write, read back and merge: on 64 sequences of 128-4096 tokens the operation takes
        // 204 / 137 / 115 / 112 us at 128 / 256 / 512 / 1024.
        const long est_tokens = (long)num_seqs * max_blocks * page_size / 2;
        const long want = est_tokens * hkv / ((long)ctx->sm_count * 8);
        chunk_tokens = 128;
        while (chunk_tokens < 1024 && chunk_tokens < want) chunk_tokens *= 2;
    }
    B2_REQUIRE(chunk_tokens % 16 == 0, B2_ERR_MSG, "b2_paged_attn_decode: chunk_tokens must be a multiple of 16");
    const int chunk_tiles = chunk_tokens / 16;
    const int page_tiles = page_size / 16;
    const long max_tiles = (long)max_blocks * page_tiles;
    const long per_seq = (max_tiles + chunk_tiles - 1) / chunk_tiles;
    const long max_work = per_seq * num_seqs;
    B2_REQUIRE(max_work < (1l << 30), B2_ERR_MSG, "b2_paged_attn_decode: work list too large");

    // scratch: partials, then (more than kInlineSeqs sequences only) the work list a first kernel builds
    const bool inline_list = num_seqs <= kInlineSeqs;
    size_t part_bytes = b2_decode_attn_scratch_bytes((int)max_work, hq, head_dim);
    part_bytes = (part_bytes + 255) & ~(size_t)255;
    const size_t list_bytes = inline_list ? 0 : ((size_t)max_work * 2 + num_seqs + 2) * sizeof(int32_t);
    void* scratch = nullptr;
    B2_CHECK(b2_ctx_scratch(ctx, part_bytes + list_bytes, &scratch));
    DecodeAttnParams p{};
    p.q = q_dev;
    p.k_pool = k_pool_dev;
    p.v_pool = v_pool_dev;
    p.block_tables = block_tables_dev;
    p.max_blocks = max_blocks;
    p.ctx_lens = ctx_lens_dev;
    p.num_seqs = num_seqs;
    p.chunk_tiles = chunk_tiles;
    p.hq = hq;
    p.hkv = hkv;
    p.page_tiles = page_tiles;
    p.scale_log2 = scale * 1.4426950408889634f;
    p.part_o = reinterpret_cast<float*>(scratch);
    p.part_ml = p.part_o + (size_t)max_work * hq * head_dim;
    p.out = out_dev;
    B2_CHECK(b2_decode_attn_counters(ctx, num_seqs, hkv, &p.merge_counters));
    if (!inline_list) {
        int32_t* lists = reinterpret_cast<int32_t*>(reinterpret_cast<uint8_t*>(scratch) + part_bytes);
        int32_t* seq_off = lists + 2 * max_work;
        p.work_seq = lists;
        p.work_chunk = lists + max_work;
        p.seq_work_off = seq_off;
        p.n_work = seq_off + num_seqs + 1;
        decode_worklist_kernel<<<1, 1024, 0, ctx->stream>>>(ctx_lens_dev, num_seqs, chunk_tiles, (int)per_seq, lists, lists + max_work, seq_off,
                                                            seq_off + num_seqs + 1);
        B2_LAUNCHED(ctx);
    }
    return b2_decode_attn_launch(ctx, p, head_dim, (int)max_work, num_seqs);
}

extern "C" int32_t b2_paged_attn_decode_host(b2_ctx* ctx, const uint16_t* q_host, const uint16_t* k_pool_dev,
                                             const uint16_t* v_pool_dev, const int32_t* block_tables_dev, int32_t max_blocks,
                                             const int32_t* ctx_lens_dev, int32_t num_seqs, int32_t hq, int32_t hkv,
                                             int32_t head_dim, int32_t page_size, float scale, int32_t chunk_tokens,
                                             uint16_t* out_host) {
    B2_REQUIRE(ctx && q_host && out_host, B2_ERR_MSG, "b2_paged_attn_decode_host: null argument");
    const size_t bytes = (size_t)num_seqs * hq * head_dim * 2;
    void* stage = nullptr;
    B2_CHECK(b2_ctx_stage(ctx, 2 * bytes, &stage));
    uint16_t* qd = reinterpret_cast<uint16_t*>(stage);
    uint16_t* od = qd + bytes / 2;
    B2_CUDA(cudaMemcpyAsync(qd, q_host, bytes, cudaMemcpyHostToDevice, ctx->stream));
    B2_CHECK(b2_paged_attn_decode(ctx, qd, k_pool_dev, v_pool_dev, block_tables_dev, max_blocks, ctx_lens_dev, num_seqs, hq, hkv,
                                  head_dim, page_size, scale, chunk_tokens, od));
    B2_CUDA(cudaMemcpyAsync(out_host, od, bytes, cudaMemcpyDeviceToHost, ctx->stream));
    B2_CUDA(cudaStreamSynchronize(ctx->stream));
    return B2_OK;
}

// ---------------------------------------------------------------------------------------------------
// Decode attention for callers that must not allocate.
//
// Some hosts of this library cannot reach cudaMalloc at the moment they need attention: a serving
// loop that has handed every free byte of HBM to its KV pool, a thread that runs under a real-time
// deadline, or an embedding runtime that owns the allocator and forbids foreign allocations.  For
// them the split-K scratch (partial outputs, running max / sum, the merge's arrival counters) lives in the fixed
// array below, which every GPU that loads this library carries until the process exits.
constexpr size_t kStaticScratchBytes = 16u << 20;  // 16 MiB per device
constexpr size_t kStaticCounterBytes = 64u << 10;  // its first 64 KiB: the merge's arrival counters
static __device__ __align__(256) unsigned char g_decode_scratch[kStaticScratchBytes];

namespace {
// Device address of g_decode_scratch per device.  In host code the array's name is only a handle
// for the runtime, not an address a kernel could use, so it is resolved once per device with
// cudaGetSymbolAddress while that device is current.  The two caches below are plain globals: two host
// threads that make their FIRST call on one device at the same moment both run the set-up and store the
// same values, which is harmless; after that the call only reads them.
unsigned char* g_scratch_addr[64] = {};
bool g_static_smem_set[64][2] = {};
int g_static_grid[64][2] = {};  // sixteen CTAs per SM of the device
}  // namespace

extern "C" int32_t b2_paged_attn_decode_static(void* stream, const uint16_t* q_dev, const uint16_t* k_pool_dev,
                                               const uint16_t* v_pool_dev, const int32_t* block_tables_dev, int32_t max_blocks,
                                               const int32_t* ctx_lens_dev, int32_t num_seqs, int32_t hq, int32_t hkv, int32_t head_dim,
                                               int32_t page_size, float scale, int32_t chunk_tokens, uint16_t* out_dev) {
    B2_REQUIRE(q_dev && k_pool_dev && v_pool_dev && block_tables_dev && ctx_lens_dev && out_dev, B2_ERR_MSG,
               "b2_paged_attn_decode_static: null argument");
    B2_REQUIRE(num_seqs >= 0 && max_blocks > 0, B2_ERR_MSG, "b2_paged_attn_decode_static: bad sizes");
    B2_REQUIRE(page_size > 0 && page_size % 16 == 0, B2_ERR_UNSUPPORTED, "b2_paged_attn_decode_static: page_size must be a multiple of 16");
    B2_REQUIRE(hkv > 0 && hq % hkv == 0, B2_ERR_MSG, "b2_paged_attn_decode_static: hq must be a multiple of hkv");
    const int group = hq / hkv;
    B2_REQUIRE(group == 1 || group == 2 || group == 4 || group == 8, B2_ERR_UNSUPPORTED,
               "b2_paged_attn_decode_static: q heads per kv head must be 1, 2, 4 or 8");
    B2_REQUIRE(head_dim == 64 || head_dim == 128, B2_ERR_UNSUPPORTED, "b2_paged_attn_decode_static: head_dim must be 64 or 128");
    if (num_seqs == 0) return B2_OK;
    if (chunk_tokens <= 0) chunk_tokens = 512;
    B2_REQUIRE(chunk_tokens % 16 == 0 && chunk_tokens <= 2048, B2_ERR_MSG, "b2_paged_attn_decode_static: chunk_tokens must be a multiple of 16, at most 2048");
    const int chunk_tiles = chunk_tokens / 16, page_tiles = page_size / 16;
    const long per_seq = ((long)max_blocks * page_tiles + chunk_tiles - 1) / chunk_tiles;
    const long max_work = per_seq * num_seqs;
    B2_REQUIRE(num_seqs <= kInlineSeqs && (long)num_seqs * hkv * sizeof(int) <= (long)kStaticCounterBytes, B2_ERR_MSG,
               "b2_paged_attn_decode_static: at most 1024 sequences and 16384 (sequence, kv head) pairs per call");
    const size_t part_bytes = (size_t)max_work * hq * (head_dim + 2) * sizeof(float);
    B2_REQUIRE(kStaticCounterBytes + part_bytes <= kStaticScratchBytes, B2_ERR_MSG,
               "b2_paged_attn_decode_static: this batch needs " + std::to_string(kStaticCounterBytes + part_bytes) +
                   " bytes of split-K scratch, the fixed array holds " + std::to_string(kStaticScratchBytes) +
                   " (raise chunk_tokens, lower max_blocks, or use b2_paged_attn_decode)");
    int dev = 0;
    B2_CUDA(cudaGetDevice(&dev));
    B2_REQUIRE(dev >= 0 && dev < 64, B2_ERR_UNSUPPORTED, "b2_paged_attn_decode_static: device index above 63");
    if (!g_scratch_addr[dev]) {
        unsigned char* ptr = nullptr;
        B2_CUDA(cudaGetSymbolAddress((void**)&ptr, g_decode_scratch));
        g_scratch_addr[dev] = ptr;
    }
    const int smem = kWarps * kStages * 2 * 16 * head_dim * 2;
    if (!g_static_smem_set[dev][head_dim == 128]) {
        if (head_dim == 128)
            B2_CUDA(cudaFuncSetAttribute(paged_attn_decode_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        else
            B2_CUDA(cudaFuncSetAttribute(paged_attn_decode_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        g_static_smem_set[dev][head_dim == 128] = true;
    }
    unsigned char* scratch = g_scratch_addr[dev];
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    if (!g_static_grid[dev][head_dim == 128]) {
        int sms = 0;
        B2_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
        g_static_grid[dev][head_dim == 128] = 16 * sms;
    }
    DecodeAttnParams p{};
    p.q = q_dev;
    p.k_pool = k_pool_dev;
    p.v_pool = v_pool_dev;
    p.block_tables = block_tables_dev;
    p.max_blocks = max_blocks;
    p.ctx_lens = ctx_lens_dev;
    p.num_seqs = num_seqs;
    p.chunk_tiles = chunk_tiles;
    p.hq = hq;
    p.hkv = hkv;
    p.page_tiles = page_tiles;
    p.scale_log2 = scale * 1.4426950408889634f;
    // Layout of the array: [arrival counters, kStaticCounterBytes][partial outputs][running max / sum].  Only the counters
    // have to start at zero: the array is zero when the library is loaded and the kernel returns every counter it used
    // to zero before it ends; every partial result the merge reads is written by this call first.
    p.merge_counters = reinterpret_cast<int*>(scratch);
    p.part_o = reinterpret_cast<float*>(scratch + kStaticCounterBytes);
    p.part_ml = p.part_o + (size_t)max_work * hq * head_dim;
    p.out = out_dev;
    const dim3 grid((unsigned)g_static_grid[dev][head_dim == 128]);
    if (head_dim == 128)
        paged_attn_decode_kernel<128><<<grid, kWarps * 32, smem, st>>>(p);
    else
        paged_attn_decode_kernel<64><<<grid, kWarps * 32, smem, st>>>(p);
    B2_CUDA(cudaGetLastError());
    return B2_OK;
}
