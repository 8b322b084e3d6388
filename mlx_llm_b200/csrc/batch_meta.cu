// Ragged-batch packer: builds one step's scheduling metadata on the GPU.
//
// The reference has no counterpart (it runs whole-prompt batch-1 prefills and per-sequence decode
// forwards, src/decode/continuous.rs:254-301); this kernel is what lets one forward carry decode
// tokens and prefill chunks of many sequences.  From the per-sequence descriptors the host scheduler
// uploads (block-table row, new-token count, cached length) it produces, in one launch:
//   block-table updates, cu_seqlens, context lengths, per-token positions / owning sequence /
//   KV slot (page * page_size + offset), rows that sample a token, the compact decode-sequence
//   arrays with their split-K work list, and the prefill query-tile work list.
// All outputs are integers and are checked bit-for-bit against a CPU restatement.
#include "common.cuh"
#include "kernels.h"

namespace {

constexpr unsigned kFull = 0xffffffffu;

// Exclusive prefix sum of v over the 1024-thread block; `total` receives the block sum.
__device__ __forceinline__ int block_scan_excl(int v, int* warp_sums, int& total) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int incl = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int n = __shfl_up_sync(kFull, incl, o);
        if (lane >= o) incl += n;
    }
    if (lane == 31) warp_sums[warp] = incl;
    __syncthreads();
    if (warp == 0) {
        int ws = warp_sums[lane];
        int wi = ws;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int n = __shfl_up_sync(kFull, wi, o);
            if (lane >= o) wi += n;
        }
        warp_sums[lane] = wi - ws;  // exclusive per-warp offset
        if (lane == 31) warp_sums[32] = wi;
    }
    __syncthreads();
    const int excl = warp_sums[warp] + incl - v;
    total = warp_sums[32];
    __syncthreads();
    return excl;
}

__global__ void __launch_bounds__(1024) batch_meta_kernel(const BatchMetaIn in, const BatchMetaOut out) {
    __shared__ int ws[33];
    __shared__ int err;
    const int tid = threadIdx.x;
    if (tid == 0) err = 0;
    for (int u = tid; u < in.U; u += 1024) {
        const int idx = in.upd_index[u];
        if (idx < 0 || idx >= in.max_blocks)
            err = 1;
        else
            out.block_tables[(size_t)in.upd_slot[u] * in.max_blocks + idx] = in.upd_page[u];
    }
    __syncthreads();

    int c_q = 0, c_lg = 0, c_dec = 0, c_dw = 0, c_pw = 0;
    for (int base = 0; base < in.B; base += 1024) {
        const int i = base + tid;
        const bool ok = i < in.B;
        const int ql = ok ? in.q_len[i] : 0;
        const int cb = ok ? in.ctx_before[i] : 0;
        const int ctx = cb + ql;
        const int want = ok && ql > 0 && in.want_logits[i] != 0;
        const int is_dec = ok && ql == 1;
        const int tiles = (ctx + 15) >> 4;
        const int n_chunks = is_dec ? (tiles + in.chunk_tiles - 1) / in.chunk_tiles : 0;
        const int n_qt = (ok && ql > 1) ? (ql + in.q_tile - 1) / in.q_tile : 0;
        int t_q, t_lg, t_dec, t_dw, t_pw;
        const int e_q = c_q + block_scan_excl(ql, ws, t_q);
        const int e_lg = c_lg + block_scan_excl(want, ws, t_lg);
        const int e_dec = c_dec + block_scan_excl(is_dec, ws, t_dec);
        const int e_dw = c_dw + block_scan_excl(n_chunks, ws, t_dw);
        const int e_pw = c_pw + block_scan_excl(n_qt, ws, t_pw);
        if (ok) {
            out.cu_seqlens[i] = e_q;
            out.context_lens[i] = ctx;
            if (want) {
                out.logit_rows[e_lg] = e_q + ql - 1;
                out.logit_seq[e_lg] = i;
            }
            if (is_dec) {
                out.dec_ctx[e_dec] = ctx;
                out.dec_qrow[e_dec] = e_q;
                out.dec_slot[e_dec] = in.seq_slot[i];
                out.dec_work_off[e_dec] = e_dw;
                for (int c = 0; c < n_chunks; c++) {
                    out.dec_work_seq[e_dw + c] = e_dec;
                    out.dec_work_chunk[e_dw + c] = c;
                }
            }
            for (int j = 0; j < n_qt; j++) {
                out.pf_seq[e_pw + j] = i;
                out.pf_qstart[e_pw + j] = j * in.q_tile;
            }
        }
        c_q += t_q;
        c_lg += t_lg;
        c_dec += t_dec;
        c_dw += t_dw;
        c_pw += t_pw;
    }
    if (tid == 0) {
        out.cu_seqlens[in.B] = c_q;
        out.dec_work_off[c_dec] = c_dw;
    }
    __syncthreads();
    // per-token metadata: owning sequence by binary search over cu_seqlens
    for (int t = tid; t < in.T; t += 1024) {
        int lo = 0, hi = in.B - 1;
        while (lo < hi) {
            const int mid = (lo + hi + 1) >> 1;
            if (out.cu_seqlens[mid] <= t)
                lo = mid;
            else
                hi = mid - 1;
        }
        // sequences with q_len == 0 share a start offset with their successor: take the last one whose
        // start is <= t (found above) — it is the one that owns t because empty ones sort before it
        const int pos = in.ctx_before[lo] + (t - out.cu_seqlens[lo]);
        out.positions[t] = pos;
        out.token_seq[t] = lo;
        const int blk = pos / in.page_size;
        if (blk >= in.max_blocks) {
            err = 1;
            out.slot_mapping[t] = -1;
        } else {
            const int page = out.block_tables[(size_t)in.seq_slot[lo] * in.max_blocks + blk];
            out.slot_mapping[t] = page * in.page_size + pos % in.page_size;
        }
    }
    __syncthreads();
    if (tid == 0) {
        out.counts[0] = c_lg;
        out.counts[1] = c_dec;
        out.counts[2] = c_dw;
        out.counts[3] = c_pw;
        out.counts[4] = err;
        out.counts[5] = c_q;
    }
}

}  // namespace

int32_t b2_batch_meta_launch(b2_ctx* ctx, const BatchMetaIn& in, const BatchMetaOut& out) {
    B2_REQUIRE(in.B >= 0 && in.T >= 0 && in.U >= 0, B2_ERR_MSG, "batch_meta: negative size");
    B2_REQUIRE(in.chunk_tiles >= 1 && in.q_tile >= 1 && in.page_size >= 1 && in.max_blocks >= 1, B2_ERR_MSG, "batch_meta: bad parameter");
    batch_meta_kernel<<<1, 1024, 0, ctx->stream>>>(in, out);
    B2_LAUNCHED(ctx);
    B2_CUDA(cudaGetLastError());
    return B2_OK;
}
