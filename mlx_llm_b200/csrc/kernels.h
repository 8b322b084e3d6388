// Internal launch interfaces shared between the kernel files, the C ABI and the engine.
#pragma once
#include <stddef.h>
#include <stdint.h>

struct b2_ctx;

// Paged-attention decode (paged_attn_decode.cu).  All pointers are device pointers.
struct DecodeAttnParams {
    const uint16_t* q;            // [rows, hq, hd] bf16; row of sequence i is q_rows[i] (or i)
    const uint16_t* k_pool;       // [pages, hkv, page, hd] bf16
    const uint16_t* v_pool;
    const int32_t* block_tables;  // [rows, max_blocks]; row of sequence i is bt_rows[i] (or i)
    int max_blocks;
    const int32_t* bt_rows;       // nullable
    const int32_t* q_rows;        // nullable
    const int32_t* ctx_lens;      // [num_seqs]
    int num_seqs;                 // used when there is no work list
    const int32_t* work_seq;      // [n_work] sequence of each split-K work item; null: the kernel derives the list from ctx_lens
    const int32_t* work_chunk;    // [n_work] chunk index inside its sequence
    const int32_t* seq_work_off;  // [num_seqs + 1] first work item of each sequence
    const int32_t* n_work;        // device scalar: number of valid work items (grid may be larger)
    int chunk_tiles;              // 16-token tiles per chunk
    int hq, hkv, page_tiles;      // page_tiles = page_size / 16
    float scale_log2;             // softmax scale * log2(e)
    float* part_o;                // [n_work, hkv, group, hd] unnormalised partial outputs
    float* part_ml;               // [n_work, hkv, group, 2] running max (log2 domain) and sum
    int* merge_counters;          // [num_seqs, hkv] arrivals per (sequence, kv head), zero between launches
    uint16_t* out;                // [rows, hq, hd] bf16
};
size_t b2_decode_attn_scratch_bytes(int max_work, int hq, int head_dim);
int32_t b2_decode_attn_counters(b2_ctx* ctx, int num_seqs, int hkv, int** out);
int32_t b2_decode_attn_launch(b2_ctx* ctx, const DecodeAttnParams& p, int head_dim, int grid_work, int num_seqs);

// ---- GEMM (gemm.cu) ----------------------------------------------------------------------------
enum { EPI_BF16 = 0, EPI_BF16_RESADD = 1, EPI_F32 = 2 };
struct GemmParams {
    const uint16_t* x;       // [M, K] bf16, row stride ldx
    const void* w;           // dense: [N, K] bf16; quantized: [N, K*bits/32] u32
    const uint16_t* scales;  // [N, K/64] bf16 (quantized only)
    const uint16_t* biases;
    int bits;                // 0 dense, 4, 8
    int group;               // 64
    int M, N, K;
    int ldx, ldo, ldres;
    int x_rows_cap;          // rows of the x allocation (0: M); lets a TMA descriptor outlive a change of M
    int epilogue;
    uint16_t* out;           // bf16 output (EPI_BF16 / EPI_BF16_RESADD)
    const uint16_t* res;     // residual input (may alias out)
    float* out_f32;          // EPI_F32
    // EPI_F32 split by column range (tensor-parallel reductions over peer memory): when f32_chunk > 0, column f of
    // the result is stored at out_f32_by_chunk[f / f32_chunk] + t*ldo + f instead, each entry being the same
    // [M, ldo] view inside another rank's memory, so that the projection's epilogue itself carries every partial
    // sum to the rank that will add it up.  f32_chunk is a multiple of 4.
    float* out_f32_by_chunk[8];
    int f32_chunk;
    // Optional (quantized, tcgen05 path): sbt[g * N + n] = scale(n, g) | bias(n, g) << 16, the scales and biases
    // transposed and interleaved so that the 32 feature rows of a warp read one 128-byte line per K group.
    const uint32_t* sbt;
};
#ifdef __CUDACC__
__device__ __forceinline__ float* gemm_f32_dst(const GemmParams& p, int t, int f) {
    float* base = p.out_f32;
    if (p.f32_chunk > 0) {
        const int q = f / p.f32_chunk;
        base = p.out_f32_by_chunk[0];
#pragma unroll
        for (int i = 1; i < 8; i++)
            if (q == i) base = p.out_f32_by_chunk[i];
    }
    return base + (size_t)t * p.ldo + f;
}
#endif
int32_t b2_gemm_launch(b2_ctx* ctx, const GemmParams& p);
// weight-streaming kernel for up to 64 tokens (gemm_stream.cu): taken by b2_gemm_launch when eligible.
bool b2_gemm_stream_eligible(const GemmParams& p);
int32_t b2_gemm_stream_launch(b2_ctx* ctx, const GemmParams& p);
// tcgen05 / TMEM path, CTA-pair form (gemm_tc.cu): taken by b2_gemm_launch when eligible.
bool b2_gemm_tc_eligible(const GemmParams& p);
int32_t b2_gemm_tc_launch(b2_ctx* ctx, const GemmParams& p);
// fills sbt (N * G words) from scales / biases [N, G] (see GemmParams::sbt); enqueued on the context's stream
int32_t b2_gemm_build_sbt(b2_ctx* ctx, const uint16_t* scales_dev, const uint16_t* biases_dev, int N, int G, uint32_t* sbt_dev);

// ---- elementwise / normalisation / embedding / sampling (fused_ops.cu) ---------------------------
// out = rmsnorm(x) * w, one row per token; rows gathered through `row_idx` when non-null.
int32_t b2_rms_norm_launch(b2_ctx* ctx, const uint16_t* x, const uint16_t* w, float eps, int rows, int dim, int ldx,
                           const int32_t* row_idx, uint16_t* out);
int32_t b2_embed_launch(b2_ctx* ctx, const uint16_t* table, const int32_t* ids, int n, int dim, int vocab, uint16_t* out);
// out[t, i] = bf16(bf16(g*bf16(sigmoid(g))) * u), g = gu[t, i], u = gu[t, inter + i]
int32_t b2_swiglu_launch(b2_ctx* ctx, const uint16_t* gate_up, int rows, int inter, uint16_t* out);
int32_t b2_swiglu2_launch(b2_ctx* ctx, const uint16_t* gate, const uint16_t* up, int64_t n, uint16_t* out);
int32_t b2_add_launch(b2_ctx* ctx, const uint16_t* a, const uint16_t* b, int64_t n, uint16_t* out);
// x = bf16(x + bf16(y)), y f32 (n a multiple of 4 for the vector path; any n works)
int32_t b2_residual_add_f32_launch(b2_ctx* ctx, const float* y, int64_t n, uint16_t* x);
// Greedy argmax per row over bf16 logits, ties -> lowest index.
int32_t b2_argmax_launch(b2_ctx* ctx, const uint16_t* logits, int rows, int vocab, int32_t* out);
int32_t b2_dequantize_launch(b2_ctx* ctx, const uint32_t* packed, const uint16_t* scales, const uint16_t* biases, int64_t rows,
                             int64_t in_dim, int bits, uint16_t* out);
int32_t b2_unpack_launch(b2_ctx* ctx, const uint32_t* packed, int64_t rows, int64_t in_dim, int bits, uint8_t* out);
int32_t b2_quantize_launch(b2_ctx* ctx, const uint16_t* w, int64_t rows, int64_t in_dim, int bits, uint32_t* packed, uint16_t* scales,
                           uint16_t* biases);

// ---- RoPE + (optional per-head q/k RMSNorm) + KV append (rope_kv.cu) ----------------------------
struct RopeKvParams {
    uint16_t* qkv;            // [T, (hq + 2*hkv) * hd] bf16: q heads, then k heads, then v heads
    int ld;                   // row stride of qkv in elements
    const int32_t* positions;     // [T]
    const int32_t* slot_mapping;  // [T] page * page_size + offset; < 0 skips the cache write
    const uint16_t* cos_table;    // [max_pos, hd/2] bf16
    const uint16_t* sin_table;
    const uint16_t* q_norm;       // [hd] or null
    const uint16_t* k_norm;
    float eps;
    int T, hq, hkv, hd, page_size;
    uint16_t* k_pool;  // [pages, hkv, page_size, hd]
    uint16_t* v_pool;
    uint16_t* q_out;   // [T, hq, hd] rotated queries (may alias the q part of qkv when ld == hq*hd)
};
int32_t b2_rope_kv_launch(b2_ctx* ctx, const RopeKvParams& p);

// ---- step metadata / ragged-batch packer (batch_meta.cu) ----------------------------------------
struct BatchMetaIn {   // device pointers into the step's staging buffer
    const int32_t* seq_slot;     // [B] row of the device block table
    const int32_t* q_len;        // [B] new tokens this step
    const int32_t* ctx_before;   // [B] tokens already cached
    const int32_t* want_logits;  // [B]
    const int32_t* upd_slot;     // [U] block-table updates: table[slot][index] = page
    const int32_t* upd_index;
    const int32_t* upd_page;
    int B, T, U;
    int chunk_tiles;     // decode split-K chunk in 16-token tiles
    int q_tile;          // prefill query tile (tokens)
    int page_size, max_blocks;
};
struct BatchMetaOut {  // device arrays owned by the engine, sized for the maxima
    int32_t* block_tables;   // [slots, max_blocks] persistent
    int32_t* cu_seqlens;     // [B + 1]
    int32_t* context_lens;   // [B]
    int32_t* positions;      // [T]
    int32_t* token_seq;      // [T]
    int32_t* slot_mapping;   // [T]
    int32_t* logit_rows;     // [B] token row of each sequence that samples this step
    int32_t* logit_seq;      // [B] batch index of it
    int32_t* dec_ctx;        // [n_dec] per decode sequence: context length,
    int32_t* dec_qrow;       //         token row,
    int32_t* dec_slot;       //         block-table row
    int32_t* dec_work_seq;   // [n_dec_work] split-K work list (index into the decode arrays)
    int32_t* dec_work_chunk;
    int32_t* dec_work_off;   // [n_dec + 1]
    int32_t* pf_seq;         // [n_pf_work] prefill work list: batch index,
    int32_t* pf_qstart;      //              first query row within the sequence's new tokens
    int32_t* counts;         // [8]: n_logits, n_dec, n_dec_work, n_pf_work, error flag
};
int32_t b2_batch_meta_launch(b2_ctx* ctx, const BatchMetaIn& in, const BatchMetaOut& out);
// Carve the output arrays (except block_tables) out of one int32 buffer in the documented order.
void b2_batch_meta_carve(int32_t* base, int B, int T, int W, int P, BatchMetaOut& o);

// ---- chunked-prefill paged attention (paged_attn_prefill.cu) -------------------------------------
struct PrefillAttnParams {
    const uint16_t* q;           // [T, hq, hd] rotated queries
    const uint16_t* k_pool;
    const uint16_t* v_pool;
    const int32_t* block_tables; // [slots, max_blocks]
    int max_blocks;
    const int32_t* seq_slot;     // [B]
    const int32_t* cu_seqlens;   // [B + 1]
    const int32_t* context_lens; // [B] including this step's tokens
    const int32_t* pf_seq;       // [n_work]
    const int32_t* pf_qstart;
    const int32_t* n_work;       // device scalar
    int hq, hkv, page_tiles;
    float scale_log2;
    uint16_t* out;               // [T, hq, hd]
    int q_tile;                  // queries per work item: b2_prefill_q_tile() at the time the work list was built
    int q_rows;                  // rows of the q allocation (>= T)
    int64_t pool_rows;           // rows of one layer's K (or V) pool = pages * hkv * page_size (or any bound >= it)
    int max_ctx;                 // host's bound on the contexts of this launch (0: unknown): lets few, long work items be split over keys
};
// 128 when the tcgen05 kernel (paged_attn_prefill_tc.cu) will take the launch, else 64.
int b2_prefill_q_tile(const b2_ctx* ctx, int head_dim);
int32_t b2_prefill_attn_launch(b2_ctx* ctx, const PrefillAttnParams& p, int head_dim, int grid_work);
bool b2_prefill_attn_tc_eligible(const PrefillAttnParams& p, int head_dim);
int32_t b2_prefill_attn_tc_launch(b2_ctx* ctx, const PrefillAttnParams& p, int grid_work);
