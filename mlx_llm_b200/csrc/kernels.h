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
    const int32_t* work_seq;      // [n_work] sequence of each split-K work item
    const int32_t* work_chunk;    // [n_work] chunk index inside its sequence
    const int32_t* seq_work_off;  // [num_seqs + 1] first work item of each sequence
    const int32_t* n_work;        // device scalar: number of valid work items (grid may be larger)
    int chunk_tiles;              // 16-token tiles per chunk
    int hq, hkv, page_tiles;      // page_tiles = page_size / 16
    float scale_log2;             // softmax scale * log2(e)
    float* part_o;                // [n_work, hkv, group, hd] unnormalised partial outputs
    float* part_ml;               // [n_work, hkv, group, 2] running max (log2 domain) and sum
    uint16_t* out;                // [rows, hq, hd] bf16
};
size_t b2_decode_attn_scratch_bytes(int max_work, int hq, int head_dim);
int32_t b2_decode_attn_launch(b2_ctx* ctx, const DecodeAttnParams& p, int head_dim, int grid_work, int num_seqs);
