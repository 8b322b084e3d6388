// Kernel-level entry points of the C ABI (parity tests and microbenchmarks call these).
#include <cmath>
#include <vector>

#include "common.cuh"
#include "kernels.h"

// Carve the packer's output arrays out of one int32 buffer, in the documented order.
void b2_batch_meta_carve(int32_t* base, int B, int T, int W, int P, BatchMetaOut& o) {
    int32_t* c = base;
    o.cu_seqlens = c; c += B + 1;
    o.context_lens = c; c += B;
    o.positions = c; c += T;
    o.token_seq = c; c += T;
    o.slot_mapping = c; c += T;
    o.logit_rows = c; c += B;
    o.logit_seq = c; c += B;
    o.dec_ctx = c; c += B;
    o.dec_qrow = c; c += B;
    o.dec_slot = c; c += B;
    o.dec_work_off = c; c += B + 1;
    o.dec_work_seq = c; c += W;
    o.dec_work_chunk = c; c += W;
    o.pf_seq = c; c += P;
    o.pf_qstart = c; c += P;
    o.counts = c;
}

extern "C" {

int32_t b2_quantize(b2_ctx* ctx, const uint16_t* w_dev, int64_t out_dim, int64_t in_dim, int32_t group, int32_t bits,
                    uint32_t* packed_dev, uint16_t* scales_dev, uint16_t* biases_dev) {
    B2_REQUIRE(ctx && w_dev && packed_dev && scales_dev && biases_dev, B2_ERR_MSG, "b2_quantize: null argument");
    B2_REQUIRE(group == 64, B2_ERR_UNSUPPORTED, "b2_quantize: only group size 64 is supported");
    B2_REQUIRE(bits == 4 || bits == 8, B2_ERR_UNSUPPORTED, "b2_quantize: bits must be 4 or 8");
    B2_REQUIRE(in_dim % group == 0, B2_ERR_MSG, "b2_quantize: group size must divide the input dimension");
    return b2_quantize_launch(ctx, w_dev, out_dim, in_dim, bits, packed_dev, scales_dev, biases_dev);
}

int32_t b2_dequantize(b2_ctx* ctx, const uint32_t* packed_dev, const uint16_t* scales_dev, const uint16_t* biases_dev,
                      int64_t out_dim, int64_t in_dim, int32_t group, int32_t bits, uint16_t* w_dev) {
    B2_REQUIRE(ctx && packed_dev && scales_dev && biases_dev && w_dev, B2_ERR_MSG, "b2_dequantize: null argument");
    B2_REQUIRE(group == 64, B2_ERR_UNSUPPORTED, "b2_dequantize: only group size 64 is supported");
    B2_REQUIRE(bits == 4 || bits == 8, B2_ERR_UNSUPPORTED, "b2_dequantize: bits must be 4 or 8");
    B2_REQUIRE(in_dim % group == 0, B2_ERR_MSG, "b2_dequantize: group size must divide the input dimension");
    return b2_dequantize_launch(ctx, packed_dev, scales_dev, biases_dev, out_dim, in_dim, bits, w_dev);
}

int32_t b2_unpack_codes(b2_ctx* ctx, const uint32_t* packed_dev, int64_t out_dim, int64_t in_dim, int32_t bits, uint8_t* codes_dev) {
    B2_REQUIRE(ctx && packed_dev && codes_dev, B2_ERR_MSG, "b2_unpack_codes: null argument");
    B2_REQUIRE(bits == 4 || bits == 8, B2_ERR_UNSUPPORTED, "b2_unpack_codes: bits must be 4 or 8");
    return b2_unpack_launch(ctx, packed_dev, out_dim, in_dim, bits, codes_dev);
}

static int32_t gemm_both(b2_ctx* ctx, GemmParams p, uint16_t* y_bf16, float* y_f32) {
    B2_REQUIRE(y_bf16 || y_f32, B2_ERR_MSG, "matmul: no output buffer");
    if (y_bf16) {
        p.epilogue = EPI_BF16;
        p.out = y_bf16;
        B2_CHECK(b2_gemm_launch(ctx, p));
    }
    if (y_f32) {
        p.epilogue = EPI_F32;
        p.out_f32 = y_f32;
        B2_CHECK(b2_gemm_launch(ctx, p));
    }
    return B2_OK;
}

int32_t b2_qmm(b2_ctx* ctx, const uint16_t* x_dev, const uint32_t* packed_dev, const uint16_t* scales_dev,
               const uint16_t* biases_dev, int32_t m, int32_t out_dim, int32_t in_dim, int32_t group, int32_t bits,
               uint16_t* y_bf16_dev, float* y_f32_dev) {
    B2_REQUIRE(ctx && x_dev && packed_dev && scales_dev && biases_dev, B2_ERR_MSG, "b2_qmm: null argument");
    B2_REQUIRE(bits == 4 || bits == 8, B2_ERR_UNSUPPORTED, "b2_qmm: bits must be 4 or 8");
    GemmParams p{};
    p.x = x_dev;
    p.w = packed_dev;
    p.scales = scales_dev;
    p.biases = biases_dev;
    p.bits = bits;
    p.group = group;
    p.M = m;
    p.N = out_dim;
    p.K = in_dim;
    p.ldx = in_dim;
    p.ldo = out_dim;
    return gemm_both(ctx, p, y_bf16_dev, y_f32_dev);
}

// h = h + x @ dequant(W)^T with the residual add fused into the projection's epilogue, in place.
int32_t b2_qmm_residual(b2_ctx* ctx, const uint16_t* x_dev, const uint32_t* packed_dev, const uint16_t* scales_dev, const uint16_t* biases_dev,
                        int32_t m, int32_t out_dim, int32_t in_dim, int32_t group, int32_t bits, uint16_t* h_dev) {
    B2_REQUIRE(ctx && x_dev && packed_dev && scales_dev && biases_dev && h_dev, B2_ERR_MSG, "b2_qmm_residual: null argument");
    B2_REQUIRE(bits == 4 || bits == 8, B2_ERR_UNSUPPORTED, "b2_qmm_residual: bits must be 4 or 8");
    GemmParams p{};
    p.x = x_dev;
    p.w = packed_dev;
    p.scales = scales_dev;
    p.biases = biases_dev;
    p.bits = bits;
    p.group = group;
    p.M = m;
    p.N = out_dim;
    p.K = in_dim;
    p.ldx = in_dim;
    p.ldo = out_dim;
    p.ldres = out_dim;
    p.epilogue = EPI_BF16_RESADD;
    p.out = h_dev;
    p.res = h_dev;
    return b2_gemm_launch(ctx, p);
}

// The same with HOST activations and a host result (pinned or pageable): x in, kernel, y out, then a stream sync.
int32_t b2_qmm_host(b2_ctx* ctx, const uint16_t* x_host, const uint32_t* packed_dev, const uint16_t* scales_dev, const uint16_t* biases_dev,
                    int32_t m, int32_t out_dim, int32_t in_dim, int32_t group, int32_t bits, uint16_t* y_bf16_host) {
    B2_REQUIRE(ctx && x_host && y_bf16_host, B2_ERR_MSG, "b2_qmm_host: null argument");
    B2_REQUIRE(m >= 0 && out_dim > 0 && in_dim > 0, B2_ERR_MSG, "b2_qmm_host: bad shape");
    const size_t xb = ((size_t)m * in_dim * 2 + 255) & ~(size_t)255, yb = (size_t)m * out_dim * 2;
    void* stage = nullptr;
    B2_CHECK(b2_ctx_stage(ctx, xb + yb, &stage));
    uint16_t* xd = reinterpret_cast<uint16_t*>(stage);
    uint16_t* yd = reinterpret_cast<uint16_t*>(reinterpret_cast<uint8_t*>(stage) + xb);
    B2_CUDA(cudaMemcpyAsync(xd, x_host, (size_t)m * in_dim * 2, cudaMemcpyHostToDevice, ctx->stream));
    B2_CHECK(b2_qmm(ctx, xd, packed_dev, scales_dev, biases_dev, m, out_dim, in_dim, group, bits, yd, nullptr));
    B2_CUDA(cudaMemcpyAsync(y_bf16_host, yd, yb, cudaMemcpyDeviceToHost, ctx->stream));
    B2_CUDA(cudaStreamSynchronize(ctx->stream));
    return B2_OK;
}

int32_t b2_linear(b2_ctx* ctx, const uint16_t* x_dev, const uint16_t* w_dev, int32_t m, int32_t out_dim, int32_t in_dim,
                  uint16_t* y_bf16_dev, float* y_f32_dev) {
    B2_REQUIRE(ctx && x_dev && w_dev, B2_ERR_MSG, "b2_linear: null argument");
    GemmParams p{};
    p.x = x_dev;
    p.w = w_dev;
    p.bits = 0;
    p.group = 64;
    p.M = m;
    p.N = out_dim;
    p.K = in_dim;
    p.ldx = in_dim;
    p.ldo = out_dim;
    return gemm_both(ctx, p, y_bf16_dev, y_f32_dev);
}

int32_t b2_rms_norm(b2_ctx* ctx, const uint16_t* x_dev, const uint16_t* w_dev, float eps, int32_t rows, int32_t dim, uint16_t* out_dev) {
    B2_REQUIRE(ctx && x_dev && w_dev && out_dev, B2_ERR_MSG, "b2_rms_norm: null argument");
    return b2_rms_norm_launch(ctx, x_dev, w_dev, eps, rows, dim, dim, nullptr, out_dev);
}
int32_t b2_swiglu(b2_ctx* ctx, const uint16_t* gate_dev, const uint16_t* up_dev, int64_t n, uint16_t* out_dev) {
    B2_REQUIRE(ctx && gate_dev && up_dev && out_dev, B2_ERR_MSG, "b2_swiglu: null argument");
    return b2_swiglu2_launch(ctx, gate_dev, up_dev, n, out_dev);
}
int32_t b2_add(b2_ctx* ctx, const uint16_t* a_dev, const uint16_t* b_dev, int64_t n, uint16_t* out_dev) {
    B2_REQUIRE(ctx && a_dev && b_dev && out_dev, B2_ERR_MSG, "b2_add: null argument");
    return b2_add_launch(ctx, a_dev, b_dev, n, out_dev);
}
int32_t b2_embed(b2_ctx* ctx, const uint16_t* table_dev, const int32_t* ids_dev, int32_t n, int32_t dim, int32_t vocab, uint16_t* out_dev) {
    B2_REQUIRE(ctx && table_dev && ids_dev && out_dev, B2_ERR_MSG, "b2_embed: null argument");
    return b2_embed_launch(ctx, table_dev, ids_dev, n, dim, vocab, out_dev);
}
int32_t b2_argmax(b2_ctx* ctx, const uint16_t* logits_dev, int32_t rows, int32_t vocab, int32_t* out_dev) {
    B2_REQUIRE(ctx && logits_dev && out_dev, B2_ERR_MSG, "b2_argmax: null argument");
    return b2_argmax_launch(ctx, logits_dev, rows, vocab, out_dev);
}

// Rope::standard / Rope::llama3 (src/primitives/rope.rs:42-52, :125-156), f32 throughout.
int32_t b2_rope_inv_freq(int32_t head_dim, float theta, int32_t kind, float factor, float low_freq_factor, float high_freq_factor,
                         float original_context, float* out_host) {
    B2_REQUIRE(out_host && head_dim > 0 && head_dim % 2 == 0, B2_ERR_MSG, "b2_rope_inv_freq: bad argument");
    const int half = head_dim / 2;
    const float two_pi = 2.0f * 3.14159265358979323846f;
    const float low_wl = original_context / low_freq_factor, high_wl = original_context / high_freq_factor;
    for (int i = 0; i < half; i++) {
        float inv = 1.0f / powf(theta, (float)(2 * i) / (float)head_dim);
        if (kind == 1) {
            const float wavelen = two_pi / inv;
            if (wavelen > low_wl) {
                inv = inv / factor;
            } else if (!(wavelen < high_wl)) {
                const float smooth = (original_context / wavelen - low_freq_factor) / (high_freq_factor - low_freq_factor);
                inv = (1.0f - smooth) * inv / factor + smooth * inv;
            }
        }
        out_host[i] = inv;
    }
    return B2_OK;
}

static inline uint16_t host_f2bf(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x0040u);
    u += 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}

int32_t b2_rope_tables(const float* inv_freq_host, int32_t half, int32_t n_pos, uint16_t* cos_host, uint16_t* sin_host) {
    B2_REQUIRE(inv_freq_host && cos_host && sin_host && half > 0 && n_pos >= 0, B2_ERR_MSG, "b2_rope_tables: bad argument");
    for (int p = 0; p < n_pos; p++)
        for (int i = 0; i < half; i++) {
            const float ang = (float)p * inv_freq_host[i];
            cos_host[(size_t)p * half + i] = host_f2bf(cosf(ang));
            sin_host[(size_t)p * half + i] = host_f2bf(sinf(ang));
        }
    return B2_OK;
}

int32_t b2_rope_kv_append(b2_ctx* ctx, uint16_t* qkv_dev, int32_t T, int32_t hq, int32_t hkv, int32_t head_dim,
                          const int32_t* positions_dev, const int32_t* slot_mapping_dev, const uint16_t* cos_dev,
                          const uint16_t* sin_dev, const uint16_t* q_norm_dev, const uint16_t* k_norm_dev, float eps,
                          int32_t page_size, uint16_t* k_pool_dev, uint16_t* v_pool_dev, uint16_t* q_out_dev) {
    B2_REQUIRE(ctx && qkv_dev && positions_dev && slot_mapping_dev && cos_dev && sin_dev && k_pool_dev && v_pool_dev && q_out_dev,
               B2_ERR_MSG, "b2_rope_kv_append: null argument");
    RopeKvParams p{};
    p.qkv = qkv_dev;
    p.ld = (hq + 2 * hkv) * head_dim;
    p.positions = positions_dev;
    p.slot_mapping = slot_mapping_dev;
    p.cos_table = cos_dev;
    p.sin_table = sin_dev;
    p.q_norm = q_norm_dev;
    p.k_norm = k_norm_dev;
    p.eps = eps;
    p.T = T;
    p.hq = hq;
    p.hkv = hkv;
    p.hd = head_dim;
    p.page_size = page_size;
    p.k_pool = k_pool_dev;
    p.v_pool = v_pool_dev;
    p.q_out = q_out_dev;
    return b2_rope_kv_launch(ctx, p);
}

int64_t b2_batch_metadata_elems(int32_t B, int32_t T, int32_t max_dec_work, int32_t max_pf_work) {
    return (int64_t)(B + 1) + B + 3 * (int64_t)T + 5 * (int64_t)B + (B + 1) + 2 * (int64_t)max_dec_work + 2 * (int64_t)max_pf_work + 8;
}

int32_t b2_build_batch_metadata(b2_ctx* ctx, const int32_t* seq_slot_host, const int32_t* q_len_host, const int32_t* ctx_before_host,
                                const int32_t* want_logits_host, int32_t B, const int32_t* upd_slot_host,
                                const int32_t* upd_index_host, const int32_t* upd_page_host, int32_t U, int32_t chunk_tokens,
                                int32_t q_tile, int32_t page_size, int32_t max_blocks, int32_t max_dec_work, int32_t max_pf_work,
                                int32_t* block_tables_dev, int32_t* out_dev) {
    B2_REQUIRE(ctx && block_tables_dev && out_dev, B2_ERR_MSG, "b2_build_batch_metadata: null argument");
    B2_REQUIRE(chunk_tokens > 0 && chunk_tokens % 16 == 0, B2_ERR_MSG, "b2_build_batch_metadata: chunk_tokens must be a positive multiple of 16");
    long T = 0;
    for (int i = 0; i < B; i++) T += q_len_host[i];
    std::vector<int32_t> stage;
    stage.reserve(4 * (size_t)B + 3 * (size_t)U);
    stage.insert(stage.end(), seq_slot_host, seq_slot_host + B);
    stage.insert(stage.end(), q_len_host, q_len_host + B);
    stage.insert(stage.end(), ctx_before_host, ctx_before_host + B);
    stage.insert(stage.end(), want_logits_host, want_logits_host + B);
    if (U > 0) {
        stage.insert(stage.end(), upd_slot_host, upd_slot_host + U);
        stage.insert(stage.end(), upd_index_host, upd_index_host + U);
        stage.insert(stage.end(), upd_page_host, upd_page_host + U);
    }
    void* dev = nullptr;
    B2_CHECK(b2_ctx_stage(ctx, stage.size() * 4 + 16, &dev));
    B2_CUDA(cudaMemcpyAsync(dev, stage.data(), stage.size() * 4, cudaMemcpyHostToDevice, ctx->stream));
    B2_CUDA(cudaStreamSynchronize(ctx->stream));  // `stage` is pageable host memory
    const int32_t* d = reinterpret_cast<const int32_t*>(dev);
    BatchMetaIn in{};
    in.seq_slot = d;
    in.q_len = d + B;
    in.ctx_before = d + 2 * B;
    in.want_logits = d + 3 * B;
    in.upd_slot = d + 4 * B;
    in.upd_index = d + 4 * B + U;
    in.upd_page = d + 4 * B + 2 * U;
    in.B = B;
    in.T = (int)T;
    in.U = U;
    in.chunk_tiles = chunk_tokens / 16;
    in.q_tile = q_tile;
    in.page_size = page_size;
    in.max_blocks = max_blocks;
    BatchMetaOut out{};
    out.block_tables = block_tables_dev;
    b2_batch_meta_carve(out_dev, B, (int)T, max_dec_work, max_pf_work, out);
    return b2_batch_meta_launch(ctx, in, out);
}

// Standalone prefill attention: builds the query-tile work list on the host.
int32_t b2_paged_attn_prefill(b2_ctx* ctx, const uint16_t* q_dev, const uint16_t* k_pool_dev, const uint16_t* v_pool_dev,
                              const int32_t* block_tables_dev, int32_t max_blocks, const int32_t* cu_seqlens_host,
                              const int32_t* ctx_lens_host, int32_t num_seqs, int32_t hq, int32_t hkv, int32_t head_dim,
                              int32_t page_size, float scale, uint16_t* out_dev) {
    B2_REQUIRE(ctx && q_dev && k_pool_dev && v_pool_dev && block_tables_dev && cu_seqlens_host && ctx_lens_host && out_dev, B2_ERR_MSG,
               "b2_paged_attn_prefill: null argument");
    B2_REQUIRE(page_size > 0 && page_size % 16 == 0, B2_ERR_UNSUPPORTED, "b2_paged_attn_prefill: page_size must be a multiple of 16");
    if (num_seqs <= 0) return B2_OK;
    const int q_tile = b2_prefill_q_tile(ctx, head_dim);
    std::vector<int32_t> host;  // slot[B] cu[B+1] ctx[B] pf_seq[P] pf_qstart[P] n_work
    std::vector<int32_t> pf_seq, pf_q;
    for (int i = 0; i < num_seqs; i++) {
        const int qn = cu_seqlens_host[i + 1] - cu_seqlens_host[i];
        B2_REQUIRE(qn >= 0 && ctx_lens_host[i] >= qn, B2_ERR_MSG, "b2_paged_attn_prefill: ctx_lens must include the new tokens");
        for (int s = 0; s < qn; s += q_tile) {
            pf_seq.push_back(i);
            pf_q.push_back(s);
        }
    }
    const int P = (int)pf_seq.size();
    if (P == 0) return B2_OK;
    for (int i = 0; i < num_seqs; i++) host.push_back(i);
    host.insert(host.end(), cu_seqlens_host, cu_seqlens_host + num_seqs + 1);
    host.insert(host.end(), ctx_lens_host, ctx_lens_host + num_seqs);
    host.insert(host.end(), pf_seq.begin(), pf_seq.end());
    host.insert(host.end(), pf_q.begin(), pf_q.end());
    host.push_back(P);
    void* dev = nullptr;
    B2_CHECK(b2_ctx_stage(ctx, host.size() * 4, &dev));
    B2_CUDA(cudaMemcpyAsync(dev, host.data(), host.size() * 4, cudaMemcpyHostToDevice, ctx->stream));
    B2_CUDA(cudaStreamSynchronize(ctx->stream));
    const int32_t* d = reinterpret_cast<const int32_t*>(dev);
    PrefillAttnParams p{};
    p.q = q_dev;
    p.k_pool = k_pool_dev;
    p.v_pool = v_pool_dev;
    p.block_tables = block_tables_dev;
    p.max_blocks = max_blocks;
    p.seq_slot = d;
    p.cu_seqlens = d + num_seqs;
    p.context_lens = d + 2 * num_seqs + 1;
    p.pf_seq = d + 3 * num_seqs + 1;
    p.pf_qstart = p.pf_seq + P;
    p.n_work = p.pf_qstart + P;
    p.hq = hq;
    p.hkv = hkv;
    p.page_tiles = page_size / 16;
    p.scale_log2 = scale * 1.4426950408889634f;
    p.out = out_dev;
    p.q_tile = q_tile;
    p.q_rows = cu_seqlens_host[num_seqs];
    // the pool's size is not an argument: the largest page the block tables name bounds the rows that are read
    {
        std::vector<int32_t> bt((size_t)num_seqs * max_blocks);
        B2_CUDA(cudaMemcpyAsync(bt.data(), block_tables_dev, bt.size() * 4, cudaMemcpyDeviceToHost, ctx->stream));
        B2_CUDA(cudaStreamSynchronize(ctx->stream));
        int32_t max_page = 0;
        for (int i = 0; i < num_seqs; i++) {
            const int used = (ctx_lens_host[i] + page_size - 1) / page_size;
            B2_REQUIRE(used <= max_blocks, B2_ERR_MSG, "b2_paged_attn_prefill: a context needs more blocks than a block-table row holds");
            for (int j = 0; j < used; j++) {
                B2_REQUIRE(bt[(size_t)i * max_blocks + j] >= 0, B2_ERR_MSG, "b2_paged_attn_prefill: negative page in a block table");
                max_page = std::max(max_page, bt[(size_t)i * max_blocks + j]);
            }
        }
        p.pool_rows = ((int64_t)max_page + 1) * hkv * page_size;
    }
    for (int i = 0; i < num_seqs; i++)
        if (cu_seqlens_host[i + 1] > cu_seqlens_host[i]) p.max_ctx = std::max(p.max_ctx, (int)ctx_lens_host[i]);
    return b2_prefill_attn_launch(ctx, p, head_dim, P);
}

}  // extern "C"
