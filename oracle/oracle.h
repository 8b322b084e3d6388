/* CPU oracle — TEST INFRASTRUCTURE ONLY (see orc_common.h).  C entry points used by the test
 * suite, the smoke check and the CPU-baseline leg of the benchmark.  The product library never
 * links or loads this. */
#ifndef ORACLE_H
#define ORACLE_H
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif

typedef struct orc_model orc_model;
typedef struct orc_pool orc_pool;
typedef struct orc_cache orc_cache;

typedef struct {
    int32_t layers, hidden, heads, kv_heads, head_dim, inter, vocab;
    float eps, theta;
    int32_t rope_kind; /* 0 standard, 1 llama3 */
    float rope_factor, rope_low, rope_high, rope_orig;
    int32_t qk_norm, quant_bits, group, f32_mode;
    int32_t sum_order; /* 0: index order; 1: another equally valid f32 summation order (sizes the rounding noise) */
} orc_model_cfg;

int orc_max_threads(void);
void orc_set_threads(int n);

uint64_t orc_splitmix64_next(uint64_t* state);
float orc_splitmix64_next_f32(uint64_t* state);
void orc_f32_to_bf16(const float* in, uint16_t* out, int64_t n);
void orc_bf16_to_f32(const uint16_t* in, float* out, int64_t n);

void orc_rope_inv_freq(int head_dim, float theta, int kind, float factor, float low_freq_factor, float high_freq_factor,
                       float original_context, float* out);
void orc_rope_cos_sin(const float* inv_freq, int half, const int32_t* pos, int n, uint16_t* cos_out, uint16_t* sin_out);
void orc_apply_rope(uint16_t* x, const uint16_t* cos_t, const uint16_t* sin_t, int n, int heads, int hd);
void orc_rms_norm(const uint16_t* x, const uint16_t* w, float eps, int rows, int dim, uint16_t* out);
void orc_swiglu(const uint16_t* gate, const uint16_t* up, int64_t n, uint16_t* out);
void orc_add_bf16(const uint16_t* a, const uint16_t* b, int64_t n, uint16_t* out);
void orc_linear(const uint16_t* x, const uint16_t* w, int m, int n, int k, float* out_f32, uint16_t* out_bf16);
int32_t orc_argmax_bf16(const uint16_t* logits, int n);
int32_t orc_argmax_f32(const float* logits, int n);

void orc_unpack_codes(const uint32_t* packed, int64_t rows, int64_t in_dim, int bits, uint8_t* codes);
void orc_dequantize(const uint32_t* packed, const uint16_t* scales, const uint16_t* biases, int64_t rows, int64_t in_dim,
                    int group, int bits, uint16_t* out);
void orc_quantize(const uint16_t* w, int64_t rows, int64_t in_dim, int group, int bits, uint32_t* packed, uint16_t* scales,
                  uint16_t* biases);
void orc_qmm(const uint16_t* x, const uint32_t* packed, const uint16_t* scales, const uint16_t* biases, int m, int n, int k,
             int group, int bits, float* out_f32, uint16_t* out_bf16);

void orc_host_attn_gqa(const float* q, const float* k, const float* v, int h, int hkv, int ql, int kl, int hd, float scale,
                       int causal, float* out);
void orc_paged_attention(const uint16_t* q, const uint16_t* kpool, const uint16_t* vpool, const int32_t* block_tables,
                         int max_blocks, const int32_t* cu_seqlens, const int32_t* ctx_lens, int num_seqs, int hq, int hkv,
                         int hd, int page, float scale, float* out);
void orc_paged_attention_decode_f32(const uint16_t* q, const uint16_t* kpool, const uint16_t* vpool,
                                    const int32_t* block_tables, int max_blocks, const int32_t* ctx_lens, int num_seqs, int hq,
                                    int hkv, int hd, int page, float scale, float* out);

void orc_synth_codes(uint64_t seed, int64_t n_words, uint32_t* out);
void orc_synth_scales_biases(uint64_t seed_scale, uint64_t seed_bias, int64_t n, float mul, float mid, uint16_t* scales,
                             uint16_t* biases);
void orc_synth_dense(uint64_t seed, int64_t n, float std_, uint16_t* out);
uint64_t orc_synth_tensor_seed(uint64_t seed, int layer, int which);

orc_model* orc_model_new(const orc_model_cfg* cfg);
void orc_model_free(orc_model* p);
void orc_model_set_dense(orc_model* p, int layer, int which, const float* data);
void orc_model_set_dense_bf16(orc_model* p, int layer, int which, const uint16_t* data);
void orc_model_set_quantized(orc_model* p, int layer, int which, const uint32_t* packed, const uint16_t* scales,
                             const uint16_t* biases, int bits, int group);
void orc_model_quantize_projection(orc_model* p, int layer, int which, int bits, int group);
void orc_model_set_norm(orc_model* p, int layer, int which, const float* data, int n);
void orc_model_fill_synthetic(orc_model* p, uint64_t seed);
void orc_model_forward(orc_model* p, int num_seqs, const int32_t* ids, const int32_t* n, orc_cache** caches,
                       const int32_t* offsets, float* logits_out, float* logits_f32_out);

orc_pool* orc_pool_new(int block_size);
void orc_pool_free(orc_pool* p);
void orc_pool_stats(orc_pool* p, int64_t* out4);
int orc_pool_is_materialized(orc_pool* p, int64_t id);
orc_cache* orc_cache_new_paged(orc_pool* p, int layers);
orc_cache* orc_cache_new_seeded(orc_pool* p, int layers, const int64_t* ids, int n);
orc_cache* orc_cache_new_contiguous(int layers);
void orc_cache_free(orc_cache* c);
int orc_cache_update(orc_cache* c, int layer, const uint16_t* k, const uint16_t* v, int step, int row_elems, int batch);
int64_t orc_cache_gather(orc_cache* c, int layer, uint16_t* k_out, uint16_t* v_out);
int32_t orc_cache_offset(orc_cache* c);
int orc_cache_truncate(orc_cache* c, int32_t len);
void orc_cache_reset(orc_cache* c);
int orc_cache_retain_sequences(orc_cache* c, const int32_t* keep, int n);
void orc_cache_paged_stats(orc_cache* c, int64_t* out4);
int orc_cache_block_ids(orc_cache* c, int64_t* out, int cap);
int orc_cache_shareable_prefix_blocks(orc_cache* c, int64_t tokens, int64_t* out, int cap);

int orc_generate(orc_model* p, const int32_t* prompt, int n_prompt, int max_new, const int32_t* stop, int n_stop,
                 int cancel_after_tokens, int use_paged, int block_size, int32_t* tokens_out, int* n_out, int* reason_out,
                 int32_t* events_out, int events_cap, int* n_events);
int orc_generate_continuous(orc_model* p, int n_req, const int32_t* prompts, const int32_t* prompt_len, const int32_t* max_new,
                            const int32_t* stops, const int32_t* n_stop, int max_batch, int block_size, int throughput,
                            int cancel_after_steps, int32_t* tokens_out, int tok_stride, int32_t* n_tokens, int32_t* reasons,
                            int32_t* events_out, int events_cap, int* n_events, int64_t* block_ids_out, int block_stride,
                            int32_t* n_blocks, int64_t* pool_stats_out, int32_t* peak_lane_blocks_out);

#ifdef __cplusplus
}
#endif
#endif
