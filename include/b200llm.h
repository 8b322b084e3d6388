/* b200llm — C ABI of the B200-native continuous-batching decode path.
 *
 * Every entry point replaces a Rust interface of SceneWorks/mlx-llm (cited per function as
 * file:line inside that project).  The reference has no FFI of its own: a `-sys` crate would bind
 * these symbols and re-expose the reference's types (KvCache, BlockPool/PagedKvCache, CausalLm,
 * Decode/generate, generate_continuous, QuantSpec/Projection) on top of them.
 *
 * Conventions
 *  - All functions return a status (B2_OK == 0, negatives are errors).  b2_last_error() returns the
 *    message of the calling thread's last failure.
 *  - Handles are opaque, owned by the caller and released with the matching *_free.
 *  - One context <-> one GPU <-> one host thread; no function is re-entrant on the same context.
 *  - Pointers named *_dev are device pointers, *_host are host pointers; bf16 tensors are passed
 *    as uint16_t.  No PyTorch type appears anywhere in this ABI.
 *  - There is no CPU fallback: without a CUDA device b2_ctx_create fails with B2_ERR_CUDA.
 */
#ifndef B200LLM_H
#define B200LLM_H
#include <stddef.h>
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif

/* Status codes.  -1..-7 map 1:1 to the reference's Error variants (src/error.rs:12-42). */
enum {
    B2_OK = 0,
    B2_ERR_CUDA = -1,          /* Error::Mlx: the device backend failed */
    B2_ERR_MISSING_TENSOR = -2,/* Error::MissingTensor */
    B2_ERR_IO = -3,            /* Error::Io */
    B2_ERR_CONFIG = -4,        /* Error::Config */
    B2_ERR_UNSUPPORTED = -5,   /* Error::Unsupported */
    B2_ERR_CANCELED = -6,      /* Error::Canceled (typed pre-inference cancel) */
    B2_ERR_MSG = -7,           /* Error::Msg: invalid argument / state */
    B2_ERR_OOM_PAGES = -8,     /* the bounded page pool is exhausted */
    B2_ERR_TIMEOUT = -9        /* a bounded device-side wait gave up */
};

typedef struct b2_ctx b2_ctx;

const char* b2_last_error(void);
int32_t b2_version(void);

/* ---- context and raw device memory (plumbing for callers without a CUDA runtime of their own) -- */
int32_t b2_ctx_create(int32_t device, b2_ctx** out);
int32_t b2_ctx_free(b2_ctx* ctx);
int32_t b2_ctx_sync(b2_ctx* ctx);
int32_t b2_device_count(int32_t* out);
int32_t b2_malloc(b2_ctx* ctx, size_t bytes, void** out_dev);
int32_t b2_free(b2_ctx* ctx, void* dev);
int32_t b2_memcpy_h2d(b2_ctx* ctx, void* dst_dev, const void* src_host, size_t bytes);
int32_t b2_memcpy_d2h(b2_ctx* ctx, void* dst_host, const void* src_dev, size_t bytes);
int32_t b2_memset(b2_ctx* ctx, void* dst_dev, int value, size_t bytes);
int32_t b2_host_alloc_pinned(size_t bytes, void** out_host);
int32_t b2_host_free_pinned(void* host);
/* CUDA-event timing on the context's stream (every kernel of this library launches there). */
int32_t b2_timer_start(b2_ctx* ctx);
int32_t b2_timer_stop_ms(b2_ctx* ctx, float* ms_out);
/* Overwrite a buffer larger than L2 so the next kernel starts cold. */
int32_t b2_flush_l2(b2_ctx* ctx);
/* Number of this library's kernels launched on the context since creation. */
int32_t b2_launch_count(b2_ctx* ctx, int64_t* out);

/* ---- paged attention (replaces primitives::attention::sdpa over PagedKvCache::gather:
 *      src/primitives/attention.rs:68-102 + src/primitives/paged_kv_cache.rs:342-354) ------------
 * KV pool layout (ours): [pages, n_kv_heads, page_size, head_dim] bf16, keys already rotated.
 * Decode: one query token per sequence, causal over its ctx_lens[i] cached positions (the query's
 * own K/V already appended).  GQA: q head h reads kv head h / (hq/hkv) (adjacent grouping,
 * attention.rs:300-301).  Split-K over chunks of `chunk_tokens` positions followed by a
 * log-sum-exp merge; chunk_tokens == 0 picks a size from the batch.  fp32 accumulate, bf16 I/O.
 *   q_dev            [num_seqs, hq, head_dim]
 *   block_tables_dev [num_seqs, max_blocks] physical page per logical block
 *   ctx_lens_dev     [num_seqs]
 *   out_dev          [num_seqs, hq, head_dim] bf16
 * Supported: head_dim 64 or 128, page_size a multiple of 16, hq/hkv in {1,2,4,8}. */
int32_t b2_paged_attn_decode(b2_ctx* ctx, const uint16_t* q_dev, const uint16_t* k_pool_dev, const uint16_t* v_pool_dev,
                             const int32_t* block_tables_dev, int32_t max_blocks, const int32_t* ctx_lens_dev,
                             int32_t num_seqs, int32_t hq, int32_t hkv, int32_t head_dim, int32_t page_size, float scale,
                             int32_t chunk_tokens, uint16_t* out_dev);
/* Same call with HOST q / out buffers (pinned or pageable): copies q in, runs, copies out back. */
int32_t b2_paged_attn_decode_host(b2_ctx* ctx, const uint16_t* q_host, const uint16_t* k_pool_dev,
                                  const uint16_t* v_pool_dev, const int32_t* block_tables_dev, int32_t max_blocks,
                                  const int32_t* ctx_lens_dev, int32_t num_seqs, int32_t hq, int32_t hkv, int32_t head_dim,
                                  int32_t page_size, float scale, int32_t chunk_tokens, uint16_t* out_host);

#ifdef __cplusplus
}
#endif
#endif
