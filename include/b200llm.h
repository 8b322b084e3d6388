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
int32_t b2_ctx_sync(b2_ctx* ctx);   /* also reports B2_ERR_TIMEOUT raised by a bounded device-side wait */
/* Projection path: 1 = tcgen05 / TMEM kernel for steps with more than 32 tokens (default), 0 = the
 * warp-level mma.sync kernel for every size (kept for comparison). */
int32_t b2_ctx_set_tensor_path(b2_ctx* ctx, int32_t use_tcgen05);
/* Limit, in milliseconds, of every device-side wait on ANOTHER rank (the flags of the peer-memory reduction);
 * default about four seconds.  When a wait runs out the kernel raises the context's error word and returns,
 * b2_ctx_sync and the engine's step return B2_ERR_TIMEOUT, and reductions launched before the error is read
 * return at once.  The waits on on-chip barriers of the tcgen05 kernels keep a fixed limit of about two seconds.
 * No counterpart in the reference (single device; its only failure path is cooperative cancel,
 * src/decode/continuous.rs:138-140, :198-214). */
int32_t b2_ctx_set_wait_limit_ms(b2_ctx* ctx, int32_t ms);
int32_t b2_device_count(int32_t* out);
int32_t b2_malloc(b2_ctx* ctx, size_t bytes, void** out_dev);
int32_t b2_free(b2_ctx* ctx, void* dev);
int32_t b2_memcpy_h2d(b2_ctx* ctx, void* dst_dev, const void* src_host, size_t bytes);
int32_t b2_memcpy_d2h(b2_ctx* ctx, void* dst_host, const void* src_dev, size_t bytes);
int32_t b2_memset(b2_ctx* ctx, void* dst_dev, int value, size_t bytes);
/* Free and total device memory of the context's GPU (for sizing the page pool). */
int32_t b2_mem_info(b2_ctx* ctx, size_t* free_bytes, size_t* total_bytes);
int32_t b2_host_alloc_pinned(size_t bytes, void** out_host);
int32_t b2_host_free_pinned(void* host);
/* CUDA-event timing on the context's stream (every kernel of this library launches there). */
int32_t b2_timer_start(b2_ctx* ctx);
int32_t b2_timer_stop_ms(b2_ctx* ctx, float* ms_out);
/* Overwrite a buffer larger than L2 so the next kernel starts cold. */
int32_t b2_flush_l2(b2_ctx* ctx);
/* Open (on != 0) or close the range an external profiler started with "--profile-from-start off"
 * looks at (cudaProfilerStart / cudaProfilerStop); the stream is drained first.  No effect otherwise. */
int32_t b2_profiler_range(b2_ctx* ctx, int32_t on);
/* NVTX ranges ("gemm", "attn_decode", "attn_prefill", "rope_kv", "elementwise", "meta_copies", "collective") around
 * the launches of each kernel class of every step, for timeline tools; off by default (also switched on by the
 * environment variable B2_NVTX=1 when the context is created).  No reference counterpart. */
int32_t b2_nvtx_enable(b2_ctx* ctx, int32_t on);
/* Environment, read when a context is created: B2_PDL_MIN_TOKENS=n makes the engine launch the small kernels of an
 * iteration (norms, SwiGLU, RoPE + KV append, attention, split-K sums) the ordinary way when the iteration has fewer
 * than n tokens, instead of with programmatic stream serialisation (default 1: always programmatic).  For comparison
 * runs; results are identical either way. */
/* Number of this library's kernels launched on the context since creation. */
int32_t b2_launch_count(b2_ctx* ctx, int64_t* out);

/* ---- paged attention (replaces primitives::attention::sdpa over PagedKvCache::gather:
 *      src/primitives/attention.rs:68-102 + src/primitives/paged_kv_cache.rs:342-354) ------------
 * KV pool layout (ours): [pages, n_kv_heads, page_size, head_dim] bf16, keys already rotated.
 * Decode: one query token per sequence, causal over its ctx_lens[i] cached positions (the query's
 * own K/V already appended).  GQA: q head h reads kv head h / (hq/hkv) (adjacent grouping,
 * attention.rs:300-301).  Split-K over chunks of `chunk_tokens` positions followed by a
 * log-sum-exp merge; chunk_tokens == 0 lets the library choose (128 to 1024 by the size of the batch).  fp32 accumulate, bf16 I/O.  A ctx_lens[i] larger than
 * max_blocks * page_size is read as that maximum; a sequence with ctx_lens[i] == 0 gets rows of zeros.
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

/* Decode attention that allocates nothing.  No counterpart in the reference: it exists for hosts that
 * cannot call the device allocator when they need attention (all of HBM already handed to the KV pool,
 * a latency-critical thread, an embedding runtime that owns the allocator).  Same arguments, meaning and
 * results as b2_paged_attn_decode, except that there is no context: the kernels are enqueued on `stream`
 * (a cudaStream_t, or NULL for the legacy default stream) of the CURRENT device and the call returns
 * without synchronising; chunk_tokens == 0 means 512.
 * The split-K scratch is a fixed 16 MiB array that lives in the library's device image, one copy per GPU.
 * A batch whose scratch need,
 *     65536 + ceil(max_blocks*page_size / chunk_tokens) * num_seqs * hq*(head_dim+2)*4  bytes,
 * exceeds 16 MiB, or that has more than 1024 sequences, is rejected with B2_ERR_MSG and a text that names the
 * sizes; nothing is launched then.  (Llama-3-8B shapes, 16 K-token tables, chunk 512: up to 31 sequences; chunk
 * 2048: up to 125.)  The whole call is one kernel launch.
 * The first call on each device looks the array's address up and sets the kernels' shared-memory limit;
 * make that call before any stream capture begins (two host threads making their first call on one device
 * at the same time both do this set-up, with the same result).  All calls on one device share the array and it keeps
 * whatever the last call left: two calls that may run at the same time (different streams, different
 * host threads) race on it, so order them on one stream or with events. */
int32_t b2_paged_attn_decode_static(void* stream, const uint16_t* q_dev, const uint16_t* k_pool_dev, const uint16_t* v_pool_dev,
                                    const int32_t* block_tables_dev, int32_t max_blocks, const int32_t* ctx_lens_dev,
                                    int32_t num_seqs, int32_t hq, int32_t hkv, int32_t head_dim, int32_t page_size, float scale,
                                    int32_t chunk_tokens, uint16_t* out_dev);

/* Chunked-prefill paged attention over a ragged batch (replaces the whole-prompt prefill attention,
 * src/decode/continuous.rs:255 -> src/models/llama.rs:837-852 -> attention.rs:68-102).  Sequence i
 * owns query rows cu_seqlens[i]..cu_seqlens[i+1]; ctx_lens[i] counts the cached positions including
 * those rows; query r of n new tokens sees keys 0..=ctx-n+r (bottom-right causal, attention.rs:31-39).
 * Block-table row of sequence i is i.  Works for any q_len >= 1 (decode rows included). */
int32_t b2_paged_attn_prefill(b2_ctx* ctx, const uint16_t* q_dev, const uint16_t* k_pool_dev, const uint16_t* v_pool_dev,
                              const int32_t* block_tables_dev, int32_t max_blocks, const int32_t* cu_seqlens_host,
                              const int32_t* ctx_lens_host, int32_t num_seqs, int32_t hq, int32_t hkv, int32_t head_dim,
                              int32_t page_size, float scale, uint16_t* out_dev);

/* ---- MLX-format group-wise affine quantization (src/primitives/quant.rs:20-82,
 *      src/primitives/projection.rs:15-102) ------------------------------------------------------
 * Weight W [out, in]; packed [out, in*bits/32] u32 with codes along `in`, lowest bits first
 * (8 nibbles or 4 bytes per word); scales/biases [out, in/group] bf16; group must be 64, bits 4/8.
 * w = bf16(code*scale + bias), one rounding. */
int32_t b2_quantize(b2_ctx* ctx, const uint16_t* w_dev, int64_t out_dim, int64_t in_dim, int32_t group, int32_t bits,
                    uint32_t* packed_dev, uint16_t* scales_dev, uint16_t* biases_dev);   /* QuantizedLinear::quantize, quant.rs:38-54 */
int32_t b2_dequantize(b2_ctx* ctx, const uint32_t* packed_dev, const uint16_t* scales_dev, const uint16_t* biases_dev,
                      int64_t out_dim, int64_t in_dim, int32_t group, int32_t bits, uint16_t* w_dev); /* dequantize_weight, quant.rs:73-82 */
int32_t b2_unpack_codes(b2_ctx* ctx, const uint32_t* packed_dev, int64_t out_dim, int64_t in_dim, int32_t bits,
                        uint8_t* codes_dev);
/* y[m, out] = x[m, in] @ dequant(W)^T (QuantizedLinear::forward, quant.rs:56-70).  Exactly one of
 * y_bf16_dev / y_f32_dev may be null; the f32 output is the unrounded accumulation. */
int32_t b2_qmm(b2_ctx* ctx, const uint16_t* x_dev, const uint32_t* packed_dev, const uint16_t* scales_dev,
               const uint16_t* biases_dev, int32_t m, int32_t out_dim, int32_t in_dim, int32_t group, int32_t bits,
               uint16_t* y_bf16_dev, float* y_f32_dev);
/* h[m, out] = bf16(h + bf16(x @ dequant(W)^T)), in place: the residual add of LlamaLayer::forward
 * (src/models/llama.rs:730-732) fused into the projection's epilogue, as the engine runs o_proj and down_proj. */
int32_t b2_qmm_residual(b2_ctx* ctx, const uint16_t* x_dev, const uint32_t* packed_dev, const uint16_t* scales_dev,
                        const uint16_t* biases_dev, int32_t m, int32_t out_dim, int32_t in_dim, int32_t group, int32_t bits,
                        uint16_t* h_dev);
/* The same call with HOST activations and a HOST bf16 result (pinned or pageable): copies x in, multiplies, copies y
 * back and waits for the stream. */
int32_t b2_qmm_host(b2_ctx* ctx, const uint16_t* x_host, const uint32_t* packed_dev, const uint16_t* scales_dev,
                    const uint16_t* biases_dev, int32_t m, int32_t out_dim, int32_t in_dim, int32_t group, int32_t bits,
                    uint16_t* y_bf16_host);
/* Dense x @ W^T (primitives::nn::linear, src/primitives/nn.rs:26-33). */
int32_t b2_linear(b2_ctx* ctx, const uint16_t* x_dev, const uint16_t* w_dev, int32_t m, int32_t out_dim, int32_t in_dim,
                  uint16_t* y_bf16_dev, float* y_f32_dev);

/* ---- fused leaves --------------------------------------------------------------------------- */
/* rms_norm (src/primitives/nn.rs:35-37): out = bf16(x / rms(x) * w), rows of `dim`. */
int32_t b2_rms_norm(b2_ctx* ctx, const uint16_t* x_dev, const uint16_t* w_dev, float eps, int32_t rows, int32_t dim,
                    uint16_t* out_dev);
/* silu(gate) * up with the reference's bf16 rounding after each op (src/models/llama.rs:1040-1045). */
int32_t b2_swiglu(b2_ctx* ctx, const uint16_t* gate_dev, const uint16_t* up_dev, int64_t n, uint16_t* out_dev);
/* bf16 residual add (src/models/llama.rs:730-732). */
int32_t b2_add(b2_ctx* ctx, const uint16_t* a_dev, const uint16_t* b_dev, int64_t n, uint16_t* out_dev);
/* embedding row gather (src/primitives/nn.rs:86-93). */
int32_t b2_embed(b2_ctx* ctx, const uint16_t* table_dev, const int32_t* ids_dev, int32_t n, int32_t dim, int32_t vocab,
                 uint16_t* out_dev);
/* greedy argmax per row, ties -> lowest index (src/primitives/sampler.rs:221-241). */
int32_t b2_argmax(b2_ctx* ctx, const uint16_t* logits_dev, int32_t rows, int32_t vocab, int32_t* out_dev);
/* RoPE inverse frequencies: kind 0 = Rope::standard (src/primitives/rope.rs:42-52), 1 = Rope::llama3
 * (rope.rs:125-156); host computation, f32 powf as the reference. */
int32_t b2_rope_inv_freq(int32_t head_dim, float theta, int32_t kind, float factor, float low_freq_factor,
                         float high_freq_factor, float original_context, float* out_host);
/* cos/sin tables for positions 0..n_pos-1 as bf16 [n_pos, head_dim/2] (Rope::cos_sin_at,
 * rope.rs:183-208: angle = pos*inv_freq in f32, evaluated on the host, cast to bf16). */
int32_t b2_rope_tables(const float* inv_freq_host, int32_t half, int32_t n_pos, uint16_t* cos_host, uint16_t* sin_host);
/* Fused [per-head q/k RMSNorm ->] NeoX RoPE -> KV append (LlamaAttention::project,
 * src/models/llama.rs:806-825 + PagedKvCache::update, src/primitives/paged_kv_cache.rs:379-394).
 * qkv_dev [T, (hq+2*hkv)*head_dim]: q heads, k heads, v heads per token.  Rotated q goes to
 * q_out_dev [T, hq, head_dim]; rotated k and raw v are scattered to slot_mapping[t] of the pools
 * ([pages, hkv, page_size, head_dim]); a negative slot skips the cache write.  q_norm/k_norm may
 * be null. */
int32_t b2_rope_kv_append(b2_ctx* ctx, uint16_t* qkv_dev, int32_t T, int32_t hq, int32_t hkv, int32_t head_dim,
                          const int32_t* positions_dev, const int32_t* slot_mapping_dev, const uint16_t* cos_dev,
                          const uint16_t* sin_dev, const uint16_t* q_norm_dev, const uint16_t* k_norm_dev, float eps,
                          int32_t page_size, uint16_t* k_pool_dev, uint16_t* v_pool_dev, uint16_t* q_out_dev);

/* ---- ragged-batch packer / step metadata (no counterpart in the reference, which never packs:
 *      src/decode/continuous.rs:254-301) ----------------------------------------------------------
 * Host inputs: per sequence the block-table row, new-token count, cached length, sample flag;
 * block-table updates (slot, block index, page).  Device outputs are written into one int32 buffer
 * `out_dev` laid out as consecutive arrays (sizes in elements):
 *   cu_seqlens[B+1] context_lens[B] positions[T] token_seq[T] slot_mapping[T] logit_rows[B]
 *   logit_seq[B] dec_ctx[B] dec_qrow[B] dec_slot[B] dec_work_off[B+1] dec_work_seq[W] dec_work_chunk[W]
 *   pf_seq[P] pf_qstart[P] counts[8]
 * with W = max_dec_work, P = max_pf_work as given.  counts = {n_logits, n_dec, n_dec_work,
 * n_pf_work, error, T}.  block_tables_dev [slots, max_blocks] is updated in place. */
int32_t b2_build_batch_metadata(b2_ctx* ctx, const int32_t* seq_slot_host, const int32_t* q_len_host,
                                const int32_t* ctx_before_host, const int32_t* want_logits_host, int32_t B,
                                const int32_t* upd_slot_host, const int32_t* upd_index_host, const int32_t* upd_page_host,
                                int32_t U, int32_t chunk_tokens, int32_t q_tile, int32_t page_size, int32_t max_blocks,
                                int32_t max_dec_work, int32_t max_pf_work, int32_t* block_tables_dev, int32_t* out_dev);
int64_t b2_batch_metadata_elems(int32_t B, int32_t T, int32_t max_dec_work, int32_t max_pf_work);

/* ================================================================================================
 * Engine API
 * ============================================================================================== */
typedef struct b2_weights b2_weights;
typedef struct b2_model b2_model;
typedef struct b2_pool b2_pool;
typedef struct b2_cache b2_cache;

/* QuantSpec (src/primitives/projection.rs:15-32). */
typedef struct { int32_t group_size, bits; } b2_quant_spec;

/* The Llama / Qwen3 subset of ModelConfig (src/config.rs:315-502). */
typedef struct {
    int32_t num_layers, hidden_size, num_heads, num_kv_heads, head_dim, intermediate_size, vocab_size;
    float rms_norm_eps, rope_theta;
    int32_t rope_kind;                /* 0 standard, 1 llama3 (build_rope, config.rs:551-581) */
    float rope_factor, rope_low_freq_factor, rope_high_freq_factor, rope_original_context;
    int32_t qk_norm;                  /* Qwen3 per-head q/k RMSNorm */
    int32_t quant_bits, quant_group;  /* `quantization` block of a pre-quantized snapshot, 0 if dense */
    int32_t tie_word_embeddings;
    /* 0 (default): every tensor is cast to bf16 and every op rounds to bf16, as CausalLm::from_weights does
     * (src/models/llama.rs:29-30, :71).  1: weights, activations, KV pages and logits stay f32 and every
     * projection adds its products in index order (one multiply and one add per term, no fused multiply-add),
     * so two implementations of the same arithmetic agree to the last bits; attention accumulates in f64.
     * A plain-CUDA-core path for small dense checkpoints (no quantization, no q/k norm, no tensor parallelism,
     * contexts up to 4096): it exists so that a tiny f32 decoder can be compared token for token. */
    int32_t compute_f32;
} b2_model_config;

enum { B2_DTYPE_F32 = 0, B2_DTYPE_BF16 = 1, B2_DTYPE_F16 = 2, B2_DTYPE_U32 = 3, B2_DTYPE_I32 = 4 };

/* Weights (src/primitives/weights.rs:17-96): a name -> tensor map, from a safetensors file or
 * directory, or assembled from host buffers (copied). */
int32_t b2_weights_new(b2_weights** out);
int32_t b2_weights_from_dir(const char* path, b2_weights** out);            /* Weights::from_dir / from_file */
int32_t b2_weights_add(b2_weights* w, const char* name, int32_t dtype, const int64_t* shape, int32_t ndim,
                       const void* data_host);
int32_t b2_weights_contains(const b2_weights* w, const char* name);        /* Weights::contains */
int32_t b2_weights_free(b2_weights* w);

/* write_snapshot (src/snapshot.rs:86-148): writes `out_dir/model.safetensors` + `out_dir/config.json` from a dense,
 * Hugging-Face-keyed tensor set.  With a QuantSpec every attention / MLP projection (PROJECTION_SUFFIXES,
 * snapshot.rs:41-49) is cast to bf16, quantized on the GPU to MLX group-64 Q4 / Q8 and stored as the packed triplet
 * `<base>.weight` (u32) / `.scales` / `.biases` (bf16); everything else is written through unchanged and config.json
 * gains the `quantization` block that makes loaders read the triplets as stored (src/models/llama.rs:77-95).
 * quant == NULL writes a dense snapshot.  *num_tensors_out (nullable) = tensors written (a triplet counts three). */
int32_t b2_write_snapshot(b2_ctx* ctx, const b2_weights* w, const char* config_json, const b2_quant_spec* quant /* nullable */,
                          const char* out_dir, int32_t* num_tensors_out);
/* ModelConfig::from_json (src/config.rs:315-502) for the Llama/Qwen3 subset. */
int32_t b2_model_config_from_json(const char* json, b2_model_config* out);
/* CausalLm::from_weights_with (src/models/llama.rs:57-303): every tensor is cast to bf16 (:71);
 * projections are read as packed triplets when `<key>.scales` exists (:77-95), else dense with
 * optional quantize-on-load (:97).  `prefix` is prepended to every key ("" for plain checkpoints). */
int32_t b2_model_from_weights(b2_ctx* ctx, const b2_weights* w, const char* prefix, const b2_model_config* cfg,
                              const b2_quant_spec* quant /* nullable */, b2_model** out);
/* Random-init model generated on the device from a counter-based recipe (benchmark / parity helper;
 * no counterpart in the reference). cfg->quant_bits selects dense / Q4 / Q8 projections. */
int32_t b2_model_synthetic(b2_ctx* ctx, const b2_model_config* cfg, uint64_t seed, b2_model** out);

/* ---- tensor parallelism over KV heads (no counterpart in the reference, which runs on one device) --------
 * Rank r of `world` owns KV heads [r*n_kv/world, (r+1)*n_kv/world) with their q heads: the matching rows of
 * q/k/v and gate/up, the matching COLUMNS of o_proj and down_proj (cut on multiples of the quantization
 * group), and pages that hold only its heads.  o_proj and down_proj then yield f32 partial sums of the hidden
 * state, which are added over the group with an NCCL all-reduce on the context's stream before the residual
 * add (src/models/llama.rs:823-831 and :1040-1045 are the two results that become partial).  Embedding,
 * norms and lm_head are replicated, every rank runs the same schedule on the same requests and gets the same
 * tokens.  One process per GPU: rank 0 draws the id, the host program hands its 128 bytes to the other ranks
 * (any channel: a file, MPI, torch.distributed), then every rank creates its group.  world == 1 is a no-op
 * group (id may be NULL).  NCCL (libnccl.so.2) is bound at run time; without it a group of more than one
 * rank fails with B2_ERR_UNSUPPORTED.  A model keeps a pointer to its group: free the model first. */
typedef struct b2_tp_group b2_tp_group;
int32_t b2_tp_unique_id(uint8_t* out128);
int32_t b2_tp_group_create(b2_ctx* ctx, const uint8_t* id128, int32_t rank, int32_t world, b2_tp_group** out);
int32_t b2_tp_group_free(b2_tp_group* g);
int32_t b2_tp_group_info(const b2_tp_group* g, int32_t* rank, int32_t* world);
/* In-place sum of an f32 device buffer over the group, enqueued on the context's stream. */
int32_t b2_tp_all_reduce_f32(b2_tp_group* g, float* buf_dev, int64_t n);
/* Reductions over peer memory instead of NCCL (ranks on one node whose GPUs reach one another over NVLink).  Rank r
 * owns the hidden-state columns [r*H/world, (r+1)*H/world).  The o_proj / down_proj kernels write their f32 partial
 * sums into slot [this rank] of a region every rank exports; one kernel then waits for every rank's projection,
 * adds up the ranks' partial sums of its own columns (loads from the peers' memory, in rank order), adds the
 * residual, and stores the new bf16 hidden state into every rank's copy.  In push mode (b2_tp_peer_set_push) the
 * projection's epilogue instead stores each column range straight into the owner's memory, so the transfer overlaps
 * the multiplication tile by tile, and the sums read local memory only: worth it when a projection runs several
 * waves of tiles (a single wave ends in one burst of remote stores that delays the kernel's end).
 * Set-up, once per group and before the group's models run: every rank
 * calls b2_tp_peer_alloc (max_tokens = the most tokens one step will carry; hidden = the model's hidden size, a
 * multiple of 4 x world) and gets the 64-byte handle of its region; the host program gathers the handles (the
 * channel that carried the id); every rank calls b2_tp_peer_attach with all of them in rank order.  From then on
 * a model of that hidden size on this group keeps its hidden state inside the region and reduces there; a step
 * of more than max_tokens tokens fails with B2_ERR_UNSUPPORTED.  If a region cannot be mapped (GPUs without peer
 * access, devices hidden from the process) attach fails with B2_ERR_UNSUPPORTED and the group stays on NCCL.  A
 * group created with id128 == NULL and world > 1 has no NCCL communicator and can only reduce this way.  Every
 * wait in the kernel is bounded (about four seconds); when one runs out the context's error word is raised,
 * b2_ctx_sync returns B2_ERR_TIMEOUT and later reductions return at once.  Ranks must enter their steps within
 * that time of one another: start them from a common point (a host barrier after loading). */
int32_t b2_tp_peer_alloc(b2_tp_group* g, int32_t max_tokens, int32_t hidden, uint8_t* handle64_out);
int32_t b2_tp_peer_attach(b2_tp_group* g, const uint8_t* handles /* world x 64 bytes */, int32_t n_handles);
/* This rank's region: `world` slots of f32 partial sums, slot s = [max_tokens, hidden] at slots_dev +
 * s * slot_stride_floats, and the bf16 hidden state.  Rank s's partial sums are read from slot s of s's own region,
 * or in push mode from slot s of the reading rank's region (its own columns only). */
int32_t b2_tp_peer_buffers(const b2_tp_group* g, float** slots_dev, int64_t* slot_stride_floats, uint16_t** x_dev,
                           int32_t* max_tokens, int32_t* hidden);
/* The first half on its own: this rank's partial projection x[m, in_dim] . W^T with `hidden` output features (W dense
 * bf16 when bits == 0, else MLX group-64 Q4 / Q8), each column range stored from the kernel's epilogue into slot
 * [this rank] of the range's owner. */
int32_t b2_tp_peer_projection(b2_tp_group* g, const uint16_t* x_dev, int32_t m, int32_t in_dim, const void* w_dev,
                              const uint16_t* scales_dev /* nullable when bits == 0 */, const uint16_t* biases_dev, int32_t bits);
/* 1: projections store by column range into the owners' regions; 0 (default): into their own region.  Every rank of
 * the group must choose the same mode, between steps. */
int32_t b2_tp_peer_set_push(b2_tp_group* g, int32_t push);
/* x[0:rows, own columns] = bf16(x + bf16(sum over s of rank s's partial sums)) stored into every rank's x; on the
 * context's stream. */
int32_t b2_tp_peer_reduce_residual(b2_tp_group* g, int32_t rows);
/* All ranks of a group inside ONE process on one device (protocol tests without N GPUs): the groups' regions
 * are used directly, and the whole group's reduction runs as a single cooperative launch, because kernels
 * that wait on one another must not be separate launches on one device. */
int32_t b2_tp_peer_attach_local(b2_tp_group* const* groups, int32_t n);
int32_t b2_tp_peer_reduce_residual_local(b2_tp_group* const* groups, int32_t n, int32_t rows);
/* One forward step (b2_model_step) of EVERY rank of a group attached with b2_tp_peer_attach_local, each rank with a model
 * and a context of its own on the one device: every rank runs on a host thread of this call, the ranks meet at each
 * reduction, and rank 0 enqueues the single launch that reduces for all of them.  caches is [n][num_seqs] (rank r's
 * caches live in rank r's pool), logits_host [n][num_seqs][vocab] bf16 and argmax_host [n][num_seqs] are nullable.  For
 * testing whole tensor-parallel models on one GPU. */
int32_t b2_model_step_local_group(b2_model* const* models, int32_t n, const int32_t* ids_host, const int32_t* n_tokens,
                                  int32_t num_seqs, b2_cache* const* caches, uint16_t* logits_host, int32_t* argmax_host);
/* The two constructors with a group (NULL: the whole model, as without the suffix).  b2_model_get_config
 * still reports the WHOLE model's dimensions. */
int32_t b2_model_from_weights_tp(b2_ctx* ctx, const b2_weights* w, const char* prefix, const b2_model_config* cfg,
                                 const b2_quant_spec* quant /* nullable */, b2_tp_group* tp, b2_model** out);
int32_t b2_model_synthetic_tp(b2_ctx* ctx, const b2_model_config* cfg, uint64_t seed, b2_tp_group* tp, b2_model** out);

int32_t b2_model_free(b2_model* m);
int32_t b2_model_get_config(const b2_model* m, b2_model_config* out);      /* CausalLm::config */
int32_t b2_model_is_quantized(const b2_model* m);                          /* CausalLm::is_quantized */
int64_t b2_model_weight_bytes(const b2_model* m);

/* BlockPool (src/primitives/paged_kv_cache.rs:72-160) with bounded physical storage: `max_pages`
 * pages of `block_size` tokens for every layer, `max_seqs` block-table rows. */
typedef struct { int64_t live_blocks, shared_blocks, peak_live_blocks, reserved_tokens, free_pages, total_pages; } b2_pool_stats_t;
int32_t b2_pool_new(b2_ctx* ctx, const b2_model* m, int32_t block_size, int64_t max_pages, int32_t max_seqs,
                    int32_t max_blocks_per_seq, b2_pool** out);                 /* BlockPool::new */
int32_t b2_pool_free(b2_pool* p);
int32_t b2_pool_stats(const b2_pool* p, b2_pool_stats_t* out);              /* live/shared/peak/reserved, :95-114 */

/* PagedKvCache + impl KvCache (src/primitives/paged_kv_cache.rs:168-516, src/primitives/kv_cache.rs:30-64). */
int32_t b2_cache_new(b2_pool* p, b2_cache** out);                           /* PagedKvCache::with_pool */
int32_t b2_cache_new_seeded(b2_pool* p, const int64_t* shared_block_ids, int32_t n, b2_cache** out); /* new_seeded :221-235 */
int32_t b2_cache_free(b2_cache* c);                                         /* Drop :507-516 */
int32_t b2_cache_offset(const b2_cache* c);                                 /* KvCache::offset */
int32_t b2_cache_batch_size(const b2_cache* c);
int32_t b2_cache_num_layers(const b2_cache* c);
int64_t b2_cache_blocks(const b2_cache* c);                                 /* frozen (full) blocks */
int64_t b2_cache_reserved_tokens(const b2_cache* c);                        /* :284-286 */
int32_t b2_cache_block_ids(const b2_cache* c, int64_t* out, int32_t cap);   /* reference-view ids; returns count */
int32_t b2_cache_truncate(b2_cache* c, int32_t len);                        /* KvCache::truncate :422-485 */
int32_t b2_cache_reset(b2_cache* c);                                        /* KvCache::reset */
int32_t b2_cache_retain_sequences(b2_cache* c, const int32_t* keep, int32_t n); /* :408-420 */
int32_t b2_cache_shareable_prefix_blocks(b2_cache* c, int64_t tokens, int64_t* out, int32_t cap); /* :250-275; returns count */
/* What KvCache::update returns (kv_cache.rs:31-33), materialised for tests: K and V of `layer`
 * as [n_kv_heads, len, head_dim] bf16 host arrays. */
int32_t b2_cache_gather(b2_cache* c, int32_t layer, uint16_t* k_host, uint16_t* v_host);
/* The same for a pool of an f32 model (b2_model_config::compute_f32): [n_kv_heads, len, head_dim] f32. */
int32_t b2_cache_gather_f32(b2_cache* c, int32_t layer, float* k_host, float* v_host);

/* One forward over a ragged batch: sequence i contributes n_tokens[i] ids at positions
 * offset(caches[i])..; returns last-position logits [num_seqs, vocab] (bf16; f32 for an f32 model) on the host and advances
 * the caches.  Covers Decode::step (src/decode/stream.rs:22-29), CausalLm::decode_logits
 * (llama.rs:351-370) and decode_logits_per_seq (llama.rs:530-558). */
int32_t b2_model_step(b2_model* m, const int32_t* ids_host, const int32_t* n_tokens, int32_t num_seqs, b2_cache** caches,
                      void* logits_host /* nullable; uint16_t (bf16) rows, float rows for an f32 model */,
                      int32_t* argmax_host /* nullable */);

/* FinishReason (src/decode/stream.rs:31-46). */
enum { B2_FINISH_STOP_TOKEN = 0, B2_FINISH_MAX_TOKENS = 1, B2_FINISH_CANCELLED = 2, B2_FINISH_STOPPED = 3 };
/* StreamEvent (stream.rs:48-64): kind 0 Token{id=a, step=b}; kind 1 Done{reason=a, generated=b}. */
typedef void (*b2_event_cb)(void* user, int32_t request_index, int32_t kind, int32_t a, int32_t b);

/* SamplingParams (src/primitives/sampler.rs:64-90). */
typedef struct { float temperature, top_p; int32_t top_k; float repetition_penalty; int32_t repetition_context; } b2_sampling;
/* GenerationConfig (stream.rs:66-89) / BatchRequest (src/decode/batch.rs:47-59). */
typedef struct {
    const int32_t* prompt_ids; int32_t n_prompt;
    b2_sampling sampling;
    uint64_t seed; int32_t has_seed;
    int32_t max_new_tokens;
    const int32_t* stop_tokens; int32_t n_stop;
    double arrival_s;              /* extension: earliest admission time since the call started */
} b2_request;
typedef struct { int32_t* tokens; int32_t capacity; int32_t n_tokens; int32_t finish_reason; } b2_gen_output;

/* ContinuousConfig (src/decode/continuous.rs:67-85) + the bounded-pool / chunking extensions. */
typedef struct {
    int32_t max_batch, block_size;
    int32_t exactness;             /* 0 Exact (per-sequence forwards), 1 Throughput (one ragged batch) */
    int32_t prefill_chunk_tokens;  /* 0: whole-prompt prefill at admission (the reference's schedule) */
    int64_t max_pages;             /* 0: sized from the requests */
    int32_t max_blocks_per_seq;    /* 0: sized from the requests */
} b2_continuous_config;
typedef struct {
    int64_t steps, decode_tokens, prefill_tokens, kernel_launches;
    double device_ms, wall_ms;
    int64_t peak_live_blocks, peak_concurrent;
    int64_t h2d_bytes, d2h_bytes;
} b2_run_stats;

/* generate (src/decode/stream.rs:113-121 + decode_loop :259-327). cancel may be null. */
int32_t b2_generate(b2_model* m, const b2_request* req, const volatile int32_t* cancel, b2_event_cb cb, void* user,
                    b2_gen_output* out);
/* PrefixCache / generate_cached (src/decode/prefix.rs:56-188): shared-prefix KV reuse for the single-sequence loop.
 * The cache keeps up to `capacity` finished sequences (prompt + generated) as paged caches in a pool of its own
 * (`max_pages` pages, least recently used sequences are dropped past the capacity or when the pool runs out); a
 * request reuses the longest stored prefix of its prompt -- the full blocks by reference, a partly covered last block
 * by one page copy -- and prefills only the rest.  The result is token for token that of b2_generate.  PrefixStats
 * (:34-47). */
typedef struct b2_prefix_cache b2_prefix_cache;
typedef struct { int64_t lookups, hits, reused_prefix_tokens, computed_prefill_tokens; } b2_prefix_stats;
int32_t b2_prefix_cache_new(b2_ctx* ctx, b2_model* m, int32_t capacity, int64_t max_pages, int32_t max_blocks_per_seq,
                            b2_prefix_cache** out);                            /* PrefixCache::new :66-72 */
int32_t b2_prefix_cache_free(b2_prefix_cache* pc);
int32_t b2_prefix_cache_stats(const b2_prefix_cache* pc, b2_prefix_stats* out); /* PrefixCache::stats :75-77 */
int32_t b2_prefix_cache_len(const b2_prefix_cache* pc);                          /* PrefixCache::len :80-82 */
int32_t b2_generate_cached(b2_model* m, const b2_request* req, const volatile int32_t* cancel, b2_event_cb cb, void* user,
                           b2_prefix_cache* pc, b2_gen_output* out);            /* generate_cached :144-188 */
/* A new cache of the same pool holding the first `len` positions of `src` (len <= offset(src)): whole blocks shared by
 * reference count as PagedKvCache::new_seeded does (src/primitives/paged_kv_cache.rs:221-235), a partly covered last
 * block copied into a private page.  Neither cache sees the other's later writes. */
int32_t b2_cache_fork(const b2_cache* src, int32_t len, b2_cache** out);

/* generate_prompt_lookup (src/decode/speculative.rs:73-171): prompt-lookup (n-gram) speculative decoding, greedy.
 * Every step verifies [last token, drafts...] in ONE forward with the logits of every position, accepts the longest
 * draft prefix the target agrees with plus one bonus token, and rolls the rejected positions back with
 * KvCache::truncate.  SpeculativeConfig (:45-60) / SpeculativeStats (:62-71).  With num_draft == 0 the result is the
 * plain greedy loop's. */
typedef struct { int32_t max_ngram, num_draft; } b2_speculative_config;
typedef struct { int64_t forwards, proposed, accepted; } b2_speculative_stats;
int32_t b2_generate_prompt_lookup(b2_model* m, const b2_request* req, const b2_speculative_config* spec,
                                  const volatile int32_t* cancel, b2_event_cb cb, void* user, b2_gen_output* out,
                                  b2_speculative_stats* stats /* nullable */);
/* The proposer on its own (core_llm::speculative::ngram_propose as speculative.rs:3-8 describes it): up to k tokens
 * that followed the most recent earlier occurrence of the history's trailing n-gram, n = max_ngram .. 1. */
int32_t b2_ngram_propose(const int32_t* history, int32_t n_history, int32_t max_ngram, int32_t k, int32_t* out, int32_t* n_out);

/* generate_continuous (src/decode/continuous.rs:117-229). outs has n entries; stats may be null. */
int32_t b2_generate_continuous(b2_model* m, const b2_request* reqs, int32_t n, const b2_continuous_config* cfg,
                               const volatile int32_t* cancel, b2_event_cb cb, void* user, b2_gen_output* outs,
                               b2_run_stats* stats);
/* The same loop one iteration at a time (one iteration == one pass of continuous.rs:167-190), so a
 * caller can time exactly K iterations.  `reqs` and the arrays it points to must outlive the engine.
 * b2_continuous_step runs up to max_steps iterations; *done_out is 1 when no work is left.  stats
 * are cumulative since b2_continuous_new. */
typedef struct b2_continuous b2_continuous;
int32_t b2_continuous_new(b2_model* m, const b2_request* reqs, int32_t n, const b2_continuous_config* cfg,
                          const volatile int32_t* cancel, b2_event_cb cb, void* user, b2_continuous** out);
int32_t b2_continuous_step(b2_continuous* e, int32_t max_steps, int32_t* done_out, b2_run_stats* stats);
/* Serving form of the same loop, for a host that routes TextLlm::generate calls (src/provider.rs:567-918) of several
 * connections through ONE batch -- which the reference does not do (its provider runs generate_with per request,
 * provider.rs:838-846): the engine starts with no requests (cfg->max_pages and cfg->max_blocks_per_seq must be given),
 * b2_continuous_submit adds one at any time between steps (the engine copies the prompt and the stop tokens; *id_out is
 * the request's index in events and results), b2_continuous_halt ends one request between steps with Done{reason}
 * -- B2_FINISH_CANCELLED for a client that went away (CancelFlag, stream.rs:9-12), B2_FINISH_STOPPED for a stop
 * string matched in the detokenised text (should_stop, provider.rs:826-828) -- and b2_continuous_result reads a
 * request's tokens so far and its finish reason (-1 while it runs).  b2_continuous_step's *done_out == 1 then means
 * "idle": more may be submitted.  Not re-entrant: one thread drives an engine. */
int32_t b2_continuous_open(b2_model* m, const b2_continuous_config* cfg, b2_event_cb cb, void* user, b2_continuous** out);
int32_t b2_continuous_submit(b2_continuous* e, const b2_request* req, int32_t* id_out);
int32_t b2_continuous_halt(b2_continuous* e, int32_t id, int32_t finish_reason);
int32_t b2_continuous_result(b2_continuous* e, int32_t id, int32_t* tokens_out, int32_t capacity, int32_t* n_out,
                             int32_t* finish_out);
int32_t b2_continuous_finish(b2_continuous* e, b2_gen_output* outs, b2_run_stats* stats);
int32_t b2_continuous_free(b2_continuous* e);

/* class index 6 = collectives (tensor-parallel all-reduce) */
/* ---- per-kernel-class timing (CUDA events on the launching stream; off by default) -------------
 * classes: 0 projections (GEMM), 1 paged-attention decode, 2 paged-attention prefill, 3 RoPE + KV
 * append, 4 norm / activation / embedding / argmax, 5 packer + step copies.  The algorithmic work of
 * the same launches is accumulated beside the times: GEMM flops (2*M*N*K) and weight bytes, decode
 * attention K/V bytes (each cached byte once per layer), prefill attention flops. */
typedef struct {
    double ms[8];
    int64_t launches[8];
    double gemm_flops, gemm_weight_bytes, attn_decode_bytes, attn_prefill_flops;
} b2_profile_t;
int32_t b2_profile_enable(b2_ctx* ctx, int32_t on);   /* also resets the accumulators */
int32_t b2_profile_read(b2_ctx* ctx, b2_profile_t* out);

#ifdef __cplusplus
}
#endif
#endif
