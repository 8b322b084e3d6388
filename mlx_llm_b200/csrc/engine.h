// Host-side engine: weights, model, bounded page pool, per-sequence paged caches, the ragged step
// and the generation loops.  Mirrors the reference's types (cited per member as file:line inside
// SceneWorks/mlx-llm); all tensor work happens in the CUDA kernels of this library.
#pragma once
#include <cstdint>
#include <map>
#include <string>
#include <vector>

#include "common.cuh"
#include "kernels.h"

// ---- Weights (src/primitives/weights.rs:17-96) -------------------------------------------------
struct HostTensor {
    int dtype = 0;
    std::vector<int64_t> shape;
    const uint8_t* ptr = nullptr;  // into `owned` or into an mmap'd file
    size_t nbytes = 0;
    std::vector<uint8_t> owned;
    int64_t numel() const {
        int64_t n = 1;
        for (auto d : shape) n *= d;
        return n;
    }
};
struct MappedFile {
    void* base = nullptr;
    size_t len = 0;
};
struct b2_weights {
    std::map<std::string, HostTensor> t;
    std::vector<MappedFile> maps;
};

// ---- Tensor-parallel group (tp.cu): rank r of `world` owns KV heads [r*hkv/world, (r+1)*hkv/world) ----
struct b2_tp_group {
    b2_ctx* ctx = nullptr;
    int rank = 0, world = 1;
    void* comm = nullptr;  // ncclComm_t (null for a group that reduces over peer memory only)
    // peer-memory reductions (tp_peer.cu): this rank's exported region and every rank's region as mapped here
    void* peer_local = nullptr;
    void* peer_base[8] = {};
    int peer_cap_rows = 0, peer_hidden = 0;
    size_t peer_x_off = 0, peer_slot_bytes = 0;
    bool peer_ready = false, peer_ipc = false, peer_push = false;
    uint32_t peer_seq = 0;  // number of the last reduction; every rank advances it in step
    // ranks emulated inside one process on one device (b2_tp_peer_attach_local): the object that lets the ranks' host
    // threads meet at every reduction, shared by the groups, owned by rank 0's
    struct b2_tp_lockstep* lockstep = nullptr;
};
// In-place sum over the group of an f32 device buffer, enqueued on the context's stream.
int32_t b2_tp_all_reduce_sum_f32(b2_tp_group* g, float* buf, size_t n);
// Peer-memory path: the projection's scattered f32 output, this rank's hidden state, the fused sum + residual add.
struct GemmParams;
void b2_tp_peer_scatter(const b2_tp_group* g, GemmParams& p);
uint16_t* b2_tp_peer_x(const b2_tp_group* g);
int32_t b2_tp_peer_reduce_residual_launch(b2_tp_group* g, int M);
void b2_tp_peer_release(b2_tp_group* g);

// ---- Model (src/models/llama.rs: CausalLm, LlamaLayer, LlamaAttention, LlamaMlp) ------------------
struct Proj {  // Projection::{Dense,Quantized} (src/primitives/projection.rs:34-47)
    int bits = 0, N = 0, K = 0;
    void* w = nullptr;
    uint16_t* scales = nullptr;
    uint16_t* biases = nullptr;
    uint32_t* sbt = nullptr;  // scales and biases once more, transposed and interleaved (GemmParams::sbt), built at load
};
struct LayerW {
    uint16_t* input_ln = nullptr;
    uint16_t* post_ln = nullptr;
    uint16_t* q_norm = nullptr;
    uint16_t* k_norm = nullptr;
    Proj qkv, o, gu, down;  // q|k|v rows fused; gate|up rows fused
};
struct Workspace {
    int t_cap = 0, b_cap = 0, w_cap = 0, p_cap = 0;
    uint16_t *x = nullptr, *xn = nullptr, *qkv = nullptr, *q = nullptr, *attn = nullptr, *gu = nullptr, *act = nullptr;
    uint16_t *last = nullptr, *logits = nullptr;
    float* tp_part = nullptr;  // [t_cap, hidden] f32 partial sums of o_proj / down_proj (tensor-parallel only)
    bool x_in_peer_region = false;  // x points into the group's exported region (not owned by the workspace)
    int32_t* argmax = nullptr;
    int32_t* ids = nullptr;
    int32_t* meta = nullptr;      // packer outputs (b2_batch_meta_carve layout)
    int32_t* stage_dev = nullptr; // packer inputs
    size_t stage_cap = 0;
    float* attn_scratch = nullptr;
    size_t attn_scratch_bytes = 0;
    // pinned host staging
    int32_t* stage_host = nullptr;
    size_t stage_host_cap = 0;
    int32_t* argmax_host = nullptr;
    uint16_t* logits_host = nullptr;
    size_t logits_host_cap = 0;
};
struct b2_model {
    b2_ctx* ctx = nullptr;
    b2_model_config cfg{};  // the WHOLE model's dimensions, also under tensor parallelism
    // this rank's share (== cfg's values without tensor parallelism)
    b2_tp_group* tp = nullptr;
    int hq_l = 0, hkv_l = 0, inter_l = 0;
    uint16_t* embed = nullptr;
    uint16_t* lm_head = nullptr;
    uint16_t* norm = nullptr;
    std::vector<LayerW> layers;
    std::vector<float> inv_freq;
    uint16_t *cos_tab = nullptr, *sin_tab = nullptr;
    int rope_positions = 0;
    std::vector<void*> allocs;
    int64_t weight_bytes = 0;
    bool quantized = false;
    bool f32 = false;  // cfg.compute_f32: every weight pointer above then holds float, not bf16
    float *cos_f32 = nullptr, *sin_f32 = nullptr;  // f32 RoPE tables of the f32 path
    struct F32Work* w32 = nullptr;                 // its activations (engine_step_f32.cu)
    Workspace ws;
    cudaEvent_t ev0 = nullptr, ev1 = nullptr;
    // accumulated by every forward
    double device_ms = 0;
    int64_t h2d_bytes = 0, d2h_bytes = 0;
};

// ---- Block-id lifetimes as the reference sees them (core_llm::paging::BlockAllocator through
// src/primitives/paged_kv_cache.rs:95-160): ids are handed out when a block FILLS ----------------
struct RefBlockAllocator {
    std::vector<uint32_t> refs;
    std::vector<int64_t> free_ids;
    int64_t live = 0, peak = 0;
    int64_t alloc();
    void retain(int64_t id);
    bool release(int64_t id);
    int64_t shared() const;
};

struct b2_pool {  // BlockPool (paged_kv_cache.rs:72-160) + bounded physical pages
    b2_ctx* ctx = nullptr;
    const b2_model* model = nullptr;
    int block_size = 16;
    int64_t max_pages = 0;
    int max_seqs = 0, max_blocks = 0;
    int layers = 0, hkv = 0, hd = 0;
    uint16_t* kv = nullptr;        // [layers][2][pages][hkv][block][hd], bf16 (f32 for an f32 model)
    int esz = 2;                   // bytes per element
    size_t page_elems = 0;         // hkv*block*hd
    int32_t* block_tables = nullptr;  // device [max_seqs][max_blocks]
    std::vector<int32_t> free_pages;  // stack, back() is handed out next
    std::vector<int32_t> page_ref;
    RefBlockAllocator ids;
    std::vector<int32_t> id_to_page;
    std::vector<int32_t> free_slots;
    std::vector<int32_t> upd_slot, upd_index, upd_page;  // block-table updates not yet on the device
    int64_t live_caches = 0;
    uint64_t step_stamp = 0;  // number of the last forward over this pool (duplicate-cache check)
    size_t page_bytes() const { return page_elems * (size_t)esz; }
    uint16_t* k_layer(int l) const { return reinterpret_cast<uint16_t*>(reinterpret_cast<uint8_t*>(kv) + ((size_t)l * 2) * (size_t)max_pages * page_bytes()); }
    uint16_t* v_layer(int l) const { return reinterpret_cast<uint16_t*>(reinterpret_cast<uint8_t*>(kv) + ((size_t)l * 2 + 1) * (size_t)max_pages * page_bytes()); }
};

struct b2_cache {  // PagedKvCache (paged_kv_cache.rs:168-516)
    b2_pool* pool = nullptr;
    int slot = -1;
    int len = 0;                     // KvCache::offset
    uint64_t step_stamp = 0;         // pool->step_stamp of the last forward this cache took part in
    std::vector<int32_t> pages;      // physical page of every started block (incl. the partial tail)
    std::vector<int64_t> block_ids;  // reference-view ids of the frozen (full) blocks
};

struct SeqStep {
    b2_cache* cache;
    const int32_t* ids;
    int n;
    bool want_logits;
    // logits / greedy ids of EVERY new position, not only the last (CausalLm::decode_logits_all, llama.rs:372-392: the
    // verify forward of speculative decoding).  Only for a step of one sequence.
    bool all_positions = false;
};
// One forward over a ragged batch.  argmax_out[i] (per sequence that wants logits, in batch order)
// and logits_out (rows in the same order: bf16, or f32 for an f32 model) are host pointers, nullable.
int32_t b2_engine_forward(b2_model* m, std::vector<SeqStep>& seqs, void* logits_out, int32_t* argmax_out);
// The f32 path's layers (engine_step_f32.cu): from the step's ids to f32 logits + greedy ids for the n_logits sampled rows;
// *logits_dev receives the device address of the [n_logits, vocab] f32 logits.
struct BatchMetaOut;
int32_t b2_forward_f32(b2_model* m, b2_pool* pool, const BatchMetaOut& mo, const int32_t* seq_slot_dev, const int32_t* ids_dev, int T, int B,
                       int n_logits, const int32_t* logit_rows, int max_ctx, float** logits_dev);
void b2_forward_f32_release(b2_model* m);
