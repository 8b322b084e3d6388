// Bounded page pool and per-sequence paged caches: host bookkeeping for the KvCache contract
// (src/primitives/kv_cache.rs:30-64) over the device-resident K/V pages.
//
// Two id spaces are kept apart on purpose.  PHYSICAL pages hold bytes and are needed as soon as the
// first token of a block arrives.  The reference's BLOCK IDS (paged_kv_cache.rs:315-340) are handed
// out only when a block fills, by a recycling allocator; they are reproduced here as pure
// bookkeeping so that block-id lists, live/shared/peak counters and reserved_tokens read exactly as
// they do in the reference.
#include <algorithm>
#include <cstring>

#include "engine.h"

int64_t RefBlockAllocator::alloc() {
    int64_t id;
    if (!free_ids.empty()) {
        id = free_ids.back();  // most recently freed first (the reference leaves the order open)
        free_ids.pop_back();
        refs[id] = 1;
    } else {
        id = (int64_t)refs.size();
        refs.push_back(1);
    }
    live++;
    peak = std::max(peak, live);
    return id;
}
void RefBlockAllocator::retain(int64_t id) { refs[id]++; }
bool RefBlockAllocator::release(int64_t id) {
    if (--refs[id] == 0) {
        free_ids.push_back(id);
        live--;
        return true;
    }
    return false;
}
int64_t RefBlockAllocator::shared() const {
    int64_t n = 0;
    for (auto r : refs) n += r > 1;
    return n;
}

namespace {

int32_t pool_alloc_page(b2_pool* p, int32_t* out) {
    B2_REQUIRE(!p->free_pages.empty(), B2_ERR_OOM_PAGES, "page pool exhausted");
    *out = p->free_pages.back();
    p->free_pages.pop_back();
    p->page_ref[*out] = 1;
    return B2_OK;
}
void pool_unref_page(b2_pool* p, int32_t page) {
    if (--p->page_ref[page] == 0) p->free_pages.push_back(page);
}
// Queue table[slot][index] = page for the next step's packer.  The packer applies the queue with many threads in no
// particular order, so the queue never holds two entries for one (slot, index): a later write (a private copy
// replacing a shared page before any step ran, a freed row handed to a new cache) replaces the earlier one here.
void push_update(b2_pool* p, int slot, int index, int page) {
    for (size_t i = p->upd_slot.size(); i-- > 0;)
        if (p->upd_slot[i] == slot && p->upd_index[i] == index) {
            p->upd_page[i] = page;
            return;
        }
    p->upd_slot.push_back(slot);
    p->upd_index.push_back(index);
    p->upd_page.push_back(page);
}
// Drop everything a cache holds from block `first_block` on (frozen ids first, then pages).
void cache_release_from(b2_cache* c, size_t first_block) {
    b2_pool* p = c->pool;
    for (size_t j = first_block; j < c->block_ids.size(); j++) p->ids.release(c->block_ids[j]);
    if (c->block_ids.size() > first_block) c->block_ids.resize(first_block);
    for (size_t j = first_block; j < c->pages.size(); j++) pool_unref_page(p, c->pages[j]);
    if (c->pages.size() > first_block) c->pages.resize(first_block);
}

}  // namespace

// Reserve pages for `n` more tokens of a cache (called by the step before the forward).
int32_t b2_cache_reserve(b2_cache* c, int n) {
    b2_pool* p = c->pool;
    const int bs = p->block_size;
    const size_t need = (size_t)((c->len + n + bs - 1) / bs);
    B2_REQUIRE((int)need <= p->max_blocks, B2_ERR_OOM_PAGES, "sequence exceeds max_blocks_per_seq of its pool");
    while (c->pages.size() < need) {
        int32_t page;
        B2_CHECK(pool_alloc_page(p, &page));
        push_update(p, c->slot, (int)c->pages.size(), page);
        c->pages.push_back(page);
    }
    return B2_OK;
}
// Advance the cache after a forward wrote `n` tokens: freeze the blocks that became full
// (freeze_full_blocks, paged_kv_cache.rs:315-340).
void b2_cache_commit(b2_cache* c, int n) {
    b2_pool* p = c->pool;
    c->len += n;
    const size_t full = (size_t)(c->len / p->block_size);
    while (c->block_ids.size() < full) {
        const int64_t id = p->ids.alloc();
        if ((size_t)id >= p->id_to_page.size()) p->id_to_page.resize((size_t)id + 1, -1);
        p->id_to_page[id] = c->pages[c->block_ids.size()];
        c->block_ids.push_back(id);
    }
}

extern "C" {

int32_t b2_pool_new(b2_ctx* ctx, const b2_model* m, int32_t block_size, int64_t max_pages, int32_t max_seqs,
                    int32_t max_blocks_per_seq, b2_pool** out) {
    B2_REQUIRE(ctx && m && out, B2_ERR_MSG, "b2_pool_new: null argument");
    B2_REQUIRE(block_size > 0, B2_ERR_MSG, "block_size must be > 0");  // BlockPool::new asserts this (:82)
    B2_REQUIRE(block_size % 16 == 0, B2_ERR_UNSUPPORTED, "b2_pool_new: the attention kernels need a block size that is a multiple of 16");
    B2_REQUIRE(max_pages > 0 && max_seqs > 0 && max_blocks_per_seq > 0, B2_ERR_MSG, "b2_pool_new: capacities must be positive");
    B2_REQUIRE(max_pages * (int64_t)block_size < (1ll << 31), B2_ERR_UNSUPPORTED, "b2_pool_new: pool too large for 32-bit slot ids");
    B2_CUDA(cudaSetDevice(ctx->device));
    b2_pool* p = new b2_pool();
    p->ctx = ctx;
    p->model = m;
    p->block_size = block_size;
    p->max_pages = max_pages;
    p->max_seqs = max_seqs;
    p->max_blocks = max_blocks_per_seq;
    p->layers = m->cfg.num_layers;
    p->hkv = m->hkv_l;  // pages hold this rank's KV heads only
    p->hd = m->cfg.head_dim;
    p->page_elems = (size_t)p->hkv * block_size * p->hd;
    p->esz = m->f32 ? 4 : 2;
    const size_t bytes = (size_t)p->layers * 2 * (size_t)max_pages * p->page_bytes();
    cudaError_t e = cudaMalloc((void**)&p->kv, bytes);
    if (e != cudaSuccess) {
        delete p;
        return b2_fail(B2_ERR_CUDA, std::string("b2_pool_new: cudaMalloc of the KV pool failed: ") + cudaGetErrorString(e));
    }
    e = cudaMalloc((void**)&p->block_tables, (size_t)max_seqs * max_blocks_per_seq * 4);
    if (e != cudaSuccess) {
        cudaFree(p->kv);
        delete p;
        return b2_fail(B2_ERR_CUDA, std::string("b2_pool_new: cudaMalloc of the block tables failed: ") + cudaGetErrorString(e));
    }
    cudaMemsetAsync(p->block_tables, 0, (size_t)max_seqs * max_blocks_per_seq * 4, ctx->stream);
    // Masked positions of a partly filled page still enter the P.V product with weight zero, and
    // 0 * NaN is NaN: the pool must never hold non-finite garbage.
    cudaMemsetAsync(p->kv, 0, bytes, ctx->stream);
    p->free_pages.resize((size_t)max_pages);
    for (int64_t i = 0; i < max_pages; i++) p->free_pages[i] = (int32_t)(max_pages - 1 - i);  // page 0 goes out first
    p->page_ref.assign((size_t)max_pages, 0);
    p->free_slots.resize(max_seqs);
    for (int i = 0; i < max_seqs; i++) p->free_slots[i] = max_seqs - 1 - i;
    *out = p;
    return B2_OK;
}

int32_t b2_pool_free(b2_pool* p) {
    if (!p) return B2_OK;
    B2_REQUIRE(p->live_caches == 0, B2_ERR_MSG, "b2_pool_free: caches of this pool are still alive");
    cudaSetDevice(p->ctx->device);
    cudaStreamSynchronize(p->ctx->stream);
    cudaFree(p->kv);
    cudaFree(p->block_tables);
    delete p;
    return B2_OK;
}

int32_t b2_pool_stats(const b2_pool* p, b2_pool_stats_t* out) {
    B2_REQUIRE(p && out, B2_ERR_MSG, "b2_pool_stats: null argument");
    out->live_blocks = p->ids.live;
    out->shared_blocks = p->ids.shared();
    out->peak_live_blocks = p->ids.peak;
    out->reserved_tokens = p->ids.live * p->block_size;  // BlockPool::reserved_tokens, :112-114
    out->free_pages = (int64_t)p->free_pages.size();
    out->total_pages = p->max_pages;
    return B2_OK;
}

int32_t b2_cache_new(b2_pool* p, b2_cache** out) {
    B2_REQUIRE(p && out, B2_ERR_MSG, "b2_cache_new: null argument");
    B2_REQUIRE(!p->free_slots.empty(), B2_ERR_OOM_PAGES, "b2_cache_new: the pool has no free block-table row (max_seqs reached)");
    b2_cache* c = new b2_cache();
    c->pool = p;
    c->slot = p->free_slots.back();
    p->free_slots.pop_back();
    p->live_caches++;
    *out = c;
    return B2_OK;
}

int32_t b2_cache_new_seeded(b2_pool* p, const int64_t* shared_block_ids, int32_t n, b2_cache** out) {
    B2_REQUIRE(p && out && (n == 0 || shared_block_ids), B2_ERR_MSG, "b2_cache_new_seeded: null argument");
    B2_REQUIRE(n <= p->max_blocks, B2_ERR_OOM_PAGES, "b2_cache_new_seeded: prefix longer than max_blocks_per_seq");
    for (int i = 0; i < n; i++) {
        const int64_t id = shared_block_ids[i];
        B2_REQUIRE(id >= 0 && (size_t)id < p->ids.refs.size() && p->ids.refs[id] > 0, B2_ERR_MSG, "b2_cache_new_seeded: block id is not live");
    }
    b2_cache* c = nullptr;
    B2_CHECK(b2_cache_new(p, &c));
    for (int i = 0; i < n; i++) {
        const int64_t id = shared_block_ids[i];
        const int32_t page = p->id_to_page[id];
        p->ids.retain(id);
        p->page_ref[page]++;
        c->block_ids.push_back(id);
        c->pages.push_back(page);
        push_update(p, c->slot, i, page);
    }
    c->len = n * p->block_size;  // starts positioned past the shared prefix (:218-220)
    *out = c;
    return B2_OK;
}

int32_t b2_cache_free(b2_cache* c) {
    if (!c) return B2_OK;
    cache_release_from(c, 0);
    c->pool->free_slots.push_back(c->slot);
    c->pool->live_caches--;
    delete c;
    return B2_OK;
}

int32_t b2_cache_offset(const b2_cache* c) { return c ? c->len : 0; }
int32_t b2_cache_batch_size(const b2_cache* c) { return c && c->len > 0 ? 1 : 0; }
int32_t b2_cache_num_layers(const b2_cache* c) { return c ? c->pool->layers : 0; }
int64_t b2_cache_blocks(const b2_cache* c) { return c ? (int64_t)c->block_ids.size() : 0; }
int64_t b2_cache_reserved_tokens(const b2_cache* c) {
    if (!c) return 0;
    const int bs = c->pool->block_size;
    return ((int64_t)c->block_ids.size() + (c->len % bs > 0 ? 1 : 0)) * bs;
}
int32_t b2_cache_block_ids(const b2_cache* c, int64_t* out, int32_t cap) {
    if (!c) return 0;
    for (size_t i = 0; i < c->block_ids.size() && (int)i < cap; i++) out[i] = c->block_ids[i];
    return (int32_t)c->block_ids.size();
}

int32_t b2_cache_reset(b2_cache* c) {
    B2_REQUIRE(c, B2_ERR_MSG, "b2_cache_reset: null cache");
    cache_release_from(c, 0);
    c->len = 0;
    return B2_OK;
}

int32_t b2_cache_retain_sequences(b2_cache* c, const int32_t* keep, int32_t n) {
    B2_REQUIRE(c, B2_ERR_MSG, "b2_cache_retain_sequences: null cache");
    if (n == 0) return b2_cache_reset(c);
    B2_REQUIRE(n == 1 && keep && keep[0] == 0, B2_ERR_MSG, "PagedKvCache is single-sequence; retain_sequences expects [] or [0]");
    return B2_OK;
}

int32_t b2_cache_truncate(b2_cache* c, int32_t len) {
    B2_REQUIRE(c, B2_ERR_MSG, "b2_cache_truncate: null cache");
    B2_REQUIRE(len >= 0, B2_ERR_MSG, "truncate: negative len");
    if (len >= c->len) return B2_OK;
    b2_pool* p = c->pool;
    const int bs = p->block_size;
    const size_t keep_full = (size_t)(len / bs);
    const int rem = len % bs;
    const size_t keep_pages = keep_full + (rem > 0 ? 1 : 0);
    // frozen ids from keep_full on are released; the boundary block (if any) becomes a private tail
    for (size_t j = keep_full; j < c->block_ids.size(); j++) p->ids.release(c->block_ids[j]);
    if (c->block_ids.size() > keep_full) c->block_ids.resize(keep_full);
    for (size_t j = keep_pages; j < c->pages.size(); j++) pool_unref_page(p, c->pages[j]);
    if (c->pages.size() > keep_pages) c->pages.resize(keep_pages);
    if (rem > 0 && p->page_ref[c->pages[keep_full]] > 1) {
        // the boundary page is shared with another sequence: unfreeze into a private copy
        int32_t fresh;
        B2_CHECK(pool_alloc_page(p, &fresh));
        const int32_t old = c->pages[keep_full];
        for (int l = 0; l < p->layers; l++) {
            uint8_t* kl = reinterpret_cast<uint8_t*>(p->k_layer(l));
            uint8_t* vl = reinterpret_cast<uint8_t*>(p->v_layer(l));
            B2_CUDA(cudaMemcpyAsync(kl + (size_t)fresh * p->page_bytes(), kl + (size_t)old * p->page_bytes(), p->page_bytes(),
                                    cudaMemcpyDeviceToDevice, p->ctx->stream));
            B2_CUDA(cudaMemcpyAsync(vl + (size_t)fresh * p->page_bytes(), vl + (size_t)old * p->page_bytes(), p->page_bytes(),
                                    cudaMemcpyDeviceToDevice, p->ctx->stream));
        }
        pool_unref_page(p, old);
        c->pages[keep_full] = fresh;
        push_update(p, c->slot, (int)keep_full, fresh);
    }
    c->len = len;
    return B2_OK;
}

int32_t b2_cache_shareable_prefix_blocks(b2_cache* c, int64_t tokens, int64_t* out, int32_t cap) {
    if (!c || tokens < 0) return 0;
    const size_t n = std::min((size_t)(tokens / c->pool->block_size), c->block_ids.size());
    for (size_t i = 0; i < n && (int)i < cap; i++) out[i] = c->block_ids[i];
    return (int32_t)n;
}

static int32_t cache_gather(b2_cache* c, int32_t layer, void* k_host, void* v_host, int esz) {
    B2_REQUIRE(c && k_host && v_host, B2_ERR_MSG, "b2_cache_gather: null argument");
    b2_pool* p = c->pool;
    B2_REQUIRE(p->esz == esz, B2_ERR_MSG, esz == 2 ? "b2_cache_gather: the pool holds f32 pages, use b2_cache_gather_f32"
                                                  : "b2_cache_gather_f32: the pool holds bf16 pages, use b2_cache_gather");
    B2_REQUIRE(layer >= 0 && layer < p->layers, B2_ERR_MSG, "b2_cache_gather: layer out of range");
    B2_REQUIRE(c->len > 0, B2_ERR_MSG, "gather on an empty paged cache");
    const int bs = p->block_size, hd = p->hd, hkv = p->hkv;
    std::vector<uint8_t> pk(p->page_bytes()), pv(p->page_bytes());
    B2_CUDA(cudaStreamSynchronize(p->ctx->stream));
    const uint8_t* kl = reinterpret_cast<const uint8_t*>(p->k_layer(layer));
    const uint8_t* vl = reinterpret_cast<const uint8_t*>(p->v_layer(layer));
    for (size_t b = 0; b < c->pages.size(); b++) {
        const int tokens = std::min(bs, c->len - (int)b * bs);
        if (tokens <= 0) break;
        B2_CUDA(cudaMemcpy(pk.data(), kl + (size_t)c->pages[b] * p->page_bytes(), p->page_bytes(), cudaMemcpyDeviceToHost));
        B2_CUDA(cudaMemcpy(pv.data(), vl + (size_t)c->pages[b] * p->page_bytes(), p->page_bytes(), cudaMemcpyDeviceToHost));
        for (int h = 0; h < hkv; h++)
            for (int t = 0; t < tokens; t++) {
                const size_t src = ((size_t)h * bs + t) * hd * esz, dst = ((size_t)h * c->len + b * bs + t) * hd * esz;
                memcpy((uint8_t*)k_host + dst, pk.data() + src, (size_t)hd * esz);
                memcpy((uint8_t*)v_host + dst, pv.data() + src, (size_t)hd * esz);
            }
    }
    return B2_OK;
}
int32_t b2_cache_gather(b2_cache* c, int32_t layer, uint16_t* k_host, uint16_t* v_host) { return cache_gather(c, layer, k_host, v_host, 2); }
int32_t b2_cache_gather_f32(b2_cache* c, int32_t layer, float* k_host, float* v_host) { return cache_gather(c, layer, k_host, v_host, 4); }

}  // extern "C"
