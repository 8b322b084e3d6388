// CPU oracle (test infrastructure): KV-cache bookkeeping with the reference's semantics.
//
// Restates src/primitives/paged_kv_cache.rs:72-516 (BlockPool, PagedKvCache, impl KvCache, Drop)
// and src/primitives/kv_cache.rs:107-190 (ContiguousKvCache).  Block-id lifetimes belong to
// core_llm::paging::BlockAllocator, whose source is not part of the reference tree; its behaviour is
// taken from the call sites (paged_kv_cache.rs:95-160): alloc() returns a recycled id when one is
// free and otherwise the next fresh id (== number of ids ever created, :119-127); retain/release are
// reference counts; release() reports when the last reference went.  Which freed id is reused first
// is NOT fixed by anything in the reference ("parity unpinned"); this oracle reuses the most
// recently freed id first.
#pragma once
#include <cstdint>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

namespace orc {

struct BlockAllocator {
    std::vector<uint32_t> refs;   // per id
    std::vector<size_t> free_ids; // stack
    size_t live = 0, peak = 0;
    size_t alloc() {
        size_t id;
        if (!free_ids.empty()) {
            id = free_ids.back();
            free_ids.pop_back();
            refs[id] = 1;
        } else {
            id = refs.size();
            refs.push_back(1);
        }
        live++;
        if (live > peak) peak = live;
        return id;
    }
    void retain(size_t id) { refs.at(id)++; }
    bool release(size_t id) {
        if (refs.at(id) == 0) throw std::runtime_error("release of a free block");
        if (--refs[id] == 0) {
            free_ids.push_back(id);
            live--;
            return true;
        }
        return false;
    }
    size_t live_blocks() const { return live; }
    size_t shared_blocks() const {
        size_t n = 0;
        for (auto r : refs) n += r > 1;
        return n;
    }
    size_t peak_live_blocks() const { return peak; }
};

// Token-major KV rows: one row = n_kv*hd bf16 values of one position.
using Rows = std::vector<uint16_t>;

struct PhysBlock {
    bool live = false;
    std::vector<Rows> k, v;  // per layer, block_size rows; empty <=> not materialised
};

struct BlockPool {
    size_t block_size;
    std::vector<PhysBlock> blocks;
    BlockAllocator alloc;
    explicit BlockPool(size_t bs) : block_size(bs) {
        if (bs == 0) throw std::runtime_error("block_size must be > 0");
    }
    size_t live_blocks() const { return alloc.live_blocks(); }
    size_t shared_blocks() const { return alloc.shared_blocks(); }
    size_t peak_live_blocks() const { return alloc.peak_live_blocks(); }
    size_t reserved_tokens() const { return live_blocks() * block_size; }
    size_t alloc_empty() {
        size_t id = alloc.alloc();
        if (id == blocks.size()) blocks.emplace_back();
        blocks[id] = PhysBlock{};
        blocks[id].live = true;
        return id;
    }
    bool is_materialized(size_t id) const { return !blocks.at(id).k.empty(); }
    void retain(size_t id) { alloc.retain(id); }
    void release(size_t id) {
        if (alloc.release(id)) blocks[id] = PhysBlock{};
    }
};

// Common view both caches give the decoder: after update(), all cached rows of a layer.
struct KvCacheBase {
    virtual ~KvCacheBase() = default;
    // Append `step` rows (token-major, row_elems each) for `layer`.
    virtual void update(size_t layer, const uint16_t* k, const uint16_t* v, size_t step, size_t row_elems) = 0;
    virtual const Rows& keys(size_t layer) = 0;
    virtual const Rows& values(size_t layer) = 0;
    virtual int32_t offset() const = 0;
    virtual size_t num_layers() const = 0;
    virtual void truncate(int32_t len) = 0;
    virtual void reset() = 0;
};

struct ContiguousKvCache : KvCacheBase {
    std::vector<Rows> k, v;
    size_t row = 0;
    explicit ContiguousKvCache(size_t layers) : k(layers), v(layers) {}
    void update(size_t layer, const uint16_t* kk, const uint16_t* vv, size_t step, size_t row_elems) override {
        row = row_elems;
        k[layer].insert(k[layer].end(), kk, kk + step * row_elems);
        v[layer].insert(v[layer].end(), vv, vv + step * row_elems);
    }
    const Rows& keys(size_t l) override { return k[l]; }
    const Rows& values(size_t l) override { return v[l]; }
    int32_t offset() const override { return row ? (int32_t)(k[0].size() / row) : 0; }
    size_t num_layers() const override { return k.size(); }
    void truncate(int32_t len) override {
        if (len < 0) throw std::runtime_error("truncate: negative len");
        if (len >= offset()) return;
        for (auto& r : k) r.resize((size_t)len * row);
        for (auto& r : v) r.resize((size_t)len * row);
    }
    void reset() override {
        for (auto& r : k) r.clear();
        for (auto& r : v) r.clear();
    }
};

struct PagedKvCache : KvCacheBase {
    size_t layers, block_size;
    std::shared_ptr<BlockPool> pool;
    std::vector<size_t> block_ids;  // frozen (full) blocks in position order
    size_t tail_len = 0;            // authoritative after the last layer of a step
    size_t row = 0;
    // all rows (frozen prefix followed by the tail) per layer; `have[l]` false for a freshly seeded
    // cache until the frozen prefix has been rebuilt from the pool (ensure_frozen, :361-375)
    std::vector<Rows> k, v;
    std::vector<bool> have;

    PagedKvCache(std::shared_ptr<BlockPool> p, size_t nl)
        : layers(nl), block_size(p->block_size), pool(std::move(p)), k(nl), v(nl), have(nl, true) {}
    // new_seeded, :221-235
    PagedKvCache(std::shared_ptr<BlockPool> p, size_t nl, const std::vector<size_t>& shared) : PagedKvCache(std::move(p), nl) {
        for (size_t id : shared) pool->retain(id);
        block_ids = shared;
        if (!shared.empty()) have.assign(nl, false);
    }
    ~PagedKvCache() override {
        for (size_t id : block_ids) pool->release(id);  // Drop, :507-516
    }
    size_t blocks() const { return block_ids.size(); }
    size_t reserved_tokens() const { return (block_ids.size() + (tail_len > 0 ? 1 : 0)) * block_size; }
    size_t len() const { return block_ids.size() * block_size + tail_len; }
    int32_t offset() const override { return (int32_t)len(); }
    size_t num_layers() const override { return layers; }
    int32_t batch_size() const {
        bool any_tail = false;
        for (size_t l = 0; l < layers; l++) any_tail = any_tail || k[l].size() > block_ids.size() * block_size * row;
        return (!block_ids.empty() || tail_len > 0 || any_tail) ? 1 : 0;
    }
    void ensure_frozen(size_t l) {
        if (have[l]) return;
        Rows kk, vv;
        for (size_t id : block_ids) {
            if (!pool->is_materialized(id)) throw std::runtime_error("ensure_frozen over an unmaterialized block");
            const auto& b = pool->blocks[id];
            kk.insert(kk.end(), b.k[l].begin(), b.k[l].end());
            vv.insert(vv.end(), b.v[l].begin(), b.v[l].end());
            row = b.k[l].size() / block_size;
        }
        // any tail appended before the rebuild stays behind the frozen prefix
        kk.insert(kk.end(), k[l].begin(), k[l].end());
        vv.insert(vv.end(), v[l].begin(), v[l].end());
        k[l].swap(kk);
        v[l].swap(vv);
        have[l] = true;
    }
    // KvCache::update, :379-394: append to the tail; freeze whole blocks once the LAST layer has the
    // step's tokens (:390-392, freeze_full_blocks :315-340).
    void update(size_t layer, const uint16_t* kk, const uint16_t* vv, size_t step, size_t row_elems) override {
        row = row_elems;
        ensure_frozen(layer);
        k[layer].insert(k[layer].end(), kk, kk + step * row_elems);
        v[layer].insert(v[layer].end(), vv, vv + step * row_elems);
        if (layer + 1 == layers) {
            tail_len += step;
            if (tail_len >= block_size) {
                size_t n_full = tail_len / block_size;
                for (size_t i = 0; i < n_full; i++) block_ids.push_back(pool->alloc_empty());
                tail_len -= n_full * block_size;
            }
        }
    }
    const Rows& keys(size_t l) override {
        ensure_frozen(l);
        return k[l];
    }
    const Rows& values(size_t l) override {
        ensure_frozen(l);
        return v[l];
    }
    // shareable_prefix_blocks, :250-275: whole blocks only; materialises the offered blocks.
    std::vector<size_t> shareable_prefix_blocks(size_t tokens) {
        size_t n = std::min(tokens / block_size, block_ids.size());
        for (size_t l = 0; l < layers; l++) ensure_frozen(l);
        for (size_t b = 0; b < n; b++) {
            size_t id = block_ids[b];
            if (pool->is_materialized(id)) continue;
            auto& pb = pool->blocks[id];
            pb.k.resize(layers);
            pb.v.resize(layers);
            for (size_t l = 0; l < layers; l++) {
                pb.k[l].assign(k[l].begin() + b * block_size * row, k[l].begin() + (b + 1) * block_size * row);
                pb.v[l].assign(v[l].begin() + b * block_size * row, v[l].begin() + (b + 1) * block_size * row);
            }
        }
        return std::vector<size_t>(block_ids.begin(), block_ids.begin() + n);
    }
    // truncate, :422-485
    void truncate(int32_t len_) override {
        if (len_ < 0) throw std::runtime_error("truncate: negative len");
        size_t n = (size_t)len_;
        if (n >= len()) return;
        size_t full = block_ids.size() * block_size;
        for (size_t l = 0; l < layers; l++) {
            ensure_frozen(l);
            k[l].resize(n * row);
            v[l].resize(n * row);
        }
        if (n >= full) {
            tail_len = n - full;
            return;
        }
        size_t keep_full = n / block_size;
        tail_len = n % block_size;
        for (size_t i = keep_full; i < block_ids.size(); i++) pool->release(block_ids[i]);
        block_ids.resize(keep_full);
    }
    void reset() override {
        for (size_t id : block_ids) pool->release(id);
        block_ids.clear();
        for (auto& r : k) r.clear();
        for (auto& r : v) r.clear();
        have.assign(layers, true);
        tail_len = 0;
    }
    // retain_sequences, :408-420: only [] (drop) or [0] (no-op) are valid.
    void retain_sequences(const int32_t* keep, size_t n) {
        if (n == 0)
            reset();
        else if (!(n == 1 && keep[0] == 0))
            throw std::runtime_error("PagedKvCache is single-sequence; retain_sequences expects [] or [0]");
    }
};

}  // namespace orc
