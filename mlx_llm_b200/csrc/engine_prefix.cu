// Shared-prefix KV reuse on pages.
//
// b2_prefix_cache / b2_generate_cached <- PrefixCache / generate_cached (src/decode/prefix.rs:56-188): the KV of every
// finished request (prompt + generated) is kept; a new request reuses the longest stored prefix of its prompt and
// prefills only the rest.  The reference copies the matched span out of contiguous tensors (slice_layers, :190-205);
// here the stored sequence IS a paged cache, and a reuse is a fork of it (b2_cache_fork): the full blocks of the
// matched span are shared by reference count, copy-on-write style (src/primitives/paged_kv_cache.rs:221-235), and only
// a partly covered last block is copied, so a hit costs at most one page copy per layer whatever the prefix length.
//
// The policy -- which stored sequence shares the longest prefix, least-recently-used eviction past `capacity` -- is
// core_llm::prefix::PrefixIndex in the reference, whose source is not part of its tree; it is restated here from its
// call sites (prefix.rs:92-131): longest common prefix over the stored sequences (ties: the most recently used), a
// match refreshes its entry, an insert evicts the least recently used entries beyond the capacity (capacity 0 keeps
// nothing), and a stored sequence that is a prefix of a newly stored one is dropped (the new entry serves every
// request the old one could).  A whole-prompt match still recomputes the last prompt token (:99-104).
#include <algorithm>
#include <memory>

#include "engine.h"

int32_t b2_cache_reserve(b2_cache* c, int n);

struct PrefixEntry {
    std::vector<int32_t> tokens;
    b2_cache* cache = nullptr;
    uint64_t used = 0;  // larger = more recent
};

struct b2_prefix_cache {
    b2_model* model = nullptr;
    b2_pool* pool = nullptr;
    int capacity = 0;
    uint64_t clock = 0;
    std::vector<PrefixEntry> entries;
    b2_prefix_stats stats{};

    void drop(size_t i) {
        b2_cache_free(entries[i].cache);
        entries.erase(entries.begin() + (long)i);
    }
    bool evict_lru() {
        if (entries.empty()) return false;
        size_t lru = 0;
        for (size_t i = 1; i < entries.size(); i++)
            if (entries[i].used < entries[lru].used) lru = i;
        drop(lru);
        return true;
    }
};

namespace {

bool is_stop(const b2_request& r, int32_t tok) {
    for (int i = 0; i < r.n_stop; i++)
        if (r.stop_tokens[i] == tok) return true;
    return false;
}

// One forward of a single sequence; when the pool is out of pages, stored sequences are evicted (least recently used
// first) until it fits.  Pages a stored sequence shares with the running one stay alive through their reference counts.
int32_t forward_evicting(b2_prefix_cache* pc, b2_cache* cache, const int32_t* ids, int n, int32_t* tok) {
    for (;;) {
        std::vector<SeqStep> s{SeqStep{cache, ids, n, true}};
        const int32_t rc = b2_engine_forward(pc->model, s, nullptr, tok);
        if (rc != B2_ERR_OOM_PAGES || !pc->evict_lru()) return rc;
    }
}

}  // namespace

extern "C" {

// A new cache holding the first `len` positions of `src`: full blocks shared, a partly covered last block copied.
int32_t b2_cache_fork(const b2_cache* src, int32_t len, b2_cache** out) {
    B2_REQUIRE(src && out, B2_ERR_MSG, "b2_cache_fork: null argument");
    B2_REQUIRE(len >= 0 && len <= src->len, B2_ERR_MSG, "b2_cache_fork: length beyond the source cache");
    b2_pool* p = src->pool;
    const int bs = p->block_size;
    const int full = len / bs, rem = len % bs;
    b2_cache* c = nullptr;
    B2_CHECK(b2_cache_new(p, &c));
    if (full > 0) {
        // the first `full` blocks of the source are frozen (full) blocks with ids: share ids and pages
        std::vector<int64_t> ids(src->block_ids.begin(), src->block_ids.begin() + full);
        b2_cache_free(c);
        c = nullptr;
        B2_CHECK(b2_cache_new_seeded(p, ids.data(), full, &c));
    }
    if (rem > 0) {
        // private copy of the boundary page: reserve a page for one more token, then copy the source's page over it
        int32_t rc = b2_cache_reserve(c, 1);
        if (rc != B2_OK) {
            b2_cache_free(c);
            return rc;
        }
        const int32_t fresh = c->pages[full], old = src->pages[full];
        for (int l = 0; l < p->layers; l++) {
            uint8_t* kl = reinterpret_cast<uint8_t*>(p->k_layer(l));
            uint8_t* vl = reinterpret_cast<uint8_t*>(p->v_layer(l));
            B2_CUDA(cudaMemcpyAsync(kl + (size_t)fresh * p->page_bytes(), kl + (size_t)old * p->page_bytes(), p->page_bytes(),
                                    cudaMemcpyDeviceToDevice, p->ctx->stream));
            B2_CUDA(cudaMemcpyAsync(vl + (size_t)fresh * p->page_bytes(), vl + (size_t)old * p->page_bytes(), p->page_bytes(),
                                    cudaMemcpyDeviceToDevice, p->ctx->stream));
        }
        c->len = len;
    }
    *out = c;
    return B2_OK;
}

int32_t b2_prefix_cache_new(b2_ctx* ctx, b2_model* m, int32_t capacity, int64_t max_pages, int32_t max_blocks_per_seq, b2_prefix_cache** out) {
    B2_REQUIRE(ctx && m && out, B2_ERR_MSG, "b2_prefix_cache_new: null argument");
    B2_REQUIRE(capacity >= 0 && max_pages > 0 && max_blocks_per_seq > 0, B2_ERR_MSG, "b2_prefix_cache_new: bad capacity");
    auto pc = std::make_unique<b2_prefix_cache>();
    pc->model = m;
    pc->capacity = capacity;
    // one block-table row per stored sequence, one for the running request, one spare for a fork in flight
    B2_CHECK(b2_pool_new(ctx, m, 16, max_pages, capacity + 2, max_blocks_per_seq, &pc->pool));
    *out = pc.release();
    return B2_OK;
}

int32_t b2_prefix_cache_free(b2_prefix_cache* pc) {
    if (!pc) return B2_OK;
    while (!pc->entries.empty()) pc->drop(pc->entries.size() - 1);
    b2_pool_free(pc->pool);
    delete pc;
    return B2_OK;
}

int32_t b2_prefix_cache_stats(const b2_prefix_cache* pc, b2_prefix_stats* out) {
    B2_REQUIRE(pc && out, B2_ERR_MSG, "b2_prefix_cache_stats: null argument");
    *out = pc->stats;
    return B2_OK;
}

int32_t b2_prefix_cache_len(const b2_prefix_cache* pc) { return pc ? (int32_t)pc->entries.size() : 0; }

int32_t b2_generate_cached(b2_model* m, const b2_request* req, const volatile int32_t* cancel, b2_event_cb cb, void* user,
                           b2_prefix_cache* pc, b2_gen_output* out) {
    B2_REQUIRE(m && req && pc, B2_ERR_MSG, "b2_generate_cached: null argument");
    B2_REQUIRE(pc->model == m, B2_ERR_MSG, "generate_cached: the prefix cache belongs to another model");
    B2_REQUIRE(req->sampling.temperature <= 0.f && (req->sampling.repetition_penalty == 1.f || req->sampling.repetition_penalty == 0.f),
               B2_ERR_UNSUPPORTED, "only greedy sampling (temperature <= 0, repetition_penalty == 1) runs on the device path");
    if (cancel && *cancel) return b2_fail(B2_ERR_CANCELED, "canceled before inference");  // typed pre-inference cancel (:154-156)
    B2_REQUIRE(req->n_prompt > 0 && req->prompt_ids, B2_ERR_MSG, "generate_cached: empty prompt");
    const int n_prompt = req->n_prompt;

    // seed_for (:92-116): longest stored prefix, capped so that the suffix keeps at least one token
    pc->stats.lookups++;
    int best = -1, best_len = 0;
    for (size_t i = 0; i < pc->entries.size(); i++) {
        const PrefixEntry& e = pc->entries[i];
        int common = 0;
        const int lim = std::min({(int)e.tokens.size(), n_prompt, e.cache->len});
        while (common < lim && e.tokens[common] == req->prompt_ids[common]) common++;
        common = std::min(common, n_prompt - 1);
        if (common > best_len || (common == best_len && common > 0 && e.used > pc->entries[best].used)) {
            best = (int)i;
            best_len = common;
        }
    }
    b2_cache* cache = nullptr;
    int matched = 0;
    if (best >= 0 && best_len > 0) {
        int32_t rc = b2_cache_fork(pc->entries[best].cache, best_len, &cache);
        while (rc == B2_ERR_OOM_PAGES && pc->entries.size() > 1) {  // make room, but never by dropping the source of the fork
            size_t lru = best == 0 ? 1 : 0;
            for (size_t i = 0; i < pc->entries.size(); i++)
                if ((int)i != best && pc->entries[i].used < pc->entries[lru].used) lru = i;
            pc->drop(lru);
            if ((int)lru < best) best--;
            rc = b2_cache_fork(pc->entries[best].cache, best_len, &cache);
        }
        if (rc == B2_OK) {
            matched = best_len;
            pc->entries[best].used = ++pc->clock;
            pc->stats.hits++;
            pc->stats.reused_prefix_tokens += matched;
        } else if (rc != B2_ERR_OOM_PAGES) {
            return rc;
        }
    }
    if (!cache) B2_CHECK(b2_cache_new(pc->pool, &cache));
    pc->stats.computed_prefill_tokens += n_prompt - matched;

    // prefill the suffix, then the plain greedy loop (decode_loop, src/decode/stream.rs:259-327)
    std::vector<int32_t> gen;
    int finish = B2_FINISH_MAX_TOKENS;
    int32_t next = 0;
    int32_t rc = forward_evicting(pc, cache, req->prompt_ids + matched, n_prompt - matched, &next);
    for (int step = 0; rc == B2_OK && step < req->max_new_tokens; step++) {
        if (cancel && *cancel) {
            finish = B2_FINISH_CANCELLED;
            break;
        }
        if (is_stop(*req, next)) {
            finish = B2_FINISH_STOP_TOKEN;
            break;
        }
        if (cb) cb(user, 0, 0, next, step);
        gen.push_back(next);
        if (step + 1 == req->max_new_tokens) break;
        const int32_t feed = next;
        rc = forward_evicting(pc, cache, &feed, 1, &next);
    }
    if (rc != B2_OK) {
        b2_cache_free(cache);
        return rc;
    }
    if (cb) cb(user, 0, 1, finish, (int32_t)gen.size());
    if (out) {
        out->n_tokens = (int32_t)gen.size();
        out->finish_reason = finish;
        if (out->tokens)
            for (size_t i = 0; i < gen.size() && (int32_t)i < out->capacity; i++) out->tokens[i] = gen[i];
    }
    // store (:118-131): prompt + generated with the cache that now holds their KV (all but the last sampled token)
    PrefixEntry e;
    e.tokens.assign(req->prompt_ids, req->prompt_ids + n_prompt);
    e.tokens.insert(e.tokens.end(), gen.begin(), gen.end());
    e.cache = cache;
    e.used = ++pc->clock;
    for (size_t i = pc->entries.size(); i-- > 0;) {  // a stored sequence that is a prefix of the new one is subsumed
        const PrefixEntry& o = pc->entries[i];
        if (o.tokens.size() <= e.tokens.size() && std::equal(o.tokens.begin(), o.tokens.end(), e.tokens.begin())) pc->drop(i);
    }
    pc->entries.push_back(std::move(e));
    while ((int)pc->entries.size() > pc->capacity) pc->evict_lru();
    return B2_OK;
}

}  // extern "C"
