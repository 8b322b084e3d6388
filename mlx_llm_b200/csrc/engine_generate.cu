// Generation loops: the single-sequence loop and iteration-level continuous batching.
//
// b2_generate            <- generate / decode_loop      (src/decode/stream.rs:113-121, :259-327)
// b2_generate_continuous <- generate_continuous         (src/decode/continuous.rs:117-340)
// b2_continuous_*        the same loop, one iteration at a time (benchmarks time K iterations)
// The admission / retirement policy restates core_llm::schedule::Scheduler as its call sites use it
// (continuous.rs:147-151, :247-252, :306-340): a stop token retires a sequence and is excluded from
// its output; a filled budget retires it including the token; a zero budget retires at admission.
#include <algorithm>
#include <chrono>
#include <cstring>
#include <deque>
#include <memory>
#include <thread>

#include "engine.h"

namespace {

struct SchedSeq {
    std::vector<int32_t> generated;
    int finish = -1;  // -1 active, else B2_FINISH_STOP_TOKEN / B2_FINISH_MAX_TOKENS
};

struct Lane {
    int req = 0;
    b2_cache* cache = nullptr;
    int32_t next_token = 0;
    int prefill_pos = 0;  // prompt tokens already in the cache
    int64_t page_budget = 0;
};

bool is_stop(const b2_request& r, int32_t tok) {
    for (int i = 0; i < r.n_stop; i++)
        if (r.stop_tokens[i] == tok) return true;
    return false;
}

int32_t check_greedy(const b2_request& r) {
    // sample()'s device fast path (src/primitives/sampler.rs:105-115) is the only sampler on this path
    B2_REQUIRE(r.sampling.temperature <= 0.f && (r.sampling.repetition_penalty == 1.f || r.sampling.repetition_penalty == 0.f),
               B2_ERR_UNSUPPORTED, "only greedy sampling (temperature <= 0, repetition_penalty == 1) runs on the device path");
    return B2_OK;
}

void fill_output(b2_gen_output* o, const std::vector<int32_t>& gen, int reason) {
    if (!o) return;
    o->n_tokens = (int32_t)gen.size();
    o->finish_reason = reason;
    if (o->tokens)
        for (size_t i = 0; i < gen.size() && (int32_t)i < o->capacity; i++) o->tokens[i] = gen[i];
}

}  // namespace

// The continuous-batching loop as an object: construct, step() until done, finish().
struct b2_continuous {
    b2_model* m = nullptr;
    const b2_request* reqs = nullptr;
    int n = 0;
    b2_continuous_config cfg{};
    const volatile int32_t* cancel = nullptr;
    b2_event_cb cb = nullptr;
    void* user = nullptr;
    b2_pool* pool = nullptr;
    std::vector<SchedSeq> sched;
    std::vector<Lane> lanes;
    int next_req = 0;
    int64_t committed_pages = 0, max_pages = 0;
    int bs = 16;
    bool chunked = false, throughput = false, cancelled = false, finished = false;
    b2_run_stats st{};
    double dev0 = 0;
    int64_t h2d0 = 0, d2h0 = 0, launch0 = 0;
    std::chrono::steady_clock::time_point t_start;
    std::vector<SeqStep> batch;
    std::vector<int> batch_lane;
    std::vector<int32_t> toks;
    // Serving mode (b2_continuous_open / _submit): requests arrive while the loop runs, so the engine keeps its own copy
    // of each (prompt and stop tokens included); `reqs` / `n` then follow `own_reqs`.
    bool open = false;
    std::vector<b2_request> own_reqs;
    std::deque<std::vector<int32_t>> own_ids;
    std::vector<char> req_cancel;  // per-request cancel / halt: 0 none, else the finish reason to report
    int max_blocks_row = 0;

    double now_s() const { return std::chrono::duration<double>(std::chrono::steady_clock::now() - t_start).count(); }
    int64_t pages_of(const b2_request& r) const { return (int64_t)((r.n_prompt + std::max(r.max_new_tokens, 0) + bs - 1) / bs); }
    void emit(int req, int kind, int a, int b) {
        if (cb) cb(user, req, kind, a, b);
    }
    // record_token (continuous.rs:306-340); returns true when the lane keeps decoding
    bool record(Lane& lane, int32_t tok) {
        SchedSeq& s = sched[lane.req];
        const b2_request& r = reqs[lane.req];
        if (is_stop(r, tok)) {
            s.finish = B2_FINISH_STOP_TOKEN;
            emit(lane.req, 1, B2_FINISH_STOP_TOKEN, (int)s.generated.size());
            return false;
        }
        s.generated.push_back(tok);
        st.decode_tokens++;
        emit(lane.req, 0, tok, (int)s.generated.size() - 1);
        if ((int)s.generated.size() >= r.max_new_tokens) {
            s.finish = B2_FINISH_MAX_TOKENS;
            emit(lane.req, 1, B2_FINISH_MAX_TOKENS, (int)s.generated.size());
            return false;
        }
        lane.next_token = tok;
        return true;
    }
    void retire(Lane& lane) {
        committed_pages -= lane.page_budget;
        b2_cache_free(lane.cache);
        lane.cache = nullptr;
    }
    int32_t forward(std::vector<SeqStep>& seqs, int32_t* argmax) {
        st.steps++;
        for (auto& s : seqs)
            if (s.n > 1 || s.cache->len == 0) st.prefill_tokens += s.n;
        return b2_engine_forward(m, seqs, nullptr, argmax);
    }
    // admit request ri: 1 lane created, 0 retired immediately, -1 must wait (arrival time or page
    // budget), -2 error (rc set)
    int admit(int ri, int32_t& rc) {
        const b2_request& r = reqs[ri];
        if (r.arrival_s > 0 && now_s() < r.arrival_s) return -1;
        if (!req_cancel.empty() && req_cancel[ri] && sched[ri].finish == -1) {  // cancelled while it waited
            sched[ri].finish = req_cancel[ri];
            emit(ri, 1, req_cancel[ri], 0);
            return 0;
        }
        if (sched[ri].finish != -1) {  // zero budget: terminal event, no prefill (continuous.rs:247-252)
            emit(ri, 1, B2_FINISH_MAX_TOKENS, 0);
            return 0;
        }
        const int64_t need = pages_of(r) + 1;
        if (committed_pages + need > max_pages) {
            if (lanes.empty()) {
                rc = b2_fail(B2_ERR_OOM_PAGES, "generate_continuous: request " + std::to_string(ri) + " does not fit the page pool");
                return -2;
            }
            return -1;
        }
        Lane lane;
        lane.req = ri;
        lane.page_budget = need;
        rc = b2_cache_new(pool, &lane.cache);  // PagedKvCache::with_pool (:254)
        if (rc != B2_OK) return -2;
        committed_pages += need;
        if (!chunked) {
            // whole-prompt batch-1 prefill at admission, first token sampled from it (:255-269)
            std::vector<SeqStep> s{SeqStep{lane.cache, r.prompt_ids, r.n_prompt, true}};
            int32_t tok = 0;
            rc = forward(s, &tok);
            if (rc != B2_OK) {
                retire(lane);
                return -2;
            }
            lane.prefill_pos = r.n_prompt;
            if (!record(lane, tok)) {
                retire(lane);
                return 0;
            }
        }
        lanes.push_back(lane);
        st.peak_concurrent = std::max<int64_t>(st.peak_concurrent, (int64_t)lanes.size());
        return 1;
    }
    int32_t fill_slots() {
        int32_t rc = B2_OK;
        while (rc == B2_OK && (int)lanes.size() < cfg.max_batch && next_req < n) {
            const int a = admit(next_req, rc);
            if (a == -1 || a == -2) break;
            next_req++;
        }
        return rc;
    }
    bool has_work() const { return !lanes.empty() || next_req < n; }

    // One iteration of the loop (continuous.rs:167-190).  *done is set when nothing is left.
    int32_t step(bool* done) {
        *done = false;
        if (finished || !has_work()) {
            *done = true;
            return B2_OK;
        }
        if (cancel && *cancel) {
            cancelled = true;
            *done = true;
            return B2_OK;
        }
        if (!req_cancel.empty()) {  // requests halted one by one (a stop string matched, a client went away)
            std::vector<Lane> keep;
            for (auto& l : lanes) {
                if (req_cancel[l.req]) {
                    sched[l.req].finish = req_cancel[l.req];
                    emit(l.req, 1, req_cancel[l.req], (int)sched[l.req].generated.size());
                    retire(l);
                } else {
                    keep.push_back(l);
                }
            }
            lanes.swap(keep);
        }
        if (chunked || lanes.empty()) B2_CHECK(fill_slots());  // lanes can be empty while requests have yet to arrive
        if (lanes.empty()) {
            if (next_req >= n) {
                *done = true;
                return B2_OK;
            }
            const double wait = reqs[next_req].arrival_s - now_s();  // nothing to run until the next arrival
            if (wait > 0) std::this_thread::sleep_for(std::chrono::duration<double>(std::min(wait, 0.002)));
            return B2_OK;
        }
        // assemble the step: every decoding lane feeds one token; prefill chunks fill the budget
        batch.clear();
        batch_lane.clear();
        int budget = chunked ? cfg.prefill_chunk_tokens : 0;
        for (size_t i = 0; i < lanes.size(); i++) {
            Lane& l = lanes[i];
            const b2_request& r = reqs[l.req];
            if (l.prefill_pos >= r.n_prompt) {
                batch.push_back(SeqStep{l.cache, &l.next_token, 1, true});
                batch_lane.push_back((int)i);
            } else if (budget > 0) {
                const int take = std::min(budget, r.n_prompt - l.prefill_pos);
                budget -= take;
                batch.push_back(SeqStep{l.cache, r.prompt_ids + l.prefill_pos, take, l.prefill_pos + take == r.n_prompt});
                batch_lane.push_back((int)i);
            }
        }
        toks.assign(batch.size(), 0);
        if (throughput) {
            B2_CHECK(forward(batch, toks.data()));
        } else {
            // Exact: every sequence is its own forward (continuous.rs:277-285)
            size_t k = 0;
            for (size_t i = 0; i < batch.size(); i++) {
                std::vector<SeqStep> one{batch[i]};
                int32_t tok = 0;
                B2_CHECK(forward(one, &tok));
                if (batch[i].want_logits) toks[k++] = tok;
            }
        }
        std::vector<char> gone(lanes.size(), 0);
        size_t k = 0;
        for (size_t i = 0; i < batch.size(); i++) {
            Lane& l = lanes[batch_lane[i]];
            if (l.prefill_pos < reqs[l.req].n_prompt) l.prefill_pos += batch[i].n;
            if (!batch[i].want_logits) continue;
            if (!record(l, toks[k++])) gone[batch_lane[i]] = 1;
        }
        std::vector<Lane> survivors;
        for (size_t i = 0; i < lanes.size(); i++) {
            if (gone[i])
                retire(lanes[i]);
            else
                survivors.push_back(lanes[i]);
        }
        lanes.swap(survivors);
        if (!chunked) B2_CHECK(fill_slots());  // admit-on-retire (continuous.rs:184-189)
        *done = !has_work();
        return B2_OK;
    }

    void snapshot_stats() {
        b2_pool_stats_t ps{};
        b2_pool_stats(pool, &ps);
        st.peak_live_blocks = ps.peak_live_blocks;
        st.device_ms = m->device_ms - dev0;
        st.wall_ms = now_s() * 1e3;
        st.h2d_bytes = m->h2d_bytes - h2d0;
        st.d2h_bytes = m->d2h_bytes - d2h0;
        st.kernel_launches = m->ctx->launches - launch0;
    }

    // Cancel epilogue + outputs (continuous.rs:198-228).
    void finish(b2_gen_output* outs, b2_run_stats* stats) {
        if (!finished) {
            if (cancelled) {
                // exactly one Done for every request still decoding or still waiting
                for (auto& l : lanes) emit(l.req, 1, B2_FINISH_CANCELLED, (int)sched[l.req].generated.size());
                for (int ri = next_req; ri < n; ri++)
                    emit(ri, 1, sched[ri].finish == B2_FINISH_MAX_TOKENS ? B2_FINISH_MAX_TOKENS : B2_FINISH_CANCELLED, 0);
            }
            snapshot_stats();
            for (auto& l : lanes) retire(l);
            lanes.clear();
            finished = true;
        }
        if (stats) *stats = st;
        if (outs)
            for (int i = 0; i < n; i++) fill_output(&outs[i], sched[i].generated, sched[i].finish == -1 ? B2_FINISH_CANCELLED : sched[i].finish);
    }
};

extern "C" {

int32_t b2_continuous_new(b2_model* m, const b2_request* reqs, int32_t n, const b2_continuous_config* cfg,
                          const volatile int32_t* cancel, b2_event_cb cb, void* user, b2_continuous** out) {
    B2_REQUIRE(m && cfg && out, B2_ERR_MSG, "b2_generate_continuous: null argument");
    B2_REQUIRE(n > 0 && reqs, B2_ERR_MSG, "generate_continuous: no requests");
    B2_REQUIRE(cfg->max_batch > 0, B2_ERR_MSG, "generate_continuous: max_batch must be > 0");
    B2_REQUIRE(cfg->block_size > 0, B2_ERR_MSG, "generate_continuous: block_size must be > 0");
    for (int i = 0; i < n; i++) {
        B2_REQUIRE(reqs[i].n_prompt > 0 && reqs[i].prompt_ids, B2_ERR_MSG,
                   "generate_continuous: request " + std::to_string(i) + " has an empty prompt");
        B2_CHECK(check_greedy(reqs[i]));
    }
    if (cancel && *cancel) return b2_fail(B2_ERR_CANCELED, "canceled before inference");

    auto e = std::make_unique<b2_continuous>();
    e->m = m;
    e->reqs = reqs;
    e->n = n;
    e->cfg = *cfg;
    e->cancel = cancel;
    e->cb = cb;
    e->user = user;
    e->bs = cfg->block_size;
    e->chunked = cfg->prefill_chunk_tokens > 0;
    e->throughput = cfg->exactness != 0;
    int max_blocks = cfg->max_blocks_per_seq;
    if (max_blocks <= 0)
        for (int i = 0; i < n; i++) max_blocks = (int)std::max<int64_t>(max_blocks, e->pages_of(reqs[i]) + 1);
    int64_t max_pages = cfg->max_pages;
    if (max_pages <= 0) {
        // room for the max_batch largest requests at full length
        std::vector<int64_t> need(n);
        for (int i = 0; i < n; i++) need[i] = e->pages_of(reqs[i]) + 1;
        std::sort(need.begin(), need.end(), std::greater<int64_t>());
        for (int i = 0; i < n && i < cfg->max_batch; i++) max_pages += need[i];
    }
    e->max_pages = max_pages;
    B2_CHECK(b2_pool_new(m->ctx, m, e->bs, max_pages, cfg->max_batch, max_blocks, &e->pool));  // BlockPool::new (:142)
    e->sched.resize(n);
    for (int i = 0; i < n; i++)
        if (reqs[i].max_new_tokens <= 0) e->sched[i].finish = B2_FINISH_MAX_TOKENS;  // retired at admission
    e->dev0 = m->device_ms;
    e->h2d0 = m->h2d_bytes;
    e->d2h0 = m->d2h_bytes;
    e->launch0 = m->ctx->launches;
    e->t_start = std::chrono::steady_clock::now();
    int32_t rc = e->fill_slots();  // initial fill (continuous.rs:157-162)
    if (rc != B2_OK) {
        e->finish(nullptr, nullptr);
        b2_pool_free(e->pool);
        return rc;
    }
    *out = e.release();
    return B2_OK;
}

int32_t b2_continuous_open(b2_model* m, const b2_continuous_config* cfg, b2_event_cb cb, void* user, b2_continuous** out) {
    B2_REQUIRE(m && cfg && out, B2_ERR_MSG, "b2_continuous_open: null argument");
    B2_REQUIRE(cfg->max_batch > 0 && cfg->block_size > 0, B2_ERR_MSG, "b2_continuous_open: max_batch and block_size must be > 0");
    B2_REQUIRE(cfg->max_pages > 0 && cfg->max_blocks_per_seq > 0, B2_ERR_MSG,
               "b2_continuous_open: max_pages and max_blocks_per_seq must be given (there are no requests to size the pool from)");
    auto e = std::make_unique<b2_continuous>();
    e->m = m;
    e->cfg = *cfg;
    e->cb = cb;
    e->user = user;
    e->bs = cfg->block_size;
    e->chunked = cfg->prefill_chunk_tokens > 0;
    e->throughput = cfg->exactness != 0;
    e->open = true;
    e->max_pages = cfg->max_pages;
    e->max_blocks_row = cfg->max_blocks_per_seq;
    B2_CHECK(b2_pool_new(m->ctx, m, e->bs, cfg->max_pages, cfg->max_batch, cfg->max_blocks_per_seq, &e->pool));
    e->dev0 = m->device_ms;
    e->h2d0 = m->h2d_bytes;
    e->d2h0 = m->d2h_bytes;
    e->launch0 = m->ctx->launches;
    e->t_start = std::chrono::steady_clock::now();
    *out = e.release();
    return B2_OK;
}

int32_t b2_continuous_submit(b2_continuous* e, const b2_request* req, int32_t* id_out) {
    B2_REQUIRE(e && req && id_out, B2_ERR_MSG, "b2_continuous_submit: null argument");
    B2_REQUIRE(e->open && !e->finished, B2_ERR_MSG, "b2_continuous_submit: the engine was not opened for submissions (b2_continuous_open) or has finished");
    B2_REQUIRE(req->n_prompt > 0 && req->prompt_ids, B2_ERR_MSG, "b2_continuous_submit: empty prompt");
    B2_CHECK(check_greedy(*req));
    const int64_t need = e->pages_of(*req) + 1;
    B2_REQUIRE(need <= e->max_blocks_row && need <= e->max_pages, B2_ERR_OOM_PAGES,
               "b2_continuous_submit: prompt + max_new_tokens needs " + std::to_string(need) + " pages, more than a block-table row (" +
                   std::to_string(e->max_blocks_row) + ") or the pool (" + std::to_string(e->max_pages) + ") holds");
    b2_request r = *req;
    e->own_ids.emplace_back(req->prompt_ids, req->prompt_ids + req->n_prompt);
    r.prompt_ids = e->own_ids.back().data();
    e->own_ids.emplace_back(req->stop_tokens, req->stop_tokens + (req->stop_tokens ? req->n_stop : 0));
    r.stop_tokens = e->own_ids.back().data();
    r.n_stop = (int32_t)e->own_ids.back().size();
    r.arrival_s = 0;  // it has arrived
    e->own_reqs.push_back(r);
    e->reqs = e->own_reqs.data();
    e->n = (int)e->own_reqs.size();
    e->sched.emplace_back();
    if (r.max_new_tokens <= 0) e->sched.back().finish = B2_FINISH_MAX_TOKENS;  // retired at admission
    e->req_cancel.push_back(0);
    *id_out = e->n - 1;
    return B2_OK;
}

int32_t b2_continuous_halt(b2_continuous* e, int32_t id, int32_t finish_reason) {
    B2_REQUIRE(e, B2_ERR_MSG, "b2_continuous_halt: null engine");
    B2_REQUIRE(id >= 0 && id < e->n, B2_ERR_MSG, "b2_continuous_halt: no such request");
    B2_REQUIRE(finish_reason == B2_FINISH_CANCELLED || finish_reason == B2_FINISH_STOPPED, B2_ERR_MSG,
               "b2_continuous_halt: the reason must be B2_FINISH_CANCELLED or B2_FINISH_STOPPED");
    if (e->req_cancel.size() < (size_t)e->n) e->req_cancel.resize(e->n, 0);
    if (e->sched[id].finish == -1 && !e->req_cancel[id]) e->req_cancel[id] = (char)finish_reason;
    return B2_OK;
}

int32_t b2_continuous_result(b2_continuous* e, int32_t id, int32_t* tokens_out, int32_t capacity, int32_t* n_out, int32_t* finish_out) {
    B2_REQUIRE(e && n_out && finish_out, B2_ERR_MSG, "b2_continuous_result: null argument");
    B2_REQUIRE(id >= 0 && id < e->n, B2_ERR_MSG, "b2_continuous_result: no such request");
    const SchedSeq& s = e->sched[id];
    *n_out = (int32_t)s.generated.size();
    *finish_out = s.finish;
    if (tokens_out)
        for (int i = 0; i < *n_out && i < capacity; i++) tokens_out[i] = s.generated[i];
    return B2_OK;
}

int32_t b2_continuous_step(b2_continuous* e, int32_t max_steps, int32_t* done_out, b2_run_stats* stats) {
    B2_REQUIRE(e, B2_ERR_MSG, "b2_continuous_step: null engine");
    B2_CUDA(cudaSetDevice(e->m->ctx->device));  // the serving thread may not be the one that built the model
    bool done = false;
    for (int i = 0; i < max_steps && !done; i++) B2_CHECK(e->step(&done));
    if (done_out) *done_out = done ? 1 : 0;
    if (stats) {
        e->snapshot_stats();
        *stats = e->st;
    }
    return B2_OK;
}

int32_t b2_continuous_finish(b2_continuous* e, b2_gen_output* outs, b2_run_stats* stats) {
    B2_REQUIRE(e, B2_ERR_MSG, "b2_continuous_finish: null engine");
    e->finish(outs, stats);
    return B2_OK;
}

int32_t b2_continuous_free(b2_continuous* e) {
    if (!e) return B2_OK;
    e->finish(nullptr, nullptr);
    b2_pool_free(e->pool);
    delete e;
    return B2_OK;
}

int32_t b2_generate_continuous(b2_model* m, const b2_request* reqs, int32_t n, const b2_continuous_config* cfg,
                               const volatile int32_t* cancel, b2_event_cb cb, void* user, b2_gen_output* outs, b2_run_stats* stats) {
    b2_continuous* e = nullptr;
    B2_CHECK(b2_continuous_new(m, reqs, n, cfg, cancel, cb, user, &e));
    int32_t rc = B2_OK;
    bool done = false;
    while (rc == B2_OK && !done) rc = e->step(&done);
    if (rc == B2_OK) e->finish(outs, stats);
    b2_continuous_free(e);
    return rc;
}

int32_t b2_generate(b2_model* m, const b2_request* req, const volatile int32_t* cancel, b2_event_cb cb, void* user, b2_gen_output* out) {
    B2_REQUIRE(m && req, B2_ERR_MSG, "b2_generate: null argument");
    B2_REQUIRE(req->n_prompt > 0 && req->prompt_ids, B2_ERR_MSG, "generate: empty prompt");
    B2_CHECK(check_greedy(*req));
    if (cancel && *cancel) return b2_fail(B2_ERR_CANCELED, "canceled before inference");
    const int bs = 16;
    const int max_blocks = (req->n_prompt + std::max(req->max_new_tokens, 0) + bs - 1) / bs + 1;
    b2_pool* pool = nullptr;
    B2_CHECK(b2_pool_new(m->ctx, m, bs, max_blocks, 1, max_blocks, &pool));
    b2_cache* cache = nullptr;
    int32_t rc = b2_cache_new(pool, &cache);
    std::vector<int32_t> gen;
    int finish = B2_FINISH_MAX_TOKENS;
    int32_t next = 0;
    if (rc == B2_OK) {
        std::vector<SeqStep> s{SeqStep{cache, req->prompt_ids, req->n_prompt, true}};
        rc = b2_engine_forward(m, s, nullptr, &next);
    }
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
        std::vector<SeqStep> s{SeqStep{cache, &feed, 1, true}};
        rc = b2_engine_forward(m, s, nullptr, &next);
    }
    if (rc == B2_OK) {
        if (cb) cb(user, 0, 1, finish, (int32_t)gen.size());
        fill_output(out, gen, finish);
    }
    if (cache) b2_cache_free(cache);
    b2_pool_free(pool);
    return rc;
}

}  // extern "C"
