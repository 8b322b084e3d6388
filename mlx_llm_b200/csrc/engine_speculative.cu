// Prompt-lookup (n-gram) speculative decoding on the paged cache.
//
// b2_generate_prompt_lookup <- generate_prompt_lookup (src/decode/speculative.rs:73-171): one prefill, then per
// step the target runs ONCE over [cur, draft_1 .. draft_k] with the logits of every position (the chunked-prefill
// kernels take the k+1 rows like any other chunk), the longest draft prefix the target's own greedy choices agree
// with is accepted plus one bonus token (decide_greedy, :301-326), and the rejected positions are rolled back with
// KvCache::truncate (:145; src/primitives/paged_kv_cache.rs:422-485 -- on real pages here).
//
// The proposer restates core_llm::speculative::ngram_propose as the reference describes it (speculative.rs:3-8:
// "copies the continuation that followed the most recent earlier occurrence of the current trailing n-gram", longest
// n-gram first); its source is not part of the reference tree, so ties and edge cases are this library's choice:
// the most recent earlier occurrence wins, the copy stops at the end of the history, no match proposes nothing.
// With num_draft = 0 the verify is a single-token forward and the loop is the plain greedy loop (the reference's
// exactness gate, tests/speculative.rs:52-66).  Sampling with temperature is not on the device path.
#include <algorithm>

#include "engine.h"

namespace {

bool is_stop(const b2_request& r, int32_t tok) {
    for (int i = 0; i < r.n_stop; i++)
        if (r.stop_tokens[i] == tok) return true;
    return false;
}

// Up to k tokens that followed the most recent earlier occurrence of the trailing n-gram, n = max_ngram .. 1.
std::vector<int32_t> ngram_propose(const std::vector<int32_t>& h, int max_ngram, int k) {
    std::vector<int32_t> out;
    const int len = (int)h.size();
    if (k <= 0 || len < 2) return out;
    for (int n = std::min(max_ngram, len - 1); n >= 1; n--) {
        const int32_t* pat = h.data() + len - n;
        for (int i = len - n - 1; i >= 0; i--) {  // start of an earlier occurrence, most recent first
            if (!std::equal(pat, pat + n, h.data() + i)) continue;
            for (int j = i + n; j < len && (int)out.size() < k; j++) out.push_back(h[j]);
            return out;
        }
    }
    return out;
}

}  // namespace

extern "C" int32_t b2_ngram_propose(const int32_t* history, int32_t n_history, int32_t max_ngram, int32_t k, int32_t* out, int32_t* n_out) {
    B2_REQUIRE(history && out && n_out && n_history >= 0, B2_ERR_MSG, "b2_ngram_propose: null argument");
    const std::vector<int32_t> h(history, history + n_history);
    const std::vector<int32_t> d = ngram_propose(h, max_ngram, k);
    for (size_t i = 0; i < d.size(); i++) out[i] = d[i];
    *n_out = (int32_t)d.size();
    return B2_OK;
}

extern "C" int32_t b2_generate_prompt_lookup(b2_model* m, const b2_request* req, const b2_speculative_config* spec, const volatile int32_t* cancel,
                                             b2_event_cb cb, void* user, b2_gen_output* out, b2_speculative_stats* stats_out) {
    B2_REQUIRE(m && req && spec, B2_ERR_MSG, "b2_generate_prompt_lookup: null argument");
    B2_REQUIRE(req->n_prompt > 0 && req->prompt_ids, B2_ERR_MSG, "generate_prompt_lookup: empty prompt");
    B2_REQUIRE(spec->max_ngram >= 1 && spec->num_draft >= 0 && spec->num_draft <= 64, B2_ERR_MSG,
               "generate_prompt_lookup: max_ngram must be >= 1 and num_draft within 0..64");
    B2_REQUIRE(req->sampling.temperature <= 0.f && (req->sampling.repetition_penalty == 1.f || req->sampling.repetition_penalty == 0.f),
               B2_ERR_UNSUPPORTED, "only greedy sampling (temperature <= 0, repetition_penalty == 1) runs on the device path");
    if (cancel && *cancel) return b2_fail(B2_ERR_CANCELED, "canceled before inference");
    b2_speculative_stats st{};
    std::vector<int32_t> gen;
    int finish = B2_FINISH_MAX_TOKENS;
    auto done = [&]() {
        if (cb) cb(user, 0, 1, finish, (int32_t)gen.size());
        if (out) {
            out->n_tokens = (int32_t)gen.size();
            out->finish_reason = finish;
            if (out->tokens)
                for (size_t i = 0; i < gen.size() && (int32_t)i < out->capacity; i++) out->tokens[i] = gen[i];
        }
        if (stats_out) *stats_out = st;
        return B2_OK;
    };
    if (req->max_new_tokens <= 0) return done();

    const int bs = 16;
    const int max_blocks = (req->n_prompt + req->max_new_tokens + spec->num_draft + 1 + bs - 1) / bs + 1;
    b2_pool* pool = nullptr;
    B2_CHECK(b2_pool_new(m->ctx, m, bs, max_blocks, 1, max_blocks, &pool));
    b2_cache* cache = nullptr;
    int32_t rc = b2_cache_new(pool, &cache);
    std::vector<int32_t> history(req->prompt_ids, req->prompt_ids + req->n_prompt), verify, argmax;
    int32_t cur = 0;
    bool stopped_early = false;
    if (rc == B2_OK) {  // prefill: the first token is sampled as usual
        std::vector<SeqStep> s{SeqStep{cache, req->prompt_ids, req->n_prompt, true}};
        rc = b2_engine_forward(m, s, nullptr, &cur);
        st.forwards++;
    }
    if (rc == B2_OK) {
        if (is_stop(*req, cur)) {
            finish = B2_FINISH_STOP_TOKEN;
            stopped_early = true;
        } else {
            if (cb) cb(user, 0, 0, cur, 0);
            gen.push_back(cur);
            history.push_back(cur);
        }
    }
    while (rc == B2_OK && !stopped_early && (int)gen.size() < req->max_new_tokens) {
        if (cancel && *cancel) {
            finish = B2_FINISH_CANCELLED;
            break;
        }
        // drafts: capped so that the commit (accepted + 1 bonus) cannot overrun the budget
        const int remaining = req->max_new_tokens - (int)gen.size();
        const int k_cap = std::min(spec->num_draft, std::max(remaining - 1, 0));
        const std::vector<int32_t> drafts = k_cap > 0 ? ngram_propose(history, spec->max_ngram, k_cap) : std::vector<int32_t>();
        st.proposed += (int64_t)drafts.size();
        verify.assign(1, cur);
        verify.insert(verify.end(), drafts.begin(), drafts.end());
        const int base = cache->len;
        argmax.assign(verify.size(), 0);
        SeqStep step{cache, verify.data(), (int)verify.size(), true};
        step.all_positions = true;
        std::vector<SeqStep> s{step};
        rc = b2_engine_forward(m, s, nullptr, argmax.data());  // argmax[i] = the target's choice after verify[i]
        if (rc != B2_OK) break;
        st.forwards++;
        int accepted = 0;
        while (accepted < (int)drafts.size() && argmax[accepted] == drafts[accepted]) accepted++;  // accept_greedy_run
        st.accepted += accepted;
        rc = b2_cache_truncate(cache, base + 1 + accepted);  // keep cur + the accepted drafts
        if (rc != B2_OK) break;
        bool end = false;
        for (int i = 0; i <= accepted && !end; i++) {  // the accepted drafts, then the bonus token
            const int32_t t = i < accepted ? drafts[i] : argmax[accepted];
            if (is_stop(*req, t)) {
                finish = B2_FINISH_STOP_TOKEN;
                end = true;
                break;
            }
            if (cb) cb(user, 0, 0, t, (int32_t)gen.size());
            gen.push_back(t);
            history.push_back(t);
            cur = t;
            if ((int)gen.size() >= req->max_new_tokens) {
                finish = B2_FINISH_MAX_TOKENS;
                end = true;
            }
        }
        if (end) break;
    }
    if (cache) b2_cache_free(cache);
    b2_pool_free(pool);
    if (rc != B2_OK) return rc;
    return done();
}
