// CPU oracle (test infrastructure): the decoder forward, the scheduler policy and the two
// generation loops, restated from the reference.
#pragma once
#include <cstdint>
#include <functional>
#include <memory>
#include <string>
#include <vector>

#include "orc_paging.h"

namespace orc {

struct ModelCfg {
    int layers = 0, hidden = 0, heads = 0, kv_heads = 0, head_dim = 0, inter = 0, vocab = 0;
    float eps = 1e-5f, theta = 500000.f;
    int rope_kind = 0;  // 0 standard, 1 llama3
    float rope_factor = 1.f, rope_low = 1.f, rope_high = 4.f, rope_orig = 8192.f;
    int qk_norm = 0;     // Qwen3 per-head q/k RMSNorm
    int quant_bits = 0;  // 0 dense, 4, 8
    int group = 64;
    int f32_mode = 0;    // 1: no bf16 rounding anywhere (weights f32)
    int sum_order = 0;   // projections: 0 = one accumulator in index order; 1 = four quarter sums, (s0+s1)+(s2+s3)
};

// A projection / dense matrix [out, in].
struct Mat {
    int out = 0, in = 0, bits = 0, group = 64;
    std::vector<uint16_t> w;       // dense bf16
    std::vector<float> wf;         // dense f32 (f32_mode)
    std::vector<uint32_t> packed;  // quantized codes
    std::vector<uint16_t> scales, biases;
};

struct Layer {
    std::vector<uint16_t> input_ln, post_ln, q_norm, k_norm;
    std::vector<float> input_ln_f, post_ln_f;
    Mat q, k, v, o, gate, up, down;
};

struct Model {
    ModelCfg cfg;
    Mat embed, lm_head;
    std::vector<uint16_t> norm;
    std::vector<float> norm_f;
    std::vector<Layer> layers;
    std::vector<float> inv_freq;
};

struct SeqIn {
    const int32_t* ids;
    int n;
    KvCacheBase* cache;
    int offset;
};

// Ragged-batch forward: every sequence contributes n tokens at positions offset..offset+n-1; returns
// last-position logits per sequence, [num_seqs, vocab] (bf16-rounded values unless f32_mode; the
// unrounded f32 accumulations are written to logits_f32 when non-null).
void forward_batch(const Model& m, std::vector<SeqIn>& seqs, std::vector<float>& logits, std::vector<float>* logits_f32);

// Scheduler — core_llm::schedule::Scheduler as seen from its call sites
// (src/decode/continuous.rs:147-151, :247-252, :306-340; src/decode/batch.rs:110-115, :175-176).
enum Finish { FIN_NONE = -1, FIN_STOP = 0, FIN_LENGTH = 1 };
struct Scheduler {
    struct Seq {
        std::vector<int32_t> prompt, stop, generated;
        size_t max_new;
        int finish = FIN_NONE;
    };
    std::vector<Seq> seqs;
    size_t admit(const std::vector<int32_t>& prompt, size_t max_new, const std::vector<int32_t>& stop) {
        Seq s;
        s.prompt = prompt;
        s.stop = stop;
        s.max_new = max_new;
        if (max_new == 0) s.finish = FIN_LENGTH;  // zero budget retires at admission
        seqs.push_back(std::move(s));
        return seqs.size() - 1;
    }
    bool is_active(size_t id) const { return seqs[id].finish == FIN_NONE; }
    int record(size_t id, int32_t tok) {
        Seq& s = seqs[id];
        for (int32_t t : s.stop)
            if (t == tok) {
                s.finish = FIN_STOP;  // stop token excluded from the output
                return FIN_STOP;
            }
        s.generated.push_back(tok);
        if (s.generated.size() >= s.max_new) {
            s.finish = FIN_LENGTH;  // budget reached: token included
            return FIN_LENGTH;
        }
        return FIN_NONE;
    }
    size_t offset(size_t id) const { return seqs[id].prompt.size() + seqs[id].generated.size(); }
};

// Event record: kind 0 = Token{id, step}, kind 1 = Done{reason, generated}
// reasons follow FinishReason (src/decode/stream.rs:31-46): 0 StopToken, 1 MaxTokens, 2 Cancelled, 3 Stopped.
struct Event {
    int32_t req, kind, a, b;
};

struct Request {
    std::vector<int32_t> prompt, stop;
    size_t max_new;
};

}  // namespace orc
