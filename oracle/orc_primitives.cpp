// CPU oracle (test infrastructure): leaf arithmetic of the decode path.
// Each function names the reference code it restates (paths inside SceneWorks/mlx-llm).
#include <omp.h>

#include "oracle.h"
#include "orc_common.h"

#include <algorithm>
#include <cfloat>
#include <cmath>
#include <vector>

using namespace orc;

extern "C" {

// ---------------------------------------------------------------------------------------------
// SplitMix64 — src/primitives/sampler.rs:36-61; known answers at :300-305.
uint64_t orc_splitmix64_next(uint64_t* state) {
    SplitMix64 r(*state);
    uint64_t v = r.next_u64();
    *state = r.s;
    return v;
}
float orc_splitmix64_next_f32(uint64_t* state) {
    SplitMix64 r(*state);
    float v = r.next_f32();
    *state = r.s;
    return v;
}

void orc_f32_to_bf16(const float* in, uint16_t* out, int64_t n) {
    for (int64_t i = 0; i < n; i++) out[i] = f2bf(in[i]);
}
void orc_bf16_to_f32(const uint16_t* in, float* out, int64_t n) {
    for (int64_t i = 0; i < n; i++) out[i] = bf2f(in[i]);
}

// ---------------------------------------------------------------------------------------------
// RoPE inverse frequencies.
//   kind 0: Rope::standard  — src/primitives/rope.rs:42-52   inv[i] = 1 / theta^(2i/hd)  (f32 powf)
//   kind 1: Rope::llama3    — src/primitives/rope.rs:125-156 NTK-by-parts wavelength schedule
// Selection between them follows ModelConfig::build_rope (src/config.rs:551-581).
void orc_rope_inv_freq(int head_dim, float theta, int kind, float factor, float low_freq_factor,
                       float high_freq_factor, float original_context, float* out) {
    int half = head_dim / 2;
    const float two_pi = 2.0f * 3.14159265358979323846f;
    float low_wl = original_context / low_freq_factor;
    float high_wl = original_context / high_freq_factor;
    for (int i = 0; i < half; i++) {
        float inv = 1.0f / std::pow(theta, (float)(2 * i) / (float)head_dim);
        if (kind == 1) {
            float wavelen = two_pi / inv;
            if (wavelen > low_wl) {
                inv = inv / factor;
            } else if (wavelen < high_wl) {
                // unchanged
            } else {
                float smooth = (original_context / wavelen - low_freq_factor) / (high_freq_factor - low_freq_factor);
                inv = (1.0f - smooth) * inv / factor + smooth * inv;
            }
        }
        out[i] = inv;
    }
}

// cos/sin tables for explicit positions — Rope::cos_sin_at, src/primitives/rope.rs:183-208:
// angle = (pos as f32) * inv_freq (f32), table laid out cat(freqs, freqs), cos/sin evaluated in
// f32 and then cast to bf16.  Output [n, 2*half] each.
void orc_rope_cos_sin(const float* inv_freq, int half, const int32_t* pos, int n, uint16_t* cos_out, uint16_t* sin_out) {
    for (int p = 0; p < n; p++) {
        for (int i = 0; i < half; i++) {
            float ang = (float)pos[p] * inv_freq[i];
            uint16_t c = f2bf(std::cos(ang)), s = f2bf(std::sin(ang));
            cos_out[(size_t)p * 2 * half + i] = c;
            cos_out[(size_t)p * 2 * half + half + i] = c;
            sin_out[(size_t)p * 2 * half + i] = s;
            sin_out[(size_t)p * 2 * half + half + i] = s;
        }
    }
}

// NeoX rotate-half — apply_rope, src/primitives/rope.rs:360-393.  x is [n, heads, hd] bf16,
// cos/sin [n, hd] bf16.  Every MLX op rounds its result to bf16:
//   out = bf16( bf16(x*cos) + bf16(rot*sin) ),   rot = cat(-x2, x1).
void orc_apply_rope(uint16_t* x, const uint16_t* cos_t, const uint16_t* sin_t, int n, int heads, int hd) {
    int half = hd / 2;
    std::vector<float> row(hd);
    for (int p = 0; p < n; p++)
        for (int h = 0; h < heads; h++) {
            uint16_t* xr = x + ((size_t)p * heads + h) * hd;
            for (int d = 0; d < hd; d++) row[d] = bf2f(xr[d]);
            for (int d = 0; d < hd; d++) {
                float rot = d < half ? -row[d + half] : row[d - half];
                float a = rbf(row[d] * bf2f(cos_t[(size_t)p * hd + d]));
                float b = rbf(rot * bf2f(sin_t[(size_t)p * hd + d]));
                xr[d] = f2bf(a + b);
            }
        }
}

// ---------------------------------------------------------------------------------------------
// RMSNorm — nn.rs:35-37 -> mlx fast::rms_norm.  Parity unpinned inside MLX; this oracle defines:
// mean of squares accumulated in f32 in index order, y = bf16( x * (1/sqrt(ms+eps)) * w ).
void orc_rms_norm(const uint16_t* x, const uint16_t* w, float eps, int rows, int dim, uint16_t* out) {
    for (int r = 0; r < rows; r++) {
        const uint16_t* xr = x + (size_t)r * dim;
        float ss = 0.f;
        for (int d = 0; d < dim; d++) {
            float v = bf2f(xr[d]);
            ss += v * v;
        }
        float inv = 1.0f / std::sqrt(ss / (float)dim + eps);
        for (int d = 0; d < dim; d++) out[(size_t)r * dim + d] = f2bf(bf2f(xr[d]) * inv * bf2f(w[d]));
    }
}

// SwiGLU gate — LlamaMlp::forward, src/models/llama.rs:1040-1045: silu(g) = g*sigmoid(g), each op
// rounded to bf16, then multiplied by up and rounded again.
void orc_swiglu(const uint16_t* gate, const uint16_t* up, int64_t n, uint16_t* out) {
    for (int64_t i = 0; i < n; i++) {
        float g = bf2f(gate[i]);
        float s = rbf(1.0f / (1.0f + std::exp(-g)));
        float a = rbf(g * s);
        out[i] = f2bf(a * bf2f(up[i]));
    }
}

// bf16 elementwise add (residual): llama.rs:730-732.
void orc_add_bf16(const uint16_t* a, const uint16_t* b, int64_t n, uint16_t* out) {
    for (int64_t i = 0; i < n; i++) out[i] = f2bf(bf2f(a[i]) + bf2f(b[i]));
}

// Dense linear x @ W^T — nn.rs:26-33.  x [m,k] bf16, w [n,k] bf16; f32 accumulate in index order.
// out_f32 (pre-rounding) and/or out_bf16 may be null.
void orc_linear(const uint16_t* x, const uint16_t* w, int m, int n, int k, float* out_f32, uint16_t* out_bf16) {
    std::vector<float> xf((size_t)m * k);
    for (size_t i = 0; i < xf.size(); i++) xf[i] = bf2f(x[i]);
    const RowsT16 xt(xf.data(), m, k);
#pragma omp parallel for schedule(static)
    for (int j = 0; j < n; j++) {
        std::vector<float> wf(k);
        for (int d = 0; d < k; d++) wf[d] = bf2f(w[(size_t)j * k + d]);
        std::vector<float> acc(m);
        dots_in_order(xt, wf.data(), acc.data());
        for (int i = 0; i < m; i++) {
            if (out_f32) out_f32[(size_t)i * n + j] = acc[i];
            if (out_bf16) out_bf16[(size_t)i * n + j] = f2bf(acc[i]);
        }
    }
}

// Greedy argmax, ties -> lowest index — sampler.rs:221-241.  Operates on bf16 logits as the
// reference does (the logits tensor is bf16).
int32_t orc_argmax_bf16(const uint16_t* logits, int n) {
    int best = 0;
    float bv = -INFINITY;
    for (int i = 0; i < n; i++) {
        float v = bf2f(logits[i]);
        if (v > bv) {
            bv = v;
            best = i;
        }
    }
    return best;
}
int32_t orc_argmax_f32(const float* logits, int n) {
    int best = 0;
    float bv = -INFINITY;
    for (int i = 0; i < n; i++)
        if (logits[i] > bv) {
            bv = logits[i];
            best = i;
        }
    return best;
}

// ---------------------------------------------------------------------------------------------
// Group-wise affine quantization in the MLX format (src/primitives/quant.rs:20-82).
// Layout (from the reference's call sites and BASELINE config): codes along `in`, `32/bits` codes
// per u32, lowest bits first; one (scale, bias) pair per `group` consecutive inputs of a row.
//
// Decoder (spec of this build; "parity unpinned" against MLX's internal rounding):
//     w = bf16_rne( float(code) * float(scale) + float(bias) )       one rounding
void orc_unpack_codes(const uint32_t* packed, int64_t rows, int64_t in_dim, int bits, uint8_t* codes) {
    int per = 32 / bits;
    uint32_t mask = (1u << bits) - 1;
    int64_t words = in_dim / per;
    for (int64_t r = 0; r < rows; r++)
        for (int64_t j = 0; j < in_dim; j++) {
            uint32_t wv = packed[r * words + j / per];
            codes[r * in_dim + j] = (uint8_t)((wv >> ((j % per) * bits)) & mask);
        }
}

void orc_dequantize(const uint32_t* packed, const uint16_t* scales, const uint16_t* biases, int64_t rows,
                    int64_t in_dim, int group, int bits, uint16_t* out) {
    int per = 32 / bits;
    uint32_t mask = (1u << bits) - 1;
    int64_t words = in_dim / per, groups = in_dim / group;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; r++)
        for (int64_t j = 0; j < in_dim; j++) {
            uint32_t c = (packed[r * words + j / per] >> ((j % per) * bits)) & mask;
            float s = bf2f(scales[r * groups + j / group]), b = bf2f(biases[r * groups + j / group]);
            out[r * in_dim + j] = f2bf(std::fmaf((float)c, s, b));
        }
}

// Encoder — restates MLX's published affine quantizer (mlx/ops.cpp `quantize`, affine mode):
// per group, with n = 2^bits-1 and eps 1e-7:
//   scale = max((wmax-wmin)/n, eps); side = |wmin| > |wmax|; scale = side ? scale : -scale;
//   edge = side ? wmin : wmax; q0 = round(edge/scale); if q0 != 0 { scale = edge/q0; bias = edge }
//   else bias = 0;  code = clamp(round((w-bias)/scale), 0, n).
// Parity unpinned: the reference's tests only bound the round-trip error (quant.rs:91-125).
// Input w is bf16 (weights are cast to bf16 before quantize-on-load: llama.rs:97).
void orc_quantize(const uint16_t* w, int64_t rows, int64_t in_dim, int group, int bits, uint32_t* packed,
                  uint16_t* scales, uint16_t* biases) {
    int per = 32 / bits;
    int64_t words = in_dim / per, groups = in_dim / group;
    float n_bins = (float)((1 << bits) - 1);
    std::fill(packed, packed + rows * words, 0u);
    for (int64_t r = 0; r < rows; r++)
        for (int64_t g = 0; g < groups; g++) {
            const uint16_t* wg = w + r * in_dim + g * group;
            float wmin = INFINITY, wmax = -INFINITY;
            for (int j = 0; j < group; j++) {
                float v = bf2f(wg[j]);
                wmin = std::min(wmin, v);
                wmax = std::max(wmax, v);
            }
            float scale = std::max((wmax - wmin) / n_bins, 1e-7f);
            bool side = std::fabs(wmin) > std::fabs(wmax);
            scale = side ? scale : -scale;
            float edge = side ? wmin : wmax;
            float q0 = std::round(edge / scale);
            float bias = 0.f;
            if (q0 != 0.f) {
                scale = edge / q0;
                bias = edge;
            }
            // scales / biases are stored in the weight dtype (bf16); the codes are chosen against the
            // f32 values before that cast, as the published kernel does.
            scales[r * groups + g] = f2bf(scale);
            biases[r * groups + g] = f2bf(bias);
            for (int j = 0; j < group; j++) {
                float q = std::round((bf2f(wg[j]) - bias) / scale);
                q = std::min(std::max(q, 0.f), n_bins);
                int64_t col = g * group + j;
                packed[r * words + col / per] |= ((uint32_t)q) << ((col % per) * bits);
            }
        }
}

// Quantized matmul x @ dequant(W)^T — QuantizedLinear::forward, quant.rs:56-70.
// x [m,k] bf16; W packed [n, k*bits/32]; f32 accumulate against the bf16-rounded dequantized
// weight.  Parity unpinned against MLX's kernel-internal order; compared with a tolerance.
void orc_qmm(const uint16_t* x, const uint32_t* packed, const uint16_t* scales, const uint16_t* biases, int m, int n,
             int k, int group, int bits, float* out_f32, uint16_t* out_bf16) {
    int per = 32 / bits;
    uint32_t mask = (1u << bits) - 1;
    int64_t words = k / per, groups = k / group;
    std::vector<float> xf((size_t)m * k);
    for (size_t i = 0; i < xf.size(); i++) xf[i] = bf2f(x[i]);
    const RowsT16 xt(xf.data(), m, k);
#pragma omp parallel for schedule(dynamic, 16)
    for (int j = 0; j < n; j++) {
        std::vector<float> wf(k);
        for (int d = 0; d < k; d++) {
            uint32_t c = (packed[(int64_t)j * words + d / per] >> ((d % per) * bits)) & mask;
            wf[d] = rbf(std::fmaf((float)c, bf2f(scales[(int64_t)j * groups + d / group]),
                                  bf2f(biases[(int64_t)j * groups + d / group])));
        }
        std::vector<float> acc(m);
        dots_in_order(xt, wf.data(), acc.data());
        for (int i = 0; i < m; i++) {
            if (out_f32) out_f32[(size_t)i * n + j] = acc[i];
            if (out_bf16) out_bf16[(size_t)i * n + j] = f2bf(acc[i]);
        }
    }
}

// ---------------------------------------------------------------------------------------------
// Attention ground truth — host_attn_gqa, src/primitives/attention.rs:373-405: f64 accumulate,
// adjacent GQA grouping (kv head = q head / groups), causal mask aligned bottom-right
// (query i sees keys 0..=kl-ql+i).  q [h,ql,hd], k/v [hkv,kl,hd] f32, out [h,ql,hd] f32.
void orc_host_attn_gqa(const float* q, const float* k, const float* v, int h, int hkv, int ql, int kl, int hd,
                       float scale, int causal, float* out) {
    int groups = h / hkv;
    long offset = (long)kl - (long)ql;
#pragma omp parallel for schedule(dynamic)
    for (int head = 0; head < h; head++) {
        const float* qb = q + (size_t)head * ql * hd;
        const float* kb = k + (size_t)(head / groups) * kl * hd;
        const float* vb = v + (size_t)(head / groups) * kl * hd;
        std::vector<double> logits(kl);
        for (int i = 0; i < ql; i++) {
            int jmax = causal ? (int)(offset + i) : kl - 1;
            double m = -DBL_MAX;
            for (int j = 0; j <= jmax; j++) {
                double dot = 0;
                for (int d = 0; d < hd; d++) dot += (double)qb[(size_t)i * hd + d] * (double)kb[(size_t)j * hd + d];
                logits[j] = dot * (double)scale;
                m = std::max(m, logits[j]);
            }
            double denom = 0;
            for (int j = 0; j <= jmax; j++) {
                logits[j] = std::exp(logits[j] - m);
                denom += logits[j];
            }
            for (int d = 0; d < hd; d++) {
                double acc = 0;
                for (int j = 0; j <= jmax; j++) acc += logits[j] / denom * (double)vb[(size_t)j * hd + d];
                out[((size_t)head * ql + i) * hd + d] = (float)acc;
            }
        }
    }
}

// Paged attention over a ragged batch, same math as above with K/V read through block tables.
//   q           [T, hq, hd] bf16, tokens of sequence s are rows cu_seqlens[s]..cu_seqlens[s+1]
//   k/v pool    [pages, hkv, page, hd] bf16 (keys already rotated)
//   block_tables[num_seqs, max_blocks] physical page per logical block
//   ctx_lens    [num_seqs] cached length INCLUDING this step's tokens
// Query r of a sequence with q_len new tokens sees keys 0..=ctx-q_len+r (bottom-right causal,
// attention.rs:31-39).  f64 accumulate; out [T, hq, hd] f32 (not rounded).
void orc_paged_attention(const uint16_t* q, const uint16_t* kpool, const uint16_t* vpool, const int32_t* block_tables,
                         int max_blocks, const int32_t* cu_seqlens, const int32_t* ctx_lens, int num_seqs, int hq,
                         int hkv, int hd, int page, float scale, float* out) {
    int groups = hq / hkv;
#pragma omp parallel for collapse(2) schedule(dynamic)
    for (int s = 0; s < num_seqs; s++)
        for (int kvh = 0; kvh < hkv; kvh++) {
            int q0 = cu_seqlens[s], qn = cu_seqlens[s + 1] - q0, ctx = ctx_lens[s];
            if (qn <= 0) continue;
            // gather this head's keys/values once
            std::vector<float> kf((size_t)ctx * hd), vf((size_t)ctx * hd);
            for (int j = 0; j < ctx; j++) {
                size_t base = (((size_t)block_tables[(size_t)s * max_blocks + j / page] * hkv + kvh) * page + j % page) * hd;
                for (int d = 0; d < hd; d++) {
                    kf[(size_t)j * hd + d] = bf2f(kpool[base + d]);
                    vf[(size_t)j * hd + d] = bf2f(vpool[base + d]);
                }
            }
            std::vector<double> logits(ctx);
            for (int g = 0; g < groups; g++) {
                int head = kvh * groups + g;
                for (int r = 0; r < qn; r++) {
                    const uint16_t* qr = q + ((size_t)(q0 + r) * hq + head) * hd;
                    int jmax = ctx - qn + r;
                    double m = -DBL_MAX;
                    for (int j = 0; j <= jmax; j++) {
                        double dot = 0;
                        for (int d = 0; d < hd; d++) dot += (double)bf2f(qr[d]) * (double)kf[(size_t)j * hd + d];
                        logits[j] = dot * (double)scale;
                        m = std::max(m, logits[j]);
                    }
                    double denom = 0;
                    for (int j = 0; j <= jmax; j++) {
                        logits[j] = std::exp(logits[j] - m);
                        denom += logits[j];
                    }
                    float* o = out + ((size_t)(q0 + r) * hq + head) * hd;
                    for (int d = 0; d < hd; d++) {
                        double acc = 0;
                        for (int j = 0; j <= jmax; j++) acc += logits[j] * (double)vf[(size_t)j * hd + d];
                        o[d] = (float)(acc / denom);
                    }
                }
            }
        }
}

// Faster f32 variant of the decode case (one query per sequence) used as the timed CPU baseline
// of the paged-attention microbenchmark: f32 accumulate, OpenMP over (sequence, kv head).
void orc_paged_attention_decode_f32(const uint16_t* q, const uint16_t* kpool, const uint16_t* vpool,
                                    const int32_t* block_tables, int max_blocks, const int32_t* ctx_lens, int num_seqs,
                                    int hq, int hkv, int hd, int page, float scale, float* out) {
    int groups = hq / hkv;
#pragma omp parallel for collapse(2) schedule(dynamic)
    for (int s = 0; s < num_seqs; s++)
        for (int kvh = 0; kvh < hkv; kvh++) {
            int ctx = ctx_lens[s];
            std::vector<float> qf((size_t)groups * hd), acc((size_t)groups * hd, 0.f), mx(groups, -INFINITY), den(groups, 0.f);
            std::vector<float> kf(hd), vf(hd);
            for (int g = 0; g < groups; g++)
                for (int d = 0; d < hd; d++) qf[(size_t)g * hd + d] = bf2f(q[((size_t)s * hq + kvh * groups + g) * hd + d]) * scale;
            for (int j = 0; j < ctx; j++) {
                size_t base = (((size_t)block_tables[(size_t)s * max_blocks + j / page] * hkv + kvh) * page + j % page) * hd;
                for (int d = 0; d < hd; d++) {
                    kf[d] = bf2f(kpool[base + d]);
                    vf[d] = bf2f(vpool[base + d]);
                }
                for (int g = 0; g < groups; g++) {
                    float dot = 0.f;
                    for (int d = 0; d < hd; d++) dot += qf[(size_t)g * hd + d] * kf[d];
                    float nm = std::max(mx[g], dot);
                    float corr = std::exp(mx[g] - nm), p = std::exp(dot - nm);
                    den[g] = den[g] * corr + p;
                    for (int d = 0; d < hd; d++) acc[(size_t)g * hd + d] = acc[(size_t)g * hd + d] * corr + p * vf[d];
                    mx[g] = nm;
                }
            }
            for (int g = 0; g < groups; g++)
                for (int d = 0; d < hd; d++)
                    out[((size_t)s * hq + kvh * groups + g) * hd + d] = acc[(size_t)g * hd + d] / den[g];
        }
}

// ---------------------------------------------------------------------------------------------
// Synthetic tensors shared with the GPU generator (see orc_common.h).
void orc_synth_codes(uint64_t seed, int64_t n_words, uint32_t* out) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n_words; i++) out[i] = synth_code_word(seed, (uint64_t)i);
}
void orc_synth_scales_biases(uint64_t seed_scale, uint64_t seed_bias, int64_t n, float mul, float mid, uint16_t* scales,
                             uint16_t* biases) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; i++) {
        scales[i] = synth_scale(seed_scale, (uint64_t)i, mul);
        biases[i] = synth_bias(seed_bias, (uint64_t)i, scales[i], mid);
    }
}
void orc_synth_dense(uint64_t seed, int64_t n, float std_, uint16_t* out) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; i++) out[i] = synth_dense(seed, (uint64_t)i, std_);
}

}  // extern "C"

// Threads the OpenMP loops above will use, and a way to set them: a launcher may export OMP_NUM_THREADS=1 to its
// children, so the timed CPU legs set the count themselves and report what they really got.
extern "C" int orc_max_threads(void) { return omp_get_max_threads(); }
extern "C" void orc_set_threads(int n) {
    if (n > 0) omp_set_num_threads(n);
}
