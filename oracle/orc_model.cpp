// CPU oracle (test infrastructure): decoder forward + generation loops.
//
// Forward math and rounding points follow src/models/llama.rs (LlamaLayer::forward/combine_ffn
// :689-735, LlamaAttention::project/forward/forward_per_seq :806-873, LlamaMlp::forward :1040-1045,
// project_logits :595-603): every MLX op materialises a bf16 tensor, so in bf16 mode each op's
// result is rounded to bf16 here; matmuls and the attention reduction accumulate wider (f32 / f64).
#include "orc_model.h"

#include <algorithm>
#include <cfloat>
#include <cmath>
#include <cstring>

#include "oracle.h"
#include "orc_common.h"

namespace orc {

static inline float R(const ModelCfg& c, float x) { return c.f32_mode ? x : rbf(x); }

// y[m, out] = x[m, in] @ W^T, f32 accumulate in index order; rounded per mode.
// With cfg.sum_order == 1 every dot product is formed as four sums over the quarters of the input dimension, added
// as (s0 + s1) + (s2 + s3): a second, equally faithful f32 order.  The distance between the two orders' logits is
// the rounding noise any two correct bf16 implementations show, which sizes the end-to-end parity gates.
static void linear(const ModelCfg& c, const Mat& w, const std::vector<float>& x, int m, std::vector<float>& y,
                   std::vector<float>* unrounded = nullptr) {
    int in = w.in, out = w.out;
    y.assign((size_t)m * out, 0.f);
    if (unrounded) unrounded->assign((size_t)m * out, 0.f);
    int per = w.bits ? 32 / w.bits : 1;
    uint32_t mask = w.bits ? (1u << w.bits) - 1 : 0;
    const int parts = (c.sum_order == 1 && in >= 4) ? 4 : 1;
    std::vector<int> cut(parts + 1);
    for (int q = 0; q <= parts; q++) cut[q] = (int)((long)in * q / parts);
    std::vector<RowsT16> xt;
    xt.reserve(parts);
    for (int q = 0; q < parts; q++) {
        if (parts == 1) {
            xt.emplace_back(x.data(), m, in);
        } else {
            std::vector<float> sub((size_t)m * (cut[q + 1] - cut[q]));
            for (int i = 0; i < m; i++)
                std::memcpy(sub.data() + (size_t)i * (cut[q + 1] - cut[q]), x.data() + (size_t)i * in + cut[q], sizeof(float) * (cut[q + 1] - cut[q]));
            xt.emplace_back(sub.data(), m, cut[q + 1] - cut[q]);
        }
    }
#pragma omp parallel for schedule(dynamic, 32)
    for (int j = 0; j < out; j++) {
        std::vector<float> wf(in);
        if (w.bits) {
            int64_t words = in / per, groups = in / w.group;
            for (int d = 0; d < in; d++) {
                uint32_t code = (w.packed[(int64_t)j * words + d / per] >> ((d % per) * w.bits)) & mask;
                wf[d] = rbf(std::fmaf((float)code, bf2f(w.scales[(int64_t)j * groups + d / w.group]),
                                      bf2f(w.biases[(int64_t)j * groups + d / w.group])));
            }
        } else if (!w.wf.empty()) {
            std::memcpy(wf.data(), w.wf.data() + (size_t)j * in, sizeof(float) * in);
        } else {
            for (int d = 0; d < in; d++) wf[d] = bf2f(w.w[(size_t)j * in + d]);
        }
        std::vector<float> acc(m);
        if (parts == 1) {
            dots_in_order(xt[0], wf.data(), acc.data());
        } else {
            std::vector<float> s[4];
            for (int q = 0; q < 4; q++) {
                s[q].resize(m);
                dots_in_order(xt[q], wf.data() + cut[q], s[q].data());
            }
            for (int i = 0; i < m; i++) acc[i] = (s[0][i] + s[1][i]) + (s[2][i] + s[3][i]);
        }
        for (int i = 0; i < m; i++) {
            if (unrounded) (*unrounded)[(size_t)i * out + j] = acc[i];
            y[(size_t)i * out + j] = R(c, acc[i]);
        }
    }
}

static void rms_norm(const ModelCfg& c, const std::vector<float>& x, const float* w, int rows, int dim, std::vector<float>& y) {
    y.resize((size_t)rows * dim);
    for (int r = 0; r < rows; r++) {
        const float* xr = x.data() + (size_t)r * dim;
        float ss = 0.f;
        for (int d = 0; d < dim; d++) ss += xr[d] * xr[d];
        float inv = 1.0f / std::sqrt(ss / (float)dim + c.eps);
        for (int d = 0; d < dim; d++) y[(size_t)r * dim + d] = R(c, xr[d] * inv * w[d]);
    }
}

static std::vector<float> to_f32(const std::vector<uint16_t>& h) {
    std::vector<float> f(h.size());
    for (size_t i = 0; i < h.size(); i++) f[i] = bf2f(h[i]);
    return f;
}

void forward_batch(const Model& m, std::vector<SeqIn>& seqs, std::vector<float>& logits, std::vector<float>* logits_f32) {
    const ModelCfg& c = m.cfg;
    int T = 0;
    for (auto& s : seqs) T += s.n;
    int H = c.hidden, hd = c.head_dim, nq = c.heads, nkv = c.kv_heads, half = hd / 2;
    float scale = std::pow((float)hd, -0.5f);  // config.rs:597-598

    // embed (nn.rs:86-93): row gather
    std::vector<float> x((size_t)T * H);
    std::vector<int> pos(T);
    {
        int t = 0;
        for (auto& s : seqs)
            for (int i = 0; i < s.n; i++, t++) {
                pos[t] = s.offset + i;
                for (int d = 0; d < H; d++)
                    x[(size_t)t * H + d] = m.embed.wf.empty() ? bf2f(m.embed.w[(size_t)s.ids[i] * H + d]) : m.embed.wf[(size_t)s.ids[i] * H + d];
            }
    }
    // rope tables for the batch's positions (rope.rs:183-208): f32 angle, cos/sin, cast to bf16
    std::vector<float> cs((size_t)T * half), sn((size_t)T * half);
    for (int t = 0; t < T; t++)
        for (int i = 0; i < half; i++) {
            float ang = (float)pos[t] * m.inv_freq[i];
            cs[(size_t)t * half + i] = R(c, std::cos(ang));
            sn[(size_t)t * half + i] = R(c, std::sin(ang));
        }
    auto rope = [&](std::vector<float>& v, int heads) {
        std::vector<float> row(hd);
        for (int t = 0; t < T; t++)
            for (int h = 0; h < heads; h++) {
                float* xr = v.data() + ((size_t)t * heads + h) * hd;
                std::memcpy(row.data(), xr, sizeof(float) * hd);
                for (int d = 0; d < hd; d++) {
                    float rot = d < half ? -row[d + half] : row[d - half];
                    float a = R(c, row[d] * cs[(size_t)t * half + d % half]);
                    float b = R(c, rot * sn[(size_t)t * half + d % half]);
                    xr[d] = R(c, a + b);
                }
            }
    };

    std::vector<float> n1, q, k, v, attn((size_t)T * nq * hd), o, h, n2, g, u, mm, dn;
    std::vector<uint16_t> kb, vb;
    for (int l = 0; l < c.layers; l++) {
        const Layer& L = m.layers[l];
        std::vector<float> ln1 = c.f32_mode ? L.input_ln_f : to_f32(L.input_ln);
        std::vector<float> ln2 = c.f32_mode ? L.post_ln_f : to_f32(L.post_ln);
        rms_norm(c, x, ln1.data(), T, H, n1);
        linear(c, L.q, n1, T, q);
        linear(c, L.k, n1, T, k);
        linear(c, L.v, n1, T, v);
        if (c.qk_norm) {  // Qwen3 per-head norm before RoPE (llama.rs:814-819)
            std::vector<float> qn = to_f32(L.q_norm), kn = to_f32(L.k_norm), tmp;
            rms_norm(c, q, qn.data(), T * nq, hd, tmp);
            q.swap(tmp);
            rms_norm(c, k, kn.data(), T * nkv, hd, tmp);
            k.swap(tmp);
        }
        rope(q, nq);
        rope(k, nkv);
        // cache update + causal GQA attention per sequence
        int t0 = 0;
        for (auto& s : seqs) {
            size_t row = (size_t)nkv * hd;
            kb.resize((size_t)s.n * row);
            vb.resize((size_t)s.n * row);
            // caches hold bf16 in bf16 mode; in f32 mode the oracle keeps a side f32 copy by packing
            // two u16 per value (row_elems doubles)
            if (!c.f32_mode) {
                for (size_t i = 0; i < kb.size(); i++) {
                    kb[i] = f2bf(k[(size_t)t0 * row + i]);
                    vb[i] = f2bf(v[(size_t)t0 * row + i]);
                }
                s.cache->update(l, kb.data(), vb.data(), s.n, row);
            } else {
                s.cache->update(l, (const uint16_t*)(k.data() + (size_t)t0 * row), (const uint16_t*)(v.data() + (size_t)t0 * row), s.n, row * 2);
            }
            const Rows& K = s.cache->keys(l);
            const Rows& V = s.cache->values(l);
            int kl = s.offset + s.n;
            auto kat = [&](int j, int kvh, int d) -> float {
                size_t idx = ((size_t)j * nkv + kvh) * hd + d;
                return c.f32_mode ? ((const float*)K.data())[idx] : bf2f(K[idx]);
            };
            auto vat = [&](int j, int kvh, int d) -> float {
                size_t idx = ((size_t)j * nkv + kvh) * hd + d;
                return c.f32_mode ? ((const float*)V.data())[idx] : bf2f(V[idx]);
            };
            int groups = nq / nkv;
#pragma omp parallel for schedule(dynamic)
            for (int head = 0; head < nq; head++) {
                int kvh = head / groups;
                std::vector<double> lg(kl);
                for (int r = 0; r < s.n; r++) {
                    const float* qr = q.data() + ((size_t)(t0 + r) * nq + head) * hd;
                    int jmax = kl - s.n + r;
                    double mx = -DBL_MAX;
                    for (int j = 0; j <= jmax; j++) {
                        double dot = 0;
                        for (int d = 0; d < hd; d++) dot += (double)qr[d] * (double)kat(j, kvh, d);
                        lg[j] = dot * (double)scale;
                        mx = std::max(mx, lg[j]);
                    }
                    double den = 0;
                    for (int j = 0; j <= jmax; j++) {
                        lg[j] = std::exp(lg[j] - mx);
                        den += lg[j];
                    }
                    float* orow = attn.data() + ((size_t)(t0 + r) * nq + head) * hd;
                    for (int d = 0; d < hd; d++) {
                        double acc = 0;
                        for (int j = 0; j <= jmax; j++) acc += lg[j] * (double)vat(j, kvh, d);
                        orow[d] = R(c, (float)(acc / den));
                    }
                }
            }
            t0 += s.n;
        }
        linear(c, L.o, attn, T, o);
        h.resize(x.size());
        for (size_t i = 0; i < x.size(); i++) h[i] = R(c, x[i] + o[i]);
        rms_norm(c, h, ln2.data(), T, H, n2);
        linear(c, L.gate, n2, T, g);
        linear(c, L.up, n2, T, u);
        mm.resize(g.size());
        for (size_t i = 0; i < g.size(); i++) {
            float sg = R(c, 1.0f / (1.0f + std::exp(-g[i])));
            float a = R(c, g[i] * sg);
            mm[i] = R(c, a * u[i]);
        }
        linear(c, L.down, mm, T, dn);
        for (size_t i = 0; i < x.size(); i++) x[i] = R(c, h[i] + dn[i]);
    }
    // last position of every sequence -> final norm -> lm_head (llama.rs:555-557, :595-603)
    int B = (int)seqs.size();
    std::vector<float> last((size_t)B * H), nf;
    {
        int t0 = 0;
        for (int b = 0; b < B; b++) {
            t0 += seqs[b].n;
            std::memcpy(last.data() + (size_t)b * H, x.data() + (size_t)(t0 - 1) * H, sizeof(float) * H);
        }
    }
    std::vector<float> fn = c.f32_mode ? m.norm_f : to_f32(m.norm);
    rms_norm(c, last, fn.data(), B, H, nf);
    linear(c, m.lm_head, nf, B, logits, logits_f32);
}

}  // namespace orc

using namespace orc;

struct OrcModel {
    Model m;
};

static void fill_inv_freq(Model& m) {
    m.inv_freq.resize(m.cfg.head_dim / 2);
    orc_rope_inv_freq(m.cfg.head_dim, m.cfg.theta, m.cfg.rope_kind, m.cfg.rope_factor, m.cfg.rope_low, m.cfg.rope_high,
                      m.cfg.rope_orig, m.inv_freq.data());
}

static ModelCfg cfg_from_c(const orc_model_cfg* c) {
    ModelCfg k;
    k.layers = c->layers; k.hidden = c->hidden; k.heads = c->heads; k.kv_heads = c->kv_heads; k.head_dim = c->head_dim;
    k.inter = c->inter; k.vocab = c->vocab; k.eps = c->eps; k.theta = c->theta; k.rope_kind = c->rope_kind;
    k.rope_factor = c->rope_factor; k.rope_low = c->rope_low; k.rope_high = c->rope_high; k.rope_orig = c->rope_orig;
    k.qk_norm = c->qk_norm; k.quant_bits = c->quant_bits; k.group = c->group ? c->group : 64; k.f32_mode = c->f32_mode;
    k.sum_order = c->sum_order;
    return k;
}

static Mat* find_mat(Model& m, int layer, int which) {
    // which: 0 q 1 k 2 v 3 o 4 gate 5 up 6 down 7 embed 8 lm_head
    if (which == 7) return &m.embed;
    if (which == 8) return &m.lm_head;
    Layer& L = m.layers.at(layer);
    Mat* t[7] = {&L.q, &L.k, &L.v, &L.o, &L.gate, &L.up, &L.down};
    return t[which];
}

static void mat_dims(const ModelCfg& c, int which, int& out, int& in) {
    int qd = c.heads * c.head_dim, kvd = c.kv_heads * c.head_dim;
    switch (which) {
        case 0: out = qd; in = c.hidden; break;
        case 1: case 2: out = kvd; in = c.hidden; break;
        case 3: out = c.hidden; in = qd; break;
        case 4: case 5: out = c.inter; in = c.hidden; break;
        case 6: out = c.hidden; in = c.inter; break;
        default: out = c.vocab; in = c.hidden; break;
    }
}

extern "C" {

orc_model* orc_model_new(const orc_model_cfg* cfg) {
    auto* om = new OrcModel();
    om->m.cfg = cfg_from_c(cfg);
    om->m.layers.resize(cfg->layers);
    fill_inv_freq(om->m);
    return (orc_model*)om;
}
void orc_model_free(orc_model* p) { delete (OrcModel*)p; }

// Dense weight from f32 data: cast to bf16 as CausalLm::from_weights does (llama.rs:71), or kept f32.
void orc_model_set_dense(orc_model* p, int layer, int which, const float* data) {
    Model& m = ((OrcModel*)p)->m;
    Mat* t = find_mat(m, layer, which);
    mat_dims(m.cfg, which, t->out, t->in);
    size_t n = (size_t)t->out * t->in;
    t->bits = 0;
    if (m.cfg.f32_mode) {
        t->wf.assign(data, data + n);
    } else {
        t->w.resize(n);
        for (size_t i = 0; i < n; i++) t->w[i] = f2bf(data[i]);
    }
}
void orc_model_set_dense_bf16(orc_model* p, int layer, int which, const uint16_t* data) {
    Model& m = ((OrcModel*)p)->m;
    Mat* t = find_mat(m, layer, which);
    mat_dims(m.cfg, which, t->out, t->in);
    t->bits = 0;
    t->w.assign(data, data + (size_t)t->out * t->in);
}
void orc_model_set_quantized(orc_model* p, int layer, int which, const uint32_t* packed, const uint16_t* scales,
                             const uint16_t* biases, int bits, int group) {
    Model& m = ((OrcModel*)p)->m;
    Mat* t = find_mat(m, layer, which);
    mat_dims(m.cfg, which, t->out, t->in);
    t->bits = bits;
    t->group = group;
    size_t words = (size_t)t->out * t->in * bits / 32, ng = (size_t)t->out * t->in / group;
    t->packed.assign(packed, packed + words);
    t->scales.assign(scales, scales + ng);
    t->biases.assign(biases, biases + ng);
}
// Quantize-on-load of a dense projection already set (Projection::load_with_bias, projection.rs:57-71).
void orc_model_quantize_projection(orc_model* p, int layer, int which, int bits, int group) {
    Model& m = ((OrcModel*)p)->m;
    Mat* t = find_mat(m, layer, which);
    size_t words = (size_t)t->out * t->in * bits / 32, ng = (size_t)t->out * t->in / group;
    t->packed.resize(words);
    t->scales.resize(ng);
    t->biases.resize(ng);
    orc_quantize(t->w.data(), t->out, t->in, group, bits, t->packed.data(), t->scales.data(), t->biases.data());
    t->bits = bits;
    t->group = group;
    t->w.clear();
}
// which: 0 input_ln 1 post_ln 2 q_norm 3 k_norm 4 final norm
void orc_model_set_norm(orc_model* p, int layer, int which, const float* data, int n) {
    Model& m = ((OrcModel*)p)->m;
    std::vector<uint16_t> h(n);
    for (int i = 0; i < n; i++) h[i] = f2bf(data[i]);
    std::vector<float> f(data, data + n);
    if (which == 4) {
        m.norm = h;
        m.norm_f = f;
        return;
    }
    Layer& L = m.layers.at(layer);
    if (which == 0) { L.input_ln = h; L.input_ln_f = f; }
    if (which == 1) { L.post_ln = h; L.post_ln_f = f; }
    if (which == 2) L.q_norm = h;
    if (which == 3) L.k_norm = h;
}

// Synthetic random-init model from the counter-based generator (orc_common.h).  Tensor seeds:
// t = mix64(seed ^ (0x5EED0000 + id)), id = 1 embed, 2 lm_head, 16*(layer+1)+which for projections;
// quantized projections use t (codes), t+1 (scales), t+2 (biases).  Norm weights are all ones.
uint64_t orc_synth_tensor_seed(uint64_t seed, int layer, int which) {
    uint64_t id = which == 7 ? 1 : which == 8 ? 2 : (uint64_t)(16 * (layer + 1) + which);
    return mix64(seed ^ (0x5EED0000ull + id));
}
void orc_model_fill_synthetic(orc_model* p, uint64_t seed) {
    Model& m = ((OrcModel*)p)->m;
    const ModelCfg& c = m.cfg;
    auto fill = [&](int layer, int which, bool allow_quant) {
        Mat* t = find_mat(m, layer, which);
        mat_dims(c, which, t->out, t->in);
        uint64_t ts = orc_synth_tensor_seed(seed, layer, which);
        size_t n = (size_t)t->out * t->in;
        if (c.quant_bits && allow_quant) {
            t->bits = c.quant_bits;
            t->group = c.group;
            t->packed.resize(n * t->bits / 32);
            t->scales.resize(n / t->group);
            t->biases.resize(n / t->group);
            orc_synth_codes(ts, (int64_t)t->packed.size(), t->packed.data());
            float mul = t->bits == 4 ? 0.02f / 7.5f : 0.02f / 127.5f;
            float mid = t->bits == 4 ? 8.f : 128.f;
            orc_synth_scales_biases(ts + 1, ts + 2, (int64_t)t->scales.size(), mul, mid, t->scales.data(), t->biases.data());
        } else {
            t->bits = 0;
            t->w.resize(n);
            orc_synth_dense(ts, (int64_t)n, 0.02f, t->w.data());
        }
    };
    fill(0, 7, false);
    fill(0, 8, false);
    std::vector<float> ones_h(c.hidden, 1.f), ones_d(c.head_dim, 1.f);
    orc_model_set_norm(p, 0, 4, ones_h.data(), c.hidden);
    for (int l = 0; l < c.layers; l++) {
        for (int w = 0; w < 7; w++) fill(l, w, true);
        orc_model_set_norm(p, l, 0, ones_h.data(), c.hidden);
        orc_model_set_norm(p, l, 1, ones_h.data(), c.hidden);
        if (c.qk_norm) {
            orc_model_set_norm(p, l, 2, ones_d.data(), c.head_dim);
            orc_model_set_norm(p, l, 3, ones_d.data(), c.head_dim);
        }
    }
}

// ---- caches exposed to the tests --------------------------------------------------------------
struct OrcPool {
    std::shared_ptr<BlockPool> p;
};
struct OrcCache {
    std::unique_ptr<KvCacheBase> c;
    PagedKvCache* paged = nullptr;
};

orc_pool* orc_pool_new(int block_size) { return (orc_pool*)new OrcPool{std::make_shared<BlockPool>((size_t)block_size)}; }
void orc_pool_free(orc_pool* p) { delete (OrcPool*)p; }
void orc_pool_stats(orc_pool* p, int64_t* out4) {
    auto& bp = *((OrcPool*)p)->p;
    out4[0] = (int64_t)bp.live_blocks();
    out4[1] = (int64_t)bp.shared_blocks();
    out4[2] = (int64_t)bp.peak_live_blocks();
    out4[3] = (int64_t)bp.reserved_tokens();
}
int orc_pool_is_materialized(orc_pool* p, int64_t id) { return ((OrcPool*)p)->p->is_materialized((size_t)id) ? 1 : 0; }
orc_cache* orc_cache_new_paged(orc_pool* p, int layers) {
    auto* oc = new OrcCache();
    auto* pc = new PagedKvCache(((OrcPool*)p)->p, (size_t)layers);
    oc->c.reset(pc);
    oc->paged = pc;
    return (orc_cache*)oc;
}
orc_cache* orc_cache_new_seeded(orc_pool* p, int layers, const int64_t* ids, int n) {
    std::vector<size_t> v(ids, ids + n);
    auto* oc = new OrcCache();
    auto* pc = new PagedKvCache(((OrcPool*)p)->p, (size_t)layers, v);
    oc->c.reset(pc);
    oc->paged = pc;
    return (orc_cache*)oc;
}
orc_cache* orc_cache_new_contiguous(int layers) {
    auto* oc = new OrcCache();
    oc->c.reset(new ContiguousKvCache((size_t)layers));
    return (orc_cache*)oc;
}
void orc_cache_free(orc_cache* c) { delete (OrcCache*)c; }
// k/v are token-major rows [step, row_elems] bf16.  Returns 0, or -1 with the batch-size rule of
// PagedKvCache::update (:380-385) when batch != 1.
int orc_cache_update(orc_cache* c, int layer, const uint16_t* k, const uint16_t* v, int step, int row_elems, int batch) {
    auto* oc = (OrcCache*)c;
    if (oc->paged && batch != 1) return -1;
    oc->c->update((size_t)layer, k, v, (size_t)step, (size_t)row_elems);
    return 0;
}
int64_t orc_cache_gather(orc_cache* c, int layer, uint16_t* k_out, uint16_t* v_out) {
    auto* oc = (OrcCache*)c;
    const Rows& K = oc->c->keys((size_t)layer);
    const Rows& V = oc->c->values((size_t)layer);
    if (k_out) std::memcpy(k_out, K.data(), K.size() * 2);
    if (v_out) std::memcpy(v_out, V.data(), V.size() * 2);
    return (int64_t)K.size();
}
int32_t orc_cache_offset(orc_cache* c) { return ((OrcCache*)c)->c->offset(); }
int orc_cache_truncate(orc_cache* c, int32_t len) {
    try {
        ((OrcCache*)c)->c->truncate(len);
    } catch (...) {
        return -1;
    }
    return 0;
}
void orc_cache_reset(orc_cache* c) { ((OrcCache*)c)->c->reset(); }
int orc_cache_retain_sequences(orc_cache* c, const int32_t* keep, int n) {
    auto* oc = (OrcCache*)c;
    if (!oc->paged) return -2;
    try {
        oc->paged->retain_sequences(keep, (size_t)n);
    } catch (...) {
        return -1;
    }
    return 0;
}
// out: [blocks, tail_len, reserved_tokens, batch_size]
void orc_cache_paged_stats(orc_cache* c, int64_t* out4) {
    auto* pc = ((OrcCache*)c)->paged;
    out4[0] = (int64_t)pc->blocks();
    out4[1] = (int64_t)pc->tail_len;
    out4[2] = (int64_t)pc->reserved_tokens();
    out4[3] = pc->batch_size();
}
int orc_cache_block_ids(orc_cache* c, int64_t* out, int cap) {
    auto* pc = ((OrcCache*)c)->paged;
    int n = (int)pc->block_ids.size();
    for (int i = 0; i < n && i < cap; i++) out[i] = (int64_t)pc->block_ids[i];
    return n;
}
int orc_cache_shareable_prefix_blocks(orc_cache* c, int64_t tokens, int64_t* out, int cap) {
    auto* pc = ((OrcCache*)c)->paged;
    auto v = pc->shareable_prefix_blocks((size_t)tokens);
    for (size_t i = 0; i < v.size() && (int)i < cap; i++) out[i] = (int64_t)v[i];
    return (int)v.size();
}

// One forward over a ragged batch through caller-owned caches (Decode::step / decode_logits /
// decode_logits_per_seq).  ids concatenated, n[i] tokens per sequence at offsets[i].
void orc_model_forward(orc_model* p, int num_seqs, const int32_t* ids, const int32_t* n, orc_cache** caches,
                       const int32_t* offsets, float* logits_out, float* logits_f32_out) {
    Model& m = ((OrcModel*)p)->m;
    std::vector<SeqIn> seqs;
    const int32_t* cur = ids;
    for (int i = 0; i < num_seqs; i++) {
        seqs.push_back(SeqIn{cur, n[i], ((OrcCache*)caches[i])->c.get(), offsets[i]});
        cur += n[i];
    }
    std::vector<float> lg, lgf;
    forward_batch(m, seqs, lg, logits_f32_out ? &lgf : nullptr);
    std::memcpy(logits_out, lg.data(), lg.size() * sizeof(float));
    if (logits_f32_out) std::memcpy(logits_f32_out, lgf.data(), lgf.size() * sizeof(float));
}

static int32_t greedy(const ModelCfg& c, const float* logits, int vocab) {
    // logits hold bf16-representable values in bf16 mode, so an f32 scan is the same comparison
    (void)c;
    return orc_argmax_f32(logits, vocab);
}

// generate — src/decode/stream.rs:113-121 + decode_loop :259-327 (greedy, contiguous cache made by
// Decode::make_cache).  cancel_after_tokens < 0 disables the cancel probe; otherwise the cancel flag
// reads as set once that many Token events have been emitted.
int orc_generate(orc_model* p, const int32_t* prompt, int n_prompt, int max_new, const int32_t* stop, int n_stop,
                 int cancel_after_tokens, int use_paged, int block_size, int32_t* tokens_out, int* n_out, int* reason_out,
                 int32_t* events_out, int events_cap, int* n_events) {
    Model& m = ((OrcModel*)p)->m;
    std::vector<Event> ev;
    if (n_prompt == 0) return -7;               // Error::Msg: empty prompt
    if (cancel_after_tokens == 0) return -6;    // Error::Canceled before any inference
    std::unique_ptr<KvCacheBase> cache;
    if (use_paged)
        cache.reset(new PagedKvCache(std::make_shared<BlockPool>((size_t)block_size), (size_t)m.cfg.layers));
    else
        cache.reset(new ContiguousKvCache((size_t)m.cfg.layers));
    std::vector<float> lg;
    std::vector<SeqIn> s{SeqIn{prompt, n_prompt, cache.get(), 0}};
    forward_batch(m, s, lg, nullptr);
    std::vector<int32_t> gen;
    int finish = 1;  // MaxTokens
    for (int step = 0; step < max_new; step++) {
        if (cancel_after_tokens >= 0 && (int)gen.size() >= cancel_after_tokens) {
            finish = 2;
            break;
        }
        int32_t next = greedy(m.cfg, lg.data(), m.cfg.vocab);
        bool is_stop = false;
        for (int i = 0; i < n_stop; i++) is_stop = is_stop || stop[i] == next;
        if (is_stop) {
            finish = 0;
            break;
        }
        ev.push_back(Event{0, 0, next, step});
        gen.push_back(next);
        if (step + 1 == max_new) break;
        int off = cache->offset();
        std::vector<SeqIn> s1{SeqIn{&next, 1, cache.get(), off}};
        forward_batch(m, s1, lg, nullptr);
    }
    ev.push_back(Event{0, 1, finish, (int32_t)gen.size()});
    for (size_t i = 0; i < gen.size(); i++) tokens_out[i] = gen[i];
    *n_out = (int)gen.size();
    *reason_out = finish;
    int ne = 0;
    for (auto& e : ev)
        if (ne < events_cap) {
            std::memcpy(events_out + 4 * ne, &e, sizeof(Event));
            ne++;
        }
    if (n_events) *n_events = ne;
    return 0;
}

// generate_continuous — src/decode/continuous.rs:117-340, reference schedule: whole-prompt batch-1
// prefill at admission, then one decode forward per step for every live lane.  `throughput` selects
// the batched forward (one ragged batch of all lanes) against per-lane forwards; in this oracle the
// two are numerically identical because its matmul is row-invariant.
//   prompts concatenated; per request prompt_len, max_new; stop tokens concatenated with n_stop.
//   cancel_after_steps < 0: never; 0: pre-set (typed error); k > 0: flag reads set at the top of
//   decode step k (1-based), i.e. after k-1 completed steps.
// Outputs: tokens_out [n_req, max over max_new] row-major with stride `tok_stride`, n_tokens[n_req],
// reasons[n_req] (0 StopToken 1 MaxTokens 2 Cancelled), events (req, kind, a, b) x n_events,
// block_ids_out: per request the reference-semantics block-id list at retirement (or at the end),
// stride block_stride, n_blocks[n_req]; pool_stats_out = live/shared/peak/reserved at the end.
int orc_generate_continuous(orc_model* p, int n_req, const int32_t* prompts, const int32_t* prompt_len,
                            const int32_t* max_new, const int32_t* stops, const int32_t* n_stop, int max_batch,
                            int block_size, int throughput, int cancel_after_steps, int32_t* tokens_out, int tok_stride,
                            int32_t* n_tokens, int32_t* reasons, int32_t* events_out, int events_cap, int* n_events,
                            int64_t* block_ids_out, int block_stride, int32_t* n_blocks, int64_t* pool_stats_out,
                            int32_t* peak_lane_blocks_out) {
    Model& m = ((OrcModel*)p)->m;
    if (n_req == 0) return -7;
    if (max_batch == 0) return -7;
    if (block_size == 0) return -7;
    for (int i = 0; i < n_req; i++)
        if (prompt_len[i] == 0) return -7;
    if (cancel_after_steps == 0) return -6;

    std::vector<Request> reqs(n_req);
    {
        const int32_t* pp = prompts;
        const int32_t* sp = stops;
        for (int i = 0; i < n_req; i++) {
            reqs[i].prompt.assign(pp, pp + prompt_len[i]);
            pp += prompt_len[i];
            reqs[i].stop.assign(sp, sp + n_stop[i]);
            sp += n_stop[i];
            reqs[i].max_new = (size_t)max_new[i];
        }
    }
    auto pool = std::make_shared<BlockPool>((size_t)block_size);
    Scheduler sched;
    for (auto& r : reqs) sched.admit(r.prompt, r.max_new, r.stop);
    struct Lane {
        size_t seq;
        std::unique_ptr<PagedKvCache> cache;
        int32_t next_token;
    };
    std::vector<Lane> lanes;
    std::vector<Event> ev;
    std::vector<std::vector<size_t>> final_blocks(n_req);
    auto emit = [&](int req, int kind, int a, int b) { ev.push_back(Event{req, kind, a, b}); };
    // record_token, continuous.rs:306-340
    auto record = [&](Lane& lane, int32_t tok) -> bool {
        int ri = (int)lane.seq;
        int fin = sched.record(lane.seq, tok);
        if (fin == FIN_STOP) {
            emit(ri, 1, 0, (int)sched.seqs[lane.seq].generated.size());
            return false;
        }
        emit(ri, 0, tok, (int)sched.seqs[lane.seq].generated.size() - 1);
        if (fin == FIN_LENGTH) {
            emit(ri, 1, 1, (int)sched.seqs[lane.seq].generated.size());
            return false;
        }
        lane.next_token = tok;
        return true;
    };
    std::vector<float> lg;
    // admit_lane, continuous.rs:235-270
    auto admit_lane = [&](size_t ri) {
        if (!sched.is_active(ri)) {
            emit((int)ri, 1, 1, 0);
            return;
        }
        Lane lane{ri, std::make_unique<PagedKvCache>(pool, (size_t)m.cfg.layers), 0};
        std::vector<SeqIn> s{SeqIn{reqs[ri].prompt.data(), (int)reqs[ri].prompt.size(), lane.cache.get(), 0}};
        forward_batch(m, s, lg, nullptr);
        int32_t tok = greedy(m.cfg, lg.data(), m.cfg.vocab);
        if (record(lane, tok))
            lanes.push_back(std::move(lane));
        else
            final_blocks[ri] = lane.cache->block_ids;
    };
    size_t next_req = 0;
    while (lanes.size() < (size_t)max_batch && next_req < (size_t)n_req) admit_lane(next_req++);
    int step_no = 0;
    bool cancelled = false;
    while (!lanes.empty()) {
        step_no++;
        if (cancel_after_steps > 0 && step_no >= cancel_after_steps) {
            cancelled = true;
            break;
        }
        size_t b = lanes.size();
        std::vector<float> all((size_t)b * m.cfg.vocab);
        if (throughput) {
            std::vector<SeqIn> s;
            for (auto& l : lanes) s.push_back(SeqIn{&l.next_token, 1, l.cache.get(), l.cache->offset()});
            forward_batch(m, s, all, nullptr);
        } else {
            for (size_t i = 0; i < b; i++) {
                std::vector<SeqIn> s{SeqIn{&lanes[i].next_token, 1, lanes[i].cache.get(), lanes[i].cache->offset()}};
                forward_batch(m, s, lg, nullptr);
                std::memcpy(all.data() + i * m.cfg.vocab, lg.data(), sizeof(float) * m.cfg.vocab);
            }
        }
        std::vector<Lane> survivors;
        for (size_t i = 0; i < b; i++) {
            int32_t tok = greedy(m.cfg, all.data() + i * m.cfg.vocab, m.cfg.vocab);
            if (record(lanes[i], tok))
                survivors.push_back(std::move(lanes[i]));
            else
                final_blocks[lanes[i].seq] = lanes[i].cache->block_ids;  // then dropped: blocks released
        }
        lanes = std::move(survivors);
        while (lanes.size() < (size_t)max_batch && next_req < (size_t)n_req) admit_lane(next_req++);
    }
    if (cancelled) {
        for (auto& l : lanes) emit((int)l.seq, 1, 2, (int)sched.seqs[l.seq].generated.size());
        for (size_t ri = next_req; ri < (size_t)n_req; ri++)
            emit((int)ri, 1, sched.seqs[ri].finish == FIN_LENGTH ? 1 : 2, 0);
    }
    for (auto& l : lanes) final_blocks[l.seq] = l.cache->block_ids;
    if (pool_stats_out) {
        pool_stats_out[0] = (int64_t)pool->live_blocks();
        pool_stats_out[1] = (int64_t)pool->shared_blocks();
        pool_stats_out[2] = (int64_t)pool->peak_live_blocks();
        pool_stats_out[3] = (int64_t)pool->reserved_tokens();
    }
    (void)peak_lane_blocks_out;
    for (int i = 0; i < n_req; i++) {
        auto& g = sched.seqs[i].generated;
        for (size_t j = 0; j < g.size() && (int)j < tok_stride; j++) tokens_out[(size_t)i * tok_stride + j] = g[j];
        n_tokens[i] = (int32_t)g.size();
        reasons[i] = sched.seqs[i].finish == FIN_STOP ? 0 : sched.seqs[i].finish == FIN_LENGTH ? 1 : 2;
        if (block_ids_out) {
            for (size_t j = 0; j < final_blocks[i].size() && (int)j < block_stride; j++)
                block_ids_out[(size_t)i * block_stride + j] = (int64_t)final_blocks[i][j];
            n_blocks[i] = (int32_t)final_blocks[i].size();
        }
    }
    int ne = 0;
    for (auto& e : ev)
        if (ne < events_cap) {
            std::memcpy(events_out + 4 * ne, &e, sizeof(Event));
            ne++;
        }
    if (n_events) *n_events = ne;
    return 0;
}

}  // extern "C"
