// The f32 path of the decoder forward (b2_model_config::compute_f32): weights, activations, K/V pages and logits
// in f32, plain CUDA-core kernels.
//
// CausalLm::from_weights casts every tensor to bf16 (src/models/llama.rs:29-30, :71), so two faithful
// implementations of the reference's arithmetic sit one bf16 rounding apart wherever a sum is formed in a different
// order, and a greedy step whose two best logits are closer than that cannot be compared.  This path removes the
// roundings instead of chasing them: the same decoder (LlamaLayer::forward :689-735, LlamaAttention :806-873,
// LlamaMlp :1040-1045, project_logits :595-603) computed in f32 with a FIXED order of operations --
//   * every projection output is one accumulator that adds x[d]*w[d] for d = 0, 1, 2, ... with a separate IEEE
//     multiply and add (no fused multiply-add), whatever the tiling;
//   * RMSNorm sums the squares in index order, then x * (1/sqrt(mean + eps)) * w, left to right;
//   * RoPE (NeoX halves): x*cos + rot(x)*sin with f32 tables built on the host (angle = pos*inv_freq in f32);
//   * attention: scores, the softmax sums and P.V in f64, keys in order, one division at the end;
//   * SwiGLU: g * (1/(1+exp(-g))) * up;  residual adds in f32;  argmax ties -> lowest index.
// Only exp / cos / sin can differ between two implementations of this, by an ulp of their library.  The kernels are
// written for small models (a thread per output, sequential inner loops): this is the comparison path, not a fast one.
#include <cfloat>

#include "engine.h"

struct F32Work {
    int t_cap = 0, b_cap = 0;
    float *x = nullptr, *xn = nullptr, *qkv = nullptr, *q = nullptr, *attn = nullptr, *gu = nullptr, *act = nullptr;
    float *last = nullptr, *logits = nullptr;
};

namespace {

constexpr int kMaxCtxF32 = 4096;  // attention keeps one f64 score per key in shared memory

__global__ void embed_f32_kernel(const float* table, const int32_t* ids, int T, int dim, int vocab, float* out) {
    const int t = blockIdx.x;
    int id = ids[t];
    id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
    for (int d = threadIdx.x; d < dim; d += blockDim.x) out[(size_t)t * dim + d] = table[(size_t)id * dim + d];
}

// out[r] = x[row(r)] / rms * w: squares summed in index order by one thread, as a scalar loop would
__global__ void rms_norm_f32_kernel(const float* x, const float* w, float eps, int dim, const int32_t* row_idx, float* out) {
    __shared__ float inv_s;
    const int r = blockIdx.x;
    const float* xr = x + (size_t)(row_idx ? row_idx[r] : r) * dim;
    if (threadIdx.x == 0) {
        float ss = 0.f;
        for (int d = 0; d < dim; d++) ss = __fadd_rn(ss, __fmul_rn(xr[d], xr[d]));
        inv_s = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, (float)dim), eps)));
    }
    __syncthreads();
    const float inv = inv_s;
    for (int d = threadIdx.x; d < dim; d += blockDim.x) out[(size_t)r * dim + d] = __fmul_rn(__fmul_rn(xr[d], inv), w[d]);
}

// y[t, j] = (res ? res[t, j] : 0) + sum_d x[t, d] * w[j, d], the sum taken in index order.  32 x 8 outputs per
// block, x and w staged through shared memory 32 inputs at a time; the staging does not touch the order.
__global__ void __launch_bounds__(256) linear_f32_kernel(const float* x, const float* w, const float* res, int M, int N, int K, float* y) {
    __shared__ float xs[8][33];
    __shared__ float ws[32][33];
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const int j = blockIdx.x * 32 + tx, t = blockIdx.y * 8 + ty;
    float acc = 0.f;
    for (int k0 = 0; k0 < K; k0 += 32) {
        const int kn = min(32, K - k0);
        {  // 8 rows of x: thread (ty, tx) loads x[t][k0 + tx];  32 rows of w: four loads per thread
            const int tt = blockIdx.y * 8 + ty;
            xs[ty][tx] = (tt < M && tx < kn) ? x[(size_t)tt * K + k0 + tx] : 0.f;
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int jr = ty * 4 + i, jj = blockIdx.x * 32 + jr;
                ws[jr][tx] = (jj < N && tx < kn) ? w[(size_t)jj * K + k0 + tx] : 0.f;
            }
        }
        __syncthreads();
        for (int d = 0; d < kn; d++) acc = __fadd_rn(acc, __fmul_rn(xs[ty][d], ws[tx][d]));
        __syncthreads();
    }
    if (t < M && j < N) y[(size_t)t * N + j] = res ? __fadd_rn(res[(size_t)t * N + j], acc) : acc;
}

// NeoX RoPE on q and k, K/V append into f32 pages [page][hkv][block][hd].  Block = one token, thread = one element.
__global__ void rope_kv_f32_kernel(const float* qkv, int ld, const int32_t* positions, const int32_t* slot_mapping, const float* cos_t,
                                   const float* sin_t, int hq, int hkv, int hd, int page_size, float* k_pool, float* v_pool, float* q_out) {
    const int t = blockIdx.x, half = hd / 2;
    const int pos = positions[t], slot = slot_mapping[t];
    const float* row = qkv + (size_t)t * ld;
    for (int e = threadIdx.x; e < (hq + 2 * hkv) * hd; e += blockDim.x) {
        const int h = e / hd, d = e % hd;
        float out;
        if (h < hq + hkv) {
            const float* hr = row + (size_t)h * hd;
            const float rot = d < half ? -hr[d + half] : hr[d - half];
            const float c = cos_t[(size_t)pos * half + d % half], s = sin_t[(size_t)pos * half + d % half];
            out = __fadd_rn(__fmul_rn(hr[d], c), __fmul_rn(rot, s));
        } else {
            out = row[e];
        }
        if (h < hq) {
            q_out[((size_t)t * hq + h) * hd + d] = out;
        } else if (slot >= 0) {
            const int kh = h < hq + hkv ? h - hq : h - hq - hkv;
            float* pool = h < hq + hkv ? k_pool : v_pool;
            pool[(((size_t)(slot / page_size) * hkv + kh) * page_size + slot % page_size) * hd + d] = out;
        }
    }
}

// Causal GQA attention of one (token, q head) over the pages of its sequence, f64 throughout, keys in order:
// the restatement of a host loop (attention.rs:373-405) on the device.
__global__ void __launch_bounds__(128) attention_f32_kernel(const float* q, const float* k_pool, const float* v_pool, const int32_t* block_tables,
                                                            int max_blocks, const int32_t* seq_slot, const int32_t* token_seq,
                                                            const int32_t* positions, int hq, int hkv, int hd, int page_size, float scale,
                                                            float* out) {
    extern __shared__ double lg[];  // [n keys]
    __shared__ double red[128];
    __shared__ double den_s;
    const int t = blockIdx.x, head = blockIdx.y, kvh = head / (hq / hkv);
    const int n = positions[t] + 1;  // the query at position p sees keys 0..p (bottom-right causal)
    const int32_t* bt = block_tables + (size_t)seq_slot[token_seq[t]] * max_blocks;
    const float* qr = q + ((size_t)t * hq + head) * hd;
    auto krow = [&](const float* pool, int j) { return pool + (((size_t)bt[j / page_size] * hkv + kvh) * page_size + j % page_size) * hd; };
    double mx = -DBL_MAX;
    for (int j = threadIdx.x; j < n; j += blockDim.x) {
        const float* kr = krow(k_pool, j);
        double dot = 0.0;
        for (int d = 0; d < hd; d++) dot = __dadd_rn(dot, __dmul_rn((double)qr[d], (double)kr[d]));
        const double v = __dmul_rn(dot, (double)scale);
        lg[j] = v;
        mx = fmax(mx, v);
    }
    red[threadIdx.x] = mx;
    __syncthreads();
    for (int s = 64; s > 0; s >>= 1) {
        if (threadIdx.x < s) red[threadIdx.x] = fmax(red[threadIdx.x], red[threadIdx.x + s]);
        __syncthreads();
    }
    mx = red[0];
    for (int j = threadIdx.x; j < n; j += blockDim.x) lg[j] = exp(lg[j] - mx);
    __syncthreads();
    if (threadIdx.x == 0) {
        double den = 0.0;
        for (int j = 0; j < n; j++) den = __dadd_rn(den, lg[j]);
        den_s = den;
    }
    __syncthreads();
    for (int d = threadIdx.x; d < hd; d += blockDim.x) {
        double acc = 0.0;
        for (int j = 0; j < n; j++) acc = __dadd_rn(acc, __dmul_rn(lg[j], (double)krow(v_pool, j)[d]));
        out[((size_t)t * hq + head) * hd + d] = (float)(acc / den_s);
    }
}

__global__ void swiglu_f32_kernel(const float* gu, int inter, int64_t n, float* out) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int64_t t = i / inter, c = i % inter;
    const float g = gu[t * 2 * inter + c], u = gu[t * 2 * inter + inter + c];
    const float sg = __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-g)));
    out[i] = __fmul_rn(__fmul_rn(g, sg), u);
}

__global__ void argmax_f32_kernel(const float* logits, int vocab, int32_t* out) {
    __shared__ float bv[256];
    __shared__ int bi[256];
    const float* row = logits + (size_t)blockIdx.x * vocab;
    float best = -INFINITY;
    int idx = 0x7fffffff;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x)
        if (row[i] > best) best = row[i], idx = i;  // strided scan visits a thread's ids in rising order
    bv[threadIdx.x] = best;
    bi[threadIdx.x] = idx;
    __syncthreads();
    for (int s = 128; s > 0; s >>= 1) {
        if (threadIdx.x < s) {
            const float ov = bv[threadIdx.x + s];
            const int oi = bi[threadIdx.x + s];
            if (ov > bv[threadIdx.x] || (ov == bv[threadIdx.x] && oi < bi[threadIdx.x])) bv[threadIdx.x] = ov, bi[threadIdx.x] = oi;
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) out[blockIdx.x] = bi[0] == 0x7fffffff ? 0 : bi[0];  // all -inf / NaN -> 0, as a host scan that starts at 0
}

template <typename T>
int32_t regrow(T*& p, size_t elems) {
    if (p) B2_CUDA(cudaFree(p));
    p = nullptr;
    B2_CUDA(cudaMalloc((void**)&p, elems * sizeof(T)));
    return B2_OK;
}

int32_t linear(b2_ctx* ctx, const float* x, const Proj& p, const float* res, int M, float* y) {
    dim3 grid((p.N + 31) / 32, (M + 7) / 8);
    linear_f32_kernel<<<grid, 256, 0, ctx->stream>>>(x, (const float*)p.w, res, M, p.N, p.K, y);
    B2_LAUNCHED(ctx);
    return B2_OK;
}

}  // namespace

void b2_forward_f32_release(b2_model* m) {
    if (!m->w32) return;
    F32Work& w = *m->w32;
    for (float* p : {w.x, w.xn, w.qkv, w.q, w.attn, w.gu, w.act, w.last, w.logits})
        if (p) cudaFree(p);
    delete m->w32;
    m->w32 = nullptr;
}

int32_t b2_forward_f32(b2_model* m, b2_pool* pool, const BatchMetaOut& mo, const int32_t* seq_slot_dev, const int32_t* ids_dev, int T, int B,
                       int n_logits, const int32_t* logit_rows, int max_ctx, float** logits_dev) {
    b2_ctx* ctx = m->ctx;
    const b2_model_config& c = m->cfg;
    B2_REQUIRE(pool->esz == 4, B2_ERR_MSG, "forward: an f32 model needs a pool created for it");
    B2_REQUIRE(max_ctx <= kMaxCtxF32, B2_ERR_UNSUPPORTED, "forward: the f32 path holds contexts of up to 4096 tokens");
    const int H = c.hidden_size, hq = c.num_heads, hkv = c.num_kv_heads, hd = c.head_dim, I = c.intermediate_size, V = c.vocab_size;
    const int qkv_w = (hq + 2 * hkv) * hd;
    if (!m->w32) m->w32 = new F32Work();
    F32Work& w = *m->w32;
    if (T > w.t_cap) {
        B2_CUDA(cudaStreamSynchronize(ctx->stream));
        const size_t t = (size_t)std::max(T, 64) * 5 / 4;
        B2_CHECK(regrow(w.x, t * H));
        B2_CHECK(regrow(w.xn, t * H));
        B2_CHECK(regrow(w.qkv, t * qkv_w));
        B2_CHECK(regrow(w.q, t * hq * hd));
        B2_CHECK(regrow(w.attn, t * hq * hd));
        B2_CHECK(regrow(w.gu, t * 2 * I));
        B2_CHECK(regrow(w.act, t * I));
        w.t_cap = (int)t;
    }
    if (std::max(B, n_logits) > w.b_cap) {
        B2_CUDA(cudaStreamSynchronize(ctx->stream));
        const size_t b = (size_t)std::max(std::max(B, n_logits), 16) * 5 / 4;
        B2_CHECK(regrow(w.last, b * H));
        B2_CHECK(regrow(w.logits, b * V));
        w.b_cap = (int)b;
    }
    cudaStream_t st = ctx->stream;
    const float scale = powf((float)hd, -0.5f);  // attn_scale, config.rs:597-598
    b2_prof_mark(ctx, B2_CLS_ELEMENTWISE);
    embed_f32_kernel<<<T, 128, 0, st>>>((const float*)m->embed, ids_dev, T, H, V, w.x);
    B2_LAUNCHED(ctx);
    Proj head;
    for (int l = 0; l < c.num_layers; l++) {
        const LayerW& L = m->layers[l];
        rms_norm_f32_kernel<<<T, 128, 0, st>>>(w.x, (const float*)L.input_ln, c.rms_norm_eps, H, nullptr, w.xn);
        B2_LAUNCHED(ctx);
        B2_CHECK(linear(ctx, w.xn, L.qkv, nullptr, T, w.qkv));
        rope_kv_f32_kernel<<<T, 256, 0, st>>>(w.qkv, qkv_w, mo.positions, mo.slot_mapping, m->cos_f32, m->sin_f32, hq, hkv, hd, pool->block_size,
                                              (float*)pool->k_layer(l), (float*)pool->v_layer(l), w.q);
        B2_LAUNCHED(ctx);
        attention_f32_kernel<<<dim3(T, hq), 128, (size_t)max_ctx * sizeof(double), st>>>(
            w.q, (const float*)pool->k_layer(l), (const float*)pool->v_layer(l), pool->block_tables, pool->max_blocks, seq_slot_dev, mo.token_seq,
            mo.positions, hq, hkv, hd, pool->block_size, scale, w.attn);
        B2_LAUNCHED(ctx);
        B2_CHECK(linear(ctx, w.attn, L.o, w.x, T, w.x));  // h = x + o_proj(attn): every output reads only its own residual
        rms_norm_f32_kernel<<<T, 128, 0, st>>>(w.x, (const float*)L.post_ln, c.rms_norm_eps, H, nullptr, w.xn);
        B2_LAUNCHED(ctx);
        B2_CHECK(linear(ctx, w.xn, L.gu, nullptr, T, w.gu));
        const int64_t n = (int64_t)T * I;
        swiglu_f32_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(w.gu, I, n, w.act);
        B2_LAUNCHED(ctx);
        B2_CHECK(linear(ctx, w.act, L.down, w.x, T, w.x));
    }
    if (n_logits > 0) {
        rms_norm_f32_kernel<<<n_logits, 128, 0, st>>>(w.x, (const float*)m->norm, c.rms_norm_eps, H, logit_rows, w.last);
        B2_LAUNCHED(ctx);
        head.bits = 0;
        head.N = V;
        head.K = H;
        head.w = m->lm_head;
        B2_CHECK(linear(ctx, w.last, head, nullptr, n_logits, w.logits));
        argmax_f32_kernel<<<n_logits, 256, 0, st>>>(w.logits, V, m->ws.argmax);
        B2_LAUNCHED(ctx);
    }
    B2_CUDA(cudaGetLastError());
    *logits_dev = w.logits;
    return B2_OK;
}
