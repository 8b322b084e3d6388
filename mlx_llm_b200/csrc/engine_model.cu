// Weights container, config parsing and model construction (from weights or synthetic).
#include <dirent.h>
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <cmath>
#include <cstring>

#include "engine.h"
#include "json_mini.h"

namespace {

inline uint16_t h_f2bf(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x0040u);
    u += 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}
inline float h_half2f(uint16_t h) {
    const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1f, man = h & 0x3ff, u;
    if (exp == 0) {
        if (man == 0) {
            u = sign;
        } else {
            exp = 127 - 15 + 1;
            while (!(man & 0x400)) {
                man <<= 1;
                exp--;
            }
            man &= 0x3ff;
            u = sign | (exp << 23) | (man << 13);
        }
    } else if (exp == 31) {
        u = sign | 0x7f800000u | (man << 13);
    } else {
        u = sign | ((exp + 127 - 15) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &u, 4);
    return f;
}

int dtype_size(int dt) { return (dt == B2_DTYPE_BF16 || dt == B2_DTYPE_F16) ? 2 : 4; }

// ---- synthetic generator: must stay bit-identical to its CPU twin used by the parity tests -----
__host__ __device__ inline uint64_t mix64(uint64_t z) {
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}
__device__ inline uint64_t synth_u64(uint64_t seed, uint64_t idx) { return mix64(seed + (idx + 1) * 0x9E3779B97F4A7C15ull); }
__device__ inline float synth_normal(uint64_t seed, uint64_t idx) {
    const uint64_t a = synth_u64(seed, 3 * idx), b = synth_u64(seed, 3 * idx + 1), c = synth_u64(seed, 3 * idx + 2);
    uint32_t sum = 0;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        sum += (uint32_t)((a >> (16 * i)) & 0xffff);
        sum += (uint32_t)((b >> (16 * i)) & 0xffff);
        sum += (uint32_t)((c >> (16 * i)) & 0xffff);
    }
    return __fmul_rn(__fsub_rn((float)sum, 393210.0f), 1.0f / 65536.0f);
}
// A slice [r0, r0+rows) x [c0, c0+cols) of a row-major tensor with `full_cols` columns: element i of the
// slice is element src(i) of the whole tensor, so a tensor-parallel rank draws exactly the values the
// whole model would hold at those positions.
struct Slice {
    int64_t rows, cols, full_cols, r0, c0;
    __host__ __device__ int64_t n() const { return rows * cols; }
    __device__ uint64_t src(int64_t i) const { return (uint64_t)((r0 + i / cols) * full_cols + c0 + i % cols); }
};
__global__ void synth_codes_kernel(uint64_t seed, Slice sl, uint32_t* out) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < sl.n()) out[i] = (uint32_t)(synth_u64(seed, sl.src(i)) >> 16);
}
__global__ void synth_sb_kernel(uint64_t seed_s, uint64_t seed_b, Slice sl, float mul, float mid, uint16_t* scales, uint16_t* biases) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= sl.n()) return;
    const uint64_t g = sl.src(i);
    const uint16_t s = f2bf(__fmul_rn(fabsf(synth_normal(seed_s, g)), mul));
    scales[i] = s;
    biases[i] = f2bf(__fmaf_rn(synth_normal(seed_b, g), 1e-3f, __fmul_rn(-mid, bf2f(s))));
}
__global__ void synth_dense_kernel(uint64_t seed, Slice sl, float std_, uint16_t* out) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < sl.n()) out[i] = f2bf(__fmul_rn(synth_normal(seed, sl.src(i)), std_));
}
__global__ void fill_bf16_kernel(uint16_t v, int64_t n, uint16_t* out) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = v;
}
uint64_t synth_tensor_seed(uint64_t seed, int layer, int which) {
    const uint64_t id = which == 7 ? 1 : which == 8 ? 2 : (uint64_t)(16 * (layer + 1) + which);
    return mix64(seed ^ (0x5EED0000ull + id));
}

int32_t dev_alloc(b2_model* m, size_t bytes, void** out) {
    B2_CUDA(cudaMalloc(out, bytes ? bytes : 16));
    m->allocs.push_back(*out);
    m->weight_bytes += (int64_t)bytes;
    return B2_OK;
}

void proj_dims(const b2_model_config& c, int which, int& out, int& in) {
    const int qd = c.num_heads * c.head_dim, kvd = c.num_kv_heads * c.head_dim;
    switch (which) {
        case 0: out = qd; in = c.hidden_size; break;
        case 1: case 2: out = kvd; in = c.hidden_size; break;
        case 3: out = c.hidden_size; in = qd; break;
        case 4: case 5: out = c.intermediate_size; in = c.hidden_size; break;
        default: out = c.hidden_size; in = c.intermediate_size; break;
    }
}

int32_t alloc_proj(b2_model* m, Proj& p, int N, int K, int bits) {
    p.N = N;
    p.K = K;
    p.bits = bits;
    if (bits == 0) {
        B2_CHECK(dev_alloc(m, (size_t)N * K * (m->f32 ? 4 : 2), &p.w));
    } else {
        B2_REQUIRE(K % 64 == 0, B2_ERR_UNSUPPORTED, "quantized projection: group size 64 must divide the input dimension");
        B2_CHECK(dev_alloc(m, (size_t)N * K * bits / 8, &p.w));
        B2_CHECK(dev_alloc(m, (size_t)N * (K / 64) * 2, (void**)&p.scales));
        B2_CHECK(dev_alloc(m, (size_t)N * (K / 64) * 2, (void**)&p.biases));
    }
    return B2_OK;
}

int32_t validate_cfg(const b2_model_config& c) {
    B2_REQUIRE(c.num_layers > 0 && c.hidden_size > 0 && c.num_heads > 0 && c.num_kv_heads > 0 && c.head_dim > 0 &&
                   c.intermediate_size > 0 && c.vocab_size > 0,
               B2_ERR_CONFIG, "model config: non-positive dimension");
    B2_REQUIRE(c.num_heads % c.num_kv_heads == 0, B2_ERR_CONFIG, "model config: num_heads must be a multiple of num_kv_heads");
    const int g = c.num_heads / c.num_kv_heads;
    B2_REQUIRE(g == 1 || g == 2 || g == 4 || g == 8, B2_ERR_UNSUPPORTED, "model config: q heads per kv head must be 1, 2, 4 or 8");
    B2_REQUIRE(c.head_dim == 64 || c.head_dim == 128, B2_ERR_UNSUPPORTED, "model config: head_dim must be 64 or 128");
    B2_REQUIRE(c.hidden_size % 8 == 0 && c.intermediate_size % 8 == 0, B2_ERR_UNSUPPORTED,
               "model config: hidden and intermediate sizes must be multiples of 8");
    B2_REQUIRE(c.quant_bits == 0 || c.quant_bits == 4 || c.quant_bits == 8, B2_ERR_UNSUPPORTED, "model config: quantization bits must be 4 or 8");
    B2_REQUIRE(c.quant_bits == 0 || c.quant_group == 64, B2_ERR_UNSUPPORTED, "model config: quantization group size must be 64");
    B2_REQUIRE(!c.compute_f32 || (c.quant_bits == 0 && c.qk_norm == 0), B2_ERR_UNSUPPORTED,
               "model config: the f32 path takes dense projections without q/k norm only");
    return B2_OK;
}

// This rank's share of the heads and of the MLP width (the whole model without a group).
int32_t set_local_dims(b2_model* m, b2_tp_group* tp) {
    const b2_model_config& c = m->cfg;
    const int world = tp ? tp->world : 1;
    B2_REQUIRE(!tp || tp->ctx == m->ctx, B2_ERR_MSG, "tensor-parallel group belongs to another context");
    B2_REQUIRE(c.num_kv_heads % world == 0, B2_ERR_UNSUPPORTED, "tensor parallelism: the group size must divide num_kv_heads");
    if (world > 1) {
        B2_REQUIRE(c.intermediate_size % (64 * world) == 0, B2_ERR_UNSUPPORTED,
                   "tensor parallelism: every rank's slice of the MLP width must be a multiple of the quantization group (64)");
        B2_REQUIRE((c.num_heads / world * c.head_dim) % 64 == 0, B2_ERR_UNSUPPORTED,
                   "tensor parallelism: every rank's slice of the attention width must be a multiple of 64");
    }
    B2_REQUIRE(world == 1 || !c.compute_f32, B2_ERR_UNSUPPORTED, "tensor parallelism: not available on the f32 path");
    m->tp = world > 1 ? tp : nullptr;
    m->hq_l = c.num_heads / world;
    m->hkv_l = c.num_kv_heads / world;
    m->inter_l = c.intermediate_size / world;
    return B2_OK;
}

// The large-M projection kernel reads scale and bias of 32 feature rows at one K group in one instruction: a second
// copy of both, transposed and interleaved, makes that one line instead of 64.  (Not counted in weight_bytes: it is a
// derived layout, 1/9 of the packed 4-bit codes.)
static int32_t build_sbt(b2_model* m, Proj& p) {
    if (p.bits == 0 || p.sbt) return B2_OK;
    const int G = p.K / 64;
    B2_CUDA(cudaMalloc((void**)&p.sbt, (size_t)p.N * G * 4));
    m->allocs.push_back(p.sbt);
    return b2_gemm_build_sbt(m->ctx, p.scales, p.biases, p.N, G, p.sbt);
}

int32_t finish_model(b2_model* m) {
    for (auto& L : m->layers) {
        B2_CHECK(build_sbt(m, L.qkv));
        B2_CHECK(build_sbt(m, L.o));
        B2_CHECK(build_sbt(m, L.gu));
        B2_CHECK(build_sbt(m, L.down));
    }
    B2_CUDA(cudaStreamSynchronize(m->ctx->stream));
    m->inv_freq.resize(m->cfg.head_dim / 2);
    B2_CHECK(b2_rope_inv_freq(m->cfg.head_dim, m->cfg.rope_theta, m->cfg.rope_kind, m->cfg.rope_factor, m->cfg.rope_low_freq_factor,
                              m->cfg.rope_high_freq_factor, m->cfg.rope_original_context, m->inv_freq.data()));
    B2_CUDA(cudaEventCreate(&m->ev0));
    B2_CUDA(cudaEventCreate(&m->ev1));
    return B2_OK;
}

}  // namespace

int32_t b2_model_ensure_rope(b2_model* m, int positions) {
    if (positions <= m->rope_positions) return B2_OK;
    int n = std::max(4096, m->rope_positions);
    while (n < positions) n *= 2;
    const int half = m->cfg.head_dim / 2;
    std::vector<uint16_t> c((size_t)n * half), s((size_t)n * half);
    B2_CHECK(b2_rope_tables(m->inv_freq.data(), half, n, c.data(), s.data()));
    B2_CUDA(cudaStreamSynchronize(m->ctx->stream));
    if (m->cos_tab) cudaFree(m->cos_tab);
    if (m->sin_tab) cudaFree(m->sin_tab);
    B2_CUDA(cudaMalloc((void**)&m->cos_tab, c.size() * 2));
    B2_CUDA(cudaMalloc((void**)&m->sin_tab, s.size() * 2));
    B2_CUDA(cudaMemcpyAsync(m->cos_tab, c.data(), c.size() * 2, cudaMemcpyHostToDevice, m->ctx->stream));
    B2_CUDA(cudaMemcpyAsync(m->sin_tab, s.data(), s.size() * 2, cudaMemcpyHostToDevice, m->ctx->stream));
    if (m->f32) {  // the f32 path rotates with unrounded tables: angle = pos*inv_freq in f32, cosf / sinf on the host (rope.rs:183-208)
        std::vector<float> cf((size_t)n * half), sf((size_t)n * half);
        for (int pos = 0; pos < n; pos++)
            for (int i = 0; i < half; i++) {
                const float ang = (float)pos * m->inv_freq[i];
                cf[(size_t)pos * half + i] = std::cos(ang);
                sf[(size_t)pos * half + i] = std::sin(ang);
            }
        if (m->cos_f32) cudaFree(m->cos_f32);
        if (m->sin_f32) cudaFree(m->sin_f32);
        B2_CUDA(cudaMalloc((void**)&m->cos_f32, cf.size() * 4));
        B2_CUDA(cudaMalloc((void**)&m->sin_f32, sf.size() * 4));
        B2_CUDA(cudaMemcpyAsync(m->cos_f32, cf.data(), cf.size() * 4, cudaMemcpyHostToDevice, m->ctx->stream));
        B2_CUDA(cudaMemcpyAsync(m->sin_f32, sf.data(), sf.size() * 4, cudaMemcpyHostToDevice, m->ctx->stream));
    }
    B2_CUDA(cudaStreamSynchronize(m->ctx->stream));  // ordered on the context stream; host buffers die here
    m->rope_positions = n;
    return B2_OK;
}

extern "C" {

// ---- Weights ------------------------------------------------------------------------------------
int32_t b2_weights_new(b2_weights** out) {
    B2_REQUIRE(out, B2_ERR_MSG, "b2_weights_new: null out");
    *out = new b2_weights();
    return B2_OK;
}
int32_t b2_weights_free(b2_weights* w) {
    if (!w) return B2_OK;
    for (auto& mf : w->maps)
        if (mf.base) munmap(mf.base, mf.len);
    delete w;
    return B2_OK;
}
int32_t b2_weights_contains(const b2_weights* w, const char* name) { return w && name && w->t.count(name) ? 1 : 0; }
int32_t b2_weights_add(b2_weights* w, const char* name, int32_t dtype, const int64_t* shape, int32_t ndim, const void* data_host) {
    B2_REQUIRE(w && name && shape && data_host && ndim >= 0, B2_ERR_MSG, "b2_weights_add: null argument");
    B2_REQUIRE(dtype >= B2_DTYPE_F32 && dtype <= B2_DTYPE_I32, B2_ERR_MSG, "b2_weights_add: unknown dtype");
    HostTensor t;
    t.dtype = dtype;
    t.shape.assign(shape, shape + ndim);
    t.nbytes = (size_t)t.numel() * dtype_size(dtype);
    t.owned.assign((const uint8_t*)data_host, (const uint8_t*)data_host + t.nbytes);
    auto& slot = w->t[name];
    slot = std::move(t);
    slot.ptr = slot.owned.data();
    return B2_OK;
}

static int32_t load_safetensors_file(b2_weights* w, const std::string& path) {
    int fd = open(path.c_str(), O_RDONLY);
    B2_REQUIRE(fd >= 0, B2_ERR_IO, "cannot open " + path);
    struct stat st;
    if (fstat(fd, &st) != 0 || st.st_size < 8) {
        close(fd);
        return b2_fail(B2_ERR_IO, "cannot stat or file too small: " + path);
    }
    void* base = mmap(nullptr, (size_t)st.st_size, PROT_READ, MAP_PRIVATE, fd, 0);
    close(fd);
    B2_REQUIRE(base != MAP_FAILED, B2_ERR_IO, "mmap failed: " + path);
    w->maps.push_back(MappedFile{base, (size_t)st.st_size});
    const uint8_t* b = (const uint8_t*)base;
    uint64_t hlen = 0;
    memcpy(&hlen, b, 8);
    B2_REQUIRE(hlen > 0 && 8 + hlen <= (uint64_t)st.st_size, B2_ERR_IO, "bad safetensors header length: " + path);
    std::string header((const char*)b + 8, (size_t)hlen), err;
    auto root = b2json::parse(header, err);
    B2_REQUIRE(root && root->kind == b2json::Value::Object, B2_ERR_IO, "bad safetensors header in " + path + ": " + err);
    const uint8_t* data = b + 8 + hlen;
    const size_t data_len = (size_t)st.st_size - 8 - (size_t)hlen;
    for (auto& kv : root->obj) {
        if (kv.first == "__metadata__") continue;
        const b2json::Value* dt = kv.second->get("dtype");
        const b2json::Value* sh = kv.second->get("shape");
        const b2json::Value* off = kv.second->get("data_offsets");
        B2_REQUIRE(dt && sh && off && off->arr.size() == 2, B2_ERR_IO, "malformed safetensors entry " + kv.first);
        HostTensor t;
        if (dt->str == "F32") t.dtype = B2_DTYPE_F32;
        else if (dt->str == "BF16") t.dtype = B2_DTYPE_BF16;
        else if (dt->str == "F16") t.dtype = B2_DTYPE_F16;
        else if (dt->str == "U32") t.dtype = B2_DTYPE_U32;
        else if (dt->str == "I32") t.dtype = B2_DTYPE_I32;
        else continue;  // tensors of other dtypes are not part of this path
        for (auto& d : sh->arr) t.shape.push_back((int64_t)d->num);
        const size_t s = (size_t)off->arr[0]->num, e = (size_t)off->arr[1]->num;
        B2_REQUIRE(s <= e && e <= data_len, B2_ERR_IO, "safetensors offsets out of range for " + kv.first);
        t.ptr = data + s;
        t.nbytes = e - s;
        B2_REQUIRE(t.nbytes == (size_t)t.numel() * dtype_size(t.dtype), B2_ERR_IO, "safetensors size mismatch for " + kv.first);
        w->t[kv.first] = std::move(t);
    }
    return B2_OK;
}

// Weights::from_dir / from_file (src/primitives/weights.rs:36-56): a file, or every *.safetensors
// of a directory.
int32_t b2_weights_from_dir(const char* path, b2_weights** out) {
    B2_REQUIRE(path && out, B2_ERR_MSG, "b2_weights_from_dir: null argument");
    struct stat st;
    B2_REQUIRE(stat(path, &st) == 0, B2_ERR_IO, std::string("no such file or directory: ") + path);
    b2_weights* w = new b2_weights();
    std::vector<std::string> files;
    if (S_ISDIR(st.st_mode)) {
        DIR* d = opendir(path);
        if (d) {
            while (dirent* e = readdir(d)) {
                std::string n = e->d_name;
                if (n.size() > 12 && n.substr(n.size() - 12) == ".safetensors") files.push_back(std::string(path) + "/" + n);
            }
            closedir(d);
        }
        std::sort(files.begin(), files.end());
    } else {
        files.push_back(path);
    }
    if (files.empty()) {
        b2_weights_free(w);
        return b2_fail(B2_ERR_IO, std::string("no .safetensors files in ") + path);
    }
    for (auto& f : files) {
        int32_t rc = load_safetensors_file(w, f);
        if (rc != B2_OK) {
            b2_weights_free(w);
            return rc;
        }
    }
    *out = w;
    return B2_OK;
}

// ---- ModelConfig::from_json (src/config.rs:315-502), Llama / Qwen3 subset -------------------------
int32_t b2_model_config_from_json(const char* json, b2_model_config* out) {
    B2_REQUIRE(json && out, B2_ERR_MSG, "b2_model_config_from_json: null argument");
    std::string err;
    auto root = b2json::parse(json, err);
    B2_REQUIRE(root && root->kind == b2json::Value::Object, B2_ERR_CONFIG, "config.json: " + (err.empty() ? std::string("not an object") : err));
    const b2json::Value* v = root.get();
    // Architecture::from_config (config.rs:64-113)
    std::string hay;
    if (auto a = v->get("architectures"))
        if (a->kind == b2json::Value::Array && !a->arr.empty() && a->arr[0]->kind == b2json::Value::String) hay += a->arr[0]->str;
    hay += " ";
    if (auto mt = v->get("model_type"))
        if (mt->kind == b2json::Value::String) hay += mt->str;
    const bool no_arch = hay == " ";
    for (auto& ch : hay) ch = (char)tolower(ch);
    auto has = [&](const char* s) { return hay.find(s) != std::string::npos; };
    int qk_norm = 0;
    if (has("qwen3_vl") || has("qwen3vl") || has("qwen3_5") || has("qwen35") || has("qwen2_moe") || has("qwen2moe") || has("gemma2") ||
        has("glm4") || has("deepseek") || has("phi3")) {
        return b2_fail(B2_ERR_UNSUPPORTED, "config.json: architecture outside the Llama / Qwen3 dense-decoder subset: " + hay);
    } else if (has("qwen3")) {
        qk_norm = 1;
    } else if (!(has("llama") || has("mistral") || has("qwen2") || no_arch)) {
        return b2_fail(B2_ERR_UNSUPPORTED, "config.json: unsupported architecture: " + hay);
    }
    auto req_int = [&](const char* key, int32_t& dst) -> int32_t {
        long long x;
        const b2json::Value* f = v->get(key);
        if (!f || !f->as_i64(x)) return b2_fail(B2_ERR_CONFIG, std::string("config.json missing integer `") + key + "`");
        dst = (int32_t)x;
        return B2_OK;
    };
    auto opt_int = [&](const char* key, int32_t dflt) -> int32_t {
        long long x;
        const b2json::Value* f = v->get(key);
        return (f && f->as_i64(x)) ? (int32_t)x : dflt;
    };
    auto opt_f32 = [&](const b2json::Value* o, const char* key, float dflt) -> float {
        double x;
        const b2json::Value* f = o ? o->get(key) : nullptr;
        return (f && f->as_f64(x)) ? (float)x : dflt;
    };
    b2_model_config c{};
    B2_CHECK(req_int("hidden_size", c.hidden_size));
    B2_CHECK(req_int("num_attention_heads", c.num_heads));
    B2_CHECK(req_int("num_hidden_layers", c.num_layers));
    B2_CHECK(req_int("intermediate_size", c.intermediate_size));
    B2_CHECK(req_int("vocab_size", c.vocab_size));
    B2_REQUIRE(c.num_heads > 0, B2_ERR_CONFIG, "config.json: num_attention_heads must be positive");
    c.head_dim = opt_int("head_dim", c.hidden_size / c.num_heads);
    c.num_kv_heads = opt_int("num_key_value_heads", c.num_heads);
    c.rms_norm_eps = opt_f32(v, "rms_norm_eps", 1e-5f);
    c.rope_theta = opt_f32(v, "rope_theta", 500000.0f);
    c.qk_norm = qk_norm;
    if (auto tw = v->get("tie_word_embeddings")) c.tie_word_embeddings = tw->kind == b2json::Value::Bool && tw->b;
    c.rope_kind = 0;
    c.rope_factor = 1.f;
    c.rope_low_freq_factor = 1.f;
    c.rope_high_freq_factor = 4.f;
    c.rope_original_context = 8192.f;
    if (auto rs = v->get("rope_scaling")) {
        if (rs->kind == b2json::Value::Object) {
            const b2json::Value* ty = rs->get("rope_type");
            if (!ty) ty = rs->get("type");
            const bool is_llama3 = !(ty && ty->kind == b2json::Value::String) || ty->str == "llama3";  // a bare factor block counts
            if (is_llama3) {
                c.rope_kind = 1;
                c.rope_factor = opt_f32(rs, "factor", 1.f);
                c.rope_low_freq_factor = opt_f32(rs, "low_freq_factor", 1.f);
                c.rope_high_freq_factor = opt_f32(rs, "high_freq_factor", 4.f);
                c.rope_original_context = opt_f32(rs, "original_max_position_embeddings", 8192.f);
            }
        }
    }
    if (auto q = v->get("quantization")) {
        long long g, b;
        const b2json::Value* gs = q->get("group_size");
        const b2json::Value* bs = q->get("bits");
        if (gs && bs && gs->as_i64(g) && bs->as_i64(b)) {
            c.quant_group = (int32_t)g;
            c.quant_bits = (int32_t)b;
        }
    }
    *out = c;
    return B2_OK;
}

// ---- CausalLm::from_weights_with (src/models/llama.rs:57-303) ---------------------------------------
// `dst` receives bf16 (every tensor is cast as llama.rs:71 does), or f32 for an f32 model (F32 sources unchanged,
// BF16 / F16 sources widened).
static int32_t upload_bf16(b2_model* m, const b2_weights* w, const std::string& key, int64_t expect_elems, uint16_t* dst) {
    auto it = w->t.find(key);
    B2_REQUIRE(it != w->t.end(), B2_ERR_MISSING_TENSOR, "missing tensor `" + key + "`");
    const HostTensor& t = it->second;
    B2_REQUIRE(t.numel() == expect_elems, B2_ERR_CONFIG, "tensor `" + key + "` has an unexpected size");
    if (m->f32) {
        B2_REQUIRE(t.dtype == B2_DTYPE_F32 || t.dtype == B2_DTYPE_F16 || t.dtype == B2_DTYPE_BF16, B2_ERR_CONFIG,
                   "tensor `" + key + "` is not a floating-point tensor");
        std::vector<float> tmp;
        const float* src = (const float*)t.ptr;
        if (t.dtype != B2_DTYPE_F32) {
            tmp.resize((size_t)expect_elems);
            const uint16_t* h = (const uint16_t*)t.ptr;
            for (int64_t i = 0; i < expect_elems; i++) {
                if (t.dtype == B2_DTYPE_F16) {
                    tmp[i] = h_half2f(h[i]);
                } else {
                    const uint32_t u = (uint32_t)h[i] << 16;
                    memcpy(&tmp[i], &u, 4);
                }
            }
            src = tmp.data();
        }
        B2_CUDA(cudaMemcpyAsync(dst, src, (size_t)expect_elems * 4, cudaMemcpyHostToDevice, m->ctx->stream));
        B2_CUDA(cudaStreamSynchronize(m->ctx->stream));
        return B2_OK;
    }
    if (t.dtype == B2_DTYPE_BF16) {
        // every copy goes through the context stream (a plain cudaMemcpy is not ordered against it)
        B2_CUDA(cudaMemcpyAsync(dst, t.ptr, (size_t)expect_elems * 2, cudaMemcpyHostToDevice, m->ctx->stream));
        B2_CUDA(cudaStreamSynchronize(m->ctx->stream));
        return B2_OK;
    }
    B2_REQUIRE(t.dtype == B2_DTYPE_F32 || t.dtype == B2_DTYPE_F16, B2_ERR_CONFIG, "tensor `" + key + "` is not a floating-point tensor");
    std::vector<uint16_t> tmp((size_t)expect_elems);
    if (t.dtype == B2_DTYPE_F32) {
        const float* f = (const float*)t.ptr;
        for (int64_t i = 0; i < expect_elems; i++) tmp[i] = h_f2bf(f[i]);
    } else {
        const uint16_t* h = (const uint16_t*)t.ptr;
        for (int64_t i = 0; i < expect_elems; i++) tmp[i] = h_f2bf(h_half2f(h[i]));
    }
    B2_CUDA(cudaMemcpyAsync(dst, tmp.data(), (size_t)expect_elems * 2, cudaMemcpyHostToDevice, m->ctx->stream));
    B2_CUDA(cudaStreamSynchronize(m->ctx->stream));
    return B2_OK;
}

// Load one logical projection into rows [row0, row0+N) of a (possibly fused) Proj.
static int32_t load_proj_rows(b2_model* m, const b2_weights* w, const std::string& key, Proj& dst, int row0, int N, int K,
                              const b2_quant_spec* quant) {
    const std::string base = key.size() > 7 && key.substr(key.size() - 7) == ".weight" ? key.substr(0, key.size() - 7) : key;
    B2_REQUIRE(!w->t.count(base + ".bias"), B2_ERR_UNSUPPORTED, "projection bias (`" + base + ".bias`) is outside the Llama / Qwen3 subset");
    const bool stored = w->t.count(base + ".scales") > 0;
    if (stored) {
        B2_REQUIRE(m->cfg.quant_bits != 0, B2_ERR_CONFIG,
                   "snapshot stores quantized tensor `" + base + ".scales` but config.json has no `quantization` block");
        B2_REQUIRE(dst.bits == m->cfg.quant_bits, B2_ERR_CONFIG, "mixed dense / quantized projections in one fused projection");
        auto wt = w->t.find(key);
        B2_REQUIRE(wt != w->t.end(), B2_ERR_MISSING_TENSOR, "missing tensor `" + key + "`");
        const size_t words = (size_t)N * K * dst.bits / 32;
        B2_REQUIRE(wt->second.dtype == B2_DTYPE_U32 && (size_t)wt->second.numel() == words, B2_ERR_CONFIG,
                   "tensor `" + key + "` is not a packed u32 weight of the expected size");
        B2_CUDA(cudaMemcpyAsync((uint32_t*)dst.w + (size_t)row0 * K * dst.bits / 32, wt->second.ptr, words * 4, cudaMemcpyHostToDevice,
                                m->ctx->stream));
        B2_CUDA(cudaStreamSynchronize(m->ctx->stream));
        B2_CHECK(upload_bf16(m, w, base + ".scales", (int64_t)N * (K / 64), dst.scales + (size_t)row0 * (K / 64)));
        B2_CHECK(upload_bf16(m, w, base + ".biases", (int64_t)N * (K / 64), dst.biases + (size_t)row0 * (K / 64)));
        return B2_OK;
    }
    if (dst.bits == 0)
        return upload_bf16(m, w, key, (int64_t)N * K, reinterpret_cast<uint16_t*>((uint8_t*)dst.w + (size_t)row0 * K * (m->f32 ? 4 : 2)));
    // quantize-on-load (Projection::load_with_bias, projection.rs:57-71)
    (void)quant;
    uint16_t* tmp = nullptr;
    B2_CUDA(cudaMalloc((void**)&tmp, (size_t)N * K * 2));
    int32_t rc = upload_bf16(m, w, key, (int64_t)N * K, tmp);
    if (rc == B2_OK)
        rc = b2_quantize_launch(m->ctx, tmp, N, K, dst.bits, (uint32_t*)dst.w + (size_t)row0 * K * dst.bits / 32,
                                dst.scales + (size_t)row0 * (K / 64), dst.biases + (size_t)row0 * (K / 64));
    cudaStreamSynchronize(m->ctx->stream);
    cudaFree(tmp);
    return rc;
}

// Tensor-parallel load: rows [r0, r0+nr) x columns [c0, c0+nc) of one logical projection go to rows
// dst_row0.. of `dst` (whose K is nc).  The whole projection is staged on the device (and quantized there
// when the snapshot is dense: groups run along the input dimension, so slicing after quantization equals
// quantizing the slice), then the slice is copied out with strided copies.
static int32_t load_proj_slice(b2_model* m, const b2_weights* w, const std::string& key, Proj& dst, int dst_row0, int N, int K, int r0,
                               int nr, int c0, int nc, const b2_quant_spec* quant) {
    if (r0 == 0 && nr == N && c0 == 0 && nc == K) return load_proj_rows(m, w, key, dst, dst_row0, N, K, quant);
    Proj full;
    full.N = N;
    full.K = K;
    full.bits = dst.bits;
    const int bits = dst.bits;
    cudaStream_t st = m->ctx->stream;
    int32_t rc = B2_OK;
    if (cudaMalloc(&full.w, bits ? (size_t)N * K * bits / 8 : (size_t)N * K * 2) != cudaSuccess) rc = b2_fail(B2_ERR_CUDA, "out of device memory while staging `" + key + "`");
    if (rc == B2_OK && bits) {
        if (cudaMalloc((void**)&full.scales, (size_t)N * (K / 64) * 2) != cudaSuccess || cudaMalloc((void**)&full.biases, (size_t)N * (K / 64) * 2) != cudaSuccess)
            rc = b2_fail(B2_ERR_CUDA, "out of device memory while staging `" + key + "`");
    }
    if (rc == B2_OK) rc = load_proj_rows(m, w, key, full, 0, N, K, quant);
    auto copy2d = [&](void* d, size_t dpitch, const void* s_, size_t spitch, size_t width) {
        if (rc == B2_OK && cudaMemcpy2DAsync(d, dpitch, s_, spitch, width, (size_t)nr, cudaMemcpyDeviceToDevice, st) != cudaSuccess)
            rc = b2_fail(B2_ERR_CUDA, "strided copy of `" + key + "` failed");
    };
    if (bits == 0) {
        copy2d((uint16_t*)dst.w + (size_t)dst_row0 * nc, (size_t)nc * 2, (const uint16_t*)full.w + (size_t)r0 * K + c0, (size_t)K * 2, (size_t)nc * 2);
    } else {
        const size_t fw = (size_t)K * bits / 8, sw = (size_t)nc * bits / 8;  // bytes of codes per row
        copy2d((uint8_t*)dst.w + (size_t)dst_row0 * sw, sw, (const uint8_t*)full.w + (size_t)r0 * fw + (size_t)c0 * bits / 8, fw, sw);
        const size_t fg = (size_t)(K / 64) * 2, sg = (size_t)(nc / 64) * 2;
        copy2d((uint8_t*)dst.scales + (size_t)dst_row0 * sg, sg, (const uint8_t*)full.scales + (size_t)r0 * fg + (size_t)(c0 / 64) * 2, fg, sg);
        copy2d((uint8_t*)dst.biases + (size_t)dst_row0 * sg, sg, (const uint8_t*)full.biases + (size_t)r0 * fg + (size_t)(c0 / 64) * 2, fg, sg);
    }
    cudaStreamSynchronize(st);
    if (full.w) cudaFree(full.w);
    if (full.scales) cudaFree(full.scales);
    if (full.biases) cudaFree(full.biases);
    return rc;
}

int32_t b2_model_from_weights_tp(b2_ctx* ctx, const b2_weights* w, const char* prefix, const b2_model_config* cfg,
                                 const b2_quant_spec* quant, b2_tp_group* tp, b2_model** out) {
    B2_REQUIRE(ctx && w && cfg && out, B2_ERR_MSG, "b2_model_from_weights: null argument");
    B2_CUDA(cudaSetDevice(ctx->device));
    b2_model_config c = *cfg;
    // a stored `quantization` block wins for stored triplets; a load-time spec quantizes dense weights
    int bits = c.quant_bits;
    if (quant) {
        B2_REQUIRE(quant->group_size == 64 && (quant->bits == 4 || quant->bits == 8), B2_ERR_UNSUPPORTED,
                   "b2_model_from_weights: QuantSpec must be group 64 with 4 or 8 bits");
        B2_REQUIRE(bits == 0 || bits == quant->bits, B2_ERR_CONFIG, "b2_model_from_weights: QuantSpec disagrees with the stored quantization");
        bits = quant->bits;
        c.quant_bits = bits;
        c.quant_group = 64;
    }
    B2_CHECK(validate_cfg(c));
    std::string pre = prefix ? prefix : "";
    auto join = [](const std::string& a, const std::string& b) { return a.empty() ? b : a + "." + b; };
    const std::string root = join(pre, "model");
    auto P = [&](const std::string& s) { return join(root, s); };

    b2_model* m = new b2_model();
    m->ctx = ctx;
    m->cfg = c;
    m->quantized = bits != 0;
    m->f32 = c.compute_f32 != 0;
    const size_t es = m->f32 ? 4 : 2;  // bytes per element of every dense tensor
    auto fail = [&](int32_t rc) {
        b2_model_free(m);
        return rc;
    };
#define TRY(x)                          \
    do {                                \
        int32_t rc__ = (x);             \
        if (rc__ != B2_OK) return fail(rc__); \
    } while (0)
    TRY(set_local_dims(m, tp));
    const int rank = m->tp ? m->tp->rank : 0, world = m->tp ? m->tp->world : 1;
    const int H = c.hidden_size, V = c.vocab_size, hd = c.head_dim;
    TRY(dev_alloc(m, (size_t)V * H * es, (void**)&m->embed));
    TRY(upload_bf16(m, w, P("embed_tokens.weight"), (int64_t)V * H, m->embed));
    TRY(dev_alloc(m, (size_t)H * es, (void**)&m->norm));
    TRY(upload_bf16(m, w, P("norm.weight"), H, m->norm));
    if (c.tie_word_embeddings) {
        m->lm_head = m->embed;  // llama.rs:124-128
    } else {
        TRY(dev_alloc(m, (size_t)V * H * es, (void**)&m->lm_head));
        TRY(upload_bf16(m, w, join(pre, "lm_head.weight"), (int64_t)V * H, m->lm_head));
    }
    m->layers.resize(c.num_layers);
    const int qd = c.num_heads * hd, kvd = c.num_kv_heads * hd, I = c.intermediate_size;
    for (int l = 0; l < c.num_layers; l++) {
        LayerW& L = m->layers[l];
        auto LP = [&](const std::string& s) { return P("layers." + std::to_string(l) + "." + s); };
        TRY(dev_alloc(m, (size_t)H * es, (void**)&L.input_ln));
        TRY(upload_bf16(m, w, LP("input_layernorm.weight"), H, L.input_ln));
        TRY(dev_alloc(m, (size_t)H * es, (void**)&L.post_ln));
        TRY(upload_bf16(m, w, LP("post_attention_layernorm.weight"), H, L.post_ln));
        if (c.qk_norm) {
            TRY(dev_alloc(m, (size_t)hd * es, (void**)&L.q_norm));
            TRY(upload_bf16(m, w, LP("self_attn.q_norm.weight"), hd, L.q_norm));
            TRY(dev_alloc(m, (size_t)hd * es, (void**)&L.k_norm));
            TRY(upload_bf16(m, w, LP("self_attn.k_norm.weight"), hd, L.k_norm));
        }
        const int qd_l = qd / world, kvd_l = kvd / world, I_l = I / world;  // this rank's rows / columns
        TRY(alloc_proj(m, L.qkv, qd_l + 2 * kvd_l, H, bits));
        TRY(load_proj_slice(m, w, LP("self_attn.q_proj.weight"), L.qkv, 0, qd, H, rank * qd_l, qd_l, 0, H, quant));
        TRY(load_proj_slice(m, w, LP("self_attn.k_proj.weight"), L.qkv, qd_l, kvd, H, rank * kvd_l, kvd_l, 0, H, quant));
        TRY(load_proj_slice(m, w, LP("self_attn.v_proj.weight"), L.qkv, qd_l + kvd_l, kvd, H, rank * kvd_l, kvd_l, 0, H, quant));
        TRY(alloc_proj(m, L.o, H, qd_l, bits));
        TRY(load_proj_slice(m, w, LP("self_attn.o_proj.weight"), L.o, 0, H, qd, 0, H, rank * qd_l, qd_l, quant));
        TRY(alloc_proj(m, L.gu, 2 * I_l, H, bits));
        TRY(load_proj_slice(m, w, LP("mlp.gate_proj.weight"), L.gu, 0, I, H, rank * I_l, I_l, 0, H, quant));
        TRY(load_proj_slice(m, w, LP("mlp.up_proj.weight"), L.gu, I_l, I, H, rank * I_l, I_l, 0, H, quant));
        TRY(alloc_proj(m, L.down, H, I_l, bits));
        TRY(load_proj_slice(m, w, LP("mlp.down_proj.weight"), L.down, 0, H, I, 0, H, rank * I_l, I_l, quant));
    }
    TRY(finish_model(m));
#undef TRY
    B2_CUDA(cudaStreamSynchronize(ctx->stream));
    *out = m;
    return B2_OK;
}

int32_t b2_model_from_weights(b2_ctx* ctx, const b2_weights* w, const char* prefix, const b2_model_config* cfg,
                              const b2_quant_spec* quant, b2_model** out) {
    return b2_model_from_weights_tp(ctx, w, prefix, cfg, quant, nullptr, out);
}

int32_t b2_model_synthetic_tp(b2_ctx* ctx, const b2_model_config* cfg, uint64_t seed, b2_tp_group* tp, b2_model** out) {
    B2_REQUIRE(ctx && cfg && out, B2_ERR_MSG, "b2_model_synthetic: null argument");
    B2_CUDA(cudaSetDevice(ctx->device));
    b2_model_config c = *cfg;
    if (c.quant_bits && !c.quant_group) c.quant_group = 64;
    B2_CHECK(validate_cfg(c));
    B2_REQUIRE(!c.compute_f32, B2_ERR_UNSUPPORTED, "b2_model_synthetic: the synthetic recipe draws bf16 weights; the f32 path loads weights");
    b2_model* m = new b2_model();
    m->ctx = ctx;
    m->cfg = c;
    m->quantized = c.quant_bits != 0;
    auto fail = [&](int32_t rc) {
        b2_model_free(m);
        return rc;
    };
#define TRY(x)                          \
    do {                                \
        int32_t rc__ = (x);             \
        if (rc__ != B2_OK) return fail(rc__); \
    } while (0)
    TRY(set_local_dims(m, tp));
    const int rank = m->tp ? m->tp->rank : 0, world = m->tp ? m->tp->world : 1;
    cudaStream_t st = ctx->stream;
    auto blocks = [](int64_t n) { return (unsigned)((n + 255) / 256); };
    auto dense = [&](uint16_t* dst, int64_t n, int layer, int which) {
        synth_dense_kernel<<<blocks(n), 256, 0, st>>>(synth_tensor_seed(seed, layer, which), Slice{1, n, n, 0, 0}, 0.02f, dst);
    };
    auto ones = [&](uint16_t* dst, int64_t n) { fill_bf16_kernel<<<blocks(n), 256, 0, st>>>(0x3f80, n, dst); };
    const int H = c.hidden_size, V = c.vocab_size, hd = c.head_dim, I = c.intermediate_size;
    TRY(dev_alloc(m, (size_t)V * H * 2, (void**)&m->embed));
    dense(m->embed, (int64_t)V * H, 0, 7);
    TRY(dev_alloc(m, (size_t)V * H * 2, (void**)&m->lm_head));
    dense(m->lm_head, (int64_t)V * H, 0, 8);
    TRY(dev_alloc(m, (size_t)H * 2, (void**)&m->norm));
    ones(m->norm, H);
    m->layers.resize(c.num_layers);
    const int bits = c.quant_bits;
    const float mul = bits == 4 ? 0.02f / 7.5f : 0.02f / 127.5f, mid = bits == 4 ? 8.f : 128.f;
    // rows [r0, r0+nr) x columns [c0, c0+nc) of logical projection `which`, written to rows dst_row0.. of p
    auto fill = [&](Proj& p, int dst_row0, int layer, int which, int r0, int nr, int c0, int nc) {
        int N, K;
        proj_dims(c, which, N, K);
        const uint64_t ts = synth_tensor_seed(seed, layer, which);
        if (bits == 0) {
            synth_dense_kernel<<<blocks((int64_t)nr * nc), 256, 0, st>>>(ts, Slice{nr, nc, K, r0, c0}, 0.02f, (uint16_t*)p.w + (size_t)dst_row0 * nc);
        } else {
            const Slice words{nr, (int64_t)nc * bits / 32, (int64_t)K * bits / 32, r0, (int64_t)c0 * bits / 32};
            const Slice grp{nr, nc / 64, K / 64, r0, c0 / 64};
            synth_codes_kernel<<<blocks(words.n()), 256, 0, st>>>(ts, words, (uint32_t*)p.w + (size_t)dst_row0 * words.cols);
            synth_sb_kernel<<<blocks(grp.n()), 256, 0, st>>>(ts + 1, ts + 2, grp, mul, mid, p.scales + (size_t)dst_row0 * grp.cols,
                                                            p.biases + (size_t)dst_row0 * grp.cols);
        }
    };
    const int qd = c.num_heads * hd, kvd = c.num_kv_heads * hd;
    const int qd_l = qd / world, kvd_l = kvd / world, I_l = I / world;
    for (int l = 0; l < c.num_layers; l++) {
        LayerW& L = m->layers[l];
        TRY(dev_alloc(m, (size_t)H * 2, (void**)&L.input_ln));
        ones(L.input_ln, H);
        TRY(dev_alloc(m, (size_t)H * 2, (void**)&L.post_ln));
        ones(L.post_ln, H);
        if (c.qk_norm) {
            TRY(dev_alloc(m, (size_t)hd * 2, (void**)&L.q_norm));
            ones(L.q_norm, hd);
            TRY(dev_alloc(m, (size_t)hd * 2, (void**)&L.k_norm));
            ones(L.k_norm, hd);
        }
        TRY(alloc_proj(m, L.qkv, qd_l + 2 * kvd_l, H, bits));  // this rank's heads: rows of q, k, v
        fill(L.qkv, 0, l, 0, rank * qd_l, qd_l, 0, H);
        fill(L.qkv, qd_l, l, 1, rank * kvd_l, kvd_l, 0, H);
        fill(L.qkv, qd_l + kvd_l, l, 2, rank * kvd_l, kvd_l, 0, H);
        TRY(alloc_proj(m, L.o, H, qd_l, bits));                // ... and the matching columns of o_proj
        fill(L.o, 0, l, 3, 0, H, rank * qd_l, qd_l);
        TRY(alloc_proj(m, L.gu, 2 * I_l, H, bits));            // rows of gate and up
        fill(L.gu, 0, l, 4, rank * I_l, I_l, 0, H);
        fill(L.gu, I_l, l, 5, rank * I_l, I_l, 0, H);
        TRY(alloc_proj(m, L.down, H, I_l, bits));              // columns of down_proj
        fill(L.down, 0, l, 6, 0, H, rank * I_l, I_l);
    }
    TRY(finish_model(m));
#undef TRY
    B2_CUDA(cudaStreamSynchronize(st));
    B2_CUDA(cudaGetLastError());
    *out = m;
    return B2_OK;
}

int32_t b2_model_synthetic(b2_ctx* ctx, const b2_model_config* cfg, uint64_t seed, b2_model** out) {
    return b2_model_synthetic_tp(ctx, cfg, seed, nullptr, out);
}

int32_t b2_model_free(b2_model* m) {
    if (!m) return B2_OK;
    cudaSetDevice(m->ctx->device);
    cudaStreamSynchronize(m->ctx->stream);
    for (void* p : m->allocs) cudaFree(p);
    if (m->cos_tab) cudaFree(m->cos_tab);
    if (m->sin_tab) cudaFree(m->sin_tab);
    if (m->cos_f32) cudaFree(m->cos_f32);
    if (m->sin_f32) cudaFree(m->sin_f32);
    b2_forward_f32_release(m);
    Workspace& w = m->ws;
    void* dev[] = {w.x_in_peer_region ? nullptr : (void*)w.x, w.tp_part, w.xn, w.qkv, w.q, w.attn, w.gu, w.act, w.last, w.logits, w.argmax, w.ids, w.meta, w.stage_dev, w.attn_scratch};
    for (void* p : dev)
        if (p) cudaFree(p);
    if (w.stage_host) cudaFreeHost(w.stage_host);
    if (w.argmax_host) cudaFreeHost(w.argmax_host);
    if (w.logits_host) cudaFreeHost(w.logits_host);
    if (m->ev0) cudaEventDestroy(m->ev0);
    if (m->ev1) cudaEventDestroy(m->ev1);
    delete m;
    return B2_OK;
}
int32_t b2_model_get_config(const b2_model* m, b2_model_config* out) {
    B2_REQUIRE(m && out, B2_ERR_MSG, "b2_model_get_config: null argument");
    *out = m->cfg;
    return B2_OK;
}
int32_t b2_model_is_quantized(const b2_model* m) { return m && m->quantized ? 1 : 0; }
int64_t b2_model_weight_bytes(const b2_model* m) { return m ? m->weight_bytes : 0; }

}  // extern "C"
