// Snapshot writer: a dense, Hugging-Face-keyed tensor set -> a directory the loader (and the reference)
// reads back, optionally with the attention / MLP projections re-quantized to MLX group-64 Q4 / Q8.
//
// Mirrors write_snapshot (src/snapshot.rs:86-148): a projection (PROJECTION_SUFFIXES, snapshot.rs:41-49) is
// cast to bf16, quantized and stored as the packed triplet `<base>.weight` (u32) / `<base>.scales` /
// `<base>.biases` (bf16); every other tensor is written through unchanged; config.json gets a matching
// `quantization` block so the loader takes its stored-triplet branch (src/models/llama.rs:77-95).  The
// quantization runs on the GPU (the same kernel as quantize-on-load), so a snapshot reloads bit-identically
// to quantizing at load time.
#include <sys/stat.h>

#include <cerrno>
#include <cstdio>
#include <cstring>

#include "engine.h"
#include "json_mini.h"

namespace {

const char* kProjectionSuffixes[7] = {"self_attn.q_proj.weight", "self_attn.k_proj.weight", "self_attn.v_proj.weight",
                                      "self_attn.o_proj.weight", "mlp.gate_proj.weight",    "mlp.up_proj.weight",
                                      "mlp.down_proj.weight"};

bool is_projection(const std::string& key) {  // snapshot.rs:52-54
    for (const char* s : kProjectionSuffixes) {
        const size_t n = strlen(s);
        if (key.size() >= n && key.compare(key.size() - n, n, s) == 0) return true;
    }
    return false;
}

struct OutTensor {
    std::string name;
    const char* dtype;
    std::vector<int64_t> shape;
    const uint8_t* ptr;  // into the source weights or into `owned`
    size_t nbytes;
    std::vector<uint8_t> owned;
};

const char* dtype_name(int dt) {
    switch (dt) {
        case B2_DTYPE_F32: return "F32";
        case B2_DTYPE_BF16: return "BF16";
        case B2_DTYPE_F16: return "F16";
        case B2_DTYPE_U32: return "U32";
        default: return "I32";
    }
}

inline uint16_t f32_to_bf16(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40);
    return (uint16_t)((u + 0x7fffu + ((u >> 16) & 1u)) >> 16);
}
inline float f16_to_f32(uint16_t h) {
    const uint32_t s = (uint32_t)(h & 0x8000u) << 16, e = (h >> 10) & 0x1f, m = h & 0x3ffu;
    uint32_t u;
    if (e == 0) {
        if (m == 0) {
            u = s;
        } else {
            int sh = 0;
            uint32_t mm = m;
            while (!(mm & 0x400u)) mm <<= 1, sh++;
            u = s | ((uint32_t)(127 - 15 - sh) << 23) | ((mm & 0x3ffu) << 13);
        }
    } else if (e == 31) {
        u = s | 0x7f800000u | (m << 13);
    } else {
        u = s | ((e + 112) << 23) | (m << 13);
    }
    float f;
    memcpy(&f, &u, 4);
    return f;
}

int32_t mkdir_p(const std::string& dir) {
    std::string cur;
    for (size_t i = 0; i <= dir.size(); i++) {
        if (i == dir.size() || dir[i] == '/') {
            if (!cur.empty() && mkdir(cur.c_str(), 0777) != 0 && errno != EEXIST) return b2_fail(B2_ERR_IO, "cannot create directory " + cur);
        }
        if (i < dir.size()) cur.push_back(dir[i]);
    }
    return B2_OK;
}

int32_t write_file(const std::string& path, const void* data, size_t n) {
    FILE* f = fopen(path.c_str(), "wb");
    B2_REQUIRE(f, B2_ERR_IO, "cannot open " + path + " for writing");
    const size_t w = n ? fwrite(data, 1, n, f) : 0;
    const int rc = fclose(f);
    B2_REQUIRE(w == n && rc == 0, B2_ERR_IO, "short write to " + path);
    return B2_OK;
}

}  // namespace

extern "C" int32_t b2_write_snapshot(b2_ctx* ctx, const b2_weights* w, const char* config_json, const b2_quant_spec* quant,
                                     const char* out_dir, int32_t* num_tensors_out) {
    B2_REQUIRE(ctx && w && config_json && out_dir, B2_ERR_MSG, "b2_write_snapshot: null argument");
    if (quant)
        B2_REQUIRE(quant->group_size == 64 && (quant->bits == 4 || quant->bits == 8), B2_ERR_UNSUPPORTED,
                   "b2_write_snapshot: QuantSpec must be group 64 with 4 or 8 bits");
    // config: must be a JSON object; a quantized snapshot of an already quantized config is refused
    std::string cfg = config_json, err;
    auto root = b2json::parse(cfg, err);
    B2_REQUIRE(root && root->kind == b2json::Value::Object, B2_ERR_CONFIG, "snapshot config.json is not a JSON object");
    if (quant) {
        B2_REQUIRE(!root->get("quantization"), B2_ERR_CONFIG, "snapshot source is already quantized");
        const size_t close = cfg.find_last_of('}');
        B2_REQUIRE(close != std::string::npos, B2_ERR_CONFIG, "snapshot config.json is not a JSON object");
        const std::string block = std::string(root->obj.empty() ? "" : ", ") + "\"quantization\": {\"group_size\": " +
                                  std::to_string(quant->group_size) + ", \"bits\": " + std::to_string(quant->bits) + "}";
        cfg.insert(close, block);
    }
    B2_CHECK(mkdir_p(out_dir));
    B2_CUDA(cudaSetDevice(ctx->device));

    std::vector<OutTensor> out;
    out.reserve(w->t.size() * 3);
    for (const auto& kv : w->t) {
        const HostTensor& t = kv.second;
        if (quant && is_projection(kv.first)) {
            B2_REQUIRE(t.shape.size() == 2, B2_ERR_CONFIG, "projection `" + kv.first + "` is not a matrix");
            B2_REQUIRE(t.dtype == B2_DTYPE_F32 || t.dtype == B2_DTYPE_BF16 || t.dtype == B2_DTYPE_F16, B2_ERR_CONFIG,
                       "projection `" + kv.first + "` is not a floating-point tensor");
            const int64_t N = t.shape[0], K = t.shape[1];
            B2_REQUIRE(K % 64 == 0, B2_ERR_UNSUPPORTED, "projection `" + kv.first + "`: group size 64 must divide the input dimension");
            // cast to bf16 (STORE_DTYPE), quantize on the device
            std::vector<uint16_t> bf((size_t)N * K);
            if (t.dtype == B2_DTYPE_BF16) {
                memcpy(bf.data(), t.ptr, bf.size() * 2);
            } else if (t.dtype == B2_DTYPE_F32) {
                const float* f = (const float*)t.ptr;
                for (size_t i = 0; i < bf.size(); i++) bf[i] = f32_to_bf16(f[i]);
            } else {
                const uint16_t* h = (const uint16_t*)t.ptr;
                for (size_t i = 0; i < bf.size(); i++) bf[i] = f32_to_bf16(f16_to_f32(h[i]));
            }
            const int bits = quant->bits;
            const size_t words = (size_t)N * K * bits / 32, groups = (size_t)N * (K / 64);
            uint16_t *d_w = nullptr, *d_s = nullptr, *d_b = nullptr;
            uint32_t* d_p = nullptr;
            int32_t rc = B2_OK;
            if (cudaMalloc((void**)&d_w, bf.size() * 2) != cudaSuccess || cudaMalloc((void**)&d_p, words * 4) != cudaSuccess ||
                cudaMalloc((void**)&d_s, groups * 2) != cudaSuccess || cudaMalloc((void**)&d_b, groups * 2) != cudaSuccess)
                rc = b2_fail(B2_ERR_CUDA, "out of device memory while quantizing `" + kv.first + "`");
            OutTensor pw, ps, pb;
            const std::string base = kv.first.substr(0, kv.first.size() - 7);  // strip ".weight"
            if (rc == B2_OK) {
                pw.owned.resize(words * 4);
                ps.owned.resize(groups * 2);
                pb.owned.resize(groups * 2);
                cudaStream_t st = ctx->stream;
                if (cudaMemcpyAsync(d_w, bf.data(), bf.size() * 2, cudaMemcpyHostToDevice, st) != cudaSuccess) rc = b2_fail(B2_ERR_CUDA, "upload failed");
                if (rc == B2_OK) rc = b2_quantize_launch(ctx, d_w, N, K, bits, d_p, d_s, d_b);
                if (rc == B2_OK &&
                    (cudaMemcpyAsync(pw.owned.data(), d_p, words * 4, cudaMemcpyDeviceToHost, st) != cudaSuccess ||
                     cudaMemcpyAsync(ps.owned.data(), d_s, groups * 2, cudaMemcpyDeviceToHost, st) != cudaSuccess ||
                     cudaMemcpyAsync(pb.owned.data(), d_b, groups * 2, cudaMemcpyDeviceToHost, st) != cudaSuccess ||
                     cudaStreamSynchronize(st) != cudaSuccess))
                    rc = b2_fail(B2_ERR_CUDA, "quantizing `" + kv.first + "` failed on the device");
            }
            cudaFree(d_w);
            cudaFree(d_p);
            cudaFree(d_s);
            cudaFree(d_b);
            if (rc != B2_OK) return rc;
            pw.name = base + ".weight", pw.dtype = "U32", pw.shape = {N, K * bits / 32};
            ps.name = base + ".scales", ps.dtype = "BF16", ps.shape = {N, K / 64};
            pb.name = base + ".biases", pb.dtype = "BF16", pb.shape = {N, K / 64};
            for (OutTensor* o : {&pw, &ps, &pb}) {
                o->nbytes = o->owned.size();
                out.push_back(std::move(*o));
                out.back().ptr = out.back().owned.data();
            }
        } else {
            OutTensor o;
            o.name = kv.first;
            o.dtype = dtype_name(t.dtype);
            o.shape = t.shape;
            o.ptr = t.ptr;
            o.nbytes = t.nbytes;
            out.push_back(std::move(o));
        }
    }

    // model.safetensors: u64 header length, JSON header (padded with spaces to 8 bytes), raw tensor bytes
    std::string header = "{";
    size_t offset = 0;
    for (size_t i = 0; i < out.size(); i++) {
        const OutTensor& o = out[i];
        if (i) header += ",";
        header += "\"" + o.name + "\":{\"dtype\":\"" + o.dtype + "\",\"shape\":[";
        for (size_t d = 0; d < o.shape.size(); d++) header += (d ? "," : "") + std::to_string(o.shape[d]);
        header += "],\"data_offsets\":[" + std::to_string(offset) + "," + std::to_string(offset + o.nbytes) + "]}";
        offset += o.nbytes;
    }
    header += "}";
    while (header.size() % 8) header.push_back(' ');
    const std::string path = std::string(out_dir) + "/model.safetensors";
    FILE* f = fopen(path.c_str(), "wb");
    B2_REQUIRE(f, B2_ERR_IO, "cannot open " + path + " for writing");
    const uint64_t hlen = header.size();
    bool ok = fwrite(&hlen, 8, 1, f) == 1 && fwrite(header.data(), 1, header.size(), f) == header.size();
    for (const OutTensor& o : out)
        if (ok && o.nbytes) ok = fwrite(o.ptr, 1, o.nbytes, f) == o.nbytes;
    ok = (fclose(f) == 0) && ok;
    B2_REQUIRE(ok, B2_ERR_IO, "short write to " + path);
    B2_CHECK(write_file(std::string(out_dir) + "/config.json", cfg.data(), cfg.size()));
    if (num_tensors_out) *num_tensors_out = (int32_t)out.size();
    return B2_OK;
}
