// CPU oracle — TEST INFRASTRUCTURE ONLY.
//
// This directory restates, on the CPU, the arithmetic and the host policy of the
// continuous-batching decode path of SceneWorks/mlx-llm so that the CUDA path can be
// checked against it.  Nothing in the product library may call into it: only the test
// suite, the smoke entry and the CPU-baseline leg of the benchmark load it.
//
// The reference runs its tensor ops through MLX (pmetal-mlx-rs 0.25.8, MLX core 0.31.2),
// whose source is not part of the reference tree.  Where a behaviour is fixed by the
// reference's own tests it is pinned here (SplitMix64 known answers, RoPE frequency
// formulas, paged-cache bookkeeping, attention vs. an f64 host loop); where only the
// third-party library fixes it (the affine quantize encoder, the exact rounding inside
// rms_norm / quantized_matmul) the header of the function says "parity unpinned".
#pragma once
#include <cmath>
#include <cstdint>
#include <cstring>
#include <vector>

namespace orc {

// ---- bf16 <-> f32, round-to-nearest-even (the dtype every cached-decode tensor uses:
// src/models/llama.rs:29-30 COMPUTE_DTYPE) ------------------------------------------
static inline uint16_t f2bf(float f) {
    uint32_t u;
    std::memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x0040u);  // quiet NaN
    uint32_t lsb = (u >> 16) & 1u;
    u += 0x7fffu + lsb;
    return (uint16_t)(u >> 16);
}
static inline float bf2f(uint16_t h) {
    uint32_t u = (uint32_t)h << 16;
    float f;
    std::memcpy(&f, &u, 4);
    return f;
}
// Round an f32 value to the nearest bf16 and return it as f32.
static inline float rbf(float f) { return bf2f(f2bf(f)); }

// ---- x @ w^T for one weight row against many activation rows ------------------------
// Every output keeps ONE f32 accumulator that adds x[i][d]*w[d] for d = 0, 1, 2, ... (a multiply, then
// an add: the build disables contraction), exactly the scalar loop `acc += x[d]*w[d]`.  The rows are
// only interleaved 32 at a time so that 32 independent accumulators sit in four 8-lane vector
// registers; no sum is split or reordered, so the result is the scalar loop's bit for bit.
typedef float orc_v8 __attribute__((vector_size(32), aligned(4)));
struct RowsT16 {  // activations re-laid as [block of 32 rows][d][32], zero padded
    int m = 0, k = 0;
    std::vector<float> t;
    RowsT16(const float* x, int m_, int k_) : m(m_), k(k_), t((size_t)((m_ + 31) / 32) * k_ * 32, 0.f) {
        for (int i = 0; i < m; i++)
            for (int d = 0; d < k; d++) t[((size_t)(i / 32) * k + d) * 32 + (i % 32)] = x[(size_t)i * k + d];
    }
};
static inline void dots_in_order(const RowsT16& x, const float* w, float* acc /* [m] */) {
    for (int b = 0; b * 32 < x.m; b++) {
        orc_v8 a0 = {0, 0, 0, 0, 0, 0, 0, 0}, a1 = a0, a2 = a0, a3 = a0;
        const float* xb = x.t.data() + (size_t)b * x.k * 32;
        for (int d = 0; d < x.k; d++) {
            const float wd = w[d];
            const orc_v8 wv = {wd, wd, wd, wd, wd, wd, wd, wd};
            const orc_v8* xr = (const orc_v8*)(xb + (size_t)d * 32);
            a0 += xr[0] * wv;  // a multiply, then an add, per lane (no contraction in this build)
            a1 += xr[1] * wv;
            a2 += xr[2] * wv;
            a3 += xr[3] * wv;
        }
        float out[32];
        std::memcpy(out, &a0, 32);
        std::memcpy(out + 8, &a1, 32);
        std::memcpy(out + 16, &a2, 32);
        std::memcpy(out + 24, &a3, 32);
        for (int i = 0; i < 32 && b * 32 + i < x.m; i++) acc[b * 32 + i] = out[i];
    }
}

// ---- SplitMix64 (src/primitives/sampler.rs:36-61) -----------------------------------
struct SplitMix64 {
    uint64_t s;
    explicit SplitMix64(uint64_t seed) : s(seed) {}
    uint64_t next_u64() {
        s += 0x9E3779B97F4A7C15ull;
        uint64_t z = s;
        z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
        z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
        return z ^ (z >> 31);
    }
    float next_f32() { return (float)(next_u64() >> 40) / (float)(1ull << 24); }
};

// ---- Counter-based synthetic tensor generator --------------------------------------
// Large random-init models (Llama-3-8B / Qwen3-32B shapes) are generated independently
// on the CPU (here) and on the GPU (the library's synthetic-model entry point) from the
// same integer recipe, so both sides hold bit-identical weights without moving them.
// Every value is a pure function of (seed, element index); only integer ops, exact
// int->float conversions, one IEEE multiply and one correctly-rounded fma are used, so
// the result does not depend on libm or on fma contraction.
static inline uint64_t mix64(uint64_t z) {
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}
static inline uint64_t synth_u64(uint64_t seed, uint64_t idx) {
    return mix64(seed + (idx + 1) * 0x9E3779B97F4A7C15ull);
}
// Approximately standard-normal value: Irwin-Hall sum of twelve 16-bit uniforms.
static inline float synth_normal(uint64_t seed, uint64_t idx) {
    uint64_t a = synth_u64(seed, 3 * idx), b = synth_u64(seed, 3 * idx + 1), c = synth_u64(seed, 3 * idx + 2);
    uint32_t sum = 0;
    for (int i = 0; i < 4; i++) {
        sum += (uint32_t)((a >> (16 * i)) & 0xffff);
        sum += (uint32_t)((b >> (16 * i)) & 0xffff);
        sum += (uint32_t)((c >> (16 * i)) & 0xffff);
    }
    return ((float)sum - 393210.0f) * (1.0f / 65536.0f);
}
// Packed quantized codes: word idx of a tensor is 32 uniformly random bits.
static inline uint32_t synth_code_word(uint64_t seed, uint64_t idx) { return (uint32_t)(synth_u64(seed, idx) >> 16); }
// Group scale: |n| * mul (mul = 0.02/7.5 gives a 4-bit grid spanning roughly +-0.02*8);
// bias = -mid*scale + n2*1e-3.
static inline uint16_t synth_scale(uint64_t seed, uint64_t idx, float mul) {
    return f2bf(std::fabs(synth_normal(seed, idx)) * mul);
}
static inline uint16_t synth_bias(uint64_t seed_bias, uint64_t idx, uint16_t scale_bf, float mid) {
    return f2bf(std::fmaf(synth_normal(seed_bias, idx), 1e-3f, -mid * bf2f(scale_bf)));
}
// Dense bf16 weight ~ std * n.
static inline uint16_t synth_dense(uint64_t seed, uint64_t idx, float std_) { return f2bf(synth_normal(seed, idx) * std_); }

}  // namespace orc
