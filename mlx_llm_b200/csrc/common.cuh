// Shared device/host helpers for the sm_100a kernels of this library.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>
#include <vector>

#include "../../include/b200llm.h"

// ---- error plumbing -------------------------------------------------------------------------
void b2_set_error(const std::string& msg);
int32_t b2_fail(int32_t code, const std::string& msg);

#define B2_CUDA(call)                                                                             \
    do {                                                                                          \
        cudaError_t e__ = (call);                                                                 \
        if (e__ != cudaSuccess)                                                                   \
            return b2_fail(B2_ERR_CUDA, std::string(#call) + ": " + cudaGetErrorString(e__));     \
    } while (0)
#define B2_CHECK(call)            \
    do {                          \
        int32_t s__ = (call);     \
        if (s__ != B2_OK) return s__; \
    } while (0)
#define B2_REQUIRE(cond, code, msg) \
    do {                            \
        if (!(cond)) return b2_fail((code), (msg)); \
    } while (0)

// ---- context --------------------------------------------------------------------------------
struct b2_ctx {
    int device = 0;
    int sm_count = 148;
    cudaStream_t stream = nullptr;
    cudaEvent_t ev0 = nullptr, ev1 = nullptr;
    int64_t launches = 0;
    // scratch owned by the context, grown on demand outside timed regions
    void* scratch = nullptr;
    size_t scratch_bytes = 0;
    void* flush_buf = nullptr;
    size_t flush_bytes = 0;
    // staging for the *_host entry points
    void* stage = nullptr;
    size_t stage_bytes = 0;
    // tcgen05 GEMM: split-K partial sums and the device error word its bounded waits raise
    float* tc_partial = nullptr;
    float* pf_part = nullptr;        // prefill attention split over keys: f32 partial outputs, maxima and sums
    size_t pf_part_bytes = 0;
    size_t tc_partial_bytes = 0;
    int* dev_err = nullptr;        // raised by a bounded device-side wait that gave up (allocated with the context)
    int* err_host = nullptr;       // pinned copy the engine step reads back with its sampled ids
    long long wait_cycles = 8000000000LL;  // limit of a wait on another rank (b2_ctx_set_wait_limit_ms), ~4 s
    int clock_khz = 1965000;
    int* attn_counters = nullptr;  // arrival counters of the decode attention's fused merge (self-resetting)
    size_t attn_counters_cap = 0;
    int* tile_counters = nullptr;  // per row-tile arrival counters of the split-K streaming kernel (self-resetting)
    bool use_tc = true;
    bool pdl_consumers = true;     // norm / SwiGLU / RoPE / attention / split-K sums launched with programmatic stream serialisation
    int pdl_min_tokens = 1;        // ... by the engine on iterations of at least this many tokens (B2_PDL_MIN_TOKENS at context creation)
    // optional per-kernel-class timing with CUDA events on the launching stream
    bool profile = false;
    // NVTX ranges around every kernel class of a step ("gemm", "attn_decode", ...), for timeline tools; off by default
    bool nvtx = false;
    bool nvtx_open = false;
    std::vector<cudaEvent_t> prof_ev;
    std::vector<int> prof_cls;
    std::vector<int64_t> prof_launch;
    size_t prof_used = 0;
    double class_ms[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    int64_t class_launches[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    double gemm_flops = 0, gemm_weight_bytes = 0, attn_decode_bytes = 0, attn_prefill_flops = 0;
};
// kernel classes for the profile
enum { B2_CLS_GEMM = 0, B2_CLS_ATTN_DECODE = 1, B2_CLS_ATTN_PREFILL = 2, B2_CLS_ROPE_KV = 3, B2_CLS_ELEMENTWISE = 4, B2_CLS_META = 5, B2_CLS_COLLECTIVE = 6 };
// Marks the start of a stretch of launches of class `cls` (-1 closes the last stretch).
void b2_prof_mark(b2_ctx* ctx, int cls);
// After the stream has been synchronised: folds the recorded stretches into class_ms.
void b2_prof_collect(b2_ctx* ctx);
int32_t b2_ctx_scratch(b2_ctx* ctx, size_t bytes, void** out);
int32_t b2_ctx_stage(b2_ctx* ctx, size_t bytes, void** out);
#define B2_LAUNCHED(ctx) ((ctx)->launches++)

// Opt a kernel into a large dynamic shared-memory size, once per (kernel, device).
#define B2_SMEM_ONCE(ctx, func, bytes)                                                                       \
    do {                                                                                                     \
        static bool done__[16] = {};                                                                         \
        if (!done__[(ctx)->device & 15]) {                                                                   \
            B2_CUDA(cudaFuncSetAttribute(func, cudaFuncAttributeMaxDynamicSharedMemorySize, (bytes)));       \
            done__[(ctx)->device & 15] = true;                                                               \
        }                                                                                                    \
    } while (0)

// ---- device helpers -------------------------------------------------------------------------
#ifdef __CUDACC__
// Launch with programmatic stream serialisation: the grid may be scheduled while the kernel before it in the stream is
// still finishing (once every CTA of that kernel has started and signalled, or exited).  The launched kernel must call
// pdl_wait() before it touches anything an earlier kernel reads or writes.
// `programmatic` false gives an ordinary launch (kept for comparison: B2_PDL_MIN_TOKENS).  Measured against ordinary
// launches: decode iterations of 4 to 32 sequences 8-15 % faster, of 64 sequences 6 %, a ~680-token iteration 3 %.  The
// weight-streaming projection kernel does NOT signal its dependents early: with that, iterations of 1 and 8 sequences
// were 2.7 % slower than with ordinary launches.
template <typename... KArgs, typename... Args>
inline cudaError_t b2_launch_pdl(bool programmatic, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                 Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = programmatic ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
// Waits until every kernel this one depends on has completed and its writes are visible (returns at once in a kernel
// launched the ordinary way).
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }
typedef __nv_bfloat16 bf16;

__device__ __forceinline__ float bf2f(uint16_t h) { return __uint_as_float((uint32_t)h << 16); }
__device__ __forceinline__ float bflo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bfhi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }
__device__ __forceinline__ uint16_t f2bf(float f) { return __bfloat16_as_ushort(__float2bfloat16_rn(f)); }
__device__ __forceinline__ float rbf(float f) { return __bfloat162float(__float2bfloat16_rn(f)); }
__device__ __forceinline__ uint32_t pack_bf2(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async16(uint32_t smem_addr, const void* gptr) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(smem_addr), "l"(gptr));
}
__device__ __forceinline__ void cp_async16_zfill(uint32_t smem_addr, const void* gptr, bool valid) {
    int sz = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_addr), "l"(gptr), "r"(sz));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x2(uint32_t& r0, uint32_t& r1, uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];\n" : "=r"(r0), "=r"(r1) : "r"(addr));
}
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a) {
    uint32_t d;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;\n" : "=r"(d) : "r"(a));
    return d;
}
// D(16x8,f32) += A(16x16,bf16,row) * B(16x8,bf16,col)
__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm volatile("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}
#endif
