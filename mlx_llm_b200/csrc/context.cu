// Context, error reporting and raw device-memory plumbing of the C ABI.
#include <cstdlib>
#include <nvtx3/nvToolsExt.h>

#include <cstdio>
#include <cstring>

#include <cuda_profiler_api.h>

#include "common.cuh"

static thread_local std::string g_last_error;

void b2_set_error(const std::string& msg) { g_last_error = msg; }
int32_t b2_fail(int32_t code, const std::string& msg) {
    g_last_error = msg;
    return code;
}

extern "C" {

const char* b2_last_error(void) { return g_last_error.c_str(); }
int32_t b2_version(void) { return 100; }

int32_t b2_device_count(int32_t* out) {
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess) {
        *out = 0;
        return b2_fail(B2_ERR_CUDA, std::string("cudaGetDeviceCount: ") + cudaGetErrorString(e));
    }
    *out = n;
    return B2_OK;
}

int32_t b2_ctx_create(int32_t device, b2_ctx** out) {
    B2_REQUIRE(out != nullptr, B2_ERR_MSG, "b2_ctx_create: null out");
    int n = 0;
    B2_CUDA(cudaGetDeviceCount(&n));
    B2_REQUIRE(n > 0, B2_ERR_CUDA, "b2_ctx_create: no CUDA device (this library has no CPU fallback)");
    B2_REQUIRE(device >= 0 && device < n, B2_ERR_MSG, "b2_ctx_create: device index out of range");
    B2_CUDA(cudaSetDevice(device));
    cudaDeviceProp prop;
    B2_CUDA(cudaGetDeviceProperties(&prop, device));
    B2_REQUIRE(prop.major >= 10, B2_ERR_UNSUPPORTED,
               std::string("b2_ctx_create: kernels are built for sm_100a only; device is ") + prop.name);
    b2_ctx* c = new b2_ctx();
    c->device = device;
    c->sm_count = prop.multiProcessorCount;
    if (prop.clockRate > 0) c->clock_khz = prop.clockRate;
    c->wait_cycles = 4000ll * c->clock_khz;
    B2_CUDA(cudaMalloc((void**)&c->dev_err, 16));
    B2_CUDA(cudaMemset(c->dev_err, 0, 16));
    B2_CUDA(cudaHostAlloc((void**)&c->err_host, 16, cudaHostAllocDefault));
    c->err_host[0] = 0;
    B2_CUDA(cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking));
    B2_CUDA(cudaEventCreate(&c->ev0));
    B2_CUDA(cudaEventCreate(&c->ev1));
    if (const char* v = std::getenv("B2_NVTX")) c->nvtx = v[0] == '1';
    if (const char* v = std::getenv("B2_PDL_MIN_TOKENS")) c->pdl_min_tokens = std::atoi(v);
    *out = c;
    return B2_OK;
}

int32_t b2_ctx_free(b2_ctx* ctx) {
    if (!ctx) return B2_OK;
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    if (ctx->scratch) cudaFree(ctx->scratch);
    if (ctx->flush_buf) cudaFree(ctx->flush_buf);
    if (ctx->stage) cudaFree(ctx->stage);
    if (ctx->tc_partial) cudaFree(ctx->tc_partial);
    if (ctx->pf_part) cudaFree(ctx->pf_part);
    if (ctx->dev_err) cudaFree(ctx->dev_err);
    if (ctx->err_host) cudaFreeHost(ctx->err_host);
    if (ctx->tile_counters) cudaFree(ctx->tile_counters);
    if (ctx->attn_counters) cudaFree(ctx->attn_counters);
    for (auto e : ctx->prof_ev) cudaEventDestroy(e);
    cudaEventDestroy(ctx->ev0);
    cudaEventDestroy(ctx->ev1);
    cudaStreamDestroy(ctx->stream);
    delete ctx;
    return B2_OK;
}

int32_t b2_ctx_sync(b2_ctx* ctx) {
    B2_CUDA(cudaStreamSynchronize(ctx->stream));
    B2_CUDA(cudaGetLastError());
    if (ctx->dev_err) {  // raised by a bounded device-side wait that gave up
        int e = 0;
        B2_CUDA(cudaMemcpyAsync(&e, ctx->dev_err, sizeof(int), cudaMemcpyDeviceToHost, ctx->stream));
        B2_CUDA(cudaStreamSynchronize(ctx->stream));
        if (e != 0) {
            B2_CUDA(cudaMemsetAsync(ctx->dev_err, 0, sizeof(int), ctx->stream));
            return b2_fail(B2_ERR_TIMEOUT, "a bounded device-side wait ran out (tcgen05 pipeline barrier or a peer-memory reduction flag)");
        }
    }
    return B2_OK;
}

// Limit of the device-side waits on another rank's flags (the peer-memory reduction).
int32_t b2_ctx_set_wait_limit_ms(b2_ctx* ctx, int32_t ms) {
    B2_REQUIRE(ctx, B2_ERR_MSG, "b2_ctx_set_wait_limit_ms: null context");
    B2_REQUIRE(ms >= 1 && ms <= 60000, B2_ERR_MSG, "b2_ctx_set_wait_limit_ms: the limit must lie between 1 ms and 60 s");
    ctx->wait_cycles = (long long)ms * ctx->clock_khz;
    return B2_OK;
}

// Selects the projection path: 1 = tcgen05/TMEM for large token counts (default), 0 = warp-level mma.sync only.
int32_t b2_ctx_set_tensor_path(b2_ctx* ctx, int32_t use_tcgen05) {
    B2_REQUIRE(ctx, B2_ERR_MSG, "b2_ctx_set_tensor_path: null context");
    ctx->use_tc = use_tcgen05 != 0;
    return B2_OK;
}

int32_t b2_malloc(b2_ctx* ctx, size_t bytes, void** out_dev) {
    B2_CUDA(cudaSetDevice(ctx->device));
    B2_CUDA(cudaMalloc(out_dev, bytes ? bytes : 16));
    return B2_OK;
}
int32_t b2_free(b2_ctx* ctx, void* dev) {
    B2_CUDA(cudaSetDevice(ctx->device));
    B2_CUDA(cudaFree(dev));
    return B2_OK;
}
int32_t b2_memcpy_h2d(b2_ctx* ctx, void* dst_dev, const void* src_host, size_t bytes) {
    B2_CUDA(cudaMemcpyAsync(dst_dev, src_host, bytes, cudaMemcpyHostToDevice, ctx->stream));
    B2_CUDA(cudaStreamSynchronize(ctx->stream));
    return B2_OK;
}
int32_t b2_memcpy_d2h(b2_ctx* ctx, void* dst_host, const void* src_dev, size_t bytes) {
    B2_CUDA(cudaMemcpyAsync(dst_host, src_dev, bytes, cudaMemcpyDeviceToHost, ctx->stream));
    B2_CUDA(cudaStreamSynchronize(ctx->stream));
    return B2_OK;
}
int32_t b2_memset(b2_ctx* ctx, void* dst_dev, int value, size_t bytes) {
    B2_CUDA(cudaMemsetAsync(dst_dev, value, bytes, ctx->stream));
    return B2_OK;
}
int32_t b2_mem_info(b2_ctx* ctx, size_t* free_bytes, size_t* total_bytes) {
    B2_REQUIRE(ctx && free_bytes && total_bytes, B2_ERR_MSG, "b2_mem_info: null argument");
    B2_CUDA(cudaSetDevice(ctx->device));
    B2_CUDA(cudaMemGetInfo(free_bytes, total_bytes));
    return B2_OK;
}

int32_t b2_host_alloc_pinned(size_t bytes, void** out_host) {
    B2_CUDA(cudaHostAlloc(out_host, bytes ? bytes : 16, cudaHostAllocDefault));
    return B2_OK;
}
int32_t b2_host_free_pinned(void* host) {
    B2_CUDA(cudaFreeHost(host));
    return B2_OK;
}

int32_t b2_timer_start(b2_ctx* ctx) {
    B2_CUDA(cudaEventRecord(ctx->ev0, ctx->stream));
    return B2_OK;
}
int32_t b2_timer_stop_ms(b2_ctx* ctx, float* ms_out) {
    B2_CUDA(cudaEventRecord(ctx->ev1, ctx->stream));
    B2_CUDA(cudaEventSynchronize(ctx->ev1));
    B2_CUDA(cudaEventElapsedTime(ms_out, ctx->ev0, ctx->ev1));
    return B2_OK;
}

int32_t b2_flush_l2(b2_ctx* ctx) {
    const size_t bytes = 256ull << 20;  // 2x the 126 MB L2
    if (!ctx->flush_buf) {
        B2_CUDA(cudaMalloc(&ctx->flush_buf, bytes));
        ctx->flush_bytes = bytes;
    }
    B2_CUDA(cudaMemsetAsync(ctx->flush_buf, 1, ctx->flush_bytes, ctx->stream));
    return B2_OK;
}

int32_t b2_profiler_range(b2_ctx* ctx, int32_t on) {
    B2_REQUIRE(ctx, B2_ERR_MSG, "b2_profiler_range: null context");
    B2_CUDA(cudaStreamSynchronize(ctx->stream));
    if (on)
        B2_CUDA(cudaProfilerStart());
    else
        B2_CUDA(cudaProfilerStop());
    return B2_OK;
}

int32_t b2_launch_count(b2_ctx* ctx, int64_t* out) {
    *out = ctx->launches;
    return B2_OK;
}

int32_t b2_nvtx_enable(b2_ctx* ctx, int32_t on) {
    B2_REQUIRE(ctx, B2_ERR_MSG, "b2_nvtx_enable: null context");
    if (ctx->nvtx_open) nvtxRangePop();
    ctx->nvtx_open = false;
    ctx->nvtx = on != 0;
    return B2_OK;
}

int32_t b2_profile_enable(b2_ctx* ctx, int32_t on) {
    B2_REQUIRE(ctx, B2_ERR_MSG, "b2_profile_enable: null context");
    B2_CUDA(cudaStreamSynchronize(ctx->stream));
    ctx->profile = on != 0;
    ctx->prof_used = 0;
    ctx->prof_cls.clear();
    ctx->prof_launch.clear();
    for (int i = 0; i < 8; i++) {
        ctx->class_ms[i] = 0;
        ctx->class_launches[i] = 0;
    }
    ctx->gemm_flops = ctx->gemm_weight_bytes = ctx->attn_decode_bytes = ctx->attn_prefill_flops = 0;
    return B2_OK;
}

int32_t b2_profile_read(b2_ctx* ctx, b2_profile_t* out) {
    B2_REQUIRE(ctx && out, B2_ERR_MSG, "b2_profile_read: null argument");
    for (int i = 0; i < 8; i++) {
        out->ms[i] = ctx->class_ms[i];
        out->launches[i] = ctx->class_launches[i];
    }
    out->gemm_flops = ctx->gemm_flops;
    out->gemm_weight_bytes = ctx->gemm_weight_bytes;
    out->attn_decode_bytes = ctx->attn_decode_bytes;
    out->attn_prefill_flops = ctx->attn_prefill_flops;
    return B2_OK;
}

}  // extern "C"

static const char* const kClassNames[8] = {"gemm", "attn_decode", "attn_prefill", "rope_kv", "elementwise", "meta_copies", "collective", "other"};

void b2_prof_mark(b2_ctx* ctx, int cls) {
    if (ctx->nvtx) {  // one range per run of launches of a class; cls < 0 closes the step's last range
        if (ctx->nvtx_open) nvtxRangePop();
        ctx->nvtx_open = cls >= 0;
        if (cls >= 0) nvtxRangePushA(kClassNames[cls & 7]);
    }
    if (!ctx->profile) return;
    if (ctx->prof_used == ctx->prof_ev.size()) {
        cudaEvent_t e;
        if (cudaEventCreate(&e) != cudaSuccess) return;
        ctx->prof_ev.push_back(e);
    }
    cudaEventRecord(ctx->prof_ev[ctx->prof_used++], ctx->stream);
    ctx->prof_cls.push_back(cls);
    ctx->prof_launch.push_back(ctx->launches);
}

void b2_prof_collect(b2_ctx* ctx) {
    if (!ctx->profile) return;
    for (size_t i = 0; i + 1 < ctx->prof_used; i++) {
        const int cls = ctx->prof_cls[i];
        if (cls < 0 || cls >= 8) continue;
        float ms = 0.f;
        if (cudaEventElapsedTime(&ms, ctx->prof_ev[i], ctx->prof_ev[i + 1]) == cudaSuccess) ctx->class_ms[cls] += ms;
        ctx->class_launches[cls] += ctx->prof_launch[i + 1] - ctx->prof_launch[i];
    }
    ctx->prof_used = 0;
    ctx->prof_cls.clear();
    ctx->prof_launch.clear();
}

int32_t b2_ctx_scratch(b2_ctx* ctx, size_t bytes, void** out) {
    if (bytes > ctx->scratch_bytes) {
        B2_CUDA(cudaStreamSynchronize(ctx->stream));
        if (ctx->scratch) B2_CUDA(cudaFree(ctx->scratch));
        ctx->scratch = nullptr;
        size_t want = bytes + (bytes >> 2) + (1 << 20);
        B2_CUDA(cudaMalloc(&ctx->scratch, want));
        ctx->scratch_bytes = want;
    }
    *out = ctx->scratch;
    return B2_OK;
}
int32_t b2_ctx_stage(b2_ctx* ctx, size_t bytes, void** out) {
    if (bytes > ctx->stage_bytes) {
        B2_CUDA(cudaStreamSynchronize(ctx->stream));
        if (ctx->stage) B2_CUDA(cudaFree(ctx->stage));
        ctx->stage = nullptr;
        size_t want = bytes + (bytes >> 2) + (1 << 16);
        B2_CUDA(cudaMalloc(&ctx->stage, want));
        ctx->stage_bytes = want;
    }
    *out = ctx->stage;
    return B2_OK;
}
