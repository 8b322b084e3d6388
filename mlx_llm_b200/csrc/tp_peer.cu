// Tensor-parallel reduction over peer memory (NVLink / NVSwitch), fused with the projection before it and the
// residual add after it:
//
//     x = bf16(x + bf16(sum over ranks of the projection's f32 partial sums))
//
// on every rank, without a library collective.  Every rank exports one region (cudaIpc) holding `world` slots of
// f32 partial sums, its copy of the hidden state x and two sets of flags; every rank maps every other rank's
// region.  Rank r owns the columns [r*H/world, (r+1)*H/world).
//   1. The projection kernels (o_proj, down_proj) store their f32 results into slot [this rank]: of their own
//      region (default), or -- push mode, b2_tp_peer_set_push -- by column range straight from the epilogue into the
//      region of the rank that owns the columns (GemmParams::out_f32_by_chunk), so the partial sums cross NVLink
//      tile by tile while other tiles are still being multiplied.  Push pays off when a projection runs several
//      waves of tiles; a single wave ends all its epilogues at once and the burst of remote stores then delays the
//      kernel's end by more than the loads of the default mode cost (measured at two ranks, 5120 wide, ~700 tokens).
//   2. One kernel (below) tells the other ranks that this rank's projection has ended (flag1), waits for theirs,
//      adds up the `world` partial sums of its own columns -- peer loads (default) or local reads (push), in rank
//      order, so the result does not depend on timing -- adds the residual, rounds, and stores the new bf16 values
//      into EVERY rank's x (peer stores).  Block g then tells block g of every other rank that its rows are in place
//      (flag2) and waits for theirs, so that when the kernel ends this rank's x is complete.
// Flags carry the number of the reduction (a counter every rank advances in step), so nothing is ever reset.
//
// Why one set of slots suffices: a rank starts its next projection only after its own kernel 2 ended, which it
// does only after every other rank signalled flag2, which a rank does only after it finished reading the slots;
// and a rank's columns of x are written by their owner only.
//
// There is no counterpart in the reference (a single-device program).  The waits are bounded: on expiry the
// kernel raises the context's error word and returns; later reductions see the word and return at once.
#include <cooperative_groups.h>

#include <chrono>
#include <condition_variable>
#include <mutex>
#include <thread>

#include "common.cuh"
#include "engine.h"

// Ranks emulated in one process (one host thread and one context each, all on one device) step in lock-step: at every
// reduction the threads meet here, rank 0's thread enqueues ONE cooperative launch that reduces for all ranks (kernels
// that wait on one another must never be separate launches on one device), and CUDA events order it after every rank's
// projection and before every rank's next kernel.
struct b2_tp_lockstep {
    int n = 0;
    b2_tp_group* groups[8] = {};
    cudaEvent_t projected[8] = {};  // rank r's projection has been enqueued up to here
    cudaEvent_t reduced = nullptr;  // the group's reduction
    std::mutex mu;
    std::condition_variable cv;
    int waiting = 0;
    uint64_t generation = 0;
    int32_t status = B2_OK;         // rank 0's launch status, read by the others after the second meeting
    // All n threads arrive, or the wait gives up after a few seconds (a rank's thread failed before the meeting point).
    bool meet() {
        std::unique_lock<std::mutex> lk(mu);
        const uint64_t gen = generation;
        if (++waiting == n) {
            waiting = 0;
            generation++;
            cv.notify_all();
            return true;
        }
        return cv.wait_for(lk, std::chrono::seconds(10), [&] { return generation != gen; });
    }
};

namespace {

constexpr int kMaxWorld = 8;
constexpr int kMaxCtas = 1024;                          // flag2 slots per source rank
constexpr size_t kFlag1Off = 0;                         // u32 [kMaxWorld]
constexpr size_t kFlag2Off = 128;                       // u32 [kMaxWorld][kMaxCtas]
constexpr size_t kDataOff = 128 + (size_t)kMaxWorld * kMaxCtas * 4 + 128;  // partial sums start here (256-byte aligned)
static_assert(kDataOff % 256 == 0, "data offset alignment");

struct PeerReduceParams {
    unsigned char* base[kMaxWorld];  // every rank's region as mapped in this process
    int rank;                        // -1: blockIdx.y is the rank (the whole group emulated by one launch)
    int push;                        // 1: rank s's partial sums of this rank's columns already sit in slot s of THIS rank's
                                     // region (stored there by s's projection); 0: they sit in slot s of s's own region
    int world, M, H, chunk;          // chunk = H / world columns owned by each rank
    uint32_t seq;
    size_t slot_bytes;               // slot s of a region sits at kDataOff + s * slot_bytes
    size_t x_off;                    // offset of x in a region
    int* err;                        // the error word of the context (of rank 0's context when emulating)
    long long wait_cycles;           // limit of every wait on another rank (the context's setting)
};

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];\n" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;\n" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ float4 ld_peer_f4(const float* p) {
    float4 v;
    asm volatile("ld.relaxed.sys.global.v4.f32 {%0,%1,%2,%3}, [%4];\n" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
    return v;
}
// Spins until *flag has reached `seq` (wrap-safe); false when the limit ran out.
__device__ bool wait_flag(const uint32_t* flag, uint32_t seq, long long limit) {
    const long long t0 = clock64();
    while ((int32_t)(ld_acquire_sys(flag) - seq) < 0) {
        if (clock64() - t0 > limit) return false;
        __nanosleep(64);
    }
    return true;
}

__global__ void __launch_bounds__(256) tp_peer_reduce_residual_kernel(const PeerReduceParams p) {
    __shared__ int gave_up;
    const int r = p.rank >= 0 ? p.rank : (int)blockIdx.y;
    const int g = blockIdx.x, G = gridDim.x, tid = threadIdx.x;
    if (tid == 0) gave_up = (*reinterpret_cast<volatile int*>(p.err) != 0);
    __syncthreads();
    if (gave_up) return;  // an earlier wait ran out: the group is broken, do not wait again
    // this rank's projection, and with it its stores into the other ranks' slots, ended before this launch began
    if (g == 0 && tid < p.world && tid != r) {
        __threadfence_system();
        st_release_sys(reinterpret_cast<uint32_t*>(p.base[tid] + kFlag1Off) + r, p.seq);
    }
    if (tid < p.world && tid != r) {
        if (!wait_flag(reinterpret_cast<const uint32_t*>(p.base[r] + kFlag1Off) + tid, p.seq, p.wait_cycles)) {
            atomicExch(p.err, 7);
            gave_up = 1;
        }
    }
    __syncthreads();
    if (gave_up) return;

    const int qpr = p.chunk >> 2;  // groups of four columns per row of this rank's range
    const int64_t items = (int64_t)p.M * qpr;
    for (int64_t i = (int64_t)g * blockDim.x + tid; i < items; i += (int64_t)G * blockDim.x) {
        const int row = (int)(i / qpr), col = r * p.chunk + (int)(i % qpr) * 4;
        const size_t off = (size_t)row * p.H + col;
        float4 part[kMaxWorld];
#pragma unroll
        for (int s = 0; s < kMaxWorld; s++)
            if (s < p.world) part[s] = ld_peer_f4(reinterpret_cast<const float*>(p.base[p.push ? r : s] + kDataOff + (size_t)s * p.slot_bytes) + off);
        float4 acc = part[0];
#pragma unroll
        for (int s = 1; s < kMaxWorld; s++)
            if (s < p.world) acc.x += part[s].x, acc.y += part[s].y, acc.z += part[s].z, acc.w += part[s].w;
        uint2 xv = *reinterpret_cast<const uint2*>(reinterpret_cast<const uint16_t*>(p.base[r] + p.x_off) + off);
        const float a0 = bf2f((uint16_t)(xv.x & 0xffff)) + rbf(acc.x), a1 = bf2f((uint16_t)(xv.x >> 16)) + rbf(acc.y);
        const float a2 = bf2f((uint16_t)(xv.y & 0xffff)) + rbf(acc.z), a3 = bf2f((uint16_t)(xv.y >> 16)) + rbf(acc.w);
        xv.x = pack_bf2(a0, a1);
        xv.y = pack_bf2(a2, a3);
#pragma unroll
        for (int s = 0; s < kMaxWorld; s++)
            if (s < p.world) *reinterpret_cast<uint2*>(reinterpret_cast<uint16_t*>(p.base[s] + p.x_off) + off) = xv;
    }
    // the rows of this block are in every rank's x: say so, then wait for the same block of every other rank
    __threadfence_system();
    __syncthreads();
    if (tid < p.world && tid != r) {
        st_release_sys(reinterpret_cast<uint32_t*>(p.base[tid] + kFlag2Off) + (size_t)r * kMaxCtas + g, p.seq);
        if (!wait_flag(reinterpret_cast<const uint32_t*>(p.base[r] + kFlag2Off) + (size_t)tid * kMaxCtas + g, p.seq, p.wait_cycles)) atomicExch(p.err, 8);
    }
}

int grid_for(int M, int chunk, int cap) {
    const int64_t items = (int64_t)M * (chunk / 4);
    return (int)std::max<int64_t>(1, std::min<int64_t>(cap, (items + 1023) / 1024));  // about four items per thread
}

int32_t ensure_err_word(b2_ctx* ctx) {
    if (!ctx->dev_err) {
        B2_CUDA(cudaMalloc((void**)&ctx->dev_err, 16));
        B2_CUDA(cudaMemsetAsync(ctx->dev_err, 0, 16, ctx->stream));
    }
    return B2_OK;
}

size_t region_bytes(int cap_rows, int hidden, int world, size_t* slot_bytes, size_t* x_off) {
    *slot_bytes = ((size_t)cap_rows * hidden * 4 + 255) / 256 * 256;
    *x_off = kDataOff + (size_t)world * *slot_bytes;
    return *x_off + ((size_t)cap_rows * hidden * 2 + 255) / 256 * 256;
}

}  // namespace

// Where this rank's projection stores its f32 result: slot [this rank] of its own region, or (push mode) the columns
// rank q owns straight into slot [this rank] of q's region.
void b2_tp_peer_scatter(const b2_tp_group* g, GemmParams& p) {
    const size_t slot = kDataOff + (size_t)g->rank * g->peer_slot_bytes;
    p.out_f32 = reinterpret_cast<float*>(static_cast<unsigned char*>(g->peer_base[g->rank]) + slot);
    p.f32_chunk = 0;
    if (!g->peer_push) return;
    p.f32_chunk = g->peer_hidden / g->world;
    for (int q = 0; q < g->world; q++) p.out_f32_by_chunk[q] = reinterpret_cast<float*>(static_cast<unsigned char*>(g->peer_base[q]) + slot);
}
uint16_t* b2_tp_peer_x(const b2_tp_group* g) { return reinterpret_cast<uint16_t*>(static_cast<unsigned char*>(g->peer_base[g->rank]) + g->peer_x_off); }

// x (the region's) += sum over ranks of the regions' partial sums, for the first M rows; on the context's stream.
int32_t b2_tp_peer_reduce_residual_launch(b2_tp_group* g, int M) {
    B2_REQUIRE(g && g->peer_ready, B2_ERR_MSG, "peer reduction: the group has no attached peer regions");
    B2_REQUIRE(M >= 0 && M <= g->peer_cap_rows, B2_ERR_MSG, "peer reduction: more rows than the regions hold");
    if (M == 0) return B2_OK;
    if (g->lockstep && g->lockstep->groups[0]->ctx != g->lockstep->groups[g->world - 1]->ctx) {
        // emulated ranks, one host thread each: meet, let rank 0 enqueue the one launch that reduces for everybody,
        // meet again; events carry the order onto the ranks' streams
        b2_tp_lockstep* ls = g->lockstep;
        B2_CUDA(cudaEventRecord(ls->projected[g->rank], g->ctx->stream));
        if (!ls->meet()) return b2_fail(B2_ERR_TIMEOUT, "peer reduction: an emulated rank did not reach the reduction");
        if (g->rank == 0) {
            int32_t rc = B2_OK;
            for (int r = 1; r < ls->n && rc == B2_OK; r++)
                if (cudaStreamWaitEvent(g->ctx->stream, ls->projected[r], 0) != cudaSuccess) rc = b2_fail(B2_ERR_CUDA, "cudaStreamWaitEvent failed");
            if (rc == B2_OK) rc = b2_tp_peer_reduce_residual_local(ls->groups, ls->n, M);
            if (rc == B2_OK && cudaEventRecord(ls->reduced, g->ctx->stream) != cudaSuccess) rc = b2_fail(B2_ERR_CUDA, "cudaEventRecord failed");
            ls->status = rc;
        }
        if (!ls->meet()) return b2_fail(B2_ERR_TIMEOUT, "peer reduction: an emulated rank did not reach the reduction");
        if (ls->status != B2_OK) return g->rank == 0 ? ls->status : b2_fail(ls->status, "peer reduction: rank 0's launch failed");
        if (g->rank != 0) B2_CUDA(cudaStreamWaitEvent(g->ctx->stream, ls->reduced, 0));
        return B2_OK;
    }
    PeerReduceParams p{};
    for (int s = 0; s < g->world; s++) p.base[s] = static_cast<unsigned char*>(g->peer_base[s]);
    p.rank = g->rank;
    p.push = g->peer_push ? 1 : 0;
    p.world = g->world;
    p.M = M;
    p.H = g->peer_hidden;
    p.chunk = g->peer_hidden / g->world;
    p.seq = ++g->peer_seq;
    p.slot_bytes = g->peer_slot_bytes;
    p.x_off = g->peer_x_off;
    p.err = g->ctx->dev_err;
    p.wait_cycles = g->ctx->wait_cycles;
    tp_peer_reduce_residual_kernel<<<grid_for(M, p.chunk, kMaxCtas), 256, 0, g->ctx->stream>>>(p);
    B2_LAUNCHED(g->ctx);
    B2_CUDA(cudaGetLastError());
    return B2_OK;
}

extern "C" {

int32_t b2_tp_peer_alloc(b2_tp_group* g, int32_t max_tokens, int32_t hidden, uint8_t* handle64_out) {
    B2_REQUIRE(g && handle64_out, B2_ERR_MSG, "b2_tp_peer_alloc: null argument");
    B2_REQUIRE(!g->peer_local, B2_ERR_MSG, "b2_tp_peer_alloc: the group already has a region");
    B2_REQUIRE(g->world <= kMaxWorld, B2_ERR_UNSUPPORTED, "peer reduction: at most 8 ranks");
    B2_REQUIRE(max_tokens > 0 && hidden > 0 && hidden % (4 * g->world) == 0, B2_ERR_MSG,
               "b2_tp_peer_alloc: hidden size must be a multiple of 4 x world");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle is 64 bytes");
    B2_CUDA(cudaSetDevice(g->ctx->device));
    B2_CHECK(ensure_err_word(g->ctx));
    size_t x_off = 0, slot_bytes = 0;
    const size_t bytes = region_bytes(max_tokens, hidden, g->world, &slot_bytes, &x_off);
    void* base = nullptr;
    B2_CUDA(cudaMalloc(&base, bytes));
    B2_CUDA(cudaMemsetAsync(base, 0, bytes, g->ctx->stream));
    B2_CUDA(cudaStreamSynchronize(g->ctx->stream));  // zeroed before any other rank can see the handle
    cudaIpcMemHandle_t h;
    if (cudaIpcGetMemHandle(&h, base) != cudaSuccess) {
        cudaGetLastError();
        memset(&h, 0, sizeof(h));  // still usable inside one process (b2_tp_peer_attach_local)
    }
    memcpy(handle64_out, &h, 64);
    g->peer_local = base;
    g->peer_cap_rows = max_tokens;
    g->peer_hidden = hidden;
    g->peer_x_off = x_off;
    g->peer_slot_bytes = slot_bytes;
    return B2_OK;
}

int32_t b2_tp_peer_attach(b2_tp_group* g, const uint8_t* handles, int32_t n_handles) {
    B2_REQUIRE(g && handles, B2_ERR_MSG, "b2_tp_peer_attach: null argument");
    B2_REQUIRE(g->peer_local && !g->peer_ready, B2_ERR_MSG, "b2_tp_peer_attach: call b2_tp_peer_alloc first, attach once");
    B2_REQUIRE(n_handles == g->world, B2_ERR_MSG, "b2_tp_peer_attach: one handle per rank, in rank order");
    B2_CUDA(cudaSetDevice(g->ctx->device));
    for (int s = 0; s < g->world; s++) {
        if (s == g->rank) {
            g->peer_base[s] = g->peer_local;
            continue;
        }
        cudaIpcMemHandle_t h;
        memcpy(&h, handles + (size_t)s * 64, 64);
        void* p = nullptr;
        const cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess) {
            cudaGetLastError();
            for (int t = 0; t < s; t++)
                if (t != g->rank && g->peer_base[t]) cudaIpcCloseMemHandle(g->peer_base[t]), g->peer_base[t] = nullptr;
            return b2_fail(B2_ERR_UNSUPPORTED, std::string("rank ") + std::to_string(s) + "'s region cannot be mapped (" + cudaGetErrorString(e) +
                                                   "): the reductions stay on NCCL");
        }
        g->peer_base[s] = p;
    }
    g->peer_ipc = true;
    g->peer_ready = true;
    return B2_OK;
}

// All ranks of a group living in ONE process on one device (no IPC): the regions are used as they are.
int32_t b2_tp_peer_attach_local(b2_tp_group* const* groups, int32_t n) {
    B2_REQUIRE(groups && n >= 1 && n <= kMaxWorld, B2_ERR_MSG, "b2_tp_peer_attach_local: bad argument");
    for (int s = 0; s < n; s++)
        B2_REQUIRE(groups[s] && groups[s]->world == n && groups[s]->rank == s && groups[s]->peer_local && !groups[s]->peer_ready &&
                       groups[s]->peer_hidden == groups[0]->peer_hidden && groups[s]->peer_cap_rows == groups[0]->peer_cap_rows &&
                       groups[s]->ctx->device == groups[0]->ctx->device,
                   B2_ERR_MSG, "b2_tp_peer_attach_local: the groups must be ranks 0..n-1 of one group with equal regions on one device");
    b2_tp_lockstep* ls = new b2_tp_lockstep();
    ls->n = n;
    B2_CUDA(cudaSetDevice(groups[0]->ctx->device));
    B2_CUDA(cudaEventCreateWithFlags(&ls->reduced, cudaEventDisableTiming));
    for (int s = 0; s < n; s++) {
        ls->groups[s] = groups[s];
        B2_CUDA(cudaEventCreateWithFlags(&ls->projected[s], cudaEventDisableTiming));
    }
    for (int s = 0; s < n; s++) {
        for (int t = 0; t < n; t++) groups[s]->peer_base[t] = groups[t]->peer_local;
        groups[s]->peer_ready = true;
        groups[s]->lockstep = ls;
    }
    return B2_OK;
}

int32_t b2_tp_peer_buffers(const b2_tp_group* g, float** slots_dev, int64_t* slot_stride_floats, uint16_t** x_dev, int32_t* max_tokens,
                           int32_t* hidden) {
    B2_REQUIRE(g && g->peer_ready, B2_ERR_MSG, "b2_tp_peer_buffers: no attached peer regions");
    if (slots_dev) *slots_dev = reinterpret_cast<float*>(static_cast<unsigned char*>(g->peer_base[g->rank]) + kDataOff);
    if (slot_stride_floats) *slot_stride_floats = (int64_t)(g->peer_slot_bytes / 4);
    if (x_dev) *x_dev = b2_tp_peer_x(g);
    if (max_tokens) *max_tokens = g->peer_cap_rows;
    if (hidden) *hidden = g->peer_hidden;
    return B2_OK;
}

int32_t b2_tp_peer_set_push(b2_tp_group* g, int32_t push) {
    B2_REQUIRE(g, B2_ERR_MSG, "b2_tp_peer_set_push: null group");
    B2_CUDA(cudaStreamSynchronize(g->ctx->stream));
    g->peer_push = push != 0;
    return B2_OK;
}

int32_t b2_tp_peer_reduce_residual(b2_tp_group* g, int32_t rows) { return b2_tp_peer_reduce_residual_launch(g, rows); }

// The first half of the fused reduction on its own: this rank's partial projection x[m, in_dim] . W^T (W dense bf16
// when bits == 0, else MLX group-64 Q4 / Q8 with its scales and biases; `hidden` output features), every column
// range stored from the kernel's epilogue into slot [this rank] of the range's owner.
int32_t b2_tp_peer_projection(b2_tp_group* g, const uint16_t* x_dev, int32_t m, int32_t in_dim, const void* w_dev, const uint16_t* scales_dev,
                              const uint16_t* biases_dev, int32_t bits) {
    B2_REQUIRE(g && g->peer_ready && x_dev && w_dev, B2_ERR_MSG, "b2_tp_peer_projection: null argument or no attached peer regions");
    B2_REQUIRE(bits == 0 || ((bits == 4 || bits == 8) && scales_dev && biases_dev), B2_ERR_UNSUPPORTED, "b2_tp_peer_projection: bits must be 0, 4 or 8");
    B2_REQUIRE(m >= 0 && m <= g->peer_cap_rows, B2_ERR_MSG, "b2_tp_peer_projection: more rows than the regions hold");
    GemmParams p{};
    p.x = x_dev;
    p.w = w_dev;
    p.scales = scales_dev;
    p.biases = biases_dev;
    p.bits = bits;
    p.group = 64;
    p.M = m;
    p.N = g->peer_hidden;
    p.K = in_dim;
    p.ldx = in_dim;
    p.ldo = g->peer_hidden;
    p.ldres = g->peer_hidden;
    p.epilogue = EPI_F32;
    b2_tp_peer_scatter(g, p);
    return b2_gemm_launch(g->ctx, p);
}

// The whole group's reduction as ONE launch (grid.y = rank) for groups attached with b2_tp_peer_attach_local:
// kernels that wait on one another must not be separate launches on one device.
int32_t b2_tp_peer_reduce_residual_local(b2_tp_group* const* groups, int32_t n, int32_t rows) {
    B2_REQUIRE(groups && n >= 1 && n <= kMaxWorld && groups[0] && groups[0]->peer_ready && !groups[0]->peer_ipc, B2_ERR_MSG,
               "b2_tp_peer_reduce_residual_local: needs groups attached with b2_tp_peer_attach_local");
    b2_tp_group* g0 = groups[0];
    B2_REQUIRE(rows >= 0 && rows <= g0->peer_cap_rows, B2_ERR_MSG, "peer reduction: more rows than the regions hold");
    if (rows == 0) return B2_OK;
    PeerReduceParams p{};
    for (int s = 0; s < n; s++) p.base[s] = static_cast<unsigned char*>(g0->peer_base[s]);
    p.rank = -1;
    p.push = g0->peer_push ? 1 : 0;
    p.world = n;
    p.M = rows;
    p.H = g0->peer_hidden;
    p.chunk = g0->peer_hidden / n;
    uint32_t seq = 0;
    for (int s = 0; s < n; s++) seq = ++groups[s]->peer_seq;
    p.seq = seq;
    p.slot_bytes = g0->peer_slot_bytes;
    p.x_off = g0->peer_x_off;
    p.err = g0->ctx->dev_err;
    p.wait_cycles = g0->ctx->wait_cycles;
    // every block of every rank resident at once: a cooperative launch, sized to fit
    int per_sm = 0;
    B2_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, tp_peer_reduce_residual_kernel, 256, 0));
    const int cap = std::max(1, per_sm * g0->ctx->sm_count / n);
    dim3 grid(grid_for(rows, p.chunk, std::min(cap, kMaxCtas)), n);
    void* args[] = {&p};
    B2_CUDA(cudaLaunchCooperativeKernel((const void*)tp_peer_reduce_residual_kernel, grid, dim3(256), args, 0, g0->ctx->stream));
    B2_LAUNCHED(g0->ctx);
    return B2_OK;
}

// One forward step of every emulated rank, each on a host thread of its own (b2_model_step per rank); the reductions
// inside meet through the group's lock-step object.  models[r] must be rank r's model of a group attached with
// b2_tp_peer_attach_local, every rank on a context of its own.
int32_t b2_model_step_local_group(b2_model* const* models, int32_t n, const int32_t* ids_host, const int32_t* n_tokens, int32_t num_seqs,
                                  b2_cache* const* caches, uint16_t* logits_host, int32_t* argmax_host) {
    B2_REQUIRE(models && ids_host && n_tokens && caches && n >= 1 && n <= kMaxWorld, B2_ERR_MSG, "b2_model_step_local_group: bad argument");
    for (int r = 0; r < n; r++) {
        B2_REQUIRE(models[r] && models[r]->tp && models[r]->tp->lockstep && models[r]->tp->rank == r && models[r]->tp->world == n, B2_ERR_MSG,
                   "b2_model_step_local_group: models[r] must be rank r of a group attached with b2_tp_peer_attach_local");
        for (int q = 0; q < r; q++)
            B2_REQUIRE(models[q]->ctx != models[r]->ctx, B2_ERR_MSG, "b2_model_step_local_group: every emulated rank needs a context of its own");
    }
    const int vocab = models[0]->cfg.vocab_size;
    std::vector<int32_t> rc(n, B2_OK);
    std::vector<std::string> msg(n);
    std::vector<std::thread> th;
    for (int r = 0; r < n; r++)
        th.emplace_back([&, r]() {
            rc[r] = b2_model_step(models[r], ids_host, n_tokens, num_seqs, const_cast<b2_cache**>(caches + (size_t)r * num_seqs),
                                  logits_host ? logits_host + (size_t)r * num_seqs * vocab : nullptr, argmax_host ? argmax_host + (size_t)r * num_seqs : nullptr);
            if (rc[r] != B2_OK) msg[r] = b2_last_error();
        });
    for (auto& t : th) t.join();
    for (int r = 0; r < n; r++)
        if (rc[r] != B2_OK) return b2_fail(rc[r], "rank " + std::to_string(r) + ": " + msg[r]);
    return B2_OK;
}

}  // extern "C"

void b2_tp_peer_release(b2_tp_group* g) {
    if (!g->peer_local) return;
    cudaStreamSynchronize(g->ctx->stream);
    if (g->lockstep) {
        b2_tp_lockstep* ls = g->lockstep;
        for (int r = 0; r < ls->n; r++)
            if (ls->groups[r] == g) ls->groups[r] = nullptr;
        bool last = true;
        for (int r = 0; r < ls->n; r++) last = last && ls->groups[r] == nullptr;
        g->lockstep = nullptr;
        if (last) {
            for (int r = 0; r < ls->n; r++) cudaEventDestroy(ls->projected[r]);
            cudaEventDestroy(ls->reduced);
            delete ls;
        }
    }
    if (g->peer_ipc)
        for (int s = 0; s < g->world; s++)
            if (s != g->rank && g->peer_base[s]) cudaIpcCloseMemHandle(g->peer_base[s]);
    cudaFree(g->peer_local);
    g->peer_local = nullptr;
    g->peer_ready = false;
}
