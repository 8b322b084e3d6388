// Tensor-parallel group: one rank per GPU, an NCCL communicator for the two reductions per layer.
//
// The reference has no tensor parallelism (it is a single-device MLX program); this is the exchange
// step the 32B configuration needs: every rank owns n_kv_heads / world KV heads with their q heads,
// the matching rows of q/k/v and gate/up and the matching COLUMNS of o_proj / down_proj, so o_proj and
// down_proj produce partial sums of the hidden state that are added across ranks
// (LlamaAttention::output, src/models/llama.rs:823-831, and LlamaMlp::forward, :1040-1045, are the two
// places whose results become partial).
//
// NCCL is bound at run time (dlopen of libnccl.so.2) so the library keeps a single hard dependency,
// the CUDA runtime; a process that already carries NCCL (for its own barriers, say) shares that copy.
#include <dlfcn.h>
#include <nccl.h>

#include "common.cuh"
#include "engine.h"

namespace {

struct NcclApi {
    ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
    const char* (*GetErrorString)(ncclResult_t) = nullptr;
    void* handle = nullptr;
    std::string why;
};

NcclApi& api() {
    static NcclApi a;
    static bool tried = false;
    if (tried) return a;
    tried = true;
    const char* names[] = {"libnccl.so.2", "libnccl.so"};
    for (const char* n : names) {
        a.handle = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
        if (a.handle) break;
    }
    if (!a.handle) {
        a.why = std::string("libnccl.so.2 could not be loaded: ") + (dlerror() ? dlerror() : "unknown");
        return a;
    }
    a.GetUniqueId = reinterpret_cast<decltype(a.GetUniqueId)>(dlsym(a.handle, "ncclGetUniqueId"));
    a.CommInitRank = reinterpret_cast<decltype(a.CommInitRank)>(dlsym(a.handle, "ncclCommInitRank"));
    a.CommDestroy = reinterpret_cast<decltype(a.CommDestroy)>(dlsym(a.handle, "ncclCommDestroy"));
    a.AllReduce = reinterpret_cast<decltype(a.AllReduce)>(dlsym(a.handle, "ncclAllReduce"));
    a.GetErrorString = reinterpret_cast<decltype(a.GetErrorString)>(dlsym(a.handle, "ncclGetErrorString"));
    if (!a.GetUniqueId || !a.CommInitRank || !a.CommDestroy || !a.AllReduce || !a.GetErrorString) {
        a.why = "libnccl.so.2 lacks one of the five entry points this library binds";
        a.handle = nullptr;
    }
    return a;
}

int32_t nccl_fail(const char* what, ncclResult_t r) {
    return b2_fail(B2_ERR_CUDA, std::string(what) + ": " + (api().GetErrorString ? api().GetErrorString(r) : "NCCL error"));
}

}  // namespace

int32_t b2_tp_all_reduce_sum_f32(b2_tp_group* g, float* buf, size_t n) {
    if (!g || g->world == 1) return B2_OK;
    B2_REQUIRE(g->comm, B2_ERR_UNSUPPORTED, "this group was created without an NCCL id: it reduces over peer memory only");
    const ncclResult_t r = api().AllReduce(buf, buf, n, ncclFloat32, ncclSum, reinterpret_cast<ncclComm_t>(g->comm), g->ctx->stream);
    if (r != ncclSuccess) return nccl_fail("ncclAllReduce", r);
    return B2_OK;
}

extern "C" {

int32_t b2_tp_unique_id(uint8_t* out128) {
    B2_REQUIRE(out128, B2_ERR_MSG, "b2_tp_unique_id: null argument");
    B2_REQUIRE(api().handle, B2_ERR_UNSUPPORTED, api().why);
    static_assert(sizeof(ncclUniqueId) == 128, "unique id is 128 bytes");
    ncclUniqueId id;
    const ncclResult_t r = api().GetUniqueId(&id);
    if (r != ncclSuccess) return nccl_fail("ncclGetUniqueId", r);
    memcpy(out128, &id, 128);
    return B2_OK;
}

int32_t b2_tp_group_create(b2_ctx* ctx, const uint8_t* id128, int32_t rank, int32_t world, b2_tp_group** out) {
    B2_REQUIRE(ctx && out, B2_ERR_MSG, "b2_tp_group_create: null argument");
    B2_REQUIRE(world >= 1 && rank >= 0 && rank < world, B2_ERR_MSG, "b2_tp_group_create: rank outside the group");
    b2_tp_group* g = new b2_tp_group();
    g->ctx = ctx;
    g->rank = rank;
    g->world = world;
    if (world > 1 && id128) {
        if (!api().handle) {
            delete g;
            return b2_fail(B2_ERR_UNSUPPORTED, api().why);
        }
        B2_CUDA(cudaSetDevice(ctx->device));
        ncclUniqueId id;
        memcpy(&id, id128, 128);
        ncclComm_t comm = nullptr;
        const ncclResult_t r = api().CommInitRank(&comm, world, id, rank);
        if (r != ncclSuccess) {
            delete g;
            return nccl_fail("ncclCommInitRank", r);
        }
        g->comm = comm;
    }
    *out = g;
    return B2_OK;
}

int32_t b2_tp_group_free(b2_tp_group* g) {
    if (!g) return B2_OK;
    b2_tp_peer_release(g);
    if (g->comm) {
        cudaStreamSynchronize(g->ctx->stream);
        api().CommDestroy(reinterpret_cast<ncclComm_t>(g->comm));
    }
    delete g;
    return B2_OK;
}

int32_t b2_tp_group_info(const b2_tp_group* g, int32_t* rank, int32_t* world) {
    B2_REQUIRE(g && rank && world, B2_ERR_MSG, "b2_tp_group_info: null argument");
    *rank = g->rank;
    *world = g->world;
    return B2_OK;
}

// In-place sum of an f32 device buffer over the group, enqueued on the context's stream.
int32_t b2_tp_all_reduce_f32(b2_tp_group* g, float* buf_dev, int64_t n) {
    B2_REQUIRE(g && buf_dev && n >= 0, B2_ERR_MSG, "b2_tp_all_reduce_f32: bad argument");
    return b2_tp_all_reduce_sum_f32(g, buf_dev, (size_t)n);
}

}  // extern "C"
