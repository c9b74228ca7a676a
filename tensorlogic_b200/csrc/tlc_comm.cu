// Tensor-parallel collectives: one process per GPU, NCCL over NVLink/NVSwitch.
//
// The reference has no multi-GPU code of any kind (no collectives, no
// multi-process launch); this is the exchange step of the Megatron-style
// sharding of the linears: an all-reduce (sum) of the [M, d] f16 partial
// results after each row-parallel projection (attn_output, ffn_down) and an
// all-gather of the vocabulary shards of the logits.
//
// NCCL is bound at run time (dlopen of libnccl.so.2) so that the library loads
// on a machine without it; in a process that already loaded PyTorch the same
// soname resolves to the copy PyTorch brought along.
#include <dlfcn.h>

#include <cstring>

#include "tlc_internal.h"

namespace {

typedef struct ncclComm *ncclComm_t;
typedef struct { char internal[128]; } ncclUniqueId;
enum { ncclSuccess = 0 };
enum { ncclFloat16 = 6, ncclSum = 0 };

struct NcclApi {
    void *handle = nullptr;
    int (*GetUniqueId)(ncclUniqueId *) = nullptr;
    int (*CommInitRank)(ncclComm_t *, int, ncclUniqueId, int) = nullptr;
    int (*CommDestroy)(ncclComm_t) = nullptr;
    int (*AllReduce)(const void *, void *, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
    int (*AllGather)(const void *, void *, size_t, int, ncclComm_t, cudaStream_t) = nullptr;
    const char *(*GetErrorString)(int) = nullptr;
    const char *(*GetLastError)(ncclComm_t) = nullptr;
    std::string error;
};

NcclApi &nccl() {
    static NcclApi api;
    static bool tried = false;
    if (tried) return api;
    tried = true;
    const char *names[] = {"libnccl.so.2", "libnccl.so"};
    for (const char *n : names) {
        api.handle = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
        if (api.handle) break;
    }
    if (!api.handle) {
        api.error = std::string("cannot load libnccl.so.2: ") + (dlerror() ? dlerror() : "unknown error");
        return api;
    }
    auto sym = [&](const char *name) -> void * {
        void *p = dlsym(api.handle, name);
        if (!p && api.error.empty()) api.error = std::string("libnccl lacks ") + name;
        return p;
    };
    api.GetUniqueId = reinterpret_cast<decltype(api.GetUniqueId)>(sym("ncclGetUniqueId"));
    api.CommInitRank = reinterpret_cast<decltype(api.CommInitRank)>(sym("ncclCommInitRank"));
    api.CommDestroy = reinterpret_cast<decltype(api.CommDestroy)>(sym("ncclCommDestroy"));
    api.AllReduce = reinterpret_cast<decltype(api.AllReduce)>(sym("ncclAllReduce"));
    api.AllGather = reinterpret_cast<decltype(api.AllGather)>(sym("ncclAllGather"));
    api.GetErrorString = reinterpret_cast<decltype(api.GetErrorString)>(sym("ncclGetErrorString"));
    return api;
}

}  // namespace

struct tlc_comm {
    tlc_ctx *ctx;
    ncclComm_t comm;
    int rank, world;
};

#define TLC_NCCL(expr)                                                                              \
    do {                                                                                            \
        int _r = (expr);                                                                            \
        if (_r != ncclSuccess)                                                                      \
            return tlc_fail(TLC_ERR_COMM, "%s failed: %s", #expr,                                   \
                            nccl().GetErrorString ? nccl().GetErrorString(_r) : "unknown NCCL error"); \
    } while (0)

extern "C" int32_t tlc_comm_unique_id(void *out128) {
    TLC_REQUIRE(out128, TLC_ERR_INVALID_OPERATION, "comm_unique_id: null pointer");
    NcclApi &api = nccl();
    TLC_REQUIRE(api.error.empty(), TLC_ERR_COMM, "%s", api.error.c_str());
    ncclUniqueId id;
    TLC_NCCL(api.GetUniqueId(&id));
    memcpy(out128, &id, sizeof(id));
    return TLC_OK;
}

extern "C" int32_t tlc_comm_init(tlc_ctx *ctx, const void *id128, int32_t rank, int32_t world, tlc_comm **out) {
    if (int32_t rc = tlc_enter(ctx)) return rc;
    TLC_REQUIRE(id128 && out, TLC_ERR_INVALID_OPERATION, "comm_init: null pointer");
    *out = nullptr;
    TLC_REQUIRE(world >= 1 && rank >= 0 && rank < world, TLC_ERR_INVALID_OPERATION, "comm_init: rank %d of %d", rank,
                world);
    NcclApi &api = nccl();
    TLC_REQUIRE(api.error.empty(), TLC_ERR_COMM, "%s", api.error.c_str());
    ncclUniqueId id;
    memcpy(&id, id128, sizeof(id));
    ncclComm_t c = nullptr;
    TLC_NCCL(api.CommInitRank(&c, world, id, rank));
    *out = new tlc_comm{ctx, c, rank, world};
    return TLC_OK;
}

extern "C" int32_t tlc_comm_destroy(tlc_comm *comm) {
    if (!comm) return TLC_OK;
    cudaSetDevice(comm->ctx->device);
    cudaStreamSynchronize(comm->ctx->stream);
    if (nccl().CommDestroy) nccl().CommDestroy(comm->comm);
    delete comm;
    return TLC_OK;
}

extern "C" int32_t tlc_comm_rank(tlc_comm *comm) { return comm ? comm->rank : -1; }
extern "C" int32_t tlc_comm_size(tlc_comm *comm) { return comm ? comm->world : 0; }

// In-place sum over the ranks of `count` f16 values, on the context's stream.
extern "C" int32_t tlc_allreduce_f16(tlc_ctx *ctx, tlc_comm *comm, void *buf_dev, size_t count) {
    if (int32_t rc = tlc_enter(ctx)) return rc;
    TLC_REQUIRE(comm && buf_dev, TLC_ERR_INVALID_OPERATION, "allreduce: null pointer");
    TLC_REQUIRE(comm->ctx->device == ctx->device, TLC_ERR_DEVICE, "allreduce: communicator lives on another device");
    if (comm->world == 1 || count == 0) return TLC_OK;
    TLC_NCCL(nccl().AllReduce(buf_dev, buf_dev, count, ncclFloat16, ncclSum, comm->comm, ctx->stream));
    ctx->launches++;
    return TLC_OK;
}

// recv[rank * count .. ] = every rank's `count` f16 values.
extern "C" int32_t tlc_allgather_f16(tlc_ctx *ctx, tlc_comm *comm, const void *send_dev, void *recv_dev,
                                     size_t count) {
    if (int32_t rc = tlc_enter(ctx)) return rc;
    TLC_REQUIRE(comm && send_dev && recv_dev, TLC_ERR_INVALID_OPERATION, "allgather: null pointer");
    TLC_REQUIRE(comm->ctx->device == ctx->device, TLC_ERR_DEVICE, "allgather: communicator lives on another device");
    if (count == 0) return TLC_OK;
    if (comm->world == 1) {
        if (send_dev != recv_dev)
            TLC_CUDA(cudaMemcpyAsync(recv_dev, send_dev, count * 2, cudaMemcpyDeviceToDevice, ctx->stream));
        return TLC_OK;
    }
    TLC_NCCL(nccl().AllGather(send_dev, recv_dev, count, ncclFloat16, comm->comm, ctx->stream));
    ctx->launches++;
    return TLC_OK;
}
