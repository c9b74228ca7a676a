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

namespace {

// ---------------------------------------------------------------------------
// One-shot all-reduce over NVLink peer memory, fused with the residual add.
//
// The row-parallel projections of a decode step leave [M, d] f16 partial sums
// on every rank (16 KB for M = 1, d = 8192): far too small for a ring, and a
// library all-reduce costs tens of microseconds per call, 160 times per step
// at 80 layers.  Here every rank owns an exchange block that its peers map
// through CUDA IPC.  One kernel per all-reduce, kChunks CTAs, each on its own
// slice of the vector and its own flags, so no CTA waits for another CTA of
// the same GPU:
//   1. store the slice of the local partial into slot [parity][rank] of every
//      peer's block (plain 16-byte stores over NVLink), fence, then store the
//      sequence number into flag [rank][chunk] of every peer (release);
//   2. wait (bounded) until the flags of all peers in the local block carry
//      that sequence number (acquire);
//   3. sum the world partials in rank order in f32 (the local one straight
//      from the GEMV's output, the others from the local block), round to f16
//      once, add the residual, store.  Every rank computes bit-identical sums.
// Two slots alternate by sequence parity: a rank can be at most one all-reduce
// ahead of a peer, because finishing one needs every peer's flag for it.  The
// sequence number lives in device memory (one per chunk), so a CUDA graph that
// replays the same launch keeps counting.
// ---------------------------------------------------------------------------
constexpr int kP2pChunks = 8;      // CTAs of a short all-reduce (each on its own slice and flags)
constexpr int kP2pMaxChunks = 32;  // CTAs of a long one (from 64 Ki values on); the flag rows are this wide
constexpr int kP2pMaxWorld = 8;
constexpr size_t kP2pFlagsOffset = 0;     // uint32 [world][kP2pMaxChunks], written by peers
constexpr size_t kP2pSeqOffset = 1024;    // uint32 [kP2pMaxChunks], local
constexpr size_t kP2pLLSeqOffset = 2048;  // uint32 [kP2pLLMaxCtas], local: the flagged-word form's call counters
constexpr size_t kP2pDataOffset = 4096;   // f16 [2][world][max_elems], written by peers
// then, 256-byte aligned: {f16 x 2, flag} [2][world][ll_cap / 2], written by peers (flagged-word form)
constexpr uint32_t kP2pLLMaxElems = 262144;  // longest vector the flagged-word form takes (32 rows of 8192)
constexpr int kP2pLLMaxCtas = kP2pLLMaxElems / (4 * 256);

struct P2pParams {
    uint8_t *peer[kP2pMaxWorld];  // exchange blocks, peer[rank] is the local one
    const __half *partial;        // [n] this rank's partial sums
    const __half *residual;       // [n] or null
    __half *out;                  // [n]
    int rank, world;
    uint32_t n, max_elems;
    size_t ll_off;    // byte offset of the flagged-word slots in an exchange block
    uint32_t ll_cap;  // elements per flagged-word slot
    tlc_dev_status *status;
    uint64_t wait_ns;  // how long the wait for the peers may last
};

__device__ __forceinline__ void st_release_sys(uint32_t *p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t *p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

__global__ void __launch_bounds__(256) allreduce_residual_kernel(const P2pParams p) {
    __shared__ int timed_out;
    tlc_pdl_prologue();  // the partial sums come from the previous kernel of the stream
    const int tid = threadIdx.x, chunk = blockIdx.x, chunks = (int)gridDim.x;  // 8 or 32 CTAs, by the vector's length
    const uint32_t per = ((p.n + chunks * 8 - 1) / (chunks * 8)) * 8;  // elements per chunk, multiple of 8
    const uint32_t lo = min(p.n, chunk * per), hi = min(p.n, lo + per);
    uint8_t *local = p.peer[p.rank];
    uint32_t *seq = reinterpret_cast<uint32_t *>(local + kP2pSeqOffset) + chunk;
    const uint32_t s = *seq + 1;
    const uint32_t parity = s & 1u;
    if (tid == 0) timed_out = 0;

    // 1. push this rank's slice to every peer
    const size_t slot_mine = ((size_t)parity * p.world + p.rank) * p.max_elems;
    for (int r = 0; r < p.world; r++) {
        if (r == p.rank) continue;
        __half *dst = reinterpret_cast<__half *>(p.peer[r] + kP2pDataOffset) + slot_mine;
        for (uint32_t i = lo + 8 * tid; i < hi; i += 8 * blockDim.x)
            *reinterpret_cast<uint4 *>(dst + i) = *reinterpret_cast<const uint4 *>(p.partial + i);
    }
    __threadfence_system();
    __syncthreads();
    if (tid < p.world && tid != p.rank)
        st_release_sys(reinterpret_cast<uint32_t *>(p.peer[tid] + kP2pFlagsOffset) + p.rank * kP2pMaxChunks + chunk, s);

    // 2. wait for every peer's slice
    if (tid < p.world && tid != p.rank) {
        const uint32_t *flag = reinterpret_cast<const uint32_t *>(local + kP2pFlagsOffset) + tid * kP2pMaxChunks + chunk;
        bool ok = false;
        const uint64_t t0 = tlc_globaltimer_ns();
        do {
            if ((int32_t)(ld_acquire_sys(flag) - s) >= 0) {
                ok = true;
                break;
            }
            __nanosleep(32);
        } while (tlc_globaltimer_ns() - t0 < p.wait_ns);
        if (!ok) {
            timed_out = 1;
            if (atomicCAS(&p.status->code, 0, 3) == 0) p.status->where = 100 + tid;
        }
    }
    __syncthreads();

    // 3. sum in rank order, add the residual
    if (!timed_out) {
        const __half *slots = reinterpret_cast<const __half *>(local + kP2pDataOffset) + (size_t)parity * p.world * p.max_elems;
        for (uint32_t i = lo + 8 * tid; i < hi; i += 8 * blockDim.x) {
            float acc[8];
#pragma unroll
            for (int j = 0; j < 8; j++) acc[j] = 0.f;
            for (int r = 0; r < p.world; r++) {
                const uint4 v = r == p.rank ? *reinterpret_cast<const uint4 *>(p.partial + i)
                                            : __ldcg(reinterpret_cast<const uint4 *>(slots + (size_t)r * p.max_elems + i));
                const __half2 *h = reinterpret_cast<const __half2 *>(&v);
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const float2 f = __half22float2(h[j]);
                    acc[2 * j] += f.x;
                    acc[2 * j + 1] += f.y;
                }
            }
            __align__(16) __half o[8];
#pragma unroll
            for (int j = 0; j < 8; j++) o[j] = __float2half_rn(acc[j]);
            if (p.residual) {
                const uint4 rv = *reinterpret_cast<const uint4 *>(p.residual + i);
                const __half *rh = reinterpret_cast<const __half *>(&rv);
#pragma unroll
                for (int j = 0; j < 8; j++) o[j] = __hadd(rh[j], o[j]);
            }
            *reinterpret_cast<uint4 *>(p.out + i) = *reinterpret_cast<const uint4 *>(o);
        }
    }
    // Every one of the kP2pMaxChunks counters follows every call, whatever its CTA count: the
    // parity of the slots is then the same for all slices of all calls, also when short and long
    // vectors alternate on one communicator.
    if (tid < kP2pMaxChunks / chunks) seq[tid * chunks] = s;
}


// ---------------------------------------------------------------------------
// The same all-reduce + residual for short vectors (a decode step's [M, d] partial sums up to
// 256 Ki values) without any fence or separate flag: every 4 bytes of data (two f16) travel in
// one 8-byte store together with the call's sequence number, and the receiver polls the very
// words it needs until they carry that number (the scheme of NCCL's LL protocol).  An 8-byte
// aligned store arrives whole, so a word whose flag matches holds this call's data.  Latency
// is one store across NVLink plus the poll, against two system-scope fences and a flag hop in
// the kernel above.  A thread owns four values: it sends them as one 16-byte store (two
// flagged words) to every peer, polls the peers' words for the same four values in its own
// block, sums in rank order in f32, rounds once, adds the residual.  Two slots alternate by
// the parity of the sequence number, as above.  Every poll is bounded.
// ---------------------------------------------------------------------------
__device__ __forceinline__ void st_volatile_v4(void *p, uint4 v) {
    asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
                 : "memory");
}
__device__ __forceinline__ uint4 ld_volatile_v4(const void *p) {
    uint4 v;
    asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}

__global__ void __launch_bounds__(256) allreduce_ll_kernel(const P2pParams p) {
    tlc_pdl_prologue();  // the partial sums come from the previous kernel of the stream
    uint8_t *local = p.peer[p.rank];
    uint32_t *seq = reinterpret_cast<uint32_t *>(local + kP2pLLSeqOffset) + blockIdx.x;
    const uint32_t s = *seq + 1;  // the first call carries 1: a zero-initialised slot matches no call; later a slot holds s - 2
    const uint32_t parity = s & 1u;
    const uint32_t i = 4u * (blockIdx.x * blockDim.x + threadIdx.x);  // first of this thread's four values
    if (i < p.n) {
        const uint2 mine = *reinterpret_cast<const uint2 *>(p.partial + i);
        // byte offset of values i .. i+3 in slot [parity][rank]: 4 bytes per value (2 of data, 2 of flag)
        const size_t word = (size_t)i * 4;
        const size_t slot_bytes = (size_t)p.ll_cap * 4;
        const uint4 packet = make_uint4(mine.x, s, mine.y, s);
        for (int r = 0; r < p.world; r++)
            if (r != p.rank) st_volatile_v4(p.peer[r] + p.ll_off + ((size_t)parity * p.world + p.rank) * slot_bytes + word, packet);
        uint2 got[kP2pMaxWorld];
        bool ok = true;
        for (int r = 0; r < p.world && ok; r++) {
            if (r == p.rank) {
                got[r] = mine;
                continue;
            }
            const uint8_t *src = local + p.ll_off + ((size_t)parity * p.world + r) * slot_bytes + word;
            uint4 v = ld_volatile_v4(src);
            if (v.y != s || v.w != s) {
                const uint64_t t0 = tlc_globaltimer_ns();
                do {
                    v = ld_volatile_v4(src);
                } while ((v.y != s || v.w != s) && tlc_globaltimer_ns() - t0 < p.wait_ns);
                if (v.y != s || v.w != s) {
                    ok = false;
                    if (atomicCAS(&p.status->code, 0, 3) == 0) p.status->where = 120 + r;
                }
            }
            got[r] = make_uint2(v.x, v.z);
        }
        if (ok) {
            float acc[4] = {0.f, 0.f, 0.f, 0.f};
            for (int r = 0; r < p.world; r++) {  // rank order: every rank computes the same bits
                const float2 a = __half22float2(*reinterpret_cast<const __half2 *>(&got[r].x));
                const float2 b = __half22float2(*reinterpret_cast<const __half2 *>(&got[r].y));
                acc[0] += a.x;
                acc[1] += a.y;
                acc[2] += b.x;
                acc[3] += b.y;
            }
            __align__(8) __half o[4];
#pragma unroll
            for (int j = 0; j < 4; j++) o[j] = __float2half_rn(acc[j]);
            if (p.residual) {
                const uint2 rv = *reinterpret_cast<const uint2 *>(p.residual + i);
                const __half *rh = reinterpret_cast<const __half *>(&rv);
#pragma unroll
                for (int j = 0; j < 4; j++) o[j] = __hadd(rh[j], o[j]);
            }
            *reinterpret_cast<uint2 *>(p.out + i) = *reinterpret_cast<const uint2 *>(o);
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) *seq = s;
}

__global__ void add_f16_kernel(const __half *__restrict__ a, const __half *__restrict__ b, __half *__restrict__ y,
                               size_t n) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) y[i] = __hadd(a[i], b[i]);
}

}  // namespace

struct tlc_comm {
    tlc_ctx *ctx;
    ncclComm_t comm;
    int rank, world;
    // peer-memory exchange (tlc_comm_p2p_export / _import)
    uint8_t *p2p_local = nullptr;
    uint8_t *p2p_peer[kP2pMaxWorld] = {};
    size_t p2p_max_elems = 0;
    size_t p2p_ll_off = 0;  // flagged-word slots of the exchange block
    uint32_t p2p_ll_cap = 0;
    bool p2p_ready = false;
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
    tlc_comm *cm = new tlc_comm();
    cm->ctx = ctx;
    cm->comm = c;
    cm->rank = rank;
    cm->world = world;
    *out = cm;
    return TLC_OK;
}

extern "C" int32_t tlc_comm_destroy(tlc_comm *comm) {
    if (!comm) return TLC_OK;
    cudaSetDevice(comm->ctx->device);
    cudaStreamSynchronize(comm->ctx->stream);
    for (int r = 0; r < comm->world && r < kP2pMaxWorld; r++)
        if (comm->p2p_ready && r != comm->rank && comm->p2p_peer[r]) cudaIpcCloseMemHandle(comm->p2p_peer[r]);
    if (comm->p2p_local) cudaFree(comm->p2p_local);
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

// ---- peer-memory exchange ----------------------------------------------------

// Allocates this rank's exchange block for all-reduces of up to max_elems f16
// values and writes its CUDA IPC handle (TLC_IPC_HANDLE_BYTES bytes) to handle_out.
extern "C" int32_t tlc_comm_p2p_export(tlc_comm *comm, size_t max_elems, void *handle_out) {
    TLC_REQUIRE(comm && handle_out, TLC_ERR_INVALID_OPERATION, "comm_p2p_export: null pointer");
    if (int32_t rc = tlc_enter(comm->ctx)) return rc;
    TLC_REQUIRE(comm->world <= kP2pMaxWorld, TLC_ERR_COMM, "peer-memory all-reduce supports up to %d ranks (got %d)",
                kP2pMaxWorld, comm->world);
    TLC_REQUIRE(!comm->p2p_local, TLC_ERR_INVALID_OPERATION, "comm_p2p_export: already exported");
    TLC_REQUIRE(max_elems > 0 && max_elems % 8 == 0, TLC_ERR_INVALID_DIMENSION,
                "comm_p2p_export: capacity %zu is not a positive multiple of 8", max_elems);
    static_assert(sizeof(cudaIpcMemHandle_t) == TLC_IPC_HANDLE_BYTES, "IPC handle size");
    const size_t ll_off = (kP2pDataOffset + (size_t)2 * comm->world * max_elems * sizeof(__half) + 255) & ~(size_t)255;
    const uint32_t ll_cap = (uint32_t)(max_elems < kP2pLLMaxElems ? max_elems : kP2pLLMaxElems);
    const size_t bytes = ll_off + (size_t)2 * comm->world * ll_cap * 4;
    void *blk = nullptr;
    cudaError_t e = cudaMalloc(&blk, bytes);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return tlc_fail(TLC_ERR_ALLOCATION, "exchange block of %zu bytes failed: %s", bytes, cudaGetErrorString(e));
    }
    TLC_CUDA(cudaMemset(blk, 0, bytes));
    TLC_CUDA(cudaDeviceSynchronize());
    cudaIpcMemHandle_t h;
    e = cudaIpcGetMemHandle(&h, blk);
    if (e != cudaSuccess) {
        cudaGetLastError();
        cudaFree(blk);
        return tlc_fail(TLC_ERR_COMM, "cudaIpcGetMemHandle failed: %s", cudaGetErrorString(e));
    }
    memcpy(handle_out, &h, sizeof(h));
    comm->p2p_local = static_cast<uint8_t *>(blk);
    comm->p2p_max_elems = max_elems;
    comm->p2p_ll_off = ll_off;
    comm->p2p_ll_cap = ll_cap;
    return TLC_OK;
}

// Maps the peers' exchange blocks: `handles` holds world handles in rank order
// (every rank's tlc_comm_p2p_export output, gathered by the host).
extern "C" int32_t tlc_comm_p2p_import(tlc_comm *comm, const void *handles) {
    TLC_REQUIRE(comm && handles, TLC_ERR_INVALID_OPERATION, "comm_p2p_import: null pointer");
    if (int32_t rc = tlc_enter(comm->ctx)) return rc;
    TLC_REQUIRE(comm->p2p_local && !comm->p2p_ready, TLC_ERR_INVALID_OPERATION,
                "comm_p2p_import: export first, import once");
    const uint8_t *hs = static_cast<const uint8_t *>(handles);
    for (int r = 0; r < comm->world; r++) {
        if (r == comm->rank) {
            comm->p2p_peer[r] = comm->p2p_local;
            continue;
        }
        cudaIpcMemHandle_t h;
        memcpy(&h, hs + (size_t)r * TLC_IPC_HANDLE_BYTES, sizeof(h));
        void *ptr = nullptr;
        cudaError_t e = cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess) {
            cudaGetLastError();
            for (int q = 0; q < r; q++)
                if (q != comm->rank && comm->p2p_peer[q]) cudaIpcCloseMemHandle(comm->p2p_peer[q]);
            return tlc_fail(TLC_ERR_COMM, "cudaIpcOpenMemHandle for rank %d failed: %s", r, cudaGetErrorString(e));
        }
        comm->p2p_peer[r] = static_cast<uint8_t *>(ptr);
    }
    comm->p2p_ready = true;
    return TLC_OK;
}

extern "C" int32_t tlc_comm_p2p_ready(tlc_comm *comm) { return comm && comm->p2p_ready ? 1 : 0; }

// out = residual + sum over ranks of partial (f32 sum in rank order, one f16
// rounding, then the f16 add).  `partial_dev` may be overwritten.  Runs as one
// peer-memory kernel when the exchange is set up and the vector fits; as NCCL
// all-reduce + add otherwise.
extern "C" int32_t tlc_allreduce_residual_f16(tlc_ctx *ctx, tlc_comm *comm, void *partial_dev,
                                              const void *residual_dev, void *out_dev, size_t count) {
    if (int32_t rc = tlc_enter(ctx)) return rc;
    TLC_REQUIRE(comm && partial_dev && out_dev, TLC_ERR_INVALID_OPERATION, "allreduce_residual: null pointer");
    TLC_REQUIRE(comm->ctx->device == ctx->device, TLC_ERR_DEVICE, "allreduce: communicator lives on another device");
    if (count == 0) return TLC_OK;
    const bool aligned = count % 8 == 0 && ((uintptr_t)partial_dev | (uintptr_t)out_dev | (uintptr_t)residual_dev) % 16 == 0;
    if (comm->world > 1 && comm->p2p_ready && aligned && count <= comm->p2p_max_elems) {
        P2pParams p{};
        for (int r = 0; r < comm->world; r++) p.peer[r] = comm->p2p_peer[r];
        p.partial = static_cast<const __half *>(partial_dev);
        p.residual = static_cast<const __half *>(residual_dev);
        p.out = static_cast<__half *>(out_dev);
        p.rank = comm->rank;
        p.world = comm->world;
        p.n = (uint32_t)count;
        p.max_elems = (uint32_t)comm->p2p_max_elems;
        p.status = ctx->dev_status;
        p.wait_ns = ctx->wait_ns;
        p.ll_off = comm->p2p_ll_off;
        p.ll_cap = comm->p2p_ll_cap;
        // short vectors: data and flag in one word, no fences (option "comm_ll")
        const bool ll = ctx->comm_ll && count <= comm->p2p_ll_cap && ((uintptr_t)partial_dev | (uintptr_t)out_dev | (uintptr_t)residual_dev) % 8 == 0;
        cudaError_t le = ll ? tlc_launch_pdl(ctx, allreduce_ll_kernel, dim3((unsigned)((count / 4 + 255) / 256)), dim3(256), 0, p)
                            : tlc_launch_pdl(ctx, allreduce_residual_kernel, dim3(count >= 65536 ? kP2pMaxChunks : kP2pChunks),
                                             dim3(256), 0, p);
        if (le != cudaSuccess) {
            cudaGetLastError();
            return tlc_fail(TLC_ERR_CUDA, "all-reduce launch failed: %s", cudaGetErrorString(le));
        }
        TLC_CHECK_LAUNCH(ctx);
        return TLC_OK;
    }
    if (comm->world > 1) {
        TLC_NCCL(nccl().AllReduce(partial_dev, partial_dev, count, ncclFloat16, ncclSum, comm->comm, ctx->stream));
        ctx->launches++;
    }
    if (residual_dev) {
        add_f16_kernel<<<(unsigned)((count + 255) / 256), 256, 0, ctx->stream>>>(
            static_cast<const __half *>(residual_dev), static_cast<const __half *>(partial_dev),
            static_cast<__half *>(out_dev), count);
        TLC_CHECK_LAUNCH(ctx);
    } else if (out_dev != partial_dev) {
        TLC_CUDA(cudaMemcpyAsync(out_dev, partial_dev, count * 2, cudaMemcpyDeviceToDevice, ctx->stream));
    }
    return TLC_OK;
}

// Failure-detection self-test (no second GPU, no communicator needed): an
// all-reduce kernel (the fenced form, or the flagged-word form) runs as "rank 0 of 2"
// over two exchange blocks on this GPU; nothing ever plays rank 1, so the wait for its
// flags (its flagged words) runs out after the context's limit, the status word is set
// and the kernel returns.
int32_t tlc_selftest_peer_wait(tlc_ctx *ctx, bool flagged_words) {
    const size_t n = 1024;
    const size_t ll_off = (kP2pDataOffset + (size_t)2 * 2 * n * sizeof(__half) + 255) & ~(size_t)255;
    const size_t bytes = ll_off + (size_t)2 * 2 * n * 4;
    uint8_t *blk[2] = {nullptr, nullptr};
    __half *vec = nullptr;
    TLC_CUDA(cudaMalloc(&blk[0], bytes));
    TLC_CUDA(cudaMalloc(&blk[1], bytes));
    TLC_CUDA(cudaMalloc(&vec, 2 * n * sizeof(__half)));
    TLC_CUDA(cudaMemsetAsync(blk[0], 0, bytes, ctx->stream));
    TLC_CUDA(cudaMemsetAsync(blk[1], 0, bytes, ctx->stream));
    TLC_CUDA(cudaMemsetAsync(vec, 0, 2 * n * sizeof(__half), ctx->stream));
    P2pParams p{};
    p.peer[0] = blk[0];
    p.peer[1] = blk[1];
    p.partial = vec;
    p.residual = nullptr;
    p.out = vec + n;
    p.rank = 0;
    p.world = 2;
    p.n = (uint32_t)n;
    p.max_elems = (uint32_t)n;
    p.ll_off = ll_off;
    p.ll_cap = (uint32_t)n;
    p.status = ctx->dev_status;
    p.wait_ns = ctx->wait_ns;
    if (flagged_words)
        allreduce_ll_kernel<<<(unsigned)((n / 4 + 255) / 256), 256, 0, ctx->stream>>>(p);
    else
        allreduce_residual_kernel<<<kP2pChunks, 256, 0, ctx->stream>>>(p);
    ctx->launches++;
    cudaError_t e = cudaGetLastError();
    cudaStreamSynchronize(ctx->stream);
    cudaFree(blk[0]);
    cudaFree(blk[1]);
    cudaFree(vec);
    if (e != cudaSuccess) return tlc_fail(TLC_ERR_CUDA, "self-test launch failed: %s", cudaGetErrorString(e));
    return TLC_OK;
}
