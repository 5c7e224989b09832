// Expert parallelism: experts are sharded E/N per rank (contiguous blocks), tokens stay data parallel.  Per layer two
// exchanges over NVLink: the dispatch all-to-all carries each assignment's bf16 token row and its local expert index
// to the owning rank, the combine all-to-all returns the expert's output row.  In between the rank runs exactly the
// single-GPU kernels over the rows it received.  The reference has no counterpart (one GPU, experts paged from SSD:
// csrc/q3_lookahead4_exl3.c); what the read pool did ("bring the expert's bytes to the rows") becomes "bring the rows
// to the expert's bytes".
//
// NCCL point-to-point (grouped ncclSend / ncclRecv with exact counts).  The counts are exchanged with one small
// all-gather and read by the host, which is the only host synchronisation of the layer.  NCCL is loaded at run time
// (dlopen), so a single-GPU process needs no NCCL at all.
#include <dlfcn.h>
#include <nccl.h>

#include <cstring>

#include "common.cuh"
#include "handle.h"

namespace {

struct NcclApi {
    void* lib = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    const char* (*GetErrorString)(ncclResult_t) = nullptr;
    ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*Send)(const void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*Recv)(void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*GroupStart)() = nullptr;
    ncclResult_t (*GroupEnd)() = nullptr;
};

NcclApi* nccl_api() {
    static NcclApi api;
    static bool tried = false;
    if (!tried) {
        tried = true;
        api.lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (!api.lib) api.lib = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
        if (api.lib) {
#define MLXS_SYM(field, name) api.field = reinterpret_cast<decltype(api.field)>(dlsym(api.lib, name))
            MLXS_SYM(GetUniqueId, "ncclGetUniqueId");
            MLXS_SYM(CommInitRank, "ncclCommInitRank");
            MLXS_SYM(CommDestroy, "ncclCommDestroy");
            MLXS_SYM(GetErrorString, "ncclGetErrorString");
            MLXS_SYM(AllGather, "ncclAllGather");
            MLXS_SYM(Send, "ncclSend");
            MLXS_SYM(Recv, "ncclRecv");
            MLXS_SYM(GroupStart, "ncclGroupStart");
            MLXS_SYM(GroupEnd, "ncclGroupEnd");
#undef MLXS_SYM
            if (!api.GetUniqueId || !api.CommInitRank || !api.CommDestroy || !api.AllGather || !api.Send || !api.Recv ||
                !api.GroupStart || !api.GroupEnd || !api.GetErrorString)
                api.lib = nullptr;
        }
    }
    return api.lib ? &api : nullptr;
}

}  // namespace

struct EpState {
    ncclComm_t comm = nullptr;
    DispatchTables rtab{};       // assignments sorted by destination rank
    int32_t *dest = nullptr, *meta = nullptr, *send_meta = nullptr, *recv_meta = nullptr;
    __nv_bfloat16 *send_x = nullptr, *recv_x = nullptr;
    void *recv_ro = nullptr, *ret_ro = nullptr;
    int32_t *counts_dev = nullptr, *all_counts_dev = nullptr, *all_counts_host = nullptr;
};

#define CU(call)                                                                                            \
    do {                                                                                                    \
        cudaError_t e__ = (call);                                                                           \
        if (e__ != cudaSuccess) return mlxs_fail(MLXS_E_CUDA, "%s: %s", #call, cudaGetErrorString(e__));  \
    } while (0)
#define NC(call)                                                                                            \
    do {                                                                                                    \
        ncclResult_t r__ = (call);                                                                          \
        if (r__ != ncclSuccess) return mlxs_fail(MLXS_E_EP, "%s: %s", #call, api->GetErrorString(r__));   \
    } while (0)

namespace mlxs {

// dest rank and local expert index of every assignment; ids outside [0, E) set the status word and go to expert 0
__global__ void ep_dest_kernel(const int32_t* __restrict__ ids, uint32_t A, uint32_t E, uint32_t e_local,
                               int32_t* __restrict__ dest, int32_t* __restrict__ meta, uint32_t* status) {
    const uint32_t a = blockIdx.x * blockDim.x + threadIdx.x;
    if (a >= A) return;
    int32_t id = ids[a];
    if (id < 0 || (uint32_t)id >= E) { atomicMax(status, (uint32_t)ST_BAD_EXPERT_ID); id = 0; }
    dest[a] = id / (int32_t)e_local;
    meta[a] = id % (int32_t)e_local;
}
// rows in destination order: send_x[i] = x[order[i] / k], send_meta[i] = meta[order[i]]; counts[r] from the offsets
__global__ void ep_gather_kernel(const __nv_bfloat16* __restrict__ x, const int32_t* __restrict__ meta,
                                 const uint32_t* __restrict__ order, const uint32_t* __restrict__ offsets, uint32_t A,
                                 uint32_t k, uint32_t H, uint32_t world, __nv_bfloat16* __restrict__ send_x,
                                 int32_t* __restrict__ send_meta, int32_t* __restrict__ counts) {
    const uint32_t i = blockIdx.x;
    if (i == 0 && threadIdx.x < world) counts[threadIdx.x] = (int32_t)(offsets[threadIdx.x + 1] - offsets[threadIdx.x]);
    if (i >= A) return;
    const uint32_t a = order[i];
    const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)(a / k) * H);
    uint4* dst = reinterpret_cast<uint4*>(send_x + (size_t)i * H);
    for (uint32_t j = threadIdx.x; j < H / 8; j += blockDim.x) dst[j] = src[j];
    if (threadIdx.x == 0) send_meta[i] = meta[a];
}
// ro[order[i]] = returned row i
__global__ void ep_scatter_kernel(const uint4* __restrict__ ret, const uint32_t* __restrict__ order, uint32_t A,
                                  uint32_t row_vec4, uint4* __restrict__ ro) {
    const uint32_t i = blockIdx.x;
    if (i >= A) return;
    const uint4* src = ret + (size_t)i * row_vec4;
    uint4* dst = ro + (size_t)order[i] * row_vec4;
    for (uint32_t j = threadIdx.x; j < row_vec4; j += blockDim.x) dst[j] = src[j];
}

}  // namespace mlxs

extern "C" int mlxs_moe_ep_unique_id(void* id128_out) {
    if (!id128_out) return mlxs_fail(MLXS_E_ARG, "ep_unique_id: null argument");
    NcclApi* api = nccl_api();
    if (!api) return mlxs_fail(MLXS_E_EP, "ep_unique_id: libnccl.so.2 could not be loaded (%s)", dlerror());
    static_assert(sizeof(ncclUniqueId) == 128, "the ABI passes the id as 128 bytes");
    ncclUniqueId id;
    NC(api->GetUniqueId(&id));
    memcpy(id128_out, &id, 128);
    return MLXS_OK;
}

extern "C" int mlxs_moe_ep_init(mlxs_moe* h, const void* id128) {
    if (!h || !id128) return mlxs_fail(MLXS_E_ARG, "ep_init: null argument");
    if (h->cfg.ep_world < 2) return mlxs_fail(MLXS_E_EP, "ep_init: the handle was created with ep_world = %u", h->cfg.ep_world);
    if (h->ep) return mlxs_fail(MLXS_E_EP, "ep_init: already initialised");
    NcclApi* api = nccl_api();
    if (!api) return mlxs_fail(MLXS_E_EP, "ep_init: libnccl.so.2 could not be loaded");
    CU(cudaSetDevice(h->cfg.device));
    EpState* ep = new EpState();
    ncclUniqueId id;
    memcpy(&id, id128, 128);
    ncclResult_t r = api->CommInitRank(&ep->comm, (int)h->cfg.ep_world, id, (int)h->cfg.ep_rank);
    if (r != ncclSuccess) { delete ep; return mlxs_fail(MLXS_E_EP, "ncclCommInitRank: %s", api->GetErrorString(r)); }
    const mlxs_moe_config& c = h->cfg;
    const size_t A = (size_t)c.max_tokens * c.top_k, R = h->rows_cap, H = c.hidden, W = c.ep_world;
    const uint32_t mc = (uint32_t)(A / h->chunk_rows + W + 1);
    ep->rtab.max_chunks = mc;
    int rc = 0;
    if ((rc = h->alloc(&ep->rtab.header, 64)) || (rc = h->alloc(&ep->rtab.offsets, (W + 1) * 4)) ||
        (rc = h->alloc(&ep->rtab.order, A * 4)) || (rc = h->alloc(&ep->rtab.chunk_expert, mc * 4)) ||
        (rc = h->alloc(&ep->rtab.chunk_row0, mc * 4)) || (rc = h->alloc(&ep->rtab.chunk_rows, mc * 4)) ||
        (rc = h->alloc(&ep->rtab.group_chunk0, mc * 4)) || (rc = h->alloc(&ep->rtab.group_mc, mc * 4)) ||
        (rc = h->alloc(&ep->dest, A * 4)) || (rc = h->alloc(&ep->meta, A * 4)) || (rc = h->alloc(&ep->send_meta, A * 4)) ||
        (rc = h->alloc(&ep->recv_meta, R * 4)) || (rc = h->alloc(&ep->send_x, A * H * 2)) ||
        (rc = h->alloc(&ep->recv_x, R * H * 2)) || (rc = h->alloc(&ep->recv_ro, R * H * 4)) ||
        (rc = h->alloc(&ep->ret_ro, A * H * 4)) || (rc = h->alloc(&ep->counts_dev, W * 4)) ||
        (rc = h->alloc(&ep->all_counts_dev, W * W * 4))) {
        api->CommDestroy(ep->comm);
        delete ep;
        return rc;
    }
    cudaError_t e = cudaMallocHost(reinterpret_cast<void**>(&ep->all_counts_host), W * W * 4);
    if (e != cudaSuccess) {
        api->CommDestroy(ep->comm);
        delete ep;
        return mlxs_fail(MLXS_E_CUDA, "cudaMallocHost: %s", cudaGetErrorString(e));
    }
    h->ep = ep;
    return MLXS_OK;
}

void mlxs_ep_destroy(mlxs_moe* h) {
    if (!h->ep) return;
    NcclApi* api = nccl_api();
    if (api && h->ep->comm) api->CommDestroy(h->ep->comm);
    if (h->ep->all_counts_host) cudaFreeHost(h->ep->all_counts_host);
    delete h->ep;
    h->ep = nullptr;
}

int mlxs_ep_routed(mlxs_moe* h, uint32_t layer, const void* x_dev, const int32_t* ids_dev, uint32_t T, void* ro,
                   int ro_bf16, cudaStream_t st) {
    EpState* ep = h->ep;
    NcclApi* api = nccl_api();
    if (!ep || !api) return mlxs_fail(MLXS_E_EP, "experts: expert-parallel exchange is not initialised (mlxs_moe_ep_init)");
    const mlxs_moe_config& c = h->cfg;
    const uint32_t A = T * c.top_k, W = c.ep_world, H = c.hidden, me = c.ep_rank;
    const size_t es = ro_bf16 ? 2 : 4;
    const ncclDataType_t ro_type = ro_bf16 ? ncclBfloat16 : ncclFloat32;
    {
        StageTimer tm(h, MLXS_STAGE_EXCHANGE, st);
        if (A) ep_dest_kernel<<<(A + 255) / 256, 256, 0, st>>>(ids_dev, A, c.n_experts, h->e_local, ep->dest, ep->meta, h->status);
        CU(launch_dispatch(ep->dest, A, W, nullptr, ep->rtab, h->chunk_rows, h->group_chunks, 0, h->status, st));
        ep_gather_kernel<<<A ? A : 1, 128, 0, st>>>(static_cast<const __nv_bfloat16*>(x_dev), ep->meta, ep->rtab.order,
                                                   ep->rtab.offsets, A, c.top_k, H, W, ep->send_x, ep->send_meta,
                                                   ep->counts_dev);
        CU(cudaGetLastError());
        NC(api->AllGather(ep->counts_dev, ep->all_counts_dev, W, ncclInt32, ep->comm, st));
        CU(cudaMemcpyAsync(ep->all_counts_host, ep->all_counts_dev, W * W * 4, cudaMemcpyDeviceToHost, st));
        CU(cudaStreamSynchronize(st));
    }
    // all_counts[s * W + d] = rows rank s sends to rank d
    const int32_t* cnt = ep->all_counts_host;
    size_t soff[64], roff[64], R = 0, S = 0;
    if (W > 64) return mlxs_fail(MLXS_E_EP, "experts: ep_world %u > 64", W);
    for (uint32_t r = 0; r < W; ++r) { soff[r] = S; S += (size_t)cnt[me * W + r]; }
    for (uint32_t s = 0; s < W; ++s) { roff[s] = R; R += (size_t)cnt[s * W + me]; }
    if (S != A) return mlxs_fail(MLXS_E_EP, "experts: exchange plan counts %zu rows, the call has %u", S, A);
    if (R > h->rows_cap)
        return mlxs_fail(MLXS_E_EP, "experts: this rank would receive %zu rows, its workspace holds %u (load imbalance beyond the capacity)", R, h->rows_cap);
    {
        StageTimer tm(h, MLXS_STAGE_EXCHANGE, st);
        NC(api->GroupStart());
        for (uint32_t r = 0; r < W; ++r) {
            const size_t ns = (size_t)cnt[me * W + r], nr = (size_t)cnt[r * W + me];
            if (ns) {
                NC(api->Send(ep->send_x + soff[r] * H, ns * H, ncclBfloat16, (int)r, ep->comm, st));
                NC(api->Send(ep->send_meta + soff[r], ns, ncclInt32, (int)r, ep->comm, st));
            }
            if (nr) {
                NC(api->Recv(ep->recv_x + roff[r] * H, nr * H, ncclBfloat16, (int)r, ep->comm, st));
                NC(api->Recv(ep->recv_meta + roff[r], nr, ncclInt32, (int)r, ep->comm, st));
            }
        }
        NC(api->GroupEnd());
    }
    h->stats.a2a_bytes_sent += (S - (size_t)cnt[me * W + me]) * ((size_t)H * 2 + 4) + (R - (size_t)cnt[me * W + me]) * H * es;
    h->stats.a2a_bytes_recv += (R - (size_t)cnt[me * W + me]) * ((size_t)H * 2 + 4) + (S - (size_t)cnt[me * W + me]) * H * es;
    // the single-GPU kernels over the received rows: every row is its own "token" with one expert
    int rc = mlxs_run_routed(h, layer, ep->recv_x, ep->recv_meta, (uint32_t)R, 1, h->e_local, h->e_first, ep->recv_ro, ro_bf16, st);
    if (rc) return rc;
    {
        StageTimer tm(h, MLXS_STAGE_EXCHANGE, st);
        NC(api->GroupStart());
        for (uint32_t r = 0; r < W; ++r) {
            const size_t ns = (size_t)cnt[r * W + me], nr = (size_t)cnt[me * W + r];
            if (ns) NC(api->Send(static_cast<char*>(ep->recv_ro) + roff[r] * H * es, ns * H, ro_type, (int)r, ep->comm, st));
            if (nr) NC(api->Recv(static_cast<char*>(ep->ret_ro) + soff[r] * H * es, nr * H, ro_type, (int)r, ep->comm, st));
        }
        NC(api->GroupEnd());
        if (A) mlxs::ep_scatter_kernel<<<A, 128, 0, st>>>(static_cast<const uint4*>(ep->ret_ro), ep->rtab.order, A,
                                                        (uint32_t)(H * es / 16), static_cast<uint4*>(ro));
        CU(cudaGetLastError());
    }
    return MLXS_OK;
}
