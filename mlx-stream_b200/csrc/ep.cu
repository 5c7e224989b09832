// Expert parallelism: experts are sharded E/N per rank (contiguous blocks), tokens stay data parallel.  Per layer two
// exchanges over NVLink: the dispatch all-to-all carries each assignment's bf16 token row and its local expert index
// to the owning rank, the combine all-to-all returns the expert's output row.  In between the rank runs exactly the
// single-GPU kernels over the rows it received.  The reference has no counterpart (one GPU, experts paged from SSD:
// csrc/q3_lookahead4_exl3.c); what the read pool did ("bring the expert's bytes to the rows") becomes "bring the rows
// to the expert's bytes".
//
// Two forms.  mlxs_ep_routed returns the unweighted row of every assignment (what the reference's Hook.routed gives):
// every assignment's token row travels and one output row per assignment comes back.  mlxs_ep_combined is the form the
// layer uses with the f32 combine: a token's row travels once per destination rank, however many of its experts live
// there, the owning rank folds w x row over the token's experts it holds (f32, in the token's k order), and one
// partial row per (token, rank) comes back; the source adds the partials in k order of their first expert, then the
// shared expert's row.
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
    ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
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
            MLXS_SYM(AllReduce, "ncclAllReduce");
            MLXS_SYM(Send, "ncclSend");
            MLXS_SYM(Recv, "ncclRecv");
            MLXS_SYM(GroupStart, "ncclGroupStart");
            MLXS_SYM(GroupEnd, "ncclGroupEnd");
#undef MLXS_SYM
            if (!api.GetUniqueId || !api.CommInitRank || !api.CommDestroy || !api.AllGather || !api.AllReduce || !api.Send || !api.Recv ||
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
    // deduplicated form
    uint32_t *urow = nullptr, *ustart = nullptr, *a_urow = nullptr, *a_first = nullptr, *xrow = nullptr;
    int32_t *send_urow = nullptr, *recv_urow = nullptr;
    float *send_w = nullptr, *recv_w = nullptr;
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

// dest rank and local slot of every assignment from the layer's placement table; ids outside [0, E) set the status
// word and go to expert 0
__global__ void ep_dest_kernel(const int32_t* __restrict__ ids, uint32_t A, uint32_t E, const uint32_t* __restrict__ place,
                               int32_t* __restrict__ dest, int32_t* __restrict__ meta, uint32_t* status) {
    const uint32_t a = blockIdx.x * blockDim.x + threadIdx.x;
    if (a >= A) return;
    int32_t id = ids[a];
    if (id < 0 || (uint32_t)id >= E) { atomicMax(status, (uint32_t)ST_BAD_EXPERT_ID); id = 0; }
    const uint32_t pl = place[id];   // rank << 16 | local slot
    dest[a] = (int32_t)(pl >> 16);
    meta[a] = (int32_t)(pl & 0xFFFFu);
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


// ---- deduplicated form ----
// Sorted position i (assignments sorted by destination rank, token order inside): is it the first assignment of its
// (token, rank) pair, and which unique row (numbered over all ranks in sorted order) does it read.  One CTA of 1024
// threads walks the positions in blocks with a running total.  ustart[r] = first unique row of rank r's segment;
// counts[2r] = assignments, counts[2r + 1] = unique rows going to rank r.
__global__ void __launch_bounds__(1024) ep_dedup_kernel(const uint32_t* __restrict__ order, const uint32_t* __restrict__ offsets,
                                                        const int32_t* __restrict__ dest, uint32_t A, uint32_t W, uint32_t k,
                                                        uint32_t* __restrict__ urow, uint32_t* __restrict__ ustart,
                                                        int32_t* __restrict__ counts) {
    __shared__ uint32_t wsum[33];
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    uint32_t carry = 0;
    for (uint32_t base = 0; base < A; base += 1024) {
        const uint32_t i = base + tid;
        uint32_t flag = 0;
        if (i < A) {
            const uint32_t a = order[i];
            if (i == 0) flag = 1;
            else {
                const uint32_t ap = order[i - 1];
                flag = (ap / k != a / k || dest[ap] != dest[a]) ? 1u : 0u;
            }
        }
        uint32_t x = flag;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const uint32_t y = __shfl_up_sync(0xFFFFFFFFu, x, o);
            if (lane >= (uint32_t)o) x += y;
        }
        if (lane == 31) wsum[warp] = x;
        __syncthreads();
        if (warp == 0) {
            const uint32_t w = wsum[lane];
            uint32_t y = w;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const uint32_t z = __shfl_up_sync(0xFFFFFFFFu, y, o);
                if (lane >= (uint32_t)o) y += z;
            }
            wsum[lane] = y - w;
            if (lane == 31) wsum[32] = y;
        }
        __syncthreads();
        if (i < A) urow[i] = carry + wsum[warp] + x - 1u;
        carry += wsum[32];
        __syncthreads();
    }
    // urow was written by this CTA: visible after the barrier above
    for (uint32_t r = tid; r <= W; r += 1024) ustart[r] = (r < W && offsets[r] < A) ? urow[offsets[r]] : carry;
    __syncthreads();
    for (uint32_t r = tid; r < W; r += 1024) {
        counts[2 * r] = (int32_t)(offsets[r + 1] - offsets[r]);
        counts[2 * r + 1] = (int32_t)(ustart[r + 1] - ustart[r]);
    }
}
// per sorted position: the unique row's copy of x (by the pair's first assignment), the assignment's local expert,
// its row inside what the destination rank receives from this rank, its weight; and the inverse maps for the final sum
__global__ void ep_gather_dedup_kernel(const __nv_bfloat16* __restrict__ x, const int32_t* __restrict__ meta,
                                       const int32_t* __restrict__ dest, const float* __restrict__ weights,
                                       const uint32_t* __restrict__ order, const uint32_t* __restrict__ urow,
                                       const uint32_t* __restrict__ ustart, uint32_t A, uint32_t k, uint32_t H,
                                       __nv_bfloat16* __restrict__ send_x, int32_t* __restrict__ send_meta,
                                       int32_t* __restrict__ send_urow, float* __restrict__ send_w,
                                       uint32_t* __restrict__ a_urow, uint32_t* __restrict__ a_first) {
    const uint32_t i = blockIdx.x;
    if (i >= A) return;
    const uint32_t a = order[i], u = urow[i];
    const bool first = i == 0 || urow[i - 1] != u;
    if (first) {
        const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)(a / k) * H);
        uint4* dst = reinterpret_cast<uint4*>(send_x + (size_t)u * H);
        for (uint32_t j = threadIdx.x; j < H / 8; j += blockDim.x) dst[j] = src[j];
    }
    if (threadIdx.x == 0) {
        send_meta[i] = meta[a];
        send_urow[i] = (int32_t)(u - ustart[dest[a]]);
        send_w[i] = weights[a];
        a_urow[a] = u;
        a_first[a] = first ? 1u : 0u;
    }
}
struct EpSegments { uint32_t a0[65], u0[65]; uint32_t W; };   // received assignments / unique rows per source rank
// received assignment -> row of recv_x: its row inside the source's block + where that block starts
__global__ void ep_rebase_kernel(const int32_t* __restrict__ recv_urow, uint32_t R, EpSegments sg, uint32_t* __restrict__ xrow) {
    const uint32_t a = blockIdx.x * blockDim.x + threadIdx.x;
    if (a >= R) return;
    uint32_t s = 0;
    while (s + 1 < sg.W && a >= sg.a0[s + 1]) ++s;
    xrow[a] = (uint32_t)recv_urow[a] + sg.u0[s];
}
// partial[u] = sum over the received assignments of unique row u of w x ro (each product rounded, folded in order, as
// the single-GPU combine does); a unique row's assignments are consecutive
__global__ void ep_partial_kernel(const float* __restrict__ ro, const float* __restrict__ w, const uint32_t* __restrict__ xrow,
                                  uint32_t R, uint32_t H, float* __restrict__ partial) {
    const uint32_t a = blockIdx.x;
    if (a >= R) return;
    const uint32_t u = xrow[a];
    if (a > 0 && xrow[a - 1] == u) return;
    for (uint32_t col = threadIdx.x * 4; col < H; col += blockDim.x * 4) {
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        for (uint32_t b = a; b < R && xrow[b] == u; ++b) {
            const float wb = w[b];
            const float4 v = *reinterpret_cast<const float4*>(ro + (size_t)b * H + col);
            const float r4[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const float p = __fadd_rn(__fmul_rn(r4[q], wb), 0.0f);
                acc[q] = b == a ? p : __fadd_rn(p, acc[q]);
            }
        }
        *reinterpret_cast<float4*>(partial + (size_t)u * H + col) = make_float4(acc[0], acc[1], acc[2], acc[3]);
    }
}
// y[t] = bf16(sum of the token's partial rows, in k order of each pair's first assignment, + shared row)
__global__ void ep_reduce_kernel(const float* __restrict__ ret, const uint32_t* __restrict__ a_urow,
                                 const uint32_t* __restrict__ a_first, const float* __restrict__ shared, uint32_t T,
                                 uint32_t k, uint32_t H, __nv_bfloat16* __restrict__ y) {
    const uint32_t col = (blockIdx.x * blockDim.x + threadIdx.x) * 4, t = blockIdx.y;
    if (col >= H) return;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    bool any = false;
    for (uint32_t j = 0; j < k; ++j) {
        const uint32_t a = t * k + j;
        if (!a_first[a]) continue;
        const float4 v = *reinterpret_cast<const float4*>(ret + (size_t)a_urow[a] * H + col);
        if (!any) { acc[0] = v.x; acc[1] = v.y; acc[2] = v.z; acc[3] = v.w; any = true; }
        else { acc[0] = __fadd_rn(v.x, acc[0]); acc[1] = __fadd_rn(v.y, acc[1]); acc[2] = __fadd_rn(v.z, acc[2]); acc[3] = __fadd_rn(v.w, acc[3]); }
    }
    float o[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) o[q] = shared ? __fadd_rn(acc[q], shared[(size_t)t * H + col + q]) : acc[q];
    __nv_bfloat162 lo = __floats2bfloat162_rn(o[0], o[1]), hi = __floats2bfloat162_rn(o[2], o[3]);
    *reinterpret_cast<uint2*>(y + (size_t)t * H + col) = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
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
        (rc = h->alloc(&ep->ret_ro, A * H * 4)) || (rc = h->alloc(&ep->counts_dev, 2 * W * 4)) ||
        (rc = h->alloc(&ep->all_counts_dev, 2 * W * W * 4)) || (rc = h->alloc(&ep->urow, A * 4)) ||
        (rc = h->alloc(&ep->ustart, (W + 1) * 4)) || (rc = h->alloc(&ep->a_urow, A * 4)) || (rc = h->alloc(&ep->a_first, A * 4)) ||
        (rc = h->alloc(&ep->xrow, R * 4)) || (rc = h->alloc(&ep->send_urow, A * 4)) || (rc = h->alloc(&ep->recv_urow, R * 4)) ||
        (rc = h->alloc(&ep->send_w, A * 4)) || (rc = h->alloc(&ep->recv_w, R * 4))) {
        api->CommDestroy(ep->comm);
        delete ep;
        return rc;
    }
    cudaError_t e = cudaMallocHost(reinterpret_cast<void**>(&ep->all_counts_host), 2 * W * W * 4);
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

int mlxs_ep_allreduce_u64(mlxs_moe* h, unsigned long long* buf_dev, size_t n, cudaStream_t st) {
    EpState* ep = h->ep;
    NcclApi* api = nccl_api();
    if (!ep || !api) return mlxs_fail(MLXS_E_EP, "expert parallelism is not initialised (mlxs_moe_ep_init)");
    NC(api->AllReduce(buf_dev, buf_dev, n, ncclUint64, ncclSum, ep->comm, st));
    return MLXS_OK;
}

// The all-ranks refusal: every rank holds the same W x W count matrix after the all-gather (counts[(s * W + d) *
// stride] = rows rank s sends to rank d) and the same row capacity, so every rank finds the same overloaded rank and
// returns the same refusal before any send or receive is queued; nobody is left waiting for a peer that bailed out.
extern "C" int32_t mlxs_moe_ep_overloaded_rank(const int32_t* counts, uint32_t world, uint32_t stride, uint64_t rows_cap) {
    if (!counts || world == 0 || stride == 0) return -2;
    for (uint32_t d = 0; d < world; ++d) {
        uint64_t recv = 0;
        for (uint32_t s = 0; s < world; ++s) {
            const int32_t c = counts[((size_t)s * world + d) * stride];
            if (c < 0) return (int32_t)d;   // a corrupt count is an overload of its destination
            recv += (uint64_t)c;
        }
        if (recv > rows_cap) return (int32_t)d;
    }
    return -1;
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
        if (A) ep_dest_kernel<<<(A + 255) / 256, 256, 0, st>>>(ids_dev, A, c.n_experts, h->layers[layer].place_dev, ep->dest, ep->meta, h->status);
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
    {
        const int32_t over = mlxs_moe_ep_overloaded_rank(cnt, W, 1, h->rows_cap);
        if (over >= 0)
            return mlxs_fail(MLXS_E_EP, "experts: rank %d would receive more rows than its workspace's %u (every rank refuses this call; capacity = min(world, 4) x max_tokens x top_k)", over, h->rows_cap);
    }
    if (S != A) return mlxs_fail(MLXS_E_EP, "experts: exchange plan counts %zu rows, the call has %u", S, A);
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
    int rc = mlxs_run_routed(h, layer, ep->recv_x, ep->recv_meta, (uint32_t)R, 1, h->e_local, 0, ep->recv_ro, ro_bf16, st);
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

int mlxs_ep_combined(mlxs_moe* h, uint32_t layer, const void* x_dev, const int32_t* ids_dev, const float* weights_dev,
                     uint32_t T, const float* shared, void* y_dev, cudaStream_t st) {
    EpState* ep = h->ep;
    NcclApi* api = nccl_api();
    if (!ep || !api) return mlxs_fail(MLXS_E_EP, "experts: expert-parallel exchange is not initialised (mlxs_moe_ep_init)");
    const mlxs_moe_config& c = h->cfg;
    const uint32_t A = T * c.top_k, W = c.ep_world, H = c.hidden, me = c.ep_rank;
    if (W > 64) return mlxs_fail(MLXS_E_EP, "experts: ep_world %u > 64", W);
    {
        StageTimer tm(h, MLXS_STAGE_EXCHANGE, st);
        if (A) mlxs::ep_dest_kernel<<<(A + 255) / 256, 256, 0, st>>>(ids_dev, A, c.n_experts, h->layers[layer].place_dev, ep->dest, ep->meta, h->status);
        CU(launch_dispatch(ep->dest, A, W, nullptr, ep->rtab, h->chunk_rows, h->group_chunks, 0, h->status, st));
        mlxs::ep_dedup_kernel<<<1, 1024, 0, st>>>(ep->rtab.order, ep->rtab.offsets, ep->dest, A, W, c.top_k, ep->urow, ep->ustart,
                                                 ep->counts_dev);
        if (A) mlxs::ep_gather_dedup_kernel<<<A, 128, 0, st>>>(static_cast<const __nv_bfloat16*>(x_dev), ep->meta, ep->dest,
                                                             weights_dev, ep->rtab.order, ep->urow, ep->ustart, A, c.top_k, H,
                                                             ep->send_x, ep->send_meta, ep->send_urow, ep->send_w, ep->a_urow,
                                                             ep->a_first);
        CU(cudaGetLastError());
        NC(api->AllGather(ep->counts_dev, ep->all_counts_dev, 2 * W, ncclInt32, ep->comm, st));
        CU(cudaMemcpyAsync(ep->all_counts_host, ep->all_counts_dev, 2 * W * W * 4, cudaMemcpyDeviceToHost, st));
        CU(cudaStreamSynchronize(st));
    }
    // cnt[(s * W + d) * 2] = assignments, [.. + 1] = unique rows rank s sends to rank d
    const int32_t* cnt = ep->all_counts_host;
    size_t sa[65], su[65], ra[65], ru[65];
    sa[0] = su[0] = ra[0] = ru[0] = 0;
    for (uint32_t r = 0; r < W; ++r) {
        sa[r + 1] = sa[r] + (size_t)cnt[(me * W + r) * 2];
        su[r + 1] = su[r] + (size_t)cnt[(me * W + r) * 2 + 1];
        ra[r + 1] = ra[r] + (size_t)cnt[(r * W + me) * 2];
        ru[r + 1] = ru[r] + (size_t)cnt[(r * W + me) * 2 + 1];
    }
    const size_t SA = sa[W], SU = su[W], RA = ra[W], RU = ru[W];
    {
        const int32_t over = mlxs_moe_ep_overloaded_rank(cnt, W, 2, h->rows_cap);
        if (over >= 0)
            return mlxs_fail(MLXS_E_EP, "experts: rank %d would receive more rows than its workspace's %u (every rank refuses this call; capacity = min(world, 4) x max_tokens x top_k)", over, h->rows_cap);
    }
    if (SA != A) return mlxs_fail(MLXS_E_EP, "experts: exchange plan counts %zu rows, the call has %u", SA, A);
    {
        StageTimer tm(h, MLXS_STAGE_EXCHANGE, st);
        NC(api->GroupStart());
        for (uint32_t r = 0; r < W; ++r) {
            const size_t na = sa[r + 1] - sa[r], nu = su[r + 1] - su[r], ma = ra[r + 1] - ra[r], mu = ru[r + 1] - ru[r];
            if (na) {
                NC(api->Send(ep->send_x + su[r] * H, nu * H, ncclBfloat16, (int)r, ep->comm, st));
                NC(api->Send(ep->send_meta + sa[r], na, ncclInt32, (int)r, ep->comm, st));
                NC(api->Send(ep->send_urow + sa[r], na, ncclInt32, (int)r, ep->comm, st));
                NC(api->Send(ep->send_w + sa[r], na, ncclFloat32, (int)r, ep->comm, st));
            }
            if (ma) {
                NC(api->Recv(ep->recv_x + ru[r] * H, mu * H, ncclBfloat16, (int)r, ep->comm, st));
                NC(api->Recv(ep->recv_meta + ra[r], ma, ncclInt32, (int)r, ep->comm, st));
                NC(api->Recv(ep->recv_urow + ra[r], ma, ncclInt32, (int)r, ep->comm, st));
                NC(api->Recv(ep->recv_w + ra[r], ma, ncclFloat32, (int)r, ep->comm, st));
            }
        }
        NC(api->GroupEnd());
        if (RA) {
            mlxs::EpSegments sg{};
            sg.W = W;
            for (uint32_t r = 0; r <= W; ++r) { sg.a0[r] = (uint32_t)ra[r]; sg.u0[r] = (uint32_t)ru[r]; }
            mlxs::ep_rebase_kernel<<<(unsigned)((RA + 255) / 256), 256, 0, st>>>(ep->recv_urow, (uint32_t)RA, sg, ep->xrow);
            CU(cudaGetLastError());
        }
    }
    const size_t self_a = (size_t)cnt[(me * W + me) * 2], self_u = (size_t)cnt[(me * W + me) * 2 + 1];
    h->stats.a2a_bytes_sent += (SU - self_u) * (size_t)H * 2 + (SA - self_a) * 12 + (RU - self_u) * (size_t)H * 4;
    h->stats.a2a_bytes_recv += (RU - self_u) * (size_t)H * 2 + (RA - self_a) * 12 + (SU - self_u) * (size_t)H * 4;
    // the single-GPU kernels over the received assignments: each is its own "token" with one expert, its row of x
    // through the table; then the weighted fold per unique row into the handle's row workspace
    h->tabs.xrow = ep->xrow;
    int rc = mlxs_run_routed(h, layer, ep->recv_x, ep->recv_meta, (uint32_t)RA, 1, h->e_local, 0, ep->recv_ro, 0, st);
    h->tabs.xrow = nullptr;
    if (rc) return rc;
    float* partial = static_cast<float*>(h->ro);
    if (RA) {
        mlxs::ep_partial_kernel<<<(unsigned)RA, 256, 0, st>>>(static_cast<const float*>(ep->recv_ro), ep->recv_w, ep->xrow,
                                                            (uint32_t)RA, H, partial);
        CU(cudaGetLastError());
    }
    {
        StageTimer tm(h, MLXS_STAGE_EXCHANGE, st);
        NC(api->GroupStart());
        for (uint32_t r = 0; r < W; ++r) {
            const size_t ns = ru[r + 1] - ru[r], nr = su[r + 1] - su[r];
            if (ns) NC(api->Send(partial + ru[r] * H, ns * H, ncclFloat32, (int)r, ep->comm, st));
            if (nr) NC(api->Recv(static_cast<float*>(ep->ret_ro) + su[r] * H, nr * H, ncclFloat32, (int)r, ep->comm, st));
        }
        NC(api->GroupEnd());
    }
    if (T) {
        StageTimer tm(h, MLXS_STAGE_COMBINE, st);
        dim3 grid((H / 4 + 255) / 256, T);
        mlxs::ep_reduce_kernel<<<grid, 256, 0, st>>>(static_cast<const float*>(ep->ret_ro), ep->a_urow, ep->a_first, shared, T,
                                                    c.top_k, H, static_cast<__nv_bfloat16*>(y_dev));
        CU(cudaGetLastError());
    }
    return MLXS_OK;
}
