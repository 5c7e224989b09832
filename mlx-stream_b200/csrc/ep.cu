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
// Transport of the layer form: stores into the peers' memory.  At init every rank allocates one window (rows, per-row
// records, returned partial rows, flag words), the ranks exchange CUDA IPC handles of their windows (one NCCL
// all-gather) and map each other's.  A call then needs no host round trip and no library collective: the gather kernel
// writes each row and its records straight into the destination rank's window over NVLink, the last block to finish
// publishes the counts and an epoch word to every peer (release at system scope); the receiver's unpack kernel waits for
// the epoch words of all sources with a bounded poll, builds the local call from the counts it finds there (the row
// count stays on the device, the launches are sized for the capacity), and after the expert kernels the partial rows go
// back the same way.  Every rank signals every rank in both phases of every call, which is also what makes one buffer
// per direction enough: a peer cannot start writing call n + 1 into a window before its owner has finished reading
// call n.  Ordinary stores and loads only: no bulk-tensor copy ever touches peer memory.
// The per-assignment form (mlxs_ep_routed) and ranks whose windows could not be mapped use NCCL point-to-point (grouped
// ncclSend / ncclRecv with exact counts after a count all-gather that the host reads).  NCCL is loaded at run time
// (dlopen), so a single-GPU process needs no NCCL at all.
#include <dlfcn.h>
#include <nccl.h>

#include <cstdlib>
#include <cstring>
#include <vector>

#include "common.cuh"
#include "dispatch_body.cuh"
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
    // peer-store transport
    bool p2p = false;
    uint8_t* win = nullptr;              // this rank's window
    void* peer_base[64] = {nullptr};     // every rank's window as mapped here (own: win)
    uint32_t epoch = 0;                  // call counter, the same on every rank
    uint32_t* ctl = nullptr;             // device words: [0] push blocks done, [1] partial blocks done, [2] received rows, [3..] a0[W + 1]
    unsigned long long* bytes_dev = nullptr;   // [2] bytes stored into / returned from peers' windows
    uint32_t wait_polls = 0;             // bound of a wait for the peers' epoch words
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
__device__ __forceinline__ void ep_dedup_body(const uint32_t* __restrict__ order, const uint32_t* __restrict__ offsets,
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
__global__ void __launch_bounds__(1024) ep_dedup_kernel(const uint32_t* __restrict__ order, const uint32_t* __restrict__ offsets,
                                                        const int32_t* __restrict__ dest, uint32_t A, uint32_t W, uint32_t k,
                                                        uint32_t* __restrict__ urow, uint32_t* __restrict__ ustart,
                                                        int32_t* __restrict__ counts) {
    ep_dedup_body(order, offsets, dest, A, W, k, urow, ustart, counts);
}
// The plan of one exchange for decode-sized calls in one launch: destination rank and local slot of every assignment,
// the stable sort by rank (the dispatch kernel's code), the first assignment of every (token, rank) pair.  One CTA; the
// three steps read what the one before wrote to global memory after a CTA barrier.  dsm: W + 99 words.
__global__ void __launch_bounds__(DTHREADS) ep_plan_kernel(const int32_t* __restrict__ ids, uint32_t A, uint32_t E,
                                                           const uint32_t* __restrict__ place, int32_t* __restrict__ dest,
                                                           int32_t* __restrict__ meta, DispatchTables rtab, uint32_t W, uint32_t k,
                                                           uint32_t chunk_rows, uint32_t group_chunks, uint32_t* __restrict__ urow,
                                                           uint32_t* __restrict__ ustart, int32_t* __restrict__ counts, uint32_t* status) {
    extern __shared__ uint32_t ep_dsm[];
    for (uint32_t a = threadIdx.x; a < A; a += DTHREADS) {
        int32_t id = ids[a];
        if (id < 0 || (uint32_t)id >= E) { atomicMax(status, (uint32_t)ST_BAD_EXPERT_ID); id = 0; }
        const uint32_t pl = place[id];   // rank << 16 | local slot
        dest[a] = (int32_t)(pl >> 16);
        meta[a] = (int32_t)(pl & 0xFFFFu);
    }
    __syncthreads();
    dispatch_body(dest, A, W, nullptr, rtab, chunk_rows, group_chunks, 0u, status, ep_dsm);
    __syncthreads();
    ep_dedup_body(rtab.order, rtab.offsets, dest, A, W, k, urow, ustart, counts);
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


// ---- peer-store transport ----
// One rank's window, the same layout on every rank (offsets in bytes):
//   disp [W] x 128 B : {assignments, unique rows, epoch} written by source rank s at slot s
//   retf [W] x 128 B : {epoch} written by rank r when its partial rows for this rank are in place
//   rx_x [W][Tm][H] bf16 : rows from source s (a token's row once per pair of ranks)
//   rx_meta [W][Tm * Kc] x 16 B : {local expert slot, row inside the source's block, weight bits, 0} per assignment
//   ret  [W][Tm][H] f32 : partial rows coming back from rank r, by the row's index inside what this rank sent to r
struct EpWin {
    uint8_t* peer[64];
    uint32_t W, me, Tm, Kc, H;
    size_t off_disp, off_retf, off_rx_x, off_rx_meta, off_ret, bytes;
};
static EpWin ep_win_layout(uint32_t W, uint32_t me, uint32_t Tm, uint32_t Kc, uint32_t H) {
    EpWin w{};
    w.W = W; w.me = me; w.Tm = Tm; w.Kc = Kc; w.H = H;
    size_t o = 0;
    auto take = [&](size_t n) { const size_t at = o; o += (n + 255) / 256 * 256; return at; };
    w.off_disp = take((size_t)W * 128);
    w.off_retf = take((size_t)W * 128);
    w.off_rx_x = take((size_t)W * Tm * H * 2);
    w.off_rx_meta = take((size_t)W * Tm * Kc * 16);
    w.off_ret = take((size_t)W * Tm * H * 4);
    w.bytes = o;
    return w;
}
extern "C" uint64_t mlxs_moe_ep_window_bytes(uint32_t world, uint32_t max_tokens, uint32_t top_k, uint32_t n_experts, uint32_t hidden) {
    if (world == 0 || n_experts % world) return 0;
    const uint32_t e_local = n_experts / world;
    return ep_win_layout(world, 0, max_tokens, top_k < e_local ? top_k : e_local, hidden).bytes;
}

namespace mlxs {

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
// bounded wait for a peer's epoch word in this rank's own window; false when it ran out
__device__ __forceinline__ bool ep_wait_epoch(const uint32_t* word, uint32_t epoch, uint32_t polls) {
    for (uint32_t i = 0; i < polls; ++i) {
        if ((int32_t)(ld_acquire_sys(word) - epoch) >= 0) return true;
        __nanosleep(i < 64 ? 100 : 1000);
    }
    return false;
}

// Sorted position i (assignments sorted by destination rank): the pair's first position stores the token's row into
// the destination's window, every position its record; the last block to finish publishes counts and epoch to all.
__global__ void __launch_bounds__(128) ep_push_kernel(const __nv_bfloat16* __restrict__ x, const int32_t* __restrict__ meta,
                                                      const int32_t* __restrict__ dest, const float* __restrict__ weights,
                                                      const uint32_t* __restrict__ order, const uint32_t* __restrict__ offsets,
                                                      const uint32_t* __restrict__ urow, const uint32_t* __restrict__ ustart,
                                                      const int32_t* __restrict__ counts, uint32_t A, uint32_t k, EpWin w,
                                                      uint32_t epoch, uint32_t* __restrict__ a_urow, uint32_t* __restrict__ a_first,
                                                      uint32_t* ctl, unsigned long long* bytes) {
    const uint32_t i = blockIdx.x;
    if (i < A) {
        const uint32_t a = order[i], u = urow[i];
        const uint32_t d = (uint32_t)dest[a];
        const bool first = i == 0 || urow[i - 1] != u;
        const uint32_t ul = u - ustart[d], il = i - offsets[d];
        uint8_t* pw = w.peer[d];
        if (first) {
            const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)(a / k) * w.H);
            uint4* dst = reinterpret_cast<uint4*>(pw + w.off_rx_x + ((size_t)w.me * w.Tm + ul) * w.H * 2);
            for (uint32_t j = threadIdx.x; j < w.H / 8; j += blockDim.x) dst[j] = src[j];
        }
        if (threadIdx.x == 0) {
            uint4* rec = reinterpret_cast<uint4*>(pw + w.off_rx_meta + ((size_t)w.me * w.Tm * w.Kc + il) * 16);
            *rec = make_uint4((uint32_t)meta[a], ul, __float_as_uint(weights[a]), 0u);
            a_urow[a] = d * w.Tm + ul;      // where this pair's partial row will land in this rank's `ret`
            a_first[a] = first ? 1u : 0u;
        }
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        const uint32_t prev = atomicAdd(&ctl[0], 1u);
        if (prev == gridDim.x - 1) {
            ctl[0] = 0;
            __threadfence_system();
            unsigned long long sent = 0, back = 0;
            for (uint32_t r = 0; r < w.W; ++r) {
                uint32_t* slot = reinterpret_cast<uint32_t*>(w.peer[r] + w.off_disp + (size_t)w.me * 128);
                const uint32_t na = A ? (uint32_t)counts[2 * r] : 0u, nu = A ? (uint32_t)counts[2 * r + 1] : 0u;
                slot[0] = na;
                slot[1] = nu;
                st_release_sys(slot + 2, epoch);
                if (r != w.me) { sent += (unsigned long long)nu * w.H * 2 + (unsigned long long)na * 16; back += (unsigned long long)nu * w.H * 4; }
            }
            atomicAdd(&bytes[0], sent);   // rows and records stored into peers' windows
            atomicAdd(&bytes[3], back);   // partial rows the peers will store into this rank's window
        }
    }
}

// Receiver: wait for every source's epoch word, lay the received assignments out as one local call (ids, the row of
// rx_x each reads, weights) and leave the row count on the device.  Every block waits by itself (the words are in
// this GPU's memory); block 0 writes the counts.
__global__ void __launch_bounds__(256) ep_unpack_kernel(EpWin w, uint32_t epoch, uint32_t polls, uint32_t rows_cap,
                                                        int32_t* __restrict__ ids, uint32_t* __restrict__ xrow,
                                                        float* __restrict__ wts, uint32_t* ctl, unsigned long long* bytes,
                                                        uint32_t* status) {
    __shared__ uint32_t a0[65];
    __shared__ int s_ok;
    const uint8_t* own = w.peer[w.me];
    if (threadIdx.x == 0) s_ok = 1;
    __syncthreads();
    if (threadIdx.x < w.W) {
        const uint32_t* slot = reinterpret_cast<const uint32_t*>(own + w.off_disp + (size_t)threadIdx.x * 128);
        if (!ep_wait_epoch(slot + 2, epoch, polls)) s_ok = 0;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        uint32_t run = 0;
        for (uint32_t s = 0; s < w.W; ++s) {
            a0[s] = run;
            const uint32_t na = s_ok ? reinterpret_cast<const uint32_t*>(own + w.off_disp + (size_t)s * 128)[0] : 0u;
            run += na <= w.Tm * w.Kc ? na : 0u;
        }
        if (!s_ok) { atomicMax(status, (uint32_t)ST_EP_TIMEOUT); run = 0; }
        else if (run > rows_cap) { atomicMax(status, (uint32_t)ST_EP_OVERFLOW); run = 0; }
        if (run == 0) for (uint32_t s = 0; s < w.W; ++s) a0[s] = 0;
        a0[w.W] = run;
        if (blockIdx.x == 0) {
            ctl[2] = run;
            for (uint32_t s = 0; s <= w.W; ++s) ctl[3 + s] = a0[s];
            unsigned long long got = 0;
            if (run)
                for (uint32_t s = 0; s < w.W; ++s)
                    if (s != w.me) {
                        const uint32_t* slot = reinterpret_cast<const uint32_t*>(own + w.off_disp + (size_t)s * 128);
                        got += (unsigned long long)slot[1] * w.H * 2 + (unsigned long long)slot[0] * 16;
                    }
            atomicAdd(&bytes[2], got);
        }
    }
    __syncthreads();
    const uint32_t RA = a0[w.W];
    for (uint32_t a = blockIdx.x * blockDim.x + threadIdx.x; a < RA; a += gridDim.x * blockDim.x) {
        uint32_t s = 0;
        while (s + 1 < w.W && a >= a0[s + 1]) ++s;
        const uint4 rec = *reinterpret_cast<const uint4*>(own + w.off_rx_meta + ((size_t)s * w.Tm * w.Kc + (a - a0[s])) * 16);
        ids[a] = (int32_t)rec.x;
        xrow[a] = s * w.Tm + (rec.y < w.Tm ? rec.y : 0u);
        wts[a] = __uint_as_float(rec.z);
    }
}

// partial[(s, ul)] = sum over the received assignments of that row of w x ro (each product rounded, folded in order, as
// the single-GPU combine does; a row's assignments are consecutive), stored straight into source s's window; the last
// block to finish tells every source that its partial rows are in place.
__global__ void __launch_bounds__(256) ep_partial_push_kernel(const float* __restrict__ ro, const float* __restrict__ wts,
                                                              const uint32_t* __restrict__ xrow, EpWin w, uint32_t epoch,
                                                              uint32_t* ctl, unsigned long long* bytes) {
    const uint32_t RA = ctl[2], H = w.H;
    unsigned long long rows_out = 0;
    for (uint32_t a = blockIdx.x; a < RA; a += gridDim.x) {
        const uint32_t u = xrow[a];
        if (a > 0 && xrow[a - 1] == u) continue;
        const uint32_t s = u / w.Tm, ul = u % w.Tm;
        float* dst = reinterpret_cast<float*>(w.peer[s] + w.off_ret + ((size_t)w.me * w.Tm + ul) * H * 4);
        for (uint32_t col = threadIdx.x * 4; col < H; col += blockDim.x * 4) {
            float acc[4] = {0.f, 0.f, 0.f, 0.f};
            for (uint32_t b = a; b < RA && xrow[b] == u; ++b) {
                const float wb = wts[b];
                const float4 v = *reinterpret_cast<const float4*>(ro + (size_t)b * H + col);
                const float r4[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const float p = __fadd_rn(__fmul_rn(r4[q], wb), 0.0f);
                    acc[q] = b == a ? p : __fadd_rn(p, acc[q]);
                }
            }
            *reinterpret_cast<float4*>(dst + col) = make_float4(acc[0], acc[1], acc[2], acc[3]);
        }
        if (s != w.me) rows_out += 1;
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        if (rows_out) atomicAdd(&bytes[1], rows_out * H * 4);
        const uint32_t prev = atomicAdd(&ctl[1], 1u);
        if (prev == gridDim.x - 1) {
            ctl[1] = 0;
            __threadfence_system();
            for (uint32_t r = 0; r < w.W; ++r)
                st_release_sys(reinterpret_cast<uint32_t*>(w.peer[r] + w.off_retf + (size_t)w.me * 128), epoch);
        }
    }
}

// y[t] = bf16(sum of the token's partial rows, in k order of each pair's first assignment, + shared row); every block
// first waits for the peers' "partial rows in place" words
__global__ void __launch_bounds__(256) ep_reduce_p2p_kernel(EpWin w, uint32_t epoch, uint32_t polls,
                                                            const uint32_t* __restrict__ a_urow, const uint32_t* __restrict__ a_first,
                                                            const float* __restrict__ shared, uint32_t T, uint32_t k,
                                                            __nv_bfloat16* __restrict__ y, uint32_t* status) {
    __shared__ int s_ok;
    const uint8_t* own = w.peer[w.me];
    if (threadIdx.x == 0) s_ok = 1;
    __syncthreads();
    if (threadIdx.x < w.W) {
        if (!ep_wait_epoch(reinterpret_cast<const uint32_t*>(own + w.off_retf + (size_t)threadIdx.x * 128), epoch, polls)) s_ok = 0;
    }
    __syncthreads();
    if (!s_ok) { if (threadIdx.x == 0) atomicMax(status, (uint32_t)ST_EP_TIMEOUT); return; }
    const uint32_t H = w.H, col = (blockIdx.x * blockDim.x + threadIdx.x) * 4, t = blockIdx.y;
    if (col >= H || t >= T) return;
    const float* ret = reinterpret_cast<const float*>(own + w.off_ret);
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
    // the peer-store transport; every rank must end up with the same answer, so the outcome is agreed with one all-reduce
    {
        int ok = getenv("MLXS_EP_NCCL_ONLY") ? 0 : 1;
        const uint32_t Kc = c.top_k < h->e_local ? c.top_k : h->e_local;
        EpWin wl = ep_win_layout((uint32_t)W, c.ep_rank, c.max_tokens, Kc, c.hidden);
        cudaIpcMemHandle_t mine;
        unsigned char* hbuf = nullptr;
        std::vector<cudaIpcMemHandle_t> all(W);
        if (W > 64) ok = 0;
        if (ok && (h->alloc(&ep->win, wl.bytes) || h->alloc(&ep->ctl, 128 * 4) || h->alloc(&ep->bytes_dev, 4 * 8) ||
                   h->alloc(&hbuf, W * sizeof(cudaIpcMemHandle_t))))
            ok = 0;
        if (ok && (cudaMemset(ep->win, 0, wl.off_rx_x) != cudaSuccess || cudaMemset(ep->ctl, 0, 128 * 4) != cudaSuccess ||
                   cudaMemset(ep->bytes_dev, 0, 32) != cudaSuccess || cudaIpcGetMemHandle(&mine, ep->win) != cudaSuccess))
            ok = 0;
        if (hbuf) {
            // the handles travel through the communicator that exists already; a rank that could not make one sends zeros
            if (!ok) memset(&mine, 0, sizeof mine);
            cudaMemcpy(hbuf + c.ep_rank * sizeof mine, &mine, sizeof mine, cudaMemcpyHostToDevice);
            ncclResult_t nr = api->AllGather(hbuf + c.ep_rank * sizeof mine, hbuf, sizeof mine, ncclUint8, ep->comm, 0);
            if (nr != ncclSuccess || cudaStreamSynchronize(0) != cudaSuccess ||
                cudaMemcpy(all.data(), hbuf, W * sizeof mine, cudaMemcpyDeviceToHost) != cudaSuccess)
                ok = 0;
        }
        if (ok) {
            for (uint32_t r = 0; r < W && ok; ++r) {
                if (r == c.ep_rank) { ep->peer_base[r] = ep->win; continue; }
                if (cudaIpcOpenMemHandle(&ep->peer_base[r], all[r], cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
                    cudaGetLastError();
                    ep->peer_base[r] = nullptr;
                    ok = 0;
                }
            }
        }
        // agree: the transport is on only if every rank mapped every window (the flag rides in the first word of ctl)
        int agreed = 0;
        if (ep->ctl) {
            const uint32_t flag = ok ? 1u : 0u;
            cudaMemcpy(ep->ctl + 100, &flag, 4, cudaMemcpyHostToDevice);
            uint32_t res = 0;
            if (api->AllReduce(ep->ctl + 100, ep->ctl + 100, 1, ncclUint32, ncclMin, ep->comm, 0) == ncclSuccess &&
                cudaStreamSynchronize(0) == cudaSuccess && cudaMemcpy(&res, ep->ctl + 100, 4, cudaMemcpyDeviceToHost) == cudaSuccess)
                agreed = res == 1u;
        }
        ep->p2p = agreed != 0;
        const char* ms = getenv("MLXS_EP_WAIT_MS");
        const double wait_ms = ms ? atof(ms) : 20000.0;      // a wait polls about once a microsecond
        ep->wait_polls = (uint32_t)(wait_ms * 1000.0 < 64.0 ? 64.0 : (wait_ms * 1000.0 > 4.0e9 ? 4.0e9 : wait_ms * 1000.0));
    }
    return MLXS_OK;
}

int mlxs_ep_transport(const mlxs_moe* h) { return !h->ep ? 0 : (h->ep->p2p ? 2 : 1); }
void mlxs_ep_bytes(mlxs_moe* h, uint64_t* sent, uint64_t* recv) {
    if (!h->ep || !h->ep->p2p || !h->ep->bytes_dev) return;
    unsigned long long b[4] = {0, 0, 0, 0};
    if (cudaMemcpy(b, h->ep->bytes_dev, sizeof b, cudaMemcpyDeviceToHost) != cudaSuccess) return;
    *sent += b[0] + b[1];
    *recv += b[2] + b[3];
    cudaMemset(h->ep->bytes_dev, 0, sizeof b);
}

void mlxs_ep_destroy(mlxs_moe* h) {
    if (!h->ep) return;
    for (uint32_t r = 0; r < h->cfg.ep_world && r < 64; ++r)
        if (r != h->cfg.ep_rank && h->ep->peer_base[r]) cudaIpcCloseMemHandle(h->ep->peer_base[r]);
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

// the layer form over peer stores: no host round trip, no library collective
static int ep_combined_p2p(mlxs_moe* h, uint32_t layer, const void* x_dev, const int32_t* ids_dev, const float* weights_dev,
                           uint32_t T, const float* shared, void* y_dev, cudaStream_t st) {
    EpState* ep = h->ep;
    const mlxs_moe_config& c = h->cfg;
    const uint32_t A = T * c.top_k, W = c.ep_world, H = c.hidden;
    const uint32_t Kc = c.top_k < h->e_local ? c.top_k : h->e_local;
    EpWin w = ep_win_layout(W, c.ep_rank, c.max_tokens, Kc, H);
    for (uint32_t r = 0; r < W; ++r) w.peer[r] = static_cast<uint8_t*>(ep->peer_base[r]);
    const uint32_t epoch = ++ep->epoch;
    {
        StageTimer tm(h, MLXS_STAGE_EXCHANGE, st);
        if (A <= 2048) {
            // decode-sized calls: destination ranks, rank sort and dedup in one launch
            mlxs::ep_plan_kernel<<<1, mlxs::DTHREADS, (W + 99) * sizeof(uint32_t), st>>>(ids_dev, A, c.n_experts, h->layers[layer].place_dev,
                                                                                     ep->dest, ep->meta, ep->rtab, W, c.top_k, h->chunk_rows,
                                                                                     h->group_chunks, ep->urow, ep->ustart, ep->counts_dev,
                                                                                     h->status);
        } else {
            mlxs::ep_dest_kernel<<<(A + 255) / 256, 256, 0, st>>>(ids_dev, A, c.n_experts, h->layers[layer].place_dev, ep->dest, ep->meta, h->status);
            CU(launch_dispatch(ep->dest, A, W, nullptr, ep->rtab, h->chunk_rows, h->group_chunks, 0, h->status, st));
            mlxs::ep_dedup_kernel<<<1, 1024, 0, st>>>(ep->rtab.order, ep->rtab.offsets, ep->dest, A, W, c.top_k, ep->urow, ep->ustart,
                                                     ep->counts_dev);
        }
        mlxs::ep_push_kernel<<<A ? A : 1, 128, 0, st>>>(static_cast<const __nv_bfloat16*>(x_dev), ep->meta, ep->dest, weights_dev,
                                                        ep->rtab.order, ep->rtab.offsets, ep->urow, ep->ustart, ep->counts_dev, A,
                                                        c.top_k, w, epoch, ep->a_urow, ep->a_first, ep->ctl, ep->bytes_dev);
        const uint32_t ub = (h->rows_cap + 255) / 256, ucap = 4u * (uint32_t)h->sm_count;
        mlxs::ep_unpack_kernel<<<ub < ucap ? (ub ? ub : 1) : ucap, 256, 0, st>>>(w, epoch, ep->wait_polls, h->rows_cap, ep->recv_meta,
                                                                            ep->xrow, ep->recv_w, ep->ctl, ep->bytes_dev, h->status);
        CU(cudaGetLastError());
    }
    // the single-GPU kernels over the received assignments: each is its own "token" with one expert, its row of x in
    // this rank's window through the table; the row count stays on the device
    h->tabs.xrow = ep->xrow;
    int rc = mlxs_run_routed(h, layer, ep->win + w.off_rx_x, ep->recv_meta, h->rows_cap, 1, h->e_local, 0, ep->recv_ro, 0, st,
                             ep->ctl + 2);
    h->tabs.xrow = nullptr;
    if (rc) return rc;   // a refused launch: the peers' next wait runs out and reports, nobody hangs
    {
        StageTimer tm(h, MLXS_STAGE_EXCHANGE, st);
        const uint32_t pcap = 8u * (uint32_t)h->sm_count;
        mlxs::ep_partial_push_kernel<<<h->rows_cap < pcap ? (h->rows_cap ? h->rows_cap : 1) : pcap, 256, 0, st>>>(
            static_cast<const float*>(ep->recv_ro), ep->recv_w, ep->xrow, w, epoch, ep->ctl, ep->bytes_dev);
        CU(cudaGetLastError());
    }
    {
        StageTimer tm(h, MLXS_STAGE_COMBINE, st);
        dim3 grid((H / 4 + 255) / 256, T ? T : 1);
        mlxs::ep_reduce_p2p_kernel<<<grid, 256, 0, st>>>(w, epoch, ep->wait_polls, ep->a_urow, ep->a_first, shared, T, c.top_k,
                                                        static_cast<__nv_bfloat16*>(y_dev), h->status);
        CU(cudaGetLastError());
    }
    return MLXS_OK;
}

int mlxs_ep_combined(mlxs_moe* h, uint32_t layer, const void* x_dev, const int32_t* ids_dev, const float* weights_dev,
                     uint32_t T, const float* shared, void* y_dev, cudaStream_t st) {
    EpState* ep = h->ep;
    NcclApi* api = nccl_api();
    if (!ep || !api) return mlxs_fail(MLXS_E_EP, "experts: expert-parallel exchange is not initialised (mlxs_moe_ep_init)");
    if (ep->p2p) return ep_combined_p2p(h, layer, x_dev, ids_dev, weights_dev, T, shared, y_dev, st);
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
