// Token dispatch: the stable sort of assignment rows by expert and the work tables the grouped kernels walk.
// Same permutation as the reference's counting sort (src/sdk_ext/quant.zig:269-290; src/arch/glm5_next/exl3_math.zig:192-225):
// order[sorted row] = assignment index, equal experts keep their routed order.  Everything stays on the device: the
// reference's host read-back of the ids (src/arch/deepseek_v41/experts.zig:1576-1587) has no counterpart here.
#include "common.cuh"
#include "kernels.h"
#include "dispatch_body.cuh"

namespace mlxs {

// A_dev: when given, the row count is read on the device (it may not exceed A, the bound the launch was sized for)
__global__ void __launch_bounds__(DTHREADS) dispatch_kernel(const int32_t* __restrict__ ids, uint32_t A, uint32_t E,
                                                            const uint8_t* __restrict__ loaded, DispatchTables t,
                                                            uint32_t CHUNK_ROWS, uint32_t GROUP_CHUNKS, uint32_t HEAVY,
                                                            uint32_t* status, const uint32_t* __restrict__ A_dev) {
    extern __shared__ uint32_t dsm[];
    if (A_dev) A = min(A, *A_dev);
    dispatch_body(ids, A, E, loaded, t, CHUNK_ROWS, GROUP_CHUNKS, HEAVY, status, dsm);
}

// ---- many assignments (prefill): the same sort over several CTAs ----
// 1: per-block histograms; 2: one CTA turns them into per-block bases and builds the tables; 3: per-block stable placement
__global__ void __launch_bounds__(DTHREADS) dispatch_count_kernel(const int32_t* __restrict__ ids, uint32_t A, uint32_t E,
                                                                  const uint8_t* __restrict__ loaded,
                                                                  uint32_t* __restrict__ blk_cnt, uint32_t* status,
                                                                  const uint32_t* __restrict__ A_dev) {
    extern __shared__ uint32_t dsm[];
    if (A_dev) A = min(A, *A_dev);
    for (uint32_t e = threadIdx.x; e < E; e += DTHREADS) dsm[e] = 0;
    __syncthreads();
    const uint32_t a = blockIdx.x * DTHREADS + threadIdx.x;
    if (a < A) {
        int32_t id = ids[a];
        if (id < 0 || (uint32_t)id >= E) { atomicMax(status, (uint32_t)ST_BAD_EXPERT_ID); id = 0; }
        else if (loaded && !loaded[id]) atomicMax(status, (uint32_t)ST_NOT_LOADED);
        atomicAdd(&dsm[id], 1u);
    }
    __syncthreads();
    for (uint32_t e = threadIdx.x; e < E; e += DTHREADS) blk_cnt[(size_t)blockIdx.x * E + e] = dsm[e];
}
__global__ void __launch_bounds__(DTHREADS) dispatch_scan_kernel(uint32_t nblk, uint32_t E, uint32_t* __restrict__ blk_cnt,
                                                                 DispatchTables t, uint32_t CHUNK_ROWS, uint32_t GROUP_CHUNKS,
                                                                 uint32_t HEAVY, const uint8_t* __restrict__ loaded, uint32_t* status) {
    extern __shared__ uint32_t dsm[];
    uint32_t* cnt = dsm;
    uint32_t* ws = dsm + E;
    const uint32_t tid = threadIdx.x;
    for (uint32_t e = tid; e < E; e += DTHREADS) {  // counts per expert; blk_cnt becomes the block's base inside the expert
        uint32_t run = 0;
        for (uint32_t b = 0; b < nblk; ++b) {
            const uint32_t v = blk_cnt[(size_t)b * E + e];
            blk_cnt[(size_t)b * E + e] = run;
            run += v;
        }
        cnt[e] = run;
    }
    __syncthreads();
    build_tables(cnt, E, loaded, t, CHUNK_ROWS, GROUP_CHUNKS, HEAVY, ws, status);
}
__global__ void __launch_bounds__(DTHREADS) dispatch_place_kernel(const int32_t* __restrict__ ids, uint32_t A, uint32_t E,
                                                                  const uint32_t* __restrict__ blk_base, DispatchTables t,
                                                                  const uint32_t* __restrict__ A_dev) {
    extern __shared__ uint32_t dsm[];   // [E] running positions of this block
    if (A_dev) A = min(A, *A_dev);
    if (blockIdx.x * DTHREADS >= A) return;   // a block beyond the device-side count
    const uint32_t tid = threadIdx.x, a0 = blockIdx.x * DTHREADS, a = a0 + tid, left = A - a0;
    for (uint32_t e = tid; e < E; e += DTHREADS) dsm[e] = t.offsets[e] + blk_base[(size_t)blockIdx.x * E + e];
    __syncthreads();
    uint32_t id = 0;
    if (a < A) {
        const int32_t v = ids[a];
        id = (v < 0 || (uint32_t)v >= E) ? 0u : (uint32_t)v;
    }
    place_block(id, a < A, a, left >= (uint32_t)DTHREADS ? DTHREADS / 32 : (left + 31) / 32, dsm, t.order);
}

cudaError_t launch_dispatch_large(const int32_t* ids, uint32_t A, uint32_t E, const uint8_t* loaded, DispatchTables t,
                                  uint32_t chunk_rows, uint32_t group_chunks, uint32_t heavy, uint32_t* blk_cnt,
                                  uint32_t* status, cudaStream_t st, const uint32_t* A_dev) {
    if (E > (uint32_t)DTHREADS) return cudaErrorInvalidValue;
    const uint32_t nblk = (A + DTHREADS - 1) / DTHREADS;
    dispatch_count_kernel<<<nblk, DTHREADS, E * sizeof(uint32_t), st>>>(ids, A, E, loaded, blk_cnt, status, A_dev);
    dispatch_scan_kernel<<<1, DTHREADS, (E + 99) * sizeof(uint32_t), st>>>(nblk, E, blk_cnt, t, chunk_rows, group_chunks, heavy, loaded, status);
    dispatch_place_kernel<<<nblk, DTHREADS, E * sizeof(uint32_t), st>>>(ids, A, E, blk_cnt, t, A_dev);
    return cudaGetLastError();
}

cudaError_t launch_dispatch(const int32_t* ids, uint32_t A, uint32_t E, const uint8_t* loaded, DispatchTables t,
                            uint32_t chunk_rows, uint32_t group_chunks, uint32_t heavy, uint32_t* status, cudaStream_t st,
                            const uint32_t* A_dev) {
    if (E > (uint32_t)DTHREADS) return cudaErrorInvalidValue;
    dispatch_kernel<<<1, DTHREADS, (E + 99) * sizeof(uint32_t), st>>>(ids, A, E, loaded, t, chunk_rows, group_chunks, heavy, status, A_dev);
    return cudaGetLastError();
}

// ---- usage tally: a block's ids are counted in shared memory first, then its non-zero counts join the layer's ----
__global__ void __launch_bounds__(256) usage_count_kernel(const int32_t* __restrict__ ids, uint64_t n, uint32_t E,
                                                          unsigned long long* __restrict__ usage) {
    extern __shared__ uint32_t hist[];
    for (uint32_t e = threadIdx.x; e < E; e += blockDim.x) hist[e] = 0;
    __syncthreads();
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) {
        const int32_t v = ids[i];
        if (v >= 0 && (uint32_t)v < E) atomicAdd(&hist[v], 1u);   // ids out of range are the dispatch's to report
    }
    __syncthreads();
    for (uint32_t e = threadIdx.x; e < E; e += blockDim.x)
        if (hist[e]) atomicAdd(&usage[e], (unsigned long long)hist[e]);
}

cudaError_t launch_usage_count(const int32_t* ids, uint64_t n, uint32_t E, unsigned long long* usage, cudaStream_t st) {
    if (n == 0) return cudaSuccess;
    const uint64_t want = (n + 2047) / 2048;
    const uint32_t grid = (uint32_t)(want < 148 ? want : 148);
    usage_count_kernel<<<grid, 256, E * sizeof(uint32_t), st>>>(ids, n, E, usage);
    return cudaGetLastError();
}

}  // namespace mlxs
