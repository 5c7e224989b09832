// Token dispatch: the stable sort of assignment rows by expert and the work tables the grouped kernels walk.
// Same permutation as the reference's counting sort (src/sdk_ext/quant.zig:269-290; src/arch/glm5_next/exl3_math.zig:192-225):
// order[sorted row] = assignment index, equal experts keep their routed order.  Everything stays on the device: the
// reference's host read-back of the ids (src/arch/deepseek_v41/experts.zig:1576-1587) has no counterpart here.
#include "common.cuh"
#include "kernels.h"

namespace mlxs {

constexpr int DTHREADS = 1024;

__global__ void __launch_bounds__(DTHREADS) dispatch_kernel(const int32_t* __restrict__ ids, uint32_t A, uint32_t E,
                                                            const uint8_t* __restrict__ loaded, DispatchTables t,
                                                            uint32_t CHUNK_ROWS, uint32_t GROUP_CHUNKS, uint32_t HEAVY,
                                                            uint32_t* status) {
    extern __shared__ uint32_t dsm[];
    uint32_t* cnt = dsm;                // [E] counts, then running write positions
    uint32_t* chunk_base = dsm + E;     // [E + 1]
    uint32_t* group_base = chunk_base + E + 1;  // [E + 1]
    uint32_t* blk = group_base + E + 1;  // [DTHREADS] ids of the block being placed
    __shared__ uint32_t s_overflow;
    const uint32_t tid = threadIdx.x;
    for (uint32_t e = tid; e < E; e += DTHREADS) cnt[e] = 0;
    if (tid == 0) s_overflow = 0;
    __syncthreads();
    for (uint32_t a = tid; a < A; a += DTHREADS) {
        int32_t id = ids[a];
        if (id < 0 || (uint32_t)id >= E) { atomicMax(status, (uint32_t)ST_BAD_EXPERT_ID); id = 0; }
        else if (loaded && !loaded[id]) atomicMax(status, (uint32_t)ST_NOT_LOADED);
        atomicAdd(&cnt[id], 1u);
    }
    __syncthreads();
    if (tid == 0) {
        uint32_t rows = 0, chunks = 0, groups = 0, distinct = 0;
        for (uint32_t e = 0; e < E; ++e) {
            uint32_t c = cnt[e];
            t.offsets[e] = rows;
            chunk_base[e] = chunks;
            group_base[e] = groups;
            // experts with HEAVY or more rows belong to the tensor-core lane: no chunks here
            uint32_t nc = takes_tensor_lane(c, HEAVY, loaded, e) ? 0u : (c + CHUNK_ROWS - 1) / CHUNK_ROWS;
            rows += c;
            chunks += nc;
            groups += (nc + GROUP_CHUNKS - 1) / GROUP_CHUNKS;
            distinct += c ? 1u : 0u;
        }
        t.offsets[E] = rows;
        chunk_base[E] = chunks;
        group_base[E] = groups;
        if (chunks > t.max_chunks) { atomicMax(status, (uint32_t)ST_WORKLIST_OVERFLOW); chunks = 0; groups = 0; s_overflow = 1; }
        t.header[HDR_NCHUNKS] = chunks;
        t.header[HDR_NGROUPS] = groups;
        t.header[HDR_CTR_GU] = 0;
        t.header[HDR_CTR_DOWN] = 0;
        t.header[HDR_CTR_AUX] = 0;
        t.header[HDR_DISTINCT] = distinct;
    }
    __syncthreads();
    if (!s_overflow) {
        for (uint32_t e = tid; e < E; e += DTHREADS) {
            const uint32_t c = cnt[e], row0 = t.offsets[e];
            const uint32_t nc = takes_tensor_lane(c, HEAVY, loaded, e) ? 0u : (c + CHUNK_ROWS - 1) / CHUNK_ROWS;
            for (uint32_t i = 0; i < nc; ++i) {
                const uint32_t ch = chunk_base[e] + i;
                t.chunk_expert[ch] = e;
                t.chunk_row0[ch] = row0 + i * CHUNK_ROWS;
                t.chunk_rows[ch] = min(CHUNK_ROWS, c - i * CHUNK_ROWS);
            }
            const uint32_t ng = (nc + GROUP_CHUNKS - 1) / GROUP_CHUNKS;
            for (uint32_t i = 0; i < ng; ++i) {
                t.group_chunk0[group_base[e] + i] = chunk_base[e] + i * GROUP_CHUNKS;
                t.group_mc[group_base[e] + i] = min(GROUP_CHUNKS, nc - i * GROUP_CHUNKS);
            }
        }
    }
    __syncthreads();
    for (uint32_t e = tid; e < E; e += DTHREADS) cnt[e] = t.offsets[e];
    __syncthreads();
    // stable placement, a block of DTHREADS assignments at a time
    for (uint32_t a0 = 0; a0 < A; a0 += DTHREADS) {
        const uint32_t a = a0 + tid;
        uint32_t id = 0xFFFFFFFFu;
        if (a < A) {
            int32_t v = ids[a];
            id = (v < 0 || (uint32_t)v >= E) ? 0u : (uint32_t)v;
        }
        blk[tid] = id;
        __syncthreads();
        if (a < A) {
            uint32_t r = 0;
            for (uint32_t j = 0; j < tid; ++j) r += (blk[j] == id) ? 1u : 0u;
            t.order[cnt[id] + r] = a;
        }
        __syncthreads();
        if (a < A) atomicAdd(&cnt[id], 1u);
        __syncthreads();
    }
}

// ---- many assignments (prefill): the same sort over several CTAs ----
// 1: per-block histograms; 2: one CTA turns them into per-block bases and builds the tables; 3: per-block stable placement
__global__ void __launch_bounds__(DTHREADS) dispatch_count_kernel(const int32_t* __restrict__ ids, uint32_t A, uint32_t E,
                                                                  const uint8_t* __restrict__ loaded,
                                                                  uint32_t* __restrict__ blk_cnt, uint32_t* status) {
    extern __shared__ uint32_t dsm[];
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
    uint32_t* chunk_base = dsm + E;
    uint32_t* group_base = chunk_base + E + 1;
    __shared__ uint32_t s_ok;
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
    if (tid == 0) {
        uint32_t rows = 0, chunks = 0, groups = 0, distinct = 0;
        for (uint32_t e = 0; e < E; ++e) {
            const uint32_t c = cnt[e];
            t.offsets[e] = rows;
            chunk_base[e] = chunks;
            group_base[e] = groups;
            const uint32_t nc = takes_tensor_lane(c, HEAVY, loaded, e) ? 0u : (c + CHUNK_ROWS - 1) / CHUNK_ROWS;
            rows += c;
            chunks += nc;
            groups += (nc + GROUP_CHUNKS - 1) / GROUP_CHUNKS;
            distinct += c ? 1u : 0u;
        }
        t.offsets[E] = rows;
        s_ok = 1;
        if (chunks > t.max_chunks) { atomicMax(status, (uint32_t)ST_WORKLIST_OVERFLOW); chunks = 0; groups = 0; s_ok = 0; }
        t.header[HDR_NCHUNKS] = chunks;
        t.header[HDR_NGROUPS] = groups;
        t.header[HDR_CTR_GU] = 0;
        t.header[HDR_CTR_DOWN] = 0;
        t.header[HDR_CTR_AUX] = 0;
        t.header[HDR_DISTINCT] = distinct;
    }
    __syncthreads();
    if (!s_ok) return;
    for (uint32_t e = tid; e < E; e += DTHREADS) {
        const uint32_t c = cnt[e], row0 = t.offsets[e];
        const uint32_t nc = takes_tensor_lane(c, HEAVY, loaded, e) ? 0u : (c + CHUNK_ROWS - 1) / CHUNK_ROWS;
        for (uint32_t i = 0; i < nc; ++i) {
            const uint32_t ch = chunk_base[e] + i;
            t.chunk_expert[ch] = e;
            t.chunk_row0[ch] = row0 + i * CHUNK_ROWS;
            t.chunk_rows[ch] = min(CHUNK_ROWS, c - i * CHUNK_ROWS);
        }
        const uint32_t ng = (nc + GROUP_CHUNKS - 1) / GROUP_CHUNKS;
        for (uint32_t i = 0; i < ng; ++i) {
            t.group_chunk0[group_base[e] + i] = chunk_base[e] + i * GROUP_CHUNKS;
            t.group_mc[group_base[e] + i] = min(GROUP_CHUNKS, nc - i * GROUP_CHUNKS);
        }
    }
}
__global__ void __launch_bounds__(DTHREADS) dispatch_place_kernel(const int32_t* __restrict__ ids, uint32_t A, uint32_t E,
                                                                  const uint32_t* __restrict__ blk_base, DispatchTables t) {
    __shared__ uint32_t blk[DTHREADS];
    const uint32_t tid = threadIdx.x, a = blockIdx.x * DTHREADS + tid;
    uint32_t id = 0xFFFFFFFFu;
    if (a < A) {
        const int32_t v = ids[a];
        id = (v < 0 || (uint32_t)v >= E) ? 0u : (uint32_t)v;
    }
    blk[tid] = id;
    __syncthreads();
    if (a < A) {
        uint32_t r = 0;
        for (uint32_t j = 0; j < tid; ++j) r += (blk[j] == id) ? 1u : 0u;
        t.order[t.offsets[id] + blk_base[(size_t)blockIdx.x * E + id] + r] = a;
    }
}

cudaError_t launch_dispatch_large(const int32_t* ids, uint32_t A, uint32_t E, const uint8_t* loaded, DispatchTables t,
                                  uint32_t chunk_rows, uint32_t group_chunks, uint32_t heavy, uint32_t* blk_cnt,
                                  uint32_t* status, cudaStream_t st) {
    const uint32_t nblk = (A + DTHREADS - 1) / DTHREADS;
    dispatch_count_kernel<<<nblk, DTHREADS, E * sizeof(uint32_t), st>>>(ids, A, E, loaded, blk_cnt, status);
    dispatch_scan_kernel<<<1, DTHREADS, (3 * E + 2) * sizeof(uint32_t), st>>>(nblk, E, blk_cnt, t, chunk_rows, group_chunks, heavy, loaded, status);
    dispatch_place_kernel<<<nblk, DTHREADS, 0, st>>>(ids, A, E, blk_cnt, t);
    return cudaGetLastError();
}

cudaError_t launch_dispatch(const int32_t* ids, uint32_t A, uint32_t E, const uint8_t* loaded, DispatchTables t,
                            uint32_t chunk_rows, uint32_t group_chunks, uint32_t heavy, uint32_t* status, cudaStream_t st) {
    size_t smem = (size_t)(3 * E + 2 + DTHREADS) * sizeof(uint32_t);
    dispatch_kernel<<<1, DTHREADS, smem, st>>>(ids, A, E, loaded, t, chunk_rows, group_chunks, heavy, status);
    return cudaGetLastError();
}

}  // namespace mlxs
