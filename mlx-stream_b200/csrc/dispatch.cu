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
                                                            uint32_t CHUNK_ROWS, uint32_t GROUP_CHUNKS,
                                                            uint32_t* status) {
    extern __shared__ uint32_t dsm[];
    uint32_t* cnt = dsm;                // [E] counts, then running write positions
    uint32_t* chunk_base = dsm + E;     // [E + 1]
    uint32_t* group_base = chunk_base + E + 1;  // [E + 1]
    uint32_t* blk = group_base + E + 1;  // [DTHREADS] ids of the block being placed
    __shared__ uint32_t s_distinct;
    const uint32_t tid = threadIdx.x;
    for (uint32_t e = tid; e < E; e += DTHREADS) cnt[e] = 0;
    if (tid == 0) s_distinct = 0;
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
            uint32_t nc = (c + CHUNK_ROWS - 1) / CHUNK_ROWS;
            rows += c;
            chunks += nc;
            groups += (nc + GROUP_CHUNKS - 1) / GROUP_CHUNKS;
            distinct += c ? 1u : 0u;
        }
        t.offsets[E] = rows;
        chunk_base[E] = chunks;
        group_base[E] = groups;
        if (chunks > t.max_chunks) { atomicMax(status, (uint32_t)ST_WORKLIST_OVERFLOW); chunks = 0; groups = 0; }
        t.header[HDR_NCHUNKS] = chunks;
        t.header[HDR_NGROUPS] = groups;
        t.header[HDR_CTR_GU] = 0;
        t.header[HDR_CTR_DOWN] = 0;
        t.header[HDR_CTR_AUX] = 0;
        t.header[HDR_DISTINCT] = distinct;
        s_distinct = chunks;
    }
    __syncthreads();
    const bool tables_ok = s_distinct != 0 || A == 0;
    if (tables_ok) {
        for (uint32_t e = tid; e < E; e += DTHREADS) {
            const uint32_t c = cnt[e], nc = (c + CHUNK_ROWS - 1) / CHUNK_ROWS, row0 = t.offsets[e];
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

cudaError_t launch_dispatch(const int32_t* ids, uint32_t A, uint32_t E, const uint8_t* loaded, DispatchTables t,
                            uint32_t chunk_rows, uint32_t group_chunks, uint32_t* status, cudaStream_t st) {
    size_t smem = (size_t)(3 * E + 2 + DTHREADS) * sizeof(uint32_t);
    dispatch_kernel<<<1, DTHREADS, smem, st>>>(ids, A, E, loaded, t, chunk_rows, group_chunks, status);
    return cudaGetLastError();
}

}  // namespace mlxs
