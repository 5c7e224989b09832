// Device code of the dispatch (stable counting sort + work tables), shared by the dispatch kernels and the fused front
// kernel.
#pragma once
#include "common.cuh"
#include "kernels.h"

namespace mlxs {

constexpr int DTHREADS = 1024;   // one thread per expert in the scans (n_experts <= 1024), one per assignment of a block

// Exclusive prefix sums of three per-thread values over the CTA (1024 threads): warp shuffles, then the 32 warp totals
// by the first warp.  ws: [3][33] words of shared memory; the totals come back in tot[3].
__device__ __forceinline__ void block_scan3(const uint32_t (&v)[3], uint32_t (&excl)[3], uint32_t (&tot)[3], uint32_t* ws) {
    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
    uint32_t inc[3];
#pragma unroll
    for (int k = 0; k < 3; ++k) {
        uint32_t x = v[k];
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const uint32_t y = __shfl_up_sync(0xFFFFFFFFu, x, o);
            if (lane >= (uint32_t)o) x += y;
        }
        inc[k] = x;
        if (lane == 31) ws[k * 33 + warp] = x;
    }
    __syncthreads();
    if (warp == 0) {
#pragma unroll
        for (int k = 0; k < 3; ++k) {
            const uint32_t w = ws[k * 33 + lane];
            uint32_t x = w;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const uint32_t y = __shfl_up_sync(0xFFFFFFFFu, x, o);
                if (lane >= (uint32_t)o) x += y;
            }
            ws[k * 33 + lane] = x - w;            // exclusive base of each warp
            if (lane == 31) ws[k * 33 + 32] = x;  // total
        }
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < 3; ++k) {
        excl[k] = ws[k * 33 + warp] + inc[k] - v[k];
        tot[k] = ws[k * 33 + 32];
    }
}

// Work tables from the per-expert counts (cnt in shared memory, one thread per expert): offsets, chunks of CHUNK_ROWS
// rows, groups of GROUP_CHUNKS chunks.  Experts that take the tensor-core lane get no chunks.  On a table overflow the
// status word is set and no chunk is written.
__device__ __forceinline__ void build_tables(const uint32_t* cnt, uint32_t E, const uint8_t* __restrict__ loaded,
                                             DispatchTables t, uint32_t CHUNK_ROWS, uint32_t GROUP_CHUNKS, uint32_t HEAVY,
                                             uint32_t* ws, uint32_t* status) {
    const uint32_t e = threadIdx.x;
    const uint32_t c = e < E ? cnt[e] : 0u;
    const uint32_t nc = (e >= E || takes_tensor_lane(c, HEAVY, loaded, e)) ? 0u : (c + CHUNK_ROWS - 1) / CHUNK_ROWS;
    const uint32_t ng = (nc + GROUP_CHUNKS - 1) / GROUP_CHUNKS;
    const uint32_t v[3] = {c, nc, ng};
    uint32_t ex[3], tot[3];
    block_scan3(v, ex, tot, ws);
    const uint32_t distinct = (uint32_t)__syncthreads_count(c != 0u);
    if (e < E) t.offsets[e] = ex[0];
    const bool ok = tot[1] <= t.max_chunks;
    if (threadIdx.x == 0) {
        t.offsets[E] = tot[0];
        if (!ok) atomicMax(status, (uint32_t)ST_WORKLIST_OVERFLOW);
        t.header[HDR_NCHUNKS] = ok ? tot[1] : 0u;
        t.header[HDR_NGROUPS] = ok ? tot[2] : 0u;
        t.header[HDR_CTR_GU] = 0;
        t.header[HDR_CTR_DOWN] = 0;
        t.header[HDR_CTR_AUX] = 0;
        t.header[HDR_DISTINCT] = distinct;
    }
    if (ok && e < E) {
        for (uint32_t i = 0; i < nc; ++i) {
            const uint32_t ch = ex[1] + i;
            t.chunk_expert[ch] = e;
            t.chunk_row0[ch] = ex[0] + i * CHUNK_ROWS;
            t.chunk_rows[ch] = min(CHUNK_ROWS, c - i * CHUNK_ROWS);
        }
        for (uint32_t i = 0; i < ng; ++i) {
            t.group_chunk0[ex[2] + i] = ex[1] + i * GROUP_CHUNKS;
            t.group_mc[ex[2] + i] = min(GROUP_CHUNKS, nc - i * GROUP_CHUNKS);
        }
    }
}

// Stable placement of one block of up to DTHREADS assignments (a = first + thread index, all threads call): the warps
// take their turn in order; inside a warp the lanes with the same expert find each other (match) and take consecutive
// positions from the expert's running position pos[id] in shared memory.
__device__ __forceinline__ void place_block(uint32_t id, bool valid, uint32_t a, uint32_t n_warps_used, uint32_t* pos,
                                            uint32_t* __restrict__ order) {
    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
    const uint32_t key = valid ? id : 0xFFFFFFFFu;
    const uint32_t peers = __match_any_sync(0xFFFFFFFFu, key);
    const uint32_t rank = __popc(peers & ((1u << lane) - 1u));
    for (uint32_t w = 0; w < n_warps_used; ++w) {
        if (w == warp && valid) {
            order[pos[id] + rank] = a;
            __syncwarp(peers);
            if (rank == 0) pos[id] += __popc(peers);
        }
        __syncthreads();
    }
}

// The whole sort by one CTA of DTHREADS threads (A <= 2048 rows in practice); dsm: E + 99 words of shared memory
__device__ __forceinline__ void dispatch_body(const int32_t* __restrict__ ids, uint32_t A, uint32_t E,
                                              const uint8_t* __restrict__ loaded, DispatchTables t, uint32_t CHUNK_ROWS,
                                              uint32_t GROUP_CHUNKS, uint32_t HEAVY, uint32_t* status, uint32_t* dsm) {
    uint32_t* cnt = dsm;                // [E] counts, then running write positions
    uint32_t* ws = dsm + E;             // [99] scan scratch
    const uint32_t tid = threadIdx.x;
    for (uint32_t e = tid; e < E; e += DTHREADS) cnt[e] = 0;
    __syncthreads();
    for (uint32_t a = tid; a < A; a += DTHREADS) {
        int32_t id = ids[a];
        if (id < 0 || (uint32_t)id >= E) { atomicMax(status, (uint32_t)ST_BAD_EXPERT_ID); id = 0; }
        else if (loaded && !loaded[id]) atomicMax(status, (uint32_t)ST_NOT_LOADED);
        atomicAdd(&cnt[id], 1u);
    }
    __syncthreads();
    build_tables(cnt, E, loaded, t, CHUNK_ROWS, GROUP_CHUNKS, HEAVY, ws, status);
    __syncthreads();
    if (tid < E) cnt[tid] = t.offsets[tid];   // the entry this thread wrote
    __syncthreads();
    for (uint32_t a0 = 0; a0 < A; a0 += DTHREADS) {
        const uint32_t a = a0 + tid, left = A - a0;
        uint32_t id = 0;
        if (a < A) {
            const int32_t v = ids[a];
            id = (v < 0 || (uint32_t)v >= E) ? 0u : (uint32_t)v;
        }
        place_block(id, a < A, a, left >= (uint32_t)DTHREADS ? DTHREADS / 32 : (left + 31) / 32, cnt, t.order);
    }
}

}  // namespace mlxs
