// The front of a decode-sized layer call in one launch: [router logits from x] -> router tail -> dispatch -> row
// staging.  Four dependent kernels of a few microseconds each cost a decode step more in launch gaps than in work
// (at one token: 37 us of a 175 us call); here they are phases of one cooperative kernel separated by grid barriers,
// and the [T, E] logits, the ids and the tables never leave the L2 between them.
//   phase 0 (only when the layer starts from x): logits = f32(x) . f32(W_g)^T, four warps per expert row, 8 token rows
//            staged in shared memory at a time (src/arch/deepseek_v41/graph.zig:2033; mimo_glue_router_rows.metal);
//   phase 1: CTA t routes token t (the router kernel's code: scoring, bias, top-k, weights);
//   phase 2: CTA 0 sorts the assignment rows by expert and builds the work tables (the dispatch kernel's code);
//   phase 3: all warps stage the rows for the streaming lane (the prep kernels' code).
// The grid barrier is a counter and a generation word in global memory: the last CTA to arrive resets the counter and
// bumps the generation, the others poll the generation with a bound.  The launch is cooperative, so all CTAs are
// resident together; a barrier that runs out still records the status word and lets the kernel finish.
#include "common.cuh"
#include "kernels.h"
#include "dispatch_body.cuh"
#include "exl3_prep_body.cuh"
#include "fp4_prep_body.cuh"
#include "logits_body.cuh"
#include "router_body.cuh"

namespace mlxs {

struct FrontParams {
    // phase 0 (w_router == null: the caller supplies logits)
    const __nv_bfloat16* w_router;   // [E, H] bf16
    float* logits_out;               // [T, E] written by phase 0
    // phase 1
    const float* logits;             // [T, E]
    const float* bias;
    int E, K, scoring, norm;
    float scale;
    int32_t* ids;
    float* weights;
    uint32_t T;
    // phase 2
    const uint8_t* loaded;
    DispatchTables t;
    uint32_t chunk_rows, group_chunks, heavy;
    uint32_t* status;
    // phase 3
    const __nv_bfloat16* x;
    uint32_t H;
    int bank_exl3;
    const __half* scales;
    size_t scales_stride;
    uint32_t* xa;
    // grid barrier: [0] arrivals, [1] generation
    uint32_t* bar;
    uint32_t poll_limit;
    int rthreads;
};

__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// All CTAs of the grid meet here.  gen: the generation this CTA saw before its first arrival, kept per thread.
__device__ __forceinline__ bool front_grid_sync(uint32_t* bar, uint32_t& gen, uint32_t limit, uint32_t* status) {
    __shared__ int s_ok;
    __syncthreads();
    if (threadIdx.x == 0) {
        bool ok = true;
        __threadfence();
        const uint32_t prev = atomicAdd(&bar[0], 1u);
        if (prev == gridDim.x - 1) {
            bar[0] = 0;
            __threadfence();
            atomicAdd(&bar[1], 1u);
        } else {
            uint32_t i = 0;
            while (ld_acquire_gpu(&bar[1]) == gen) {
                if (++i > limit) { ok = false; atomicMax(status, (uint32_t)ST_WAIT_FULL); break; }
                __nanosleep(32);
            }
        }
        __threadfence();
        s_ok = ok ? 1 : 0;
    }
    gen += 1;
    __syncthreads();
    return s_ok != 0;
}

__global__ void __launch_bounds__(1024, 1) front_kernel(const FrontParams P) {
    extern __shared__ __align__(16) uint8_t fsm[];
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u, nwarp = blockDim.x >> 5;
    // the barrier's generation before this CTA's first arrival (it cannot advance until every CTA, this one too, arrives)
    __shared__ uint32_t s_gen;
    if (threadIdx.x == 0) s_gen = ld_acquire_gpu(&P.bar[1]);
    __syncthreads();
    uint32_t gen = s_gen;
    const uint32_t T = P.T;

    // ---- phase 0: logits from x (the logits kernel's code: four warps per expert row) ----
    if (P.w_router) {
        logits_rows(P.x, P.w_router, T, (uint32_t)P.E, P.H, P.logits_out, fsm, blockIdx.x, gridDim.x);
        front_grid_sync(P.bar, gen, P.poll_limit, P.status);
    }

    // ---- phase 1: the router's tail, a CTA per token ----
    for (uint32_t t = blockIdx.x; t < T; t += gridDim.x)
        route_row(P.logits, P.bias, P.E, P.K, P.scoring, P.norm, P.scale, P.ids, P.weights, (int)t, reinterpret_cast<float*>(fsm), P.rthreads);
    front_grid_sync(P.bar, gen, P.poll_limit, P.status);

    // ---- phase 2: dispatch by CTA 0 ----
    if (blockIdx.x == 0)
        dispatch_body(P.ids, T * (uint32_t)P.K, (uint32_t)P.E, P.loaded, P.t, P.chunk_rows, P.group_chunks, P.heavy, P.status,
                      reinterpret_cast<uint32_t*>(fsm));
    front_grid_sync(P.bar, gen, P.poll_limit, P.status);

    // ---- phase 3: row staging, a warp per (chunk, row, 128-block) or per (chunk, row) ----
    const uint32_t n_chunks = P.t.header[HDR_NCHUNKS];
    const uint32_t gw = blockIdx.x * nwarp + warp, gstride = gridDim.x * nwarp;
    if (P.bank_exl3) {
        const uint32_t nb = P.H / 128, per_chunk = P.chunk_rows * nb;
        for (uint32_t task = gw; task < n_chunks * per_chunk; task += gstride) {
            const uint32_t chunk = task / per_chunk, rem = task % per_chunk, row = rem / nb, b = rem % nb;
            const uint32_t e = P.t.chunk_expert[chunk], rows = P.t.chunk_rows[chunk];
            const bool valid = row < rows;
            const uint32_t assign = valid ? P.t.order[P.t.chunk_row0[chunk] + row] : 0u;
            exl3_prep_row_block<false>(P.x, x_row_of(P.t, assign, (uint32_t)P.K), valid, e, P.H, P.scales, P.scales_stride, chunk, row, b,
                                       lane, P.xa);
        }
    } else {
        // a row's 8-input groups are split over 4 warps
        for (uint32_t task = gw; task < n_chunks * P.chunk_rows * 4u; task += gstride) {
            const uint32_t chunk = task / (P.chunk_rows * 4u), rem = task % (P.chunk_rows * 4u), row = rem / 4u, part = rem % 4u;
            const bool valid = row < P.t.chunk_rows[chunk];
            const uint32_t tok = valid ? x_row_of(P.t, P.t.order[P.t.chunk_row0[chunk] + row], (uint32_t)P.K) : 0u;
            fp4_prep_row(P.x, tok, valid, P.H, chunk, row, part * 32u + lane, 128u, P.xa);
        }
    }
}

// smem: the larger of the phases' needs
static size_t front_smem_bytes(const FrontArgs& a, int rthreads) {
    size_t s = router_smem_floats(a.E, a.K, rthreads) * sizeof(float);
    const size_t d = ((size_t)a.E + 99) * sizeof(uint32_t);
    if (d > s) s = d;
    if (a.w_router) { const size_t l = logits_smem_bytes(a.H, 32); if (l > s) s = l; }
    return s;
}

cudaError_t launch_front(const FrontArgs& a, cudaStream_t st) {
    if (a.T == 0) return cudaSuccess;
    FrontParams P{};
    P.w_router = a.w_router; P.logits_out = a.logits_out; P.logits = a.w_router ? a.logits_out : a.logits; P.bias = a.bias;
    P.E = a.E; P.K = a.K; P.scoring = a.scoring; P.norm = a.norm; P.scale = a.scale; P.ids = a.ids; P.weights = a.weights; P.T = a.T;
    P.loaded = a.loaded; P.t = a.t; P.chunk_rows = a.chunk_rows; P.group_chunks = a.group_chunks; P.heavy = a.heavy; P.status = a.status;
    P.x = a.x; P.H = a.H; P.bank_exl3 = a.bank_exl3; P.scales = a.scales; P.scales_stride = a.scales_stride; P.xa = a.xa;
    P.bar = a.bar; P.poll_limit = 1u << 22;
    const int rt = ((a.E > a.K ? a.E : a.K) + 31) / 32 * 32;
    P.rthreads = rt;
    const size_t smem = front_smem_bytes(a, rt);
    cudaError_t e = cudaFuncSetAttribute(front_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    void* args[] = {&P};
    // enough CTAs for the staging of the call's rows (a CTA per SM above 16 tokens); every CTA of a cooperative launch
    // is resident at once
    const unsigned grid = a.T > 16 ? (unsigned)(a.sm_count > 0 ? a.sm_count : 32) : (a.T > 4 ? 32u : (a.T > 1 ? 16u : 8u));
    return cudaLaunchCooperativeKernel(reinterpret_cast<void*>(front_kernel), dim3(grid), dim3(1024), args, smem, st);
}

}  // namespace mlxs
