// Router tail: fp32 logits -> top-k expert ids (rank order) + normalised weights.
// One CTA per token row, one thread per expert (n_experts <= 1024), top_k <= 64.
// Semantics: src/kernels/exl3/q3rc_router_tail.metal:12-40 (sqrt(softplus)), src/arch/mimo_v2/kernels/mimo_glue_top8.metal
// and src/arch/glm5_next/kernels/glm5n_glue_top8.metal (sigmoid): key = score + bias, rank = number of experts that
// precede (key descending, ties to the lower index, NaN last), ids[rank] = expert, weights from the unbiased score,
// sum folded in rank order (total = w[j] + total), / (sum + 1e-20), x scale.
#include "common.cuh"
#include "kernels.h"
#include "router_body.cuh"

namespace mlxs {

__global__ void router_kernel(const float* __restrict__ logits, const float* __restrict__ bias, int E, int K,
                              int scoring, int norm, float scale, int32_t* __restrict__ ids,
                              float* __restrict__ weights) {
    extern __shared__ float sm[];
    route_row(logits, bias, E, K, scoring, norm, scale, ids, weights, (int)blockIdx.x, sm, (int)blockDim.x);
}

// Router logits for decode-sized batches: logits[t, e] = sum_k f32(x[t, k]) * f32(W[e, k]), f32 accumulate
// (src/arch/deepseek_v41/graph.zig:2033; kernels q3rc_gate_part.metal, mimo_glue_router_rows.metal).  A warp owns one
// expert row; the CTA's eight warps share eight token rows at a time through shared memory.  The sum order is fixed: a
// lane adds its strided products in k order, then an xor butterfly.
constexpr int RL_WARPS = 8;
constexpr int RL_TOK = 8;        // token rows staged per pass
__global__ void __launch_bounds__(RL_WARPS * 32) router_logits_kernel(const __nv_bfloat16* __restrict__ x,
                                                                     const __nv_bfloat16* __restrict__ w, uint32_t T,
                                                                     uint32_t E, uint32_t H, float* __restrict__ logits) {
    extern __shared__ __align__(16) uint8_t rl_sm[];
    uint4* xs = reinterpret_cast<uint4*>(rl_sm);           // [RL_TOK][H / 8] vectors of 8 bf16
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t e = blockIdx.x * RL_WARPS + warp;
    const uint32_t nv = H / 8;
    const uint4* wrow = reinterpret_cast<const uint4*>(w + (size_t)(e < E ? e : 0) * H);
    for (uint32_t t0 = 0; t0 < T; t0 += RL_TOK) {
        const uint32_t nt = T - t0 < (uint32_t)RL_TOK ? T - t0 : (uint32_t)RL_TOK;
        __syncthreads();
        for (uint32_t v = threadIdx.x; v < nt * nv; v += RL_WARPS * 32)
            xs[v] = reinterpret_cast<const uint4*>(x + (size_t)t0 * H)[v];
        __syncthreads();
        float acc[RL_TOK];
#pragma unroll
        for (int tt = 0; tt < RL_TOK; ++tt) acc[tt] = 0.f;
        for (uint32_t v = lane; v < nv; v += 32) {
            const uint4 wv = wrow[v];
            const uint32_t ww[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
            for (int tt = 0; tt < RL_TOK; ++tt) {
                if ((uint32_t)tt < nt) {
                    const uint4 xv = xs[tt * nv + v];
                    const uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        acc[tt] = __fmaf_rn(__uint_as_float(xw[q] << 16), __uint_as_float(ww[q] << 16), acc[tt]);
                        acc[tt] = __fmaf_rn(__uint_as_float(xw[q] & 0xFFFF0000u), __uint_as_float(ww[q] & 0xFFFF0000u), acc[tt]);
                    }
                }
            }
        }
#pragma unroll
        for (int tt = 0; tt < RL_TOK; ++tt) {
            float a = acc[tt];
#pragma unroll
            for (int o = 16; o >= 1; o >>= 1) a = __fadd_rn(a, __shfl_xor_sync(0xFFFFFFFFu, a, o));
            if (lane == 0 && e < E && (uint32_t)tt < nt) logits[(size_t)(t0 + tt) * E + e] = a;
        }
    }
}

cudaError_t launch_router_logits(const __nv_bfloat16* x, const __nv_bfloat16* w, uint32_t T, uint32_t E, uint32_t H,
                                 float* logits, cudaStream_t st) {
    if (T == 0) return cudaSuccess;
    if (H % 8) return cudaErrorInvalidValue;
    const size_t smem = (size_t)RL_TOK * H * 2;
    cudaError_t err = cudaFuncSetAttribute(router_logits_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (err != cudaSuccess) return err;
    router_logits_kernel<<<(E + RL_WARPS - 1) / RL_WARPS, RL_WARPS * 32, smem, st>>>(x, w, T, E, H, logits);
    return cudaGetLastError();
}

cudaError_t launch_router(const float* logits, const float* bias, int T, int E, int K, int scoring, int norm,
                          float scale, int32_t* ids, float* weights, cudaStream_t st) {
    if (T == 0) return cudaSuccess;
    int threads = ((E > K ? E : K) + 31) / 32 * 32;
    const int nwarps = threads / 32;
    (void)nwarps;
    size_t smem = router_smem_floats(E, K, threads) * sizeof(float);
    router_kernel<<<T, threads, smem, st>>>(logits, bias, E, K, scoring, norm, scale, ids, weights);
    return cudaGetLastError();
}

}  // namespace mlxs
