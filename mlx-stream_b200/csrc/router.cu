// Router tail: fp32 logits -> top-k expert ids (rank order) + normalised weights.
// One CTA per token row, one thread per expert (n_experts <= 1024), top_k <= 64.
// Semantics: src/kernels/exl3/q3rc_router_tail.metal:12-40 (sqrt(softplus)), src/arch/mimo_v2/kernels/mimo_glue_top8.metal
// and src/arch/glm5_next/kernels/glm5n_glue_top8.metal (sigmoid): key = score + bias, rank = number of experts that
// precede (key descending, ties to the lower index, NaN last), ids[rank] = expert, weights from the unbiased score,
// sum folded in rank order (total = w[j] + total), / (sum + 1e-20), x scale.
#include "common.cuh"
#include "kernels.h"
#include "logits_body.cuh"
#include "router_body.cuh"

namespace mlxs {

__global__ void router_kernel(const float* __restrict__ logits, const float* __restrict__ bias, int E, int K,
                              int scoring, int norm, float scale, int32_t* __restrict__ ids,
                              float* __restrict__ weights) {
    extern __shared__ float sm[];
    route_row(logits, bias, E, K, scoring, norm, scale, ids, weights, (int)blockIdx.x, sm, (int)blockDim.x);
}

// Router logits for decode-sized batches: the shared device code of logits_body.cuh, two expert rows per CTA of 8 warps
constexpr int RL_WARPS = 8;
__global__ void __launch_bounds__(RL_WARPS * 32) router_logits_kernel(const __nv_bfloat16* __restrict__ x,
                                                                     const __nv_bfloat16* __restrict__ w, uint32_t T,
                                                                     uint32_t E, uint32_t H, float* __restrict__ logits) {
    extern __shared__ __align__(16) uint8_t rl_sm[];
    logits_rows(x, w, T, E, H, logits, rl_sm, blockIdx.x, gridDim.x);
}

cudaError_t launch_router_logits(const __nv_bfloat16* x, const __nv_bfloat16* w, uint32_t T, uint32_t E, uint32_t H,
                                 float* logits, cudaStream_t st) {
    if (T == 0) return cudaSuccess;
    if (H % 8) return cudaErrorInvalidValue;
    const size_t smem = logits_smem_bytes(H, RL_WARPS);
    cudaError_t err = cudaFuncSetAttribute(router_logits_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (err != cudaSuccess) return err;
    const uint32_t slots = RL_WARPS / LG_PARTS;
    router_logits_kernel<<<(E + slots - 1) / slots, RL_WARPS * 32, smem, st>>>(x, w, T, E, H, logits);
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
