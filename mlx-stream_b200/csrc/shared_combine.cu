// The bf16 dense shared expert at decode widths (larger batches: dense_gemm.cu), and the weighted combine.
//
// Shared expert (src/arch/deepseek_v41/graph.zig:2162-2172): h = silu(min(w1 x, lim)) * clip(w3 x, +-lim) in f32,
// rounded to the activation dtype, then w2 h.  Memory-bound on the 3 H I bf16 weights: a CTA owns 16 output features,
// its 8 warps split the reduction dimension, weights stream as 128-bit loads straight into mma A fragments (the k
// order inside a 32-wide chunk is permuted identically for both operands, which a dot product does not see).
//
// Combine (src/arch/deepseek_v41/graph.zig:2182-2184; src/arch/mimo_v2/kernels/mimo_moe_combine.metal;
// src/arch/glm5_next/kernels/glm5n_moe_combine.metal): fixed fold order k = 0..top_k-1, one bf16 rounding.
#include "common.cuh"
#include "kernels.h"

namespace mlxs {

// warps of a CTA (they split the reduction dimension).  The down kernel has 320 row tiles for 148 SMs: with 4 warps
// and about 100 registers every CTA is resident at once (2-3 per SM) instead of running in two waves.
constexpr int sh_warps(int mode) { return mode == 0 ? 8 : 4; }
constexpr int SH_TOK = 64;  // tokens per pass
constexpr int SH_AHEAD = 2;  // weight chunks in flight per warp

template <int MODE>  // 0: gate/up + activation -> h bf16 [T, N]; 1: down -> out f32 [T, N]
__global__ void __launch_bounds__(sh_warps(MODE) * 32) shared_kernel(const __nv_bfloat16* __restrict__ x, uint32_t T,
                                                               uint32_t Kdim, uint32_t N,
                                                               const __nv_bfloat16* __restrict__ wa,
                                                               const __nv_bfloat16* __restrict__ wb, float limit,
                                                               __nv_bfloat16* __restrict__ h_out,
                                                               float* __restrict__ f_out) {
    extern __shared__ float red[];  // [SH_WARPS][NW][8 tiles][32 lanes][4]
    constexpr int SH_WARPS = sh_warps(MODE);
    constexpr int NW = MODE == 0 ? 2 : 1;
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u, g = lane >> 2, c = lane & 3u;
    const uint32_t row0 = blockIdx.x * 16;
    for (uint32_t t0 = 0; t0 < T; t0 += SH_TOK) {
        const uint32_t nt_n = min((uint32_t)SH_TOK, T - t0);
        const uint32_t ntiles = (nt_n + 7) / 8;
        float acc[NW][8][4];
#pragma unroll
        for (int w = 0; w < NW; ++w)
#pragma unroll
            for (int i = 0; i < 8; ++i)
#pragma unroll
                for (int q = 0; q < 4; ++q) acc[w][i][q] = 0.f;
        // A warp walks its share of the reduction dimension 32 inputs at a time.  The weights come straight from HBM and
        // are used once, so the loads of the next SH_AHEAD chunks are always in flight (a register ring, statically
        // indexed) while the current chunk's mma run: with one chunk in flight the kernel was bound by the load latency.
        const uint32_t nchunk = Kdim / 32;
        uint4 ring[SH_AHEAD][2 * NW];
        auto load_chunk = [&](uint4 (&dst)[2 * NW], uint32_t kc) {
            if (kc < nchunk) {
                const size_t ko = (size_t)kc * 32 + c * 8;
                dst[0] = __ldcs(reinterpret_cast<const uint4*>(wa + (size_t)(row0 + g) * Kdim + ko));
                dst[1] = __ldcs(reinterpret_cast<const uint4*>(wa + (size_t)(row0 + g + 8) * Kdim + ko));
                if (NW == 2) {
                    dst[2 * NW - 2] = __ldcs(reinterpret_cast<const uint4*>(wb + (size_t)(row0 + g) * Kdim + ko));
                    dst[2 * NW - 1] = __ldcs(reinterpret_cast<const uint4*>(wb + (size_t)(row0 + g + 8) * Kdim + ko));
                }
            }
        };
        // the rows of a chunk's token tiles come from L2: they too are loaded one chunk ahead, all eight at once
        // (predicated, no branch between them)
        static_assert(SH_AHEAD == 2, "the row buffers alternate with the chunk's place in the weight ring");
        uint4 xr[2][8];
        auto load_rows = [&](uint4 (&dst)[8], uint32_t kc) {
            const size_t ko = (size_t)kc * 32 + c * 8;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const uint32_t tok = t0 + i * 8 + g;
                dst[i] = make_uint4(0, 0, 0, 0);
                if (kc < nchunk && i < (int)ntiles && tok < T) dst[i] = *reinterpret_cast<const uint4*>(x + (size_t)tok * Kdim + ko);
            }
        };
#pragma unroll
        for (int r = 0; r < SH_AHEAD; ++r) load_chunk(ring[r], warp + r * SH_WARPS);
        load_rows(xr[0], warp);
        for (uint32_t kc0 = warp; kc0 < nchunk; kc0 += SH_AHEAD * SH_WARPS) {
#pragma unroll
            for (int r = 0; r < SH_AHEAD; ++r) {
                const uint32_t kc = kc0 + r * SH_WARPS;
                if (kc < nchunk) {
                    uint4 a[2 * NW];
#pragma unroll
                    for (int q = 0; q < 2 * NW; ++q) a[q] = ring[r][q];
                    load_chunk(ring[r], kc + SH_AHEAD * SH_WARPS);
                    load_rows(xr[r ^ 1], kc + SH_WARPS);
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        if (i < (int)ntiles) {
#pragma unroll
                            for (int w = 0; w < NW; ++w) {
                                const uint32_t a1[4] = {a[2 * w].x, a[2 * w + 1].x, a[2 * w].y, a[2 * w + 1].y};
                                const uint32_t a2[4] = {a[2 * w].z, a[2 * w + 1].z, a[2 * w].w, a[2 * w + 1].w};
                                mma_bf16(acc[w][i], a1, xr[r][i].x, xr[r][i].y);
                                mma_bf16(acc[w][i], a2, xr[r][i].z, xr[r][i].w);
                            }
                        }
                    }
                }
            }
        }
        // cross-warp reduction of the split reduction dimension
#pragma unroll
        for (int w = 0; w < NW; ++w)
#pragma unroll
            for (int i = 0; i < 8; ++i)
                if (i < (int)ntiles)
                    *reinterpret_cast<float4*>(red + ((((size_t)warp * NW + w) * 8 + i) * 32 + lane) * 4) =
                        make_float4(acc[w][i][0], acc[w][i][1], acc[w][i][2], acc[w][i][3]);
        __syncthreads();
        for (uint32_t idx = threadIdx.x; idx < ntiles * 128; idx += SH_WARPS * 32) {
            const uint32_t i = idx / 128, ln = (idx / 4) % 32, q = idx % 4;
            float s[NW];
#pragma unroll
            for (int w = 0; w < NW; ++w) {
                float v = 0.f;
                for (int ww = 0; ww < SH_WARPS; ++ww) v += red[((((size_t)ww * NW + w) * 8 + i) * 32 + ln) * 4 + q];
                s[w] = v;
            }
            const uint32_t row = row0 + (ln >> 2) + ((q & 2) ? 8 : 0);
            const uint32_t tok = t0 + i * 8 + 2 * (ln & 3) + (q & 1);
            if (tok < T) {
                if (MODE == 0) {
                    float gate = s[0], up = s[NW - 1];
                    if (limit > 0.f) {
                        gate = (gate != gate) ? gate : (gate < limit ? gate : limit);
                        up = (up != up) ? up : (up > limit ? limit : (up < -limit ? -limit : up));
                    }
                    const float yv = 1.0f / (1.0f + expf(fabsf(gate)));
                    const float sg = gate < 0.f ? yv : 1.0f - yv;
                    h_out[(size_t)tok * N + row] = __float2bfloat16_rn((gate * sg) * up);
                } else {
                    f_out[(size_t)tok * N + row] = s[0];
                }
            }
        }
        __syncthreads();
    }
}

cudaError_t launch_shared_expert(const __nv_bfloat16* x, const __nv_bfloat16* w1, const __nv_bfloat16* w3,
                                 const __nv_bfloat16* w2, uint32_t T, uint32_t H, uint32_t I, float limit,
                                 __nv_bfloat16* h_ws, float* out, cudaStream_t st) {
    if (T == 0) return cudaSuccess;
    const size_t smem0 = (size_t)sh_warps(0) * 2 * 8 * 32 * 4 * sizeof(float), smem1 = (size_t)sh_warps(1) * 8 * 32 * 4 * sizeof(float);
    cudaError_t e = cudaFuncSetAttribute(shared_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem0);
    if (e != cudaSuccess) return e;
    shared_kernel<0><<<I / 16, sh_warps(0) * 32, smem0, st>>>(x, T, H, I, w1, w3, limit, h_ws, nullptr);
    e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    shared_kernel<1><<<H / 16, sh_warps(1) * 32, smem1, st>>>(h_ws, T, I, H, w2, nullptr, 0.f, nullptr, out);
    return cudaGetLastError();
}

// thread = 4 columns of one token
__global__ void combine_kernel(const void* __restrict__ ro, int ro_bf16, const float* __restrict__ weights,
                               const float* __restrict__ shared, uint32_t T, uint32_t K, uint32_t H, int chain,
                               __nv_bfloat16* __restrict__ y) {
    const uint32_t col = (blockIdx.x * blockDim.x + threadIdx.x) * 4, t = blockIdx.y;
    if (col >= H) return;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (uint32_t k = 0; k < K; ++k) {
        const float w = weights[(size_t)t * K + k];
        float r[4];
        if (ro_bf16) {
            const uint2 v = *reinterpret_cast<const uint2*>(static_cast<const __nv_bfloat16*>(ro) +
                                                            ((size_t)t * K + k) * H + col);
            r[0] = __uint_as_float(v.x << 16); r[1] = __uint_as_float(v.x & 0xFFFF0000u);
            r[2] = __uint_as_float(v.y << 16); r[3] = __uint_as_float(v.y & 0xFFFF0000u);
        } else {
            const float4 v = *reinterpret_cast<const float4*>(static_cast<const float*>(ro) + ((size_t)t * K + k) * H + col);
            r[0] = v.x; r[1] = v.y; r[2] = v.z; r[3] = v.w;
        }
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const float p = __fadd_rn(__fmul_rn(r[q], w), 0.0f);  // each product rounded, no contraction
            acc[q] = k == 0 ? p : __fadd_rn(p, acc[q]);
        }
    }
    float o[4];
    if (chain) {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            float routed = bf16_round_f(acc[q]);
            if (shared) routed = __fadd_rn(routed, bf16_round_f(shared[(size_t)t * H + col + q]));
            o[q] = routed;
        }
    } else {
#pragma unroll
        for (int q = 0; q < 4; ++q) o[q] = shared ? __fadd_rn(acc[q], shared[(size_t)t * H + col + q]) : acc[q];
    }
    __nv_bfloat162 lo = __floats2bfloat162_rn(o[0], o[1]), hi = __floats2bfloat162_rn(o[2], o[3]);
    uint2 pk = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
    *reinterpret_cast<uint2*>(y + (size_t)t * H + col) = pk;
}

cudaError_t launch_combine(const void* ro, int ro_bf16, const float* weights, const float* shared, uint32_t T,
                           uint32_t K, uint32_t H, int chain, __nv_bfloat16* y, cudaStream_t st) {
    if (T == 0) return cudaSuccess;
    dim3 grid((H / 4 + 255) / 256, T);
    combine_kernel<<<grid, 256, 0, st>>>(ro, ro_bf16, weights, shared, T, K, H, chain, y);
    return cudaGetLastError();
}

}  // namespace mlxs
