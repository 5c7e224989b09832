// The router's logits for decode-sized batches (device code shared by the logits kernel and the fused front kernel):
// logits[t, e] = sum_k f32(x[t, k]) * f32(W[e, k]), f32 accumulate (src/arch/deepseek_v41/graph.zig:2033; kernels
// q3rc_gate_part.metal, mimo_glue_router_rows.metal).
// Four warps share one expert row: warp s sums the s-th quarter of the inputs (a lane adds its strided products in k
// order, then an xor butterfly), and the four partial sums are folded left, ((p0 + p1) + p2) + p3.  The order is a function
// of the shape only, so both kernels give the same bits.  Up to LG_TOK token rows are staged in shared memory per pass.
#pragma once
#include "common.cuh"

namespace mlxs {

constexpr int LG_TOK = 8;     // token rows staged per pass
constexpr int LG_PARTS = 4;   // warps per expert row

// shared memory of a CTA of `nwarps` warps: the staged rows, then the partial sums [nwarps][LG_TOK]
__host__ __device__ inline size_t logits_smem_bytes(uint32_t H, uint32_t nwarps) {
    return (size_t)LG_TOK * H * 2 + (size_t)nwarps * LG_TOK * sizeof(float);
}

// All threads of the CTA call this (it holds CTA-wide barriers).  The CTA's warps form nwarps / 4 expert slots; CTA
// `cta` of `n_cta` takes the experts e = (cta * slots + slot), stepping by n_cta * slots.
__device__ __forceinline__ void logits_rows(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                                            uint32_t T, uint32_t E, uint32_t H, float* __restrict__ logits, uint8_t* sm,
                                            uint32_t cta, uint32_t n_cta) {
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u, nwarps = blockDim.x >> 5;
    const uint32_t slots = nwarps / LG_PARTS, slot = warp / LG_PARTS, part = warp % LG_PARTS;
    const uint32_t nv = H / 8;
    uint4* xs = reinterpret_cast<uint4*>(sm);                                  // [LG_TOK][nv] vectors of 8 bf16
    float* ps = reinterpret_cast<float*>(sm + (size_t)LG_TOK * H * 2);         // [nwarps][LG_TOK]
    const uint32_t v_begin = part * nv / LG_PARTS, v_end = (part + 1) * nv / LG_PARTS;
    const uint32_t e_step = n_cta * slots, rounds = (E + e_step - 1) / e_step;
    for (uint32_t t0 = 0; t0 < T; t0 += LG_TOK) {
        const uint32_t nt = T - t0 < (uint32_t)LG_TOK ? T - t0 : (uint32_t)LG_TOK;
        __syncthreads();
        for (uint32_t v = threadIdx.x; v < nt * nv; v += blockDim.x) xs[v] = reinterpret_cast<const uint4*>(x + (size_t)t0 * H)[v];
        __syncthreads();
        for (uint32_t rd = 0; rd < rounds; ++rd) {
            const uint32_t e = rd * e_step + cta * slots + slot;
            const bool live = slot < slots && e < E;
            float acc[LG_TOK];
#pragma unroll
            for (int tt = 0; tt < LG_TOK; ++tt) acc[tt] = 0.f;
            if (live) {
                const uint4* wrow = reinterpret_cast<const uint4*>(w + (size_t)e * H);
                for (uint32_t v = v_begin + lane; v < v_end; v += 32) {
                    const uint4 wv = wrow[v];
                    const uint32_t ww[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
                    for (int tt = 0; tt < LG_TOK; ++tt) {
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
            }
#pragma unroll
            for (int tt = 0; tt < LG_TOK; ++tt) {
                float a = acc[tt];
#pragma unroll
                for (int o = 16; o >= 1; o >>= 1) a = __fadd_rn(a, __shfl_xor_sync(0xFFFFFFFFu, a, o));
                if (lane == 0) ps[warp * LG_TOK + tt] = a;
            }
            __syncthreads();
            if (live && part == 0 && lane < nt) {
                const float* p0 = ps + (slot * LG_PARTS) * LG_TOK + lane;
                float a = p0[0];
#pragma unroll
                for (int s = 1; s < LG_PARTS; ++s) a = __fadd_rn(a, p0[s * LG_TOK]);
                logits[(size_t)(t0 + lane) * E + e] = a;
            }
            __syncthreads();
        }
    }
}

}  // namespace mlxs
