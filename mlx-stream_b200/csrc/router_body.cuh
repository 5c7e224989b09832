// The router's tail for one token row (device code shared by the router kernel and the fused front kernel).
#pragma once
#include "common.cuh"

namespace mlxs {

__device__ __forceinline__ float rt_log1p(float x) {  // src/kernels/exl3/header_router_tail.metal
    float xp1 = __fadd_rn(1.0f, x);
    if (xp1 == __int_as_float(0x7F800000)) return xp1;
    if (xp1 == 1.0f) return x;
    return __fmul_rn(x, __fdiv_rn(det_logf(xp1), __fsub_rn(xp1, 1.0f)));
}
__device__ __forceinline__ float rt_softplus(float g) {
    if (g != g) return __int_as_float(0x7FC00000);
    float maxval = g > 0.0f ? g : 0.0f, minval = g > 0.0f ? 0.0f : g;
    const float inf = __int_as_float(0x7F800000);
    if (minval == -inf || maxval == inf) return maxval;
    return __fadd_rn(maxval, rt_log1p(det_expf(__fsub_rn(minval, maxval))));
}

// One token row by the whole CTA: thread e < E scores expert e; `rthreads` = the E (and K) rounded up to whole warps,
// the threads beyond it only keep the barriers company.  sm: router_smem_floats(E, K, rthreads) floats.
__host__ __device__ inline size_t router_smem_floats(int E, int K, int rthreads) {
    const int nwarps = rthreads / 32;
    return (size_t)(E + 34 + K + (nwarps * K <= 256 ? nwarps * K : 0));
}
__device__ __forceinline__ void route_row(const float* __restrict__ logits, const float* __restrict__ bias, int E, int K,
                                          int scoring, int norm, float scale, int32_t* __restrict__ ids,
                                          float* __restrict__ weights, int row, float* sm, int rthreads) {
    float* key_sh = sm;          // [E]
    float* red = sm + E;         // [32] softmax partials, then [0] = sum, [1] = max
    float* picked = red + 34;    // [K]
    const int e = threadIdx.x;
    const float x = e < E ? logits[(size_t)row * E + e] : 0.0f;
    float score = 0.0f;
    if (scoring == 1) {
        float y = __fdiv_rn(1.0f, __fadd_rn(1.0f, det_expf(fabsf(x))));
        score = x < 0.0f ? y : __fsub_rn(1.0f, y);
    } else if (scoring == 0) {
        score = __fsqrt_rn(rt_softplus(x));
    } else {
        // softmax: max (exact in any order), exp(x - max), sum = 32 strided partials in index order then an
        // xor butterfly 16, 8, 4, 2, 1 (the order the host restatement folds in)
        if (e < E) key_sh[e] = x;
        __syncthreads();
        if (threadIdx.x < 32) {
            float m = -__int_as_float(0x7F800000);
            bool has_nan = false;
            for (int j = threadIdx.x; j < E; j += 32) {
                float v = key_sh[j];
                if (v != v) has_nan = true; else if (v > m) m = v;
            }
            for (int o = 16; o >= 1; o >>= 1) {
                float om = __shfl_xor_sync(0xFFFFFFFFu, m, o);
                m = om > m ? om : m;
            }
            has_nan = __any_sync(0xFFFFFFFFu, has_nan);
            if (threadIdx.x == 0) { red[33] = m; red[32] = has_nan ? 1.0f : 0.0f; }
        }
        __syncthreads();
        const float m = red[33];
        const bool has_nan = red[32] != 0.0f;
        float ex = has_nan ? __int_as_float(0x7FC00000) : det_expf(__fsub_rn(x, m));
        __syncthreads();
        if (e < E) key_sh[e] = ex;
        __syncthreads();
        if (threadIdx.x < 32) {
            float p = 0.0f;
            for (int j = threadIdx.x; j < E; j += 32) p = __fadd_rn(p, key_sh[j]);
            for (int o = 16; o >= 1; o >>= 1) p = __fadd_rn(p, __shfl_xor_sync(0xFFFFFFFFu, p, o));
            if (threadIdx.x == 0) red[0] = p;
        }
        __syncthreads();
        score = __fdiv_rn(ex, red[0]);
        __syncthreads();
    }
    const float biased = bias ? __fadd_rn(score, e < E ? bias[e] : 0.0f) : score;
    const int nwarps = rthreads >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (K <= 32 && nwarps * K <= 256 && 2 * nwarps * K <= E + 34) {
        // Selection by repeated maximum of a total order that is the rank rule: the float key mapped monotonically to
        // an unsigned (NaN lowest, -0 folded into +0 so that equal floats tie), ties to the lower index.  Each warp
        // takes the K best of its 32 experts with warp-wide max / min reductions, warp 0 then takes the K best of the
        // nwarps x K candidates.  The result is the same permutation the rank count gives.
        uint32_t* cand_key = reinterpret_cast<uint32_t*>(key_sh);          // [nwarps * K]
        uint32_t* cand_idx = cand_key + nwarps * K;                         // needs 2 * nwarps * K <= E + 34 + K words
        float* cand_score = picked + K;                                     // [nwarps * K]
        uint32_t mykey = 0;
        if (e < E && biased == biased) {
            const uint32_t b = __float_as_uint(__fadd_rn(biased, 0.0f));
            mykey = (b & 0x80000000u) ? ~b : (b | 0x80000000u);
            // a NaN stays 0, the lowest; a real key is >= 1 (~0xFF800000 for -inf is 0x007FFFFF)
        }
        bool alive = e < E;
        for (int r = 0; r < K && warp < nwarps; ++r) {
            const uint32_t k = alive ? mykey : 0u;
            const uint32_t best = __reduce_max_sync(0xFFFFFFFFu, k);
            const uint32_t who = __reduce_min_sync(0xFFFFFFFFu, (alive && k == best) ? (uint32_t)lane : 0xFFFFFFFFu);
            if (who == 0xFFFFFFFFu) {  // fewer than K experts in this warp
                if (lane == 0) { cand_key[warp * K + r] = 0; cand_idx[warp * K + r] = 0xFFFFFFFFu; }
                continue;
            }
            if ((uint32_t)lane == who) {
                cand_key[warp * K + r] = mykey; cand_idx[warp * K + r] = (uint32_t)e; cand_score[warp * K + r] = score;
                alive = false;
            }
        }
        __syncthreads();
        if (warp == 0) {
            const int C = nwarps * K, per = (C + 31) / 32;   // per <= 8
            uint32_t ck[8], ci[8];
            float cs[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int c = lane + 32 * i;
                const bool ok = i < per && c < C;
                ck[i] = ok ? cand_key[c] : 0u;
                ci[i] = ok ? cand_idx[c] : 0xFFFFFFFFu;
                cs[i] = ok ? cand_score[c] : 0.0f;
            }
            for (int r = 0; r < K; ++r) {
                // this lane's best live candidate: highest key, then lowest expert index
                uint32_t bk = 0, bi = 0xFFFFFFFFu;
                int bslot = -1;
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    if (ci[i] != 0xFFFFFFFFu && (bslot < 0 || ck[i] > bk || (ck[i] == bk && ci[i] < bi))) { bk = ck[i]; bi = ci[i]; bslot = i; }
                }
                const uint32_t best = __reduce_max_sync(0xFFFFFFFFu, bslot >= 0 ? bk : 0u);
                const uint32_t who = __reduce_min_sync(0xFFFFFFFFu, (bslot >= 0 && bk == best) ? bi : 0xFFFFFFFFu);
                if (bslot >= 0 && bi == who) {
                    float sc = 0.0f;
#pragma unroll
                    for (int i = 0; i < 8; ++i) if (i == bslot) { sc = cs[i]; ci[i] = 0xFFFFFFFFu; }
                    ids[(size_t)row * K + r] = (int32_t)who;
                    picked[r] = sc;
                }
            }
        }
    } else {
        if (e < E) key_sh[e] = biased;
        __syncthreads();
        if (e < E) {
            const bool mn = biased != biased;
            int rank = 0;
            for (int j = 0; j < E; ++j) {
                const float o = key_sh[j];
                const bool on = o != o;
                const bool before = mn ? (!on || j < e) : (!on && (o > biased || (o == biased && j < e)));
                rank += before ? 1 : 0;
            }
            if (rank < K) {
                ids[(size_t)row * K + rank] = e;
                picked[rank] = score;
            }
        }
    }
    __syncthreads();
    if (e < K) {
        float total = 0.0f;
        for (int j = 0; j < K; ++j) total = __fadd_rn(picked[j], total);
        const float den = __fadd_rn(total, 1e-20f);
        const float q = norm ? __fdiv_rn(picked[e], den) : picked[e];
        weights[(size_t)row * K + e] = __fmul_rn(q, scale);
    }
    __syncthreads();   // the shared arrays are free for the next row
}


}  // namespace mlxs
