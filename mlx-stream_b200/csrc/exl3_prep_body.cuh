// Device code of the EXL3 streaming lane's row staging (shared by the prep kernel and the fused front kernel).
#pragma once
#include "common.cuh"
#include "kernels.h"

namespace mlxs {

constexpr int A_TILE_WORDS = 64;   // one chunk x k-tile of activations in B-fragment order: 32 lanes x 2 u32

// One chunk x k-tile block is 32 lanes x 2 u32: lane (g = token slot, c) holds b0 = x[slot g][k 2c,2c+1],
// b1 = x[slot g][k 2c+8,2c+9]; slots 0..3 are the f16 hi halves of rows 0..3, slots 4..7 their lo halves.  A warp lane
// that owns elements 4*lane..4*lane+3 of a 128-block writes k-tile lane/4, k = 4*(lane&3) + q.
__device__ __forceinline__ void store_frag4(uint32_t* tile_base /* the 128-block's first k-tile */, uint32_t row,
                                            uint32_t lane, const float (&v)[4]) {
    const uint32_t cq = lane & 3u;
    uint32_t* kt = tile_base + (lane >> 2) * A_TILE_WORDS;
    const uint32_t c0 = 2u * (cq & 1u), reg = cq >> 1;
    __half h0, l0, h1, l1, h2, l2, h3, l3;
    split_hi_lo(v[0], h0, l0); split_hi_lo(v[1], h1, l1); split_hi_lo(v[2], h2, l2); split_hi_lo(v[3], h3, l3);
    kt[(row * 4u + c0) * 2u + reg] = pack_h2(h0, h1);
    kt[((row + 4u) * 4u + c0) * 2u + reg] = pack_h2(l0, l1);
    kt[(row * 4u + c0 + 1u) * 2u + reg] = pack_h2(h2, h3);
    kt[((row + 4u) * 4u + c0 + 1u) * 2u + reg] = pack_h2(l2, l3);
}

// One warp stages one 128-block b of one row of a chunk (both projections, or the raw row): xg = H128(x * suh) *
// 128^-0.5 as f16 hi / lo in fragment order.  row = the row's slot inside its chunk; tok = the row of x it reads.
template <bool RAW>
__device__ __forceinline__ void exl3_prep_row_block(const void* __restrict__ xin, uint32_t tok, bool valid, uint32_t e,
                                                    uint32_t in_dim, const __half* __restrict__ scales, size_t scales_stride,
                                                    uint32_t chunk, uint32_t row, uint32_t b, uint32_t lane,
                                                    uint32_t* __restrict__ xa) {
    const uint32_t nkt = in_dim / 16;
    constexpr int NP = RAW ? 1 : 2;
    const float S = __uint_as_float(SCALE_BITS);
    for (int p = 0; p < NP; ++p) {
        uint32_t* dst = xa + ((size_t)chunk * NP + p) * nkt * A_TILE_WORDS;
        float v[4] = {0.f, 0.f, 0.f, 0.f};
        if (valid) {
            if (RAW) {
                const float4 f = *reinterpret_cast<const float4*>(static_cast<const float*>(xin) +
                                                                  (size_t)tok * in_dim + b * 128 + lane * 4);
                v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
            } else {
                const uint2 xb = *reinterpret_cast<const uint2*>(static_cast<const __nv_bfloat16*>(xin) +
                                                                 (size_t)tok * in_dim + b * 128 + lane * 4);
                const uint2 sb = *reinterpret_cast<const uint2*>(scales + (size_t)e * scales_stride +
                                                                 (size_t)p * in_dim + b * 128 + lane * 4);
                const float x0 = __uint_as_float(xb.x << 16), x1 = __uint_as_float(xb.x & 0xFFFF0000u);
                const float x2 = __uint_as_float(xb.y << 16), x3 = __uint_as_float(xb.y & 0xFFFF0000u);
                const float2 s01 = __half22float2(*reinterpret_cast<const __half2*>(&sb.x));
                const float2 s23 = __half22float2(*reinterpret_cast<const __half2*>(&sb.y));
                v[0] = x0 * s01.x; v[1] = x1 * s01.y; v[2] = x2 * s23.x; v[3] = x3 * s23.y;
                hadamard128_warp(v, lane);
                v[0] *= S; v[1] *= S; v[2] *= S; v[3] *= S;
            }
        }
        store_frag4(dst + (size_t)b * 8 * A_TILE_WORDS, row, lane, v);
    }
}

}  // namespace mlxs
