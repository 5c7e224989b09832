// Device code of the FP4 streaming lane's row staging (shared by the prep kernel and the fused front kernel).
#pragma once
#include "common.cuh"
#include "kernels.h"

namespace mlxs {

constexpr int F4_XA_SB_WORDS = 128;  // one chunk x one 32-block of activations: 32 lanes x 4 u32

// One row of a chunk (row slot `slot` of 8): bf16 -> f16, 8 consecutive inputs per step, idx = idx0, idx0 + stride, ...
// (block sb = idx / 4, word c = idx % 4); the four u32 of a lane hold the inputs in natural order.
__device__ __forceinline__ void fp4_prep_row(const __nv_bfloat16* __restrict__ x, uint32_t tok, bool valid, uint32_t H,
                                             uint32_t chunk, uint32_t slot, uint32_t idx0, uint32_t stride,
                                             uint32_t* __restrict__ xa) {
    for (uint32_t idx = idx0; idx < H / 8; idx += stride) {
        uint4 raw = make_uint4(0, 0, 0, 0);
        if (valid) raw = *reinterpret_cast<const uint4*>(x + (size_t)tok * H + (size_t)idx * 8);
        const uint32_t wds[4] = {raw.x, raw.y, raw.z, raw.w};
        __half h[8];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            h[2 * i] = __float2half_rn(__uint_as_float(wds[i] << 16));
            h[2 * i + 1] = __float2half_rn(__uint_as_float(wds[i] & 0xFFFF0000u));
        }
        const uint32_t sb = idx / 4, c = idx % 4;
        uint4 o = make_uint4(pack_h2(h[0], h[1]), pack_h2(h[2], h[3]), pack_h2(h[4], h[5]), pack_h2(h[6], h[7]));
        *reinterpret_cast<uint4*>(xa + ((size_t)chunk * (H / 32) + sb) * F4_XA_SB_WORDS + (slot * 4 + c) * 4) = o;
    }
}

}  // namespace mlxs
