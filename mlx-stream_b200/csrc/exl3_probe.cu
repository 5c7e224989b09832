// Measured ceiling of the EXL3 in-register decode: the streaming kernel's decode statements alone, fed from registers
// (no global or shared loads, no barriers), with or without the one mma per tile.  Every consumer warp of the real
// kernel spends its issue slots on exactly these statements, so tiles per second here x bytes per tile is the rate of
// code the decode can consume on this GPU, whatever the memory system delivers.
#include <cuda_runtime.h>

#include "../../include/mlxs_moe.h"
#include "common.cuh"

int mlxs_fail(int rc, const char* fmt, ...);

namespace mlxs {

// One warp decodes `tiles` 16x16 tiles.  The two code words of a lane evolve by a cheap recurrence that does not
// depend on the decode's result (so the compiler can neither hoist nor fold the decode), the decoded fragments are
// folded into a checksum that is stored once.
template <int KB, bool MMA>
__global__ void __launch_bounds__(512, 2) exl3_decode_probe_kernel(uint32_t tiles, uint32_t seed, uint32_t* __restrict__ sink) {
    const uint32_t lane = threadIdx.x & 31u;
    uint32_t wi, wj, lp;
    exl3_lane_plan_kb<KB>(lane, wi, wj, lp);
    uint32_t lo = seed ^ (blockIdx.x * 2654435761u + threadIdx.x * 40503u), hi = lo * 747796405u + 2891336453u;
    uint32_t chk = 0;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    const uint32_t bx = lo | 0x3C003C00u, by = hi | 0x3C003C00u;   // stand-ins for the rows' fragment
#pragma unroll 8
    for (uint32_t t = 0; t < tiles; ++t) {
        uint32_t b[4];
        exl3_decode_lane_kb<KB>(lo, hi, lp, b);
        if (MMA) {
            const uint32_t a[4] = {b[0], b[2], b[1], b[3]};
            mma_f16(acc, a, bx, by);
        } else {
            chk ^= b[0] ^ b[1] ^ b[2] ^ b[3];
        }
        lo += 0x9E3779B9u;      // one add per word stands in for the two shared-memory loads of the real loop
        hi += 0x7F4A7C15u;
    }
    if (MMA) chk = __float_as_uint(acc[0]) ^ __float_as_uint(acc[1]) ^ __float_as_uint(acc[2]) ^ __float_as_uint(acc[3]);
    if (chk == 0x12345u) sink[0] = chk;   // practically never: keeps the loop alive
}

}  // namespace mlxs

extern "C" int mlxs_moe_exl3_decode_rate(int32_t device, uint32_t bits, int with_mma, uint32_t tiles_per_warp,
                                         double* tiles_per_s) {
    using namespace mlxs;
    if (!tiles_per_s) return mlxs_fail(MLXS_E_ARG, "exl3_decode_rate: null argument");
    if (bits != 2 && bits != 3) return mlxs_fail(MLXS_E_CONFIG, "exl3_decode_rate: K=%u not implemented (KNotImplemented)", bits);
    if (tiles_per_warp == 0 || tiles_per_warp > (1u << 24)) return mlxs_fail(MLXS_E_ARG, "exl3_decode_rate: tiles_per_warp out of range");
    cudaError_t e = cudaSetDevice(device);
    if (e != cudaSuccess) return mlxs_fail(MLXS_E_CUDA, "exl3_decode_rate: cudaSetDevice: %s", cudaGetErrorString(e));
    cudaDeviceProp prop;
    if ((e = cudaGetDeviceProperties(&prop, device)) != cudaSuccess)
        return mlxs_fail(MLXS_E_CUDA, "exl3_decode_rate: %s", cudaGetErrorString(e));
    uint32_t* sink = nullptr;
    if ((e = cudaMalloc(&sink, 16)) != cudaSuccess) return mlxs_fail(MLXS_E_CUDA, "exl3_decode_rate: cudaMalloc: %s", cudaGetErrorString(e));
    cudaEvent_t a, b;
    cudaEventCreate(&a);
    cudaEventCreate(&b);
    const int grid = 2 * prop.multiProcessorCount, threads = 512;   // the gate/up kernel's residency: 32 decode warps per SM
    auto launch = [&](uint32_t tiles) {
        if (bits == 3) {
            if (with_mma) exl3_decode_probe_kernel<3, true><<<grid, threads>>>(tiles, 1u, sink);
            else exl3_decode_probe_kernel<3, false><<<grid, threads>>>(tiles, 1u, sink);
        } else {
            if (with_mma) exl3_decode_probe_kernel<2, true><<<grid, threads>>>(tiles, 1u, sink);
            else exl3_decode_probe_kernel<2, false><<<grid, threads>>>(tiles, 1u, sink);
        }
    };
    launch(tiles_per_warp / 8 + 1);   // warm-up
    float best = 0.f;
    for (int rep = 0; rep < 3; ++rep) {
        cudaEventRecord(a, 0);
        launch(tiles_per_warp);
        cudaEventRecord(b, 0);
        if ((e = cudaEventSynchronize(b)) != cudaSuccess) break;
        float ms = 0.f;
        cudaEventElapsedTime(&ms, a, b);
        if (rep == 0 || ms < best) best = ms;
    }
    if (e == cudaSuccess) e = cudaGetLastError();
    cudaEventDestroy(a);
    cudaEventDestroy(b);
    cudaFree(sink);
    if (e != cudaSuccess) return mlxs_fail(MLXS_E_CUDA, "exl3_decode_rate: %s", cudaGetErrorString(e));
    const double warps = (double)grid * (threads / 32);
    *tiles_per_s = warps * (double)tiles_per_warp / ((double)best * 1e-3);
    return MLXS_OK;
}
