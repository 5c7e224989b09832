// An allocation-free EXL3 projection (K = 3 code planes only: 24 words per 16x16 tile): z = xh . W_hat for one code
// plane, with its scratch in a fixed device array.
//
// Who needs it: a host that settles its device-memory budget when the model loads and allows no device allocation
// afterwards, and any code that runs while a stream is being captured into a graph, where cudaMalloc is not allowed.
// Those callers cannot create a handle (mlxs_moe_create allocates the bank and the workspaces), so this entry takes
// only caller-owned buffers: the code plane as it sits in the bank file, the input rows and the output rows.
//
// The scratch (the rows rearranged into tensor-core fragment order, f16 hi / lo) lives in `g_scratch` below: 1 MiB
// that every device which loads this library keeps until the process exits.  All calls share it and it keeps the
// last call's contents: each call rewrites every word it later reads (padding rows are written as zeros), and two
// calls that overlap on the GPU (different streams) race on it; callers serialise them.
#include <cuda_runtime.h>

#include <mutex>

#include "../../include/mlxs_moe.h"
#include "common.cuh"

namespace mlxs {

constexpr uint32_t NA_MAX_ROWS = 32;    // rows per call
constexpr uint32_t NA_MAX_IN = 8192;    // input width
constexpr uint32_t NA_FRAG_WORDS = 64;  // one 4-row chunk x one 16-input tile: 32 lanes x 2 u32
constexpr size_t NA_SCRATCH_WORDS = (size_t)(NA_MAX_ROWS / 4) * (NA_MAX_IN / 16) * NA_FRAG_WORDS;  // 262,144 = 1 MiB

static __device__ __align__(256) uint32_t g_scratch[NA_SCRATCH_WORDS];

// rows -> fragment order: lane (g = token slot, c) of a (chunk, k-tile) block holds x[slot g][k 2c,2c+1] and
// x[slot g][k 2c+8,2c+9]; slots 0..3 are the f16 hi halves of the chunk's rows, slots 4..7 their lo halves
__global__ void __launch_bounds__(128) na_stage_kernel(const float* __restrict__ xh, uint32_t rows, uint32_t in_dim,
                                                       uint32_t* __restrict__ xa) {
    const uint32_t chunk = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t r = chunk * 4 + warp, nkt = in_dim / 16;
    const bool valid = r < rows;
    for (uint32_t b = blockIdx.y; b < in_dim / 128; b += gridDim.y) {
        float v[4] = {0.f, 0.f, 0.f, 0.f};  // padding rows are staged as zeros: nothing stale is ever read
        if (valid) {
            const float4 f = *reinterpret_cast<const float4*>(xh + (size_t)r * in_dim + b * 128 + lane * 4);
            v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
        }
        const uint32_t cq = lane & 3u, c0 = 2u * (cq & 1u), reg = cq >> 1;
        uint32_t* kt = xa + ((size_t)chunk * nkt + b * 8 + (lane >> 2)) * NA_FRAG_WORDS;
        __half h0, l0, h1, l1, h2, l2, h3, l3;
        split_hi_lo(v[0], h0, l0); split_hi_lo(v[1], h1, l1); split_hi_lo(v[2], h2, l2); split_hi_lo(v[3], h3, l3);
        kt[(warp * 4u + c0) * 2u + reg] = pack_h2(h0, h1);
        kt[((warp + 4u) * 4u + c0) * 2u + reg] = pack_h2(l0, l1);
        kt[(warp * 4u + c0 + 1u) * 2u + reg] = pack_h2(h2, h3);
        kt[((warp + 4u) * 4u + c0 + 1u) * 2u + reg] = pack_h2(l2, l3);
    }
}

// one warp = one 16-column tile of the output for one 4-row chunk; code in the bank file's order
// [in/16][out/16][24 u32] (src/expert/bank.zig:116-118)
__global__ void __launch_bounds__(128) na_gemv_kernel(const uint32_t* __restrict__ code, uint32_t in_dim,
                                                      uint32_t out_dim, const uint32_t* __restrict__ xa, uint32_t rows,
                                                      float* __restrict__ z) {
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t tn = blockIdx.x * 4 + warp, chunk = blockIdx.y, nkt = in_dim / 16, ntn = out_dim / 16;
    if (tn >= ntn) return;
    uint32_t wi, wj, lp;
    exl3_lane_plan(lane, wi, wj, lp);
    const uint2* xv = reinterpret_cast<const uint2*>(xa + (size_t)chunk * nkt * NA_FRAG_WORDS) + lane;
    // the sum over the inputs in the same equal parts, folded left, as the handle's streaming kernel takes it (4 parts
    // when the k-tiles divide by 32, else 2 by 16, else one): the two entries then agree bit for bit
    const uint32_t parts = nkt % 32 == 0 ? 4u : (nkt % 16 == 0 ? 2u : 1u), part_kt = nkt / parts;
    const uint32_t g = lane >> 2, c = lane & 3u;
    float v[4] = {0.f, 0.f, 0.f, 0.f};
    for (uint32_t part = 0; part < parts; ++part) {
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        for (uint32_t kt = part * part_kt; kt < (part + 1) * part_kt; ++kt) {
            const uint32_t* tile = code + ((size_t)kt * ntn + tn) * 24;
            uint32_t b[4];
            exl3_decode_lane(tile[wi], tile[wj], lp, b);
            const uint32_t a[4] = {b[0], b[2], b[1], b[3]};
            const uint2 x2 = xv[(size_t)kt * 32];
            mma_f16(acc, a, x2.x, x2.y);
        }
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const float pv = acc[q] + __shfl_xor_sync(0xFFFFFFFFu, acc[q], 2);
            v[q] = part == 0 ? pv : v[q] + pv;
        }
    }
    if (c < 2) {
        const uint32_t r0 = chunk * 4 + 2 * c;
        if (r0 < rows) {
            z[(size_t)r0 * out_dim + tn * 16 + g] = v[0];
            z[(size_t)r0 * out_dim + tn * 16 + g + 8] = v[2];
        }
        if (r0 + 1 < rows) {
            z[(size_t)(r0 + 1) * out_dim + tn * 16 + g] = v[1];
            z[(size_t)(r0 + 1) * out_dim + tn * 16 + g + 8] = v[3];
        }
    }
}

}  // namespace mlxs

// in api.cu
int mlxs_fail(int rc, const char* fmt, ...);

// Set-up, once per device, with that device current: the array's name is only a host-side handle, the kernels need
// its device address.
static int scratch_address(uint32_t** out) {
    static std::mutex mu;
    static uint32_t* ptrs[64] = {nullptr};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return mlxs_fail(MLXS_E_CUDA, "exl3_gemv_noalloc: cudaGetDevice: %s", cudaGetErrorString(e));
    if (dev < 0 || dev >= 64) return mlxs_fail(MLXS_E_ARG, "exl3_gemv_noalloc: device ordinal %d not supported", dev);
    std::lock_guard<std::mutex> lk(mu);
    if (!ptrs[dev]) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, mlxs::g_scratch);
        if (e != cudaSuccess || !p)
            return mlxs_fail(MLXS_E_CUDA, "exl3_gemv_noalloc: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
        ptrs[dev] = static_cast<uint32_t*>(p);
    }
    *out = ptrs[dev];
    return MLXS_OK;
}

extern "C" int mlxs_moe_exl3_gemv_noalloc(const void* code_dev, uint32_t in_dim, uint32_t out_dim, const float* xh_dev,
                                          uint32_t rows, float* z_dev, void* stream) {
    using namespace mlxs;
    if (!code_dev || !xh_dev || !z_dev) return mlxs_fail(MLXS_E_ARG, "exl3_gemv_noalloc: null buffer");
    if (rows > NA_MAX_ROWS)
        return mlxs_fail(MLXS_E_TOO_MANY_TOKENS, "exl3_gemv_noalloc: %u rows, the fixed scratch holds %u", rows, NA_MAX_ROWS);
    if (in_dim == 0 || in_dim % 128 || in_dim > NA_MAX_IN)
        return mlxs_fail(MLXS_E_ARG, "exl3_gemv_noalloc: in_dim %u must be a multiple of 128 up to %u", in_dim, NA_MAX_IN);
    if (out_dim == 0 || out_dim % 16) return mlxs_fail(MLXS_E_ARG, "exl3_gemv_noalloc: out_dim %u must be a multiple of 16", out_dim);
    // the staging kernel reads the rows as 16-byte vectors (row offsets are multiples of 512 bytes, so only the base
    // matters); code and output are read and written as 4-byte words
    if (reinterpret_cast<uintptr_t>(xh_dev) & 15u)
        return mlxs_fail(MLXS_E_ARG, "exl3_gemv_noalloc: xh_dev must be 16-byte aligned");
    if (reinterpret_cast<uintptr_t>(code_dev) & 3u)
        return mlxs_fail(MLXS_E_ARG, "exl3_gemv_noalloc: code_dev must be 4-byte aligned");
    if (reinterpret_cast<uintptr_t>(z_dev) & 3u)
        return mlxs_fail(MLXS_E_ARG, "exl3_gemv_noalloc: z_dev must be 4-byte aligned");
    if (rows == 0) return MLXS_OK;
    uint32_t* scratch = nullptr;
    int rc = scratch_address(&scratch);
    if (rc) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    const uint32_t chunks = (rows + 3) / 4;
    na_stage_kernel<<<dim3(chunks, 8), 128, 0, st>>>(xh_dev, rows, in_dim, scratch);
    na_gemv_kernel<<<dim3((out_dim / 16 + 3) / 4, chunks), 128, 0, st>>>(static_cast<const uint32_t*>(code_dev), in_dim,
                                                                        out_dim, scratch, rows, z_dev);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return mlxs_fail(MLXS_E_CUDA, "exl3_gemv_noalloc: launch: %s", cudaGetErrorString(e));
    return MLXS_OK;
}
