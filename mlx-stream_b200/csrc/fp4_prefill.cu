// MXFP4 / NVFP4 expert kernels for experts with many rows: tcgen05 tensor cores over codes decoded in shared memory.
//
// The reference sends prefill-sized FP4 work to a grouped quantised GEMM over rows sorted by expert
// (src/arch/mimo_v2/math.zig:426-447, src/arch/glm5_next/nvfp4.zig:36-56): bf16 rows times dequantised weights, f32
// accumulate.  Here a CTA owns (expert, up to 128 of its rows, 256 output columns of gate and up | 512 of down).  W^T
// is the MMA's A operand (M = 128 output columns per accumulator group), the rows are the B operand (N = rows rounded
// to 16), four accumulator groups fill the SM's tensor memory, and one staged copy of the rows serves all four groups
// (gate and up read the same rows).
//   * a producer thread streams the same repacked code/scale stream the decode-batch kernel reads (bulk copies, one
//     stage = 128 inputs of a 128-column block) and the rows, which a prep kernel laid out in the core-matrix order;
//   * 16 decode warps turn codes into 16-bit operands, two codes per integer op
//     (src/arch/mimo_v2/kernels/header_mimo_moe_k1.metal:7-12), 8 weights of one output column per 16-byte store, which
//     is exactly one row of a K-major core matrix.  The k order inside a group of 8 is the decode's (0,4,1,5,2,6,3,7)
//     and the prep kernel stores the rows in the same order;
//   * MXFP4: operands are bf16.  The code's 3 magnitude bits placed at bits 6..8 are e2m1 x 2^-126 as bf16 (the 0.5
//     code is a bf16 subnormal); one bf16x2 multiply by 2^(b-1) gives e2m1 x 2^(b-127) exactly, and the rows stay the
//     bf16 they arrived as, so every product is exact.  This needs 2^(b-1) to be a bf16, b <= 128 (block scale <= 2):
//     an expert with a larger scale byte is marked at load and always takes the streaming lane;
//   * NVFP4: operands are f16, weights e2m1 x 2^-14 times the block's E4M3 scale (exact in f16, as in the streaming
//     lane), rows rounded bf16 -> f16, the global g/2688 x 2^14 applied in the epilogue (decode_kernels_ref.zig:13-65);
//   * one thread issues tcgen05.mma.kind::f16 (K = 16) and commits to mbarriers; the decode warps run the epilogue
//     straight from tensor memory (a thread owns one output column of 16 rows): the reference's bf16 rounding chain
//     for gate/up (mimo_moe_k1_gateup.metal:115-128, glm5n_nvfp4_gateup.metal:109-129), stores for down.
// Every wait is bounded; on a give-up the CTA sets the status word, skips work and still frees its tensor memory.
#include <cstdlib>

#include "common.cuh"
#include "kernels.h"
#include "umma.cuh"

namespace mlxs {

constexpr int Q_NT = PREFILL_TILE_ROWS;       // rows per tile (MMA N, rounded up to 16 per item)
constexpr int Q_KS = 128;                     // inputs per raw stage (the stream's stage)
constexpr int Q_SB = 32;                      // inputs per operand stage
constexpr int Q_RAW_STAGES = 2;
constexpr int Q_A_STAGES = 2;
constexpr int Q_B_STAGES = 4;
constexpr int Q_NG = 4;                       // accumulator groups
constexpr int Q_LBO_A = 16 * 128 + 32;        // K-direction distance of A core matrices; + 32 B keeps the 16-byte stores
                                              // of a quarter warp (2 columns x 4 k-groups) on distinct banks
constexpr int Q_A_BYTES = 4 * Q_LBO_A;        // one group's 128 columns x 32 inputs
constexpr int Q_LBO_B = (Q_NT / 8) * 128;     // 2048
constexpr int Q_B_BYTES = 4 * Q_LBO_B;        // 128 rows x 32 inputs: 8 KB
constexpr int Q_SBO = 128;
constexpr int Q_W_STAGE = 8192;               // code bytes per projection per raw stage (fp4.cu F4_W_STAGE)

__host__ __device__ inline uint32_t q_scale_stage_bytes(bool nv) { return nv ? 1024u : 512u; }
// position of input k % 8 inside its 16-byte group: the order the two-codes-per-op decode produces
__host__ __device__ inline uint32_t q_pos8(uint32_t j) { return (j & 3u) * 2u + (j >> 2); }
// element offset of (row, k) inside a tile's operand: [k/32][(k%32)/8][row/8][row%8][pos]
__device__ __forceinline__ size_t q_b_off(uint32_t row, uint32_t k) {
    return (size_t)(k / Q_SB) * (Q_B_BYTES / 2) + ((k % Q_SB) / 8) * (Q_LBO_B / 2) + (row / 8) * 64 + (row % 8) * 8 + q_pos8(k % 8);
}

// ------------------------------------------------------------------------------------------------------------
// prep: gather the tile's rows into the B-operand order (bf16 kept for MXFP4, rounded to f16 for NVFP4)
// ------------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) q_prep_kernel(const __nv_bfloat16* __restrict__ x, uint32_t top_k, uint32_t H, int nv,
                                                     DispatchTables t, const uint32_t* __restrict__ tiles,
                                                     uint16_t* __restrict__ xa) {
    const uint32_t tile = blockIdx.x;
    if (tile >= tiles[0]) return;
    const uint32_t row0 = tiles[2 + 3 * tile], rows = tiles[3 + 3 * tile];
    const uint32_t rows16 = (rows + 15) / 16 * 16, groups = H / 8;
    uint16_t* dst = xa + (size_t)tile * Q_NT * H;
    // a thread moves 8 consecutive inputs of one row; consecutive threads take consecutive rows (one core matrix = 128 B)
    for (uint32_t i = blockIdx.y * blockDim.x + threadIdx.x; i < rows16 * groups; i += gridDim.y * blockDim.x) {
        const uint32_t r = i % rows16, kg = i / rows16;
        uint4 raw = make_uint4(0, 0, 0, 0);
        if (r < rows) raw = *reinterpret_cast<const uint4*>(x + (size_t)(t.order[row0 + r] / top_k) * H + (size_t)kg * 8);
        const uint32_t wds[4] = {raw.x, raw.y, raw.z, raw.w};
        uint16_t e[8];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            if (nv) {
                e[2 * q] = __half_as_ushort(__float2half_rn(__uint_as_float(wds[q] << 16)));
                e[2 * q + 1] = __half_as_ushort(__float2half_rn(__uint_as_float(wds[q] & 0xFFFF0000u)));
            } else {
                e[2 * q] = (uint16_t)(wds[q] & 0xFFFFu);
                e[2 * q + 1] = (uint16_t)(wds[q] >> 16);
            }
        }
        // stored order 0,4,1,5,2,6,3,7
        const uint4 o = make_uint4(e[0] | ((uint32_t)e[4] << 16), e[1] | ((uint32_t)e[5] << 16), e[2] | ((uint32_t)e[6] << 16),
                                   e[3] | ((uint32_t)e[7] << 16));
        *reinterpret_cast<uint4*>(dst + q_b_off(r, kg * 8)) = o;
    }
}

// ------------------------------------------------------------------------------------------------------------
// the kernel
// ------------------------------------------------------------------------------------------------------------
struct QParams {
    const uint8_t* w;            // layer base of the gate/up or down stream
    size_t expert_stride;
    const float* gscale;         // NVFP4: [E][3]
    uint32_t n_blocks, n_stages_k;  // out / 128, in / 128
    uint32_t w_bytes;            // bytes of one (block, stage) of the stream
    const uint16_t* xa;          // B operand: [tile][in/32][8 KB]
    const uint32_t* tiles;
    DispatchTables t;
    uint32_t H, I;
    uint16_t* xd;                // gate/up output = down's B operand
    void* out;                   // down: ro [A, H] bf16 (chain) or f32
    int out_bf16;
    float limit;
    uint32_t* status;
};

// MXFP4: 8 codes of a word -> 4 bf16x2 of e2m1 x 2^-126 (pairs (0,4), (1,5), (2,6), (3,7))
__device__ __forceinline__ void q_decode8_bf16(uint32_t w, uint32_t (&h)[4]) {
    h[0] = ((w << 6) & 0x01C001C0u) | ((w << 12) & 0x80008000u);
    h[1] = ((w << 2) & 0x01C001C0u) | ((w << 8) & 0x80008000u);
    h[2] = ((w >> 2) & 0x01C001C0u) | ((w << 4) & 0x80008000u);
    h[3] = ((w >> 6) & 0x01C001C0u) | (w & 0x80008000u);
}
// NVFP4: the same to f16x2 of e2m1 x 2^-14
__device__ __forceinline__ void q_decode8_f16(uint32_t w, uint32_t (&h)[4]) {
    h[0] = ((w << 9) & 0x0E000E00u) | ((w << 12) & 0x80008000u);
    h[1] = ((w << 5) & 0x0E000E00u) | ((w << 8) & 0x80008000u);
    h[2] = ((w << 1) & 0x0E000E00u) | ((w << 4) & 0x80008000u);
    h[3] = ((w >> 3) & 0x0E000E00u) | (w & 0x80008000u);
}
__device__ __forceinline__ uint32_t q_mul_bf16x2(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}
__device__ __forceinline__ uint32_t q_mul_f16x2(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}
// E4M3 byte -> f16x2 (both halves) of its value: bits << 7 is the value x 2^-8 as f16, x 256 is exact
__device__ __forceinline__ uint32_t q_e4m3_f16x2(uint32_t b) {
    const uint32_t v = b & 127u;
    const uint32_t u = (v << 7) | (((v + 1u) >> 7) << 14) | ((b & 128u) << 8);
    return q_mul_f16x2(u * 0x00010001u, 0x5C005C00u);
}
__device__ __forceinline__ float q_sigmoid(float x) {  // src/arch/mimo_v2/moe.zig:341-344
    const float y = 1.0f / (1.0f + expf(fabsf(x)));
    return x < 0.f ? y : 1.0f - y;
}

// NPROJ projections x CB adjacent 128-column blocks = 4 accumulator groups of 128 tensor-memory columns
template <int NPROJ, int CB, bool NV>
__global__ void __launch_bounds__(512 + 64, 1) fp4_prefill_kernel(const QParams P) {
    static_assert(NPROJ * CB == Q_NG, "four accumulator groups fill the 512 tensor-memory columns at 128 rows");
    extern __shared__ __align__(128) uint8_t smem_raw[];
    constexpr int NCW = 16;
    constexpr int TMEM_COLS = Q_NG * Q_NT;
    constexpr uint32_t SSTAGE = NV ? 1024u : 512u;
    constexpr uint32_t W_BYTES = NPROJ * (Q_W_STAGE + SSTAGE);   // one block's stage of the stream
    constexpr uint32_t RAW_BYTES = CB * W_BYTES;
    __shared__ __align__(8) uint64_t raw_full[Q_RAW_STAGES], raw_empty[Q_RAW_STAGES];
    __shared__ __align__(8) uint64_t b_full[Q_B_STAGES], b_empty[Q_B_STAGES], a_full[Q_A_STAGES], a_empty[Q_A_STAGES];
    __shared__ __align__(8) uint64_t acc_full, acc_empty;
    __shared__ uint32_t s_tmem;
    __shared__ volatile int s_abort;
    uint8_t* a_ring = smem_raw;                                        // [stage][group][Q_A_BYTES]
    uint8_t* b_ring = a_ring + Q_A_STAGES * Q_NG * Q_A_BYTES;          // [stage][Q_B_BYTES]
    uint8_t* raw_ring = b_ring + Q_B_STAGES * Q_B_BYTES;               // [stage][CB][W_BYTES]
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t nbg = P.n_blocks / CB;
    // a CTA without work leaves before it takes tensor memory (the whole CTA reads the same count)
    if (blockIdx.x >= P.tiles[0] * nbg) return;

    if (threadIdx.x == 0) {
        for (int s = 0; s < Q_RAW_STAGES; ++s) { mbar_init(&raw_full[s], 1); mbar_init(&raw_empty[s], NCW); }
        for (int s = 0; s < Q_A_STAGES; ++s) { mbar_init(&a_full[s], NCW); mbar_init(&a_empty[s], 1); }
        for (int s = 0; s < Q_B_STAGES; ++s) { mbar_init(&b_full[s], 1); mbar_init(&b_empty[s], 1); }
        mbar_init(&acc_full, 1);
        mbar_init(&acc_empty, NCW);
        s_abort = 0;
        mbar_fence_init();
    }
    if (warp == 0) tmem_alloc(&s_tmem, TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = s_tmem;
    const uint32_t n_items = P.tiles[0] * nbg;
    const uint32_t nstage = P.n_stages_k;
    auto give_up = [&](uint32_t code) { if (!s_abort) atomicMax(P.status, code); s_abort = 1; };

    if (warp == NCW) {
        // ---------------- producer: code/scale stream + rows ----------------
        if (lane == 0) {
            uint32_t rit = 0, bit = 0;
            for (uint32_t item = blockIdx.x; item < n_items && !s_abort; item += gridDim.x) {
                const uint32_t tile = item / nbg, nb0 = (item % nbg) * CB, expert = P.tiles[1 + 3 * tile];
                const uint8_t* wsrc = P.w + (size_t)expert * P.expert_stride + (size_t)nb0 * nstage * W_BYTES;
                const uint16_t* xsrc = P.xa + (size_t)tile * Q_NT * (nstage * Q_KS);
                bool ok = true;
                for (uint32_t ks = 0; ks < nstage && ok; ++ks, ++rit) {
                    const uint32_t rs = rit % Q_RAW_STAGES, rph = (rit / Q_RAW_STAGES) & 1u;
                    if (!mbar_wait_bounded(&raw_empty[rs], rph ^ 1u, &s_abort, 128)) { give_up(ST_WAIT_EMPTY); ok = false; break; }
                    mbar_expect_tx(&raw_full[rs], RAW_BYTES);
                    for (int cb = 0; cb < CB; ++cb)
                        bulk_g2s(raw_ring + rs * RAW_BYTES + cb * W_BYTES, wsrc + ((size_t)cb * nstage + ks) * W_BYTES, W_BYTES,
                                 &raw_full[rs]);
                    for (uint32_t sb = 0; sb < Q_KS / Q_SB; ++sb, ++bit) {
                        const uint32_t bs = bit % Q_B_STAGES, bph = (bit / Q_B_STAGES) & 1u;
                        if (!mbar_wait_bounded(&b_empty[bs], bph ^ 1u, &s_abort, 128)) { give_up(ST_WAIT_EMPTY); ok = false; break; }
                        mbar_expect_tx(&b_full[bs], Q_B_BYTES);
                        bulk_g2s(b_ring + bs * Q_B_BYTES, xsrc + (size_t)(ks * (Q_KS / Q_SB) + sb) * (Q_B_BYTES / 2), Q_B_BYTES,
                                 &b_full[bs]);
                    }
                }
                if (!ok) break;
            }
            if (s_abort) for (int i = 0; i < 2000; ++i) __nanosleep(1000);
        }
    } else if (warp == NCW + 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            uint32_t bit = 0, nitem = 0;
            for (uint32_t item = blockIdx.x; item < n_items && !s_abort; item += gridDim.x, ++nitem) {
                const uint32_t tile = item / nbg, rows = P.tiles[3 + 3 * tile];
                const uint32_t idesc = umma_idesc(NV ? UMMA_F16 : UMMA_BF16, (rows + 15) / 16 * 16);
                if (!mbar_wait_bounded(&acc_empty, (nitem & 1u) ^ 1u, &s_abort, 64)) { give_up(ST_WAIT_EMPTY); break; }
                tc_fence_after();
                bool ok = true;
                for (uint32_t kk = 0; kk < nstage * (Q_KS / Q_SB); ++kk, ++bit) {
                    const uint32_t as = bit % Q_A_STAGES, aph = (bit / Q_A_STAGES) & 1u;
                    const uint32_t bs = bit % Q_B_STAGES, bph = (bit / Q_B_STAGES) & 1u;
                    if (!mbar_wait_bounded(&a_full[as], aph, &s_abort, 32) || !mbar_wait_bounded(&b_full[bs], bph, &s_abort, 32)) {
                        give_up(ST_WAIT_FULL); ok = false; break;
                    }
                    tc_fence_after();
                    const uint32_t b0 = smem_u32(b_ring + bs * Q_B_BYTES);
#pragma unroll
                    for (int gq = 0; gq < Q_NG; ++gq) {
                        const uint32_t a0 = smem_u32(a_ring + (as * Q_NG + gq) * Q_A_BYTES);
#pragma unroll
                        for (int i = 0; i < Q_SB / 16; ++i)
                            umma_f16(tmem + gq * Q_NT, umma_smem_desc(a0 + i * 2 * Q_LBO_A, Q_LBO_A, Q_SBO),
                                     umma_smem_desc(b0 + i * 2 * Q_LBO_B, Q_LBO_B, Q_SBO), idesc, (kk | (uint32_t)i) ? 1u : 0u);
                    }
                    umma_commit(&a_empty[as]);
                    umma_commit(&b_empty[bs]);
                }
                if (!ok) break;
                umma_commit(&acc_full);
            }
        }
    } else {
        // ---------------- decode warps + epilogue ----------------
        // a warp owns 16 output columns (j) of two accumulator groups: gate/up: projection hi, both column blocks;
        // down: column blocks 2 hi and 2 hi + 1
        const uint32_t hi = warp >> 3, j = warp & 7u, g = lane >> 2, c = lane & 3u;
        uint32_t rit = 0, nitem = 0;
        for (uint32_t item = blockIdx.x; item < n_items && !s_abort; item += gridDim.x, ++nitem) {
            const uint32_t tile = item / nbg, nb0 = (item % nbg) * CB;
            const uint32_t expert = P.tiles[1 + 3 * tile], row0 = P.tiles[2 + 3 * tile], rows = P.tiles[3 + 3 * tile];
            bool ok = true;
            for (uint32_t ks = 0; ks < nstage && ok; ++ks, ++rit) {
                const uint32_t rs = rit % Q_RAW_STAGES, rph = (rit / Q_RAW_STAGES) & 1u;
                if (!mbar_wait_bounded(&raw_full[rs], rph, &s_abort)) { give_up(ST_WAIT_FULL); ok = false; break; }
                const uint8_t* raw = raw_ring + rs * RAW_BYTES;
#pragma unroll
                for (int sb = 0; sb < Q_KS / Q_SB; ++sb) {
                    // 4 operand stages per raw stage and an even ring: stage and parity are compile-time
                    const uint32_t as = sb % Q_A_STAGES, aph = (sb / Q_A_STAGES) & 1u;
                    if (!mbar_wait_bounded(&a_empty[as], aph ^ 1u, &s_abort)) { give_up(ST_WAIT_FULL); ok = false; break; }
#pragma unroll
                    for (int u = 0; u < 2; ++u) {
                        const uint32_t cb = NPROJ == 2 ? (uint32_t)u : 2u * hi + u, p = NPROJ == 2 ? hi : 0u;
                        const uint32_t gq = NPROJ == 2 ? hi * CB + u : cb;
                        const uint8_t* blk = raw + cb * W_BYTES;
                        const uint2 ww = *(reinterpret_cast<const uint2*>(blk + p * Q_W_STAGE) + (j * 4 + sb) * 32 + lane);
                        const uint8_t* sc = blk + NPROJ * Q_W_STAGE + p * SSTAGE;
                        uint32_t hx[4], hy[4];
                        if (NV) {
                            const uint32_t bb = *reinterpret_cast<const uint16_t*>(sc + (((j * 4 + sb) * 2 + (c >> 1)) * 8 + g) * 2);
                            const uint32_t s0 = q_e4m3_f16x2(bb & 0xFFu), s1 = q_e4m3_f16x2(bb >> 8);
                            q_decode8_f16(ww.x, hx);
                            q_decode8_f16(ww.y, hy);
#pragma unroll
                            for (int i = 0; i < 4; ++i) { hx[i] = q_mul_f16x2(hx[i], s0); hy[i] = q_mul_f16x2(hy[i], s1); }
                        } else {
                            const uint32_t bb = *reinterpret_cast<const uint16_t*>(sc + ((j * 4 + sb) * 8 + g) * 2);
                            const uint32_t s0 = (((bb & 0xFFu) + 126u) << 7) * 0x00010001u;   // 2^(b - 1) in both halves
                            const uint32_t s1 = (((bb >> 8) + 126u) << 7) * 0x00010001u;
                            q_decode8_bf16(ww.x, hx);
                            q_decode8_bf16(ww.y, hy);
#pragma unroll
                            for (int i = 0; i < 4; ++i) { hx[i] = q_mul_bf16x2(hx[i], s0); hy[i] = q_mul_bf16x2(hy[i], s1); }
                        }
                        // columns 16 j + g and 16 j + g + 8 are row g of core matrices 2 j and 2 j + 1; k-group c
                        uint8_t* ad = a_ring + (as * Q_NG + gq) * Q_A_BYTES + c * Q_LBO_A + (2 * j) * Q_SBO + g * 16;
                        *reinterpret_cast<uint4*>(ad) = make_uint4(hx[0], hx[1], hx[2], hx[3]);
                        *reinterpret_cast<uint4*>(ad + Q_SBO) = make_uint4(hy[0], hy[1], hy[2], hy[3]);
                    }
                    fence_async_smem();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&a_full[as]);
                }
                if (!ok) break;
                __syncwarp();
                if (lane == 0) mbar_arrive(&raw_empty[rs]);
            }
            if (!ok) break;
            // ---- epilogue: a thread owns output column 32 q + lane of a group, 16 rows per tensor-memory load ----
            if (!mbar_wait_bounded(&acc_full, nitem & 1u, &s_abort)) { give_up(ST_WAIT_FULL); break; }
            tc_fence_after();
            const uint32_t q = warp & 3u, sub = warp >> 2;
            const uint32_t rows16 = (rows + 15) / 16 * 16, nrb = rows16 / 16;
            if (NPROJ == 2) {
                float gs_g = 1.f, gs_u = 1.f;
                if (NV) {
                    gs_g = (P.gscale[expert * 3 + 0] / 2688.0f) * 16384.0f;
                    gs_u = (P.gscale[expert * 3 + 1] / 2688.0f) * 16384.0f;
                }
                uint16_t* xd_tile = P.xd + (size_t)tile * Q_NT * P.I;
                for (uint32_t unit = sub; unit < CB * nrb; unit += 4) {
                    const uint32_t cb = unit / nrb, rb = (unit % nrb) * 16;
                    uint32_t vg[16], vu[16];
                    tmem_ld16(tmem + ((q * 32u) << 16) + (0 * CB + cb) * Q_NT + rb, vg);
                    tmem_ld16(tmem + ((q * 32u) << 16) + (1 * CB + cb) * Q_NT + rb, vu);
                    const uint32_t col = (nb0 + cb) * 128 + q * 32 + lane;
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        // mimo_moe_k1_gateup.metal:115-128 / glm5n_nvfp4_gateup.metal:109-129
                        float gf = bf16_round_f(__uint_as_float(vg[i]) * gs_g), uf = bf16_round_f(__uint_as_float(vu[i]) * gs_u);
                        if (P.limit > 0.f) {
                            gf = gf > P.limit ? P.limit : gf;
                            uf = uf > P.limit ? P.limit : (uf < -P.limit ? -P.limit : uf);
                        }
                        const float hq = bf16_round_f(bf16_round_f(gf * q_sigmoid(gf)) * uf);
                        const uint32_t r = rb + i;
                        uint16_t bits = 0;
                        if (r < rows) bits = NV ? __half_as_ushort(__float2half_rn(hq)) : (uint16_t)(__float_as_uint(hq) >> 16);
                        xd_tile[q_b_off(r, col)] = bits;
                    }
                }
            } else {
                float gs = 1.f;
                if (NV) gs = (P.gscale[expert * 3 + 2] / 2688.0f) * 16384.0f;
                for (uint32_t unit = sub; unit < CB * nrb; unit += 4) {
                    const uint32_t cb = unit / nrb, rb = (unit % nrb) * 16;
                    uint32_t v[16];
                    tmem_ld16(tmem + ((q * 32u) << 16) + cb * Q_NT + rb, v);
                    const uint32_t col = (nb0 + cb) * 128 + q * 32 + lane;
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        const uint32_t r = rb + i;
                        if (r >= rows) continue;
                        const uint32_t assign = P.t.order[row0 + r];
                        const float z = __uint_as_float(v[i]) * gs;
                        if (P.out_bf16) static_cast<__nv_bfloat16*>(P.out)[(size_t)assign * P.H + col] = __float2bfloat16_rn(z);
                        else static_cast<float*>(P.out)[(size_t)assign * P.H + col] = z;
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty);
        }
    }
    // every thread comes here, also after a give-up: the tensor memory is always released
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (warp == 0) tmem_free(tmem, TMEM_COLS);
}

static size_t q_smem_bytes(int nproj, int cb, bool nv) {
    return (size_t)Q_A_STAGES * Q_NG * Q_A_BYTES + (size_t)Q_B_STAGES * Q_B_BYTES +
           (size_t)Q_RAW_STAGES * cb * nproj * (Q_W_STAGE + q_scale_stage_bytes(nv));
}

bool fp4_prefill_supported(uint32_t H, uint32_t I) { return H % 128 == 0 && I % 128 == 0 && (I / 128) % 2 == 0 && (H / 128) % 4 == 0; }

template <int NPROJ, int CB, bool NV>
static cudaError_t q_launch(const QParams& P, int sm_count, cudaStream_t st) {
    const size_t smem = q_smem_bytes(NPROJ, CB, NV);
    cudaError_t e = cudaFuncSetAttribute(fp4_prefill_kernel<NPROJ, CB, NV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    fp4_prefill_kernel<NPROJ, CB, NV><<<sm_count, 512 + 64, smem, st>>>(P);
    return cudaGetLastError();
}

cudaError_t launch_fp4_prefill(const Fp4PrefillArgs& a, cudaStream_t st) {
    cudaError_t e = launch_prefill_plan(a.t, a.n_experts, a.lane_flags, a.min_rows, a.max_tiles, a.tiles, a.status, st);
    if (e != cudaSuccess) return e;
    q_prep_kernel<<<dim3(a.max_tiles, 8), 256, 0, st>>>(a.x, a.top_k, a.H, a.nv, a.t, a.tiles, a.xa);
    if ((e = cudaGetLastError()) != cudaSuccess) return e;
    const uint32_t sstage = q_scale_stage_bytes(a.nv != 0);
    QParams P{};
    P.gscale = a.gscale; P.tiles = a.tiles; P.t = a.t; P.H = a.H; P.I = a.I; P.limit = a.limit; P.status = a.status;
    // gate / up: two projections x two adjacent column blocks per CTA, one copy of the rows
    P.w = a.gu; P.w_bytes = 2 * (Q_W_STAGE + sstage); P.n_blocks = a.I / 128; P.n_stages_k = a.H / Q_KS;
    P.expert_stride = (size_t)P.n_blocks * P.n_stages_k * P.w_bytes;
    P.xa = a.xa; P.xd = a.xd; P.out = nullptr; P.out_bf16 = 0;
    e = a.nv ? q_launch<2, 2, true>(P, a.sm_count, st) : q_launch<2, 2, false>(P, a.sm_count, st);
    if (e != cudaSuccess) return e;
    // down: four adjacent column blocks per CTA
    P.w = a.dn; P.w_bytes = Q_W_STAGE + sstage; P.n_blocks = a.H / 128; P.n_stages_k = a.I / Q_KS;
    P.expert_stride = (size_t)P.n_blocks * P.n_stages_k * P.w_bytes;
    P.xa = a.xd; P.xd = nullptr; P.out = a.ro; P.out_bf16 = a.ro_bf16;
    return a.nv ? q_launch<1, 4, true>(P, a.sm_count, st) : q_launch<1, 4, false>(P, a.sm_count, st);
}

}  // namespace mlxs
