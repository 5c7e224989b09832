// EXL3 expert kernels for prefill-sized batches: tcgen05 tensor cores with the trellis decoded into shared memory.
//
// The reference's prefill lane (src/exl3/quant.zig:1040-1271; texts dsv41_prefill_dig_gemm_*_m128*.metal) decodes
// trellis tiles to f16 in threadgroup memory per K stage and feeds its MMA units with f16 rotated activations and an
// f32 accumulator.  Here the same roles map to Blackwell: a CTA owns (expert, 256 output columns of gate and up | 512
// of down, up to 128 of the expert's rows).  W^T is the MMA's A operand (M = 128 output columns per accumulator
// group) and the rows are the B operand (N = rows rounded to 16), so a ragged expert pads to 16 rows, not 128, and the
// four accumulator groups D[128 columns x rows] fill the SM's tensor memory (512 columns).  One staged copy of the rows
// serves all four groups: the rows, not the weights, are what travels most through L2 in this lane.
//   * a producer warp streams the raw code (bulk copies) and the rows' rotated f16 activations, which a prep kernel
//     laid out in global memory in the K-major core-matrix order the MMA reads, so a stage is one contiguous copy;
//   * decode warps (one per 16-column tile and projection) turn each 16x16 tile into f16 with the same in-register
//     decode as the decode-batch kernel and store it as K-major core matrices (no swizzle: a lane's four half2 land at
//     row*16 + 4c bytes of a 128-byte core matrix, conflict free), then fence to the async proxy;
//   * one thread issues tcgen05.mma.kind::f16 (K = 16 per instruction) and commits to mbarriers;
//   * the decode warps run the epilogue: tcgen05.ld, transpose through shared memory, then the same row-wise math as
//     the decode-batch kernel (Hadamard-128, svh, clamped SwiGLU, suh_d, Hadamard for gate/up; Hadamard, svh_d for down).
// Every wait is bounded; on a give-up the CTA sets the status word, skips work and still frees its tensor memory.
#include <cstdlib>

#include "common.cuh"
#include "kernels.h"
#include "umma.cuh"

namespace mlxs {

constexpr int PF_NT = 128;        // rows per tile (MMA N, rounded up to 16 per item)
constexpr int PF_KS = 32;         // inputs per pipeline stage (2 k-tiles)
constexpr int PF_KT = PF_KS / 16; // k-tiles per stage
constexpr int PF_RAW_STAGES = 4;  // raw code ring
constexpr int PF_A_STAGES = 2;    // decoded-A ring (decode -> MMA is a short hop)
constexpr int PF_B_STAGES = 4;    // B-operand ring: deep, the rows come through L2 with a long latency
constexpr int PF_A_BYTES = 128 * PF_KS * 2;     // decoded W^T (128 columns x 32 inputs f16) per projection per stage: 8 KB
constexpr int PF_B_BYTES = PF_NT * PF_KS * 2;   // rows (128 x 32 f16) per projection per stage: 8 KB
constexpr int PF_LBO_A = (128 / 8) * 128;       // byte distance of two core matrices along K, A operand
constexpr int PF_LBO_B = (PF_NT / 8) * 128;     // the same, B operand
constexpr int PF_SBO = 128;                     // byte distance of two core matrices along M / N
constexpr int PF_EPI_ROWS = 32;                 // rows per epilogue batch
constexpr int PF_ZS_STRIDE = 132;

// ------------------------------------------------------------------------------------------------------------
// plan: row tiles per expert from the dispatch tables
// ------------------------------------------------------------------------------------------------------------
// Tile table: [0] = tiles of list 0 (experts with up to cap0 rows: one tile each; with cap1 = 0 every expert, in tiles
// of up to cap0 rows), [1] = tiles of list 1 (the other experts, tiles of up to cap1 rows), then the entries {expert,
// first sorted row, rows, first staging row}: list 0 from entry 0, list 1 from entry max_tiles.  An expert's rows are
// split evenly over its tiles (a 16-row remainder tile would cost a full decode).
// Staging rows: a tile's rows padded to 16, tiles in sorted order, so tile number n starts at its first row + 16 n.
__global__ void pf_plan_kernel(DispatchTables t, uint32_t E, const uint8_t* __restrict__ flags, uint32_t min_rows,
                               uint32_t cap0, uint32_t cap1, uint32_t max_tiles, uint32_t* __restrict__ tiles,
                               uint32_t* status) {
    __shared__ uint32_t base0[1025], base1[1025];
    const uint32_t tid = threadIdx.x;
    // tiles per expert in parallel (base0 / base1 hold the counts first), then one thread turns them into offsets
    for (uint32_t e = tid; e < E; e += blockDim.x) {
        const uint32_t c = t.offsets[e + 1] - t.offsets[e];
        const bool lane = takes_tensor_lane(c, min_rows, flags, e), list1 = cap1 && c > cap0;
        base0[e] = lane && !list1 ? (c + cap0 - 1) / cap0 : 0u;
        base1[e] = lane && list1 ? (c + cap1 - 1) / cap1 : 0u;
    }
    __syncthreads();
    if (tid == 0) {
        uint32_t n0 = 0, n1 = 0;
        for (uint32_t e = 0; e < E; ++e) {
            const uint32_t c0 = base0[e], c1 = base1[e];
            base0[e] = n0;
            base1[e] = n1;
            n0 += c0;
            n1 += c1;
        }
        if (n0 > max_tiles || n1 > max_tiles) { atomicMax(status, (uint32_t)ST_WORKLIST_OVERFLOW); n0 = 0; n1 = 0; }
        base0[E] = n0;
        base1[E] = n1;
        tiles[0] = n0;
        tiles[1] = n1;
    }
    __syncthreads();
    if (base0[E] + base1[E] == 0) return;
    for (uint32_t e = tid; e < E; e += blockDim.x) {
        const uint32_t c = t.offsets[e + 1] - t.offsets[e], r0 = t.offsets[e];
        if (!takes_tensor_lane(c, min_rows, flags, e)) continue;
        const bool list1 = cap1 && c > cap0;
        const uint32_t cap = list1 ? cap1 : cap0;
        const uint32_t nt = (c + cap - 1) / cap;
        const uint32_t per = ((c + nt - 1) / nt + 15) / 16 * 16;
        const uint32_t first = list1 ? base1[e] : base0[e], ordinal = base0[e] + base1[e];
        for (uint32_t i = 0; i < nt; ++i) {
            uint32_t* d = prefill_tile(tiles, list1 ? 1 : 0, max_tiles, first + i);
            d[0] = e; d[1] = r0 + i * per; d[2] = min(per, c - i * per); d[3] = r0 + i * per + 16 * (ordinal + i);
        }
    }
}

// ------------------------------------------------------------------------------------------------------------
// prep: rows -> rotated f16 activations in the MMA's B-operand order
// ------------------------------------------------------------------------------------------------------------
// xa[tile][proj][stage = k/32][kc = (k%32)/8][rc = row/8][row%8][k%8] f16
__device__ __forceinline__ size_t pf_xa_off(uint32_t nstage, uint32_t tile, uint32_t np, uint32_t p, uint32_t row, uint32_t k) {
    return ((((size_t)tile * np + p) * nstage + k / PF_KS) * (PF_KS / 8) + (k % PF_KS) / 8) * (PF_NT * 8) + (row / 8) * 64 + (row % 8) * 8 + k % 8;
}
__global__ void __launch_bounds__(256) pf_prep_kernel(const __nv_bfloat16* __restrict__ x, uint32_t top_k, uint32_t H,
                                                      const __half* __restrict__ scales, size_t scales_stride,
                                                      DispatchTables t, const uint32_t* __restrict__ tiles,
                                                      __half* __restrict__ xa) {
    const uint32_t tile = blockIdx.x;
    if (tile >= tiles[0]) return;
    const uint32_t* te = prefill_tile(tiles, 0, 0, tile);
    const uint32_t e = te[0], row0 = te[1], rows = te[2];
    const uint32_t rows16 = (rows + 15) / 16 * 16, warp = threadIdx.x >> 5, lane = threadIdx.x & 31u, b = blockIdx.y;
    const float S = __uint_as_float(SCALE_BITS);
    const uint32_t nstage = H / PF_KS;
    for (uint32_t r = warp; r < rows16; r += 8) {
        const bool valid = r < rows;
        const uint32_t tok = valid ? x_row_of(t, t.order[row0 + r], top_k) : 0u;
        uint2 xb = make_uint2(0, 0);
        if (valid) xb = *reinterpret_cast<const uint2*>(x + (size_t)tok * H + b * 128 + lane * 4);
        const float x0 = __uint_as_float(xb.x << 16), x1 = __uint_as_float(xb.x & 0xFFFF0000u);
        const float x2 = __uint_as_float(xb.y << 16), x3 = __uint_as_float(xb.y & 0xFFFF0000u);
#pragma unroll
        for (int p = 0; p < 2; ++p) {
            float v[4] = {0.f, 0.f, 0.f, 0.f};
            if (valid) {
                const uint2 sb = *reinterpret_cast<const uint2*>(scales + (size_t)e * scales_stride + (size_t)p * H + b * 128 + lane * 4);
                const float2 s01 = __half22float2(*reinterpret_cast<const __half2*>(&sb.x));
                const float2 s23 = __half22float2(*reinterpret_cast<const __half2*>(&sb.y));
                v[0] = x0 * s01.x; v[1] = x1 * s01.y; v[2] = x2 * s23.x; v[3] = x3 * s23.y;
                hadamard128_warp(v, lane);
            }
            // src/kernels/exl3/dsv41_prefill_dig_take2v_5120.metal:57-58: the rotated input is rounded to f16
            const __half2 h01 = __floats2half2_rn(v[0] * S, v[1] * S), h23 = __floats2half2_rn(v[2] * S, v[3] * S);
            *reinterpret_cast<uint2*>(xa + pf_xa_off(nstage, tile, 2, p, r, b * 128 + lane * 4)) =
                make_uint2(*reinterpret_cast<const uint32_t*>(&h01), *reinterpret_cast<const uint32_t*>(&h23));
        }
    }
}

// ------------------------------------------------------------------------------------------------------------
// the kernel
// ------------------------------------------------------------------------------------------------------------
struct PfParams {
    const uint32_t* code;        // layer base of the block stream (8 tiles of 8 K words per k-tile and projection)
    size_t expert_stride_words;
    uint32_t n_blocks, nkt;      // out / 128, in / 16
    const __half* xa;            // B operand, layout of pf_xa_off
    const uint32_t* tiles;
    DispatchTables t;
    const __half* scales;
    size_t scales_stride;
    uint32_t H, I;
    __half* xd;                  // gate/up output = down's B operand
    float* ro;                   // down output [A, H]
    float limit;
    uint32_t* status;
};

// NPROJ projections x CB adjacent 128-column blocks = 4 accumulator groups of 128 TMEM columns each
template <int NPROJ, int CB, int KB>
__global__ void __launch_bounds__(512 + 64, 1) exl3_prefill_kernel(const PfParams P) {
    static_assert(NPROJ * CB == 4, "four accumulator groups fill the 512 tensor-memory columns at 128 rows");
    extern __shared__ __align__(128) uint8_t smem_raw[];
    constexpr int NCW = 16;                            // decode warps
    constexpr int NG = NPROJ * CB;                     // accumulator groups
    constexpr int TW = 8 * KB;                         // words per 16x16 tile (KB bits per weight)
    constexpr int KSTRIDE = NPROJ * 8 * TW;            // words per k-tile in one block's code stream
    constexpr int RAW_BLK = PF_KT * KSTRIDE * 4;       // bytes of one block's k-tiles of a stage
    constexpr int RAW_BYTES = CB * RAW_BLK;
    constexpr int TMEM_COLS = NG * PF_NT;
    __shared__ __align__(8) uint64_t raw_full[PF_RAW_STAGES], raw_empty[PF_RAW_STAGES];
    __shared__ __align__(8) uint64_t b_full[PF_B_STAGES], b_empty[PF_B_STAGES], a_full[PF_A_STAGES], a_empty[PF_A_STAGES];
    __shared__ __align__(8) uint64_t acc_full, acc_empty, epi_bar;
    __shared__ uint32_t s_tmem;
    __shared__ volatile int s_abort;
    // carve: [A ring: NG groups per stage][B ring: NPROJ operands per stage][raw ring][epilogue staging zs]
    uint8_t* a_ring = smem_raw;
    uint8_t* b_ring = a_ring + PF_A_STAGES * NG * PF_A_BYTES;
    uint8_t* raw_ring = b_ring + PF_B_STAGES * NPROJ * PF_B_BYTES;
    float* zs = reinterpret_cast<float*>(raw_ring + PF_RAW_STAGES * RAW_BYTES);
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    // a CTA without work leaves before it takes tensor memory (the whole CTA reads the same count)
    if (blockIdx.x >= P.tiles[0] * (P.n_blocks / CB)) return;

    if (threadIdx.x == 0) {
        for (int s = 0; s < PF_RAW_STAGES; ++s) { mbar_init(&raw_full[s], 1); mbar_init(&raw_empty[s], NCW); }
        for (int s = 0; s < PF_A_STAGES; ++s) { mbar_init(&a_full[s], NCW); mbar_init(&a_empty[s], 1); }
        for (int s = 0; s < PF_B_STAGES; ++s) { mbar_init(&b_full[s], 1); mbar_init(&b_empty[s], 1); }
        mbar_init(&acc_full, 1);
        mbar_init(&acc_empty, NCW);
        mbar_init(&epi_bar, NCW);
        s_abort = 0;
        mbar_fence_init();
    }
    if (warp == 0) tmem_alloc(&s_tmem, TMEM_COLS);  // tensor memory for the accumulators (one warp allocates and frees)
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = s_tmem;
    const uint32_t n_tiles = P.tiles[0];
    const uint32_t nbg = P.n_blocks / CB;              // column-block groups per row tile
    const uint32_t n_items = n_tiles * nbg;
    const uint32_t nstage = P.nkt / PF_KT;
    auto give_up = [&](uint32_t code) { if (!s_abort) atomicMax(P.status, code); s_abort = 1; };

    if (warp == NCW) {
        // ---------------- producer: raw code + B operand ----------------
        if (lane == 0) {
            uint32_t rit = 0, bit = 0;
            for (uint32_t item = blockIdx.x; item < n_items && !s_abort; item += gridDim.x) {
                const uint32_t tile = item / nbg, nb0 = (item % nbg) * CB, expert = prefill_tile(P.tiles, 0, 0, tile)[0];
                const uint32_t* wsrc = P.code + (size_t)expert * P.expert_stride_words + (size_t)nb0 * P.nkt * KSTRIDE;
                for (uint32_t ks = 0; ks < nstage; ++ks, ++rit, ++bit) {
                    const uint32_t rs = rit % PF_RAW_STAGES, rph = (rit / PF_RAW_STAGES) & 1u;
                    if (!mbar_wait_bounded(&raw_empty[rs], rph ^ 1u, &s_abort, 128)) { give_up(ST_WAIT_EMPTY); break; }
                    mbar_expect_tx(&raw_full[rs], RAW_BYTES);
                    for (int cb = 0; cb < CB; ++cb)
                        bulk_g2s(raw_ring + rs * RAW_BYTES + cb * RAW_BLK,
                                 wsrc + (size_t)cb * P.nkt * KSTRIDE + (size_t)ks * PF_KT * KSTRIDE, RAW_BLK, &raw_full[rs]);
                    const uint32_t bs = bit % PF_B_STAGES, bph = (bit / PF_B_STAGES) & 1u;
                    if (!mbar_wait_bounded(&b_empty[bs], bph ^ 1u, &s_abort, 128)) { give_up(ST_WAIT_EMPTY); break; }
                    mbar_expect_tx(&b_full[bs], NPROJ * PF_B_BYTES);
                    for (int p = 0; p < NPROJ; ++p)
                        bulk_g2s(b_ring + (bs * NPROJ + p) * PF_B_BYTES,
                                 P.xa + (((size_t)tile * NPROJ + p) * nstage + ks) * (PF_B_BYTES / 2), PF_B_BYTES, &b_full[bs]);
                }
            }
            if (s_abort) for (int i = 0; i < 2000; ++i) __nanosleep(1000);
        }
    } else if (warp == NCW + 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            uint32_t bit = 0, nitem = 0;
            for (uint32_t item = blockIdx.x; item < n_items && !s_abort; item += gridDim.x, ++nitem) {
                const uint32_t tile = item / nbg, rows = prefill_tile(P.tiles, 0, 0, tile)[2];
                const uint32_t idesc = umma_idesc(UMMA_F16, (rows + 15) / 16 * 16);
                if (!mbar_wait_bounded(&acc_empty, (nitem & 1u) ^ 1u, &s_abort, 64)) { give_up(ST_WAIT_EMPTY); break; }
                tc_fence_after();
                bool ok = true;
                for (uint32_t ks = 0; ks < nstage; ++ks, ++bit) {
                    const uint32_t as = bit % PF_A_STAGES, aph = (bit / PF_A_STAGES) & 1u;
                    const uint32_t bs = bit % PF_B_STAGES, bph = (bit / PF_B_STAGES) & 1u;
                    if (!mbar_wait_bounded(&a_full[as], aph, &s_abort, 32) || !mbar_wait_bounded(&b_full[bs], bph, &s_abort, 32)) {
                        give_up(ST_WAIT_FULL); ok = false; break;
                    }
                    tc_fence_after();
#pragma unroll
                    for (int gq = 0; gq < NG; ++gq) {
                        const int p = gq / CB;  // group = (projection, column block)
                        const uint32_t a0 = smem_u32(a_ring + (as * NG + gq) * PF_A_BYTES);
                        const uint32_t b0 = smem_u32(b_ring + (bs * NPROJ + p) * PF_B_BYTES);
#pragma unroll
                        for (int i = 0; i < PF_KS / 16; ++i)
                            umma_f16(tmem + gq * PF_NT, umma_smem_desc(a0 + i * 2 * PF_LBO_A, PF_LBO_A, PF_SBO),
                                     umma_smem_desc(b0 + i * 2 * PF_LBO_B, PF_LBO_B, PF_SBO), idesc, (ks | (uint32_t)i) ? 1u : 0u);
                    }
                    umma_commit(&a_empty[as]);  // the stage's operands are free once these MMAs have read them
                    umma_commit(&b_empty[bs]);
                }
                if (!ok) break;
                umma_commit(&acc_full);
            }
        }
    } else {
        // ---------------- decode warps + epilogue ----------------
        // a warp owns 16-column tile j of two accumulator groups: gate/up: projection hi, both column blocks;
        // down: column blocks 2 hi and 2 hi + 1.  Group index = NPROJ == 2 ? hi * CB + cb : 2 hi + cb.
        const uint32_t hi = warp >> 3, j = warp & 7u;
        uint32_t wi, wj, lp;
        exl3_lane_plan_kb<KB>(lane, wi, wj, lp);
        const uint32_t g = lane >> 2, c = lane & 3u;
        const float S = __uint_as_float(SCALE_BITS);
        uint32_t rit = 0, bit = 0, nitem = 0, epi_ph = 0;
        auto epi_sync = [&]() -> bool {
            __syncwarp();
            if (lane == 0) mbar_arrive(&epi_bar);
            const bool ok = mbar_wait_bounded(&epi_bar, epi_ph, &s_abort);
            epi_ph ^= 1u;
            if (!ok) give_up(ST_WAIT_FULL);
            return ok;
        };
        for (uint32_t item = blockIdx.x; item < n_items && !s_abort; item += gridDim.x, ++nitem) {
            const uint32_t tile = item / nbg, nb0 = (item % nbg) * CB;
            const uint32_t* te = prefill_tile(P.tiles, 0, 0, tile);
            const uint32_t expert = te[0], row0 = te[1], rows = te[2];
            bool ok = true;
            for (uint32_t ks = 0; ks < nstage; ++ks, ++rit, ++bit) {
                const uint32_t rs = rit % PF_RAW_STAGES, rph = (rit / PF_RAW_STAGES) & 1u;
                const uint32_t as = bit % PF_A_STAGES, aph = (bit / PF_A_STAGES) & 1u;
                if (!mbar_wait_bounded(&raw_full[rs], rph, &s_abort) || !mbar_wait_bounded(&a_empty[as], aph ^ 1u, &s_abort)) {
                    give_up(ST_WAIT_FULL); ok = false; break;
                }
#pragma unroll
                for (int u = 0; u < 2; ++u) {
                    const uint32_t cb = NPROJ == 2 ? (uint32_t)u : 2u * hi + u, p = NPROJ == 2 ? hi : 0u;
                    const uint32_t gq = NPROJ == 2 ? hi * CB + u : cb;
                    const uint32_t* wt = reinterpret_cast<const uint32_t*>(raw_ring + rs * RAW_BYTES + cb * RAW_BLK) + p * (8u * TW) + j * TW;
                    // the warp's 16 columns are core-matrix rows 2j and 2j+1; a lane's half2 pairs sit at g*16 + 4c bytes
                    uint8_t* ad = a_ring + (as * NG + gq) * PF_A_BYTES + (2 * j) * PF_SBO + g * 16 + c * 4;
#pragma unroll
                    for (int kt = 0; kt < PF_KT; ++kt) {
                        uint32_t bq[4];
                        exl3_decode_lane_kb<KB>(wt[kt * KSTRIDE + wi], wt[kt * KSTRIDE + wj], lp, bq);
                        uint8_t* d = ad + (2 * kt) * PF_LBO_A;
                        *reinterpret_cast<uint32_t*>(d) = bq[0];                        // k 2c,2c+1      column g
                        *reinterpret_cast<uint32_t*>(d + PF_LBO_A) = bq[1];             // k 2c+8,2c+9    column g
                        *reinterpret_cast<uint32_t*>(d + PF_SBO) = bq[2];               // k 2c,2c+1      column g+8
                        *reinterpret_cast<uint32_t*>(d + PF_SBO + PF_LBO_A) = bq[3];    // k 2c+8,2c+9    column g+8
                    }
                }
                fence_async_smem();
                __syncwarp();
                if (lane == 0) { mbar_arrive(&a_full[as]); mbar_arrive(&raw_empty[rs]); }
            }
            if (!ok) break;
            // ---- epilogue: per column block, 32 rows at a time ----
            if (!mbar_wait_bounded(&acc_full, nitem & 1u, &s_abort)) { give_up(ST_WAIT_FULL); break; }
            tc_fence_after();
            const uint32_t q = warp & 3u, sub = warp >> 2;
            const uint32_t rows16 = (rows + 15) / 16 * 16;
            for (uint32_t cb = 0; cb < (uint32_t)CB && ok; ++cb) {
                for (uint32_t rb = 0; rb < rows16 && ok; rb += PF_EPI_ROWS) {
                    // 16 warps: lane quarter q, then (projection, 16-row half) for gate/up; down uses warps 0..7
                    if (sub < 2u * NPROJ) {
                        const uint32_t ep = sub % NPROJ, half = sub / NPROJ;
                        uint32_t v[16];
                        tmem_ld16(tmem + ((q * 32u) << 16) + (ep * CB + cb) * PF_NT + rb + half * 16, v);
#pragma unroll
                        for (int i = 0; i < 16; ++i) zs[(ep * PF_EPI_ROWS + half * 16 + i) * PF_ZS_STRIDE + q * 32 + lane] = __uint_as_float(v[i]);
                    }
                    if (!epi_sync()) { ok = false; break; }
                    for (uint32_t rr = warp; rr < PF_EPI_ROWS; rr += NCW) {
                        const uint32_t r = rb + rr;
                        if (r >= rows16) continue;
                        const bool valid = r < rows;
                        const uint32_t col = (nb0 + cb) * 128 + lane * 4;
                        if (NPROJ == 2) {
                            float vv[4] = {0.f, 0.f, 0.f, 0.f};
                            if (valid) {
                                const float4 zg = *reinterpret_cast<const float4*>(zs + (0 * PF_EPI_ROWS + rr) * PF_ZS_STRIDE + lane * 4);
                                const float4 zu = *reinterpret_cast<const float4*>(zs + (1 * PF_EPI_ROWS + rr) * PF_ZS_STRIDE + lane * 4);
                                float gq4[4] = {zg.x, zg.y, zg.z, zg.w}, uq4[4] = {zu.x, zu.y, zu.z, zu.w};
                                hadamard128_warp(gq4, lane);
                                hadamard128_warp(uq4, lane);
                                const __half* sc = P.scales + (size_t)expert * P.scales_stride;
                                const uint2 sg = *reinterpret_cast<const uint2*>(sc + 2 * (size_t)P.H + col);
                                const uint2 su = *reinterpret_cast<const uint2*>(sc + 2 * (size_t)P.H + P.I + col);
                                const uint2 sd = *reinterpret_cast<const uint2*>(sc + 2 * (size_t)P.H + 2 * (size_t)P.I + col);
                                const float2 sg01 = __half22float2(*reinterpret_cast<const __half2*>(&sg.x));
                                const float2 sg23 = __half22float2(*reinterpret_cast<const __half2*>(&sg.y));
                                const float2 su01 = __half22float2(*reinterpret_cast<const __half2*>(&su.x));
                                const float2 su23 = __half22float2(*reinterpret_cast<const __half2*>(&su.y));
                                const float2 sd01 = __half22float2(*reinterpret_cast<const __half2*>(&sd.x));
                                const float2 sd23 = __half22float2(*reinterpret_cast<const __half2*>(&sd.y));
                                const float svg[4] = {sg01.x, sg01.y, sg23.x, sg23.y}, svu[4] = {su01.x, su01.y, su23.x, su23.y};
                                const float shd[4] = {sd01.x, sd01.y, sd23.x, sd23.y};
#pragma unroll
                                for (int qq = 0; qq < 4; ++qq) {
                                    const float gm = (gq4[qq] * S) * svg[qq], um = (uq4[qq] * S) * svu[qq];
                                    float gate = gm, up = um;
                                    if (P.limit > 0.f) {
                                        gate = (gm != gm) ? gm : (gm < P.limit ? gm : P.limit);
                                        const float u0 = (um != um) ? um : (um > -P.limit ? um : -P.limit);
                                        up = (u0 != u0) ? u0 : (u0 < P.limit ? u0 : P.limit);
                                    }
                                    const float yv = 1.0f / (1.0f + expf(fabsf(gate)));
                                    const float sgm = gate < 0.f ? yv : 1.0f - yv;
                                    vv[qq] = ((gate * sgm) * up) * shd[qq];
                                }
                                hadamard128_warp(vv, lane);
                            }
                            // src/kernels/exl3/header_dig2_x.metal:104: the down input is rounded to f16
                            const __half2 h01 = __floats2half2_rn(vv[0] * S, vv[1] * S), h23 = __floats2half2_rn(vv[2] * S, vv[3] * S);
                            *reinterpret_cast<uint2*>(P.xd + pf_xa_off(P.I / PF_KS, tile, 1, 0, r, col)) =
                                make_uint2(*reinterpret_cast<const uint32_t*>(&h01), *reinterpret_cast<const uint32_t*>(&h23));
                        } else if (valid) {
                            const float4 z4 = *reinterpret_cast<const float4*>(zs + rr * PF_ZS_STRIDE + lane * 4);
                            float vv[4] = {z4.x, z4.y, z4.z, z4.w};
                            hadamard128_warp(vv, lane);
                            const __half* sc = P.scales + (size_t)expert * P.scales_stride + 2 * (size_t)P.H + 3 * (size_t)P.I;
                            const uint2 so = *reinterpret_cast<const uint2*>(sc + col);
                            const float2 s01 = __half22float2(*reinterpret_cast<const __half2*>(&so.x));
                            const float2 s23 = __half22float2(*reinterpret_cast<const __half2*>(&so.y));
                            const uint32_t assign = P.t.order[row0 + r];
                            *reinterpret_cast<float4*>(P.ro + (size_t)assign * P.H + col) =
                                make_float4((vv[0] * S) * s01.x, (vv[1] * S) * s01.y, (vv[2] * S) * s23.x, (vv[3] * S) * s23.y);
                        }
                    }
                    if (!epi_sync()) { ok = false; break; }
                }
            }
            if (!ok) break;
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

static size_t pf_smem_bytes(int nproj) {
    return (size_t)PF_A_STAGES * 4 * PF_A_BYTES + (size_t)PF_B_STAGES * nproj * PF_B_BYTES +
           (size_t)PF_RAW_STAGES * PF_KT * 4 * 192 * 4 + (size_t)nproj * PF_EPI_ROWS * PF_ZS_STRIDE * sizeof(float);
}

bool exl3_prefill_supported(Exl3Dims d) { return (d.I / 128) % 2 == 0 && (d.H / 128) % 4 == 0; }

cudaError_t launch_prefill_plan(DispatchTables t, uint32_t n_experts, const uint8_t* lane_flags, uint32_t min_rows,
                                uint32_t cap0, uint32_t cap1, uint32_t max_tiles, uint32_t* tiles, uint32_t* status,
                                cudaStream_t st) {
    pf_plan_kernel<<<1, 256, 0, st>>>(t, n_experts, lane_flags, min_rows, cap0, cap1, max_tiles, tiles, status);
    return cudaGetLastError();
}

cudaError_t launch_exl3_prefill(const Exl3PrefillArgs& a, cudaStream_t st) {
    cudaError_t e = launch_prefill_plan(a.t, a.n_experts, nullptr, a.min_rows, PF_NT, 0, a.max_tiles, a.tiles, a.status, st);
    if (e != cudaSuccess) return e;
    pf_prep_kernel<<<dim3(a.max_tiles, a.d.H / 128), 256, 0, st>>>(a.x, a.top_k, a.d.H, a.L.scales, exl3_scales_per_expert(a.d),
                                                                  a.t, a.tiles, a.xa);
    if ((e = cudaGetLastError()) != cudaSuccess) return e;
    PfParams P{};
    P.tiles = a.tiles; P.t = a.t; P.scales = a.L.scales; P.scales_stride = exl3_scales_per_expert(a.d);
    P.H = a.d.H; P.I = a.d.I; P.limit = a.limit; P.status = a.status;
    // gate / up: two projections x two adjacent column blocks per CTA
    P.code = a.L.gu_code; P.expert_stride_words = 2 * exl3_code_words(a.d); P.n_blocks = a.d.I / 128; P.nkt = a.d.H / 16;
    P.xa = a.xa; P.xd = a.xd; P.ro = nullptr;
    size_t smem = pf_smem_bytes(2);
    if (a.d.K == 3) {
        if ((e = cudaFuncSetAttribute(exl3_prefill_kernel<2, 2, 3>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)) != cudaSuccess) return e;
        exl3_prefill_kernel<2, 2, 3><<<a.sm_count, 512 + 64, smem, st>>>(P);
    } else {
        if ((e = cudaFuncSetAttribute(exl3_prefill_kernel<2, 2, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)) != cudaSuccess) return e;
        exl3_prefill_kernel<2, 2, 2><<<a.sm_count, 512 + 64, smem, st>>>(P);
    }
    if ((e = cudaGetLastError()) != cudaSuccess) return e;
    // down: four adjacent column blocks per CTA
    P.code = a.L.d_code; P.expert_stride_words = exl3_code_words(a.d); P.n_blocks = a.d.H / 128; P.nkt = a.d.I / 16;
    P.xa = a.xd; P.xd = nullptr; P.ro = a.ro;
    smem = pf_smem_bytes(1);
    if (a.d.K == 3) {
        if ((e = cudaFuncSetAttribute(exl3_prefill_kernel<1, 4, 3>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)) != cudaSuccess) return e;
        exl3_prefill_kernel<1, 4, 3><<<a.sm_count, 512 + 64, smem, st>>>(P);
    } else {
        if ((e = cudaFuncSetAttribute(exl3_prefill_kernel<1, 4, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)) != cudaSuccess) return e;
        exl3_prefill_kernel<1, 4, 2><<<a.sm_count, 512 + 64, smem, st>>>(P);
    }
    return cudaGetLastError();
}

}  // namespace mlxs
