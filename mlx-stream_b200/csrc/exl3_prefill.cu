// EXL3 expert kernels for experts with many rows: tcgen05 tensor cores, the trellis decoded straight into tensor memory.
//
// The reference's prefill lane (src/exl3/quant.zig:1040-1271; texts dsv41_prefill_dig_gemm_*_m128*.metal) decodes
// trellis tiles to f16 in threadgroup memory per K stage and feeds its MMA units with f16 rotated activations and an
// f32 accumulator.  Here a CTA owns (expert, a tile of its rows, a group of 128-column blocks).  W^T is the MMA's A
// operand (M = 128 output columns per accumulator group) and lives in tensor memory; the rows are the B operand in
// shared memory (N = rows rounded to 16), so a ragged expert pads to 16 rows.
//   * the in-register decode of a 16x16 tile leaves a lane (g, c) with W[k 2c,2c+1 | 2c+8,2c+9][column g | g+8]: that
//     is one tcgen05.st.16x256b fragment (thread (g, c): lanes g and g + 8, two adjacent 32-bit columns) once the K
//     order inside a 16-block is taken as k' = 4c + 2 (k / 8) + k % 2, c = (k % 8) / 2; the rows are staged in the same
//     order, which a dot product does not see.  One tile costs its decode plus one tensor-memory store: no shared-memory
//     stores, no address arithmetic, no proxy fence;
//   * tensor memory holds the f32 accumulators and a ring of two decoded stages of 64 inputs (32 columns per group
//     and stage).  Two shapes, each 2 groups (gate and up of one column block, or two column blocks of down): 64 rows
//     (experts with up to 64 rows) in 256 columns, two CTAs per SM, so that one CTA's barrier waits and epilogue run
//     under the other's decode; and 192 rows (the others) in 512 columns, where one decode serves three times the rows;
//   * a producer thread streams the raw code (bulk copies, one stage = 4 k-tiles of the group's blocks) and the rows'
//     rotated f16 activations, which a prep kernel laid out as K-major core matrices;
//   * 16 decode warps in two teams that take the stages alternately (team = stage parity = slot of the operand ring):
//     a warp's chain per stage is barrier wait, decode, tensor-memory store latency, arrive, and with one team that
//     chain, not the decode's instructions, set the stage time; two teams overlap each other's latencies.  A warp
//     = (lane quarter q, team, half of the groups) decodes the tiles 2q and 2q + 1 of its groups for all 4 k-tiles;
//   * one thread issues tcgen05.mma.kind::f16 (K = 16, A from tensor memory) and commits once per stage (a commit costs
//     it about as much as an MMA): the commit frees the operand slot, and the decode team that sees the slot free
//     arrives on the rows' slot of the same stage on the MMAs' behalf; the thread waits on one barrier per stage (decode
//     warp 0 arrives only after it has seen the stage's rows land);
//   * the decode warps run the epilogue: tcgen05.ld, transpose through shared memory, then the same row-wise math as
//     the decode-batch kernel (Hadamard-128, svh, clamped SwiGLU, suh_d, Hadamard for gate/up; Hadamard, svh_d for down).
// Every wait is bounded; on a give-up the CTA sets the status word, skips work and still frees its tensor memory.
#include <cstdlib>

#include "common.cuh"
#include "kernels.h"
#include "umma.cuh"

// -DMLXS_LANE_COUNTERS: cycle counters around the waits, the decode and the MMA issue of one CTA, printed once per launch
// (how the lane's bound was found; off in the library)
#ifdef MLXS_LANE_COUNTERS
#include <cstdio>
#define LC(...) __VA_ARGS__
#else
#define LC(...)
#endif

namespace mlxs {

constexpr int PF_KST = 64;          // inputs per operand stage (4 k-tiles)
constexpr int PF_KT = PF_KST / 16;
constexpr int PF_A_COLS = PF_KST / 2;   // tensor-memory columns of one group's decoded stage
constexpr int PF_CAP0 = 64, PF_CAP1 = 192;   // rows per tile of the two shapes
constexpr int PF_RAW_STAGES = 4, PF_B_MAX = 8;  // stages of the code ring; most stages of the row ring
constexpr int PF_SBO = 128;                  // byte distance of two core matrices along N
constexpr int PF_EPI_ROWS = 32;              // rows per epilogue batch
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
// position of input k % 16 inside its 16-block: the order in which the decode's registers fill a tensor-memory fragment
__host__ __device__ inline uint32_t pf_pos16(uint32_t k16) { return 4u * ((k16 & 7u) >> 1) + 2u * (k16 >> 3) + (k16 & 1u); }
// Staged rows of a tile with rows16 rows over `width` inputs, as K-major core matrices:
// [k / 64][kc = position / 8 of the stage][row / 8][row % 8][position % 8], so a stage of 64 inputs is rows16 x 128
// contiguous bytes and the K-direction distance of two core matrices is rows16 x 16 bytes.  Element offset of (row, k):
__device__ __forceinline__ size_t pf_b_off(uint32_t rows16, uint32_t row, uint32_t k) {
    const uint32_t pos = (k % PF_KST) / 16 * 16 + pf_pos16(k % 16);   // position inside the stage
    return (size_t)(k / PF_KST) * (rows16 * PF_KST) + (pos / 8) * (rows16 * 8) + (row / 8) * 64 + (row % 8) * 8 + pos % 8;
}
// a lane that holds the four consecutive inputs 4 (lane % 4) + q of a 16-block stores them as two half2: positions
// p0, p0 + 1 and p0 + 4, p0 + 5 with p0 = {0, 8, 2, 10}[lane % 4]
__device__ __forceinline__ void pf_store4(__half* tile_base, uint32_t rows16, uint32_t row, uint32_t k0, float v0, float v1, float v2, float v3) {
    const __half2 h01 = __floats2half2_rn(v0, v1), h23 = __floats2half2_rn(v2, v3);
    *reinterpret_cast<__half2*>(tile_base + pf_b_off(rows16, row, k0)) = h01;
    *reinterpret_cast<__half2*>(tile_base + pf_b_off(rows16, row, k0 + 2)) = h23;
}

// xa: [projection][staging rows][H] (a tile's rows start at its first staging row, padded to 16)
__global__ void __launch_bounds__(256) pf_prep_kernel(const __nv_bfloat16* __restrict__ x, uint32_t top_k, uint32_t H,
                                                      const __half* __restrict__ scales, size_t scales_stride,
                                                      DispatchTables t, const uint32_t* __restrict__ tiles, uint32_t max_tiles,
                                                      size_t proj_stride, __half* __restrict__ xa) {
    const int list = blockIdx.x >= max_tiles;
    const uint32_t tile = blockIdx.x - (list ? max_tiles : 0u);
    if (tile >= tiles[list]) return;
    const uint32_t* te = prefill_tile(tiles, list, max_tiles, tile);
    const uint32_t e = te[0], row0 = te[1], rows = te[2];
    const uint32_t rows16 = (rows + 15) / 16 * 16, warp = threadIdx.x >> 5, lane = threadIdx.x & 31u, b = blockIdx.y;
    const float S = __uint_as_float(SCALE_BITS);
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
            pf_store4(xa + p * proj_stride + (size_t)te[3] * H, rows16, r, b * 128 + lane * 4, v[0] * S, v[1] * S, v[2] * S, v[3] * S);
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
    const __half* xa;            // B operand: [projection][staging rows][in]
    size_t xa_proj_stride;       // elements between the projections' staged rows
    const uint32_t* tiles;
    uint32_t max_tiles;
    DispatchTables t;
    const __half* scales;
    size_t scales_stride;
    uint32_t H, I;
    __half* xd;                  // gate/up output = down's B operand, [staging rows][I]
    float* ro;                   // down output [A, H]
    float limit;
    uint32_t* status;
    uint32_t b_stages;
};

__device__ __forceinline__ void tmem_st_16x256(uint32_t taddr, const uint32_t (&v)[4]) {
    asm volatile("tcgen05.st.sync.aligned.16x256b.x1.b32 [%0], {%1,%2,%3,%4};" ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]) : "memory");
}
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// NPROJ projections x CB adjacent 128-column blocks = NG accumulator groups of NT tensor-memory columns each; PER_SM
// CTAs share an SM (and its 512 tensor-memory columns)
template <int NPROJ, int CB, int NT, int KB, int PER_SM>
__global__ void __launch_bounds__(512 + 64, PER_SM) exl3_prefill_kernel(const PfParams P) {
    constexpr int NG = NPROJ * CB;
    constexpr int A_STAGES = 2;                        // one per decode team
    constexpr int TCOLS = 512 / PER_SM;                // tensor-memory columns of this CTA
    static_assert((NG == 2 || NG == 4) && NG * NT + A_STAGES * NG * PF_A_COLS <= TCOLS, "shape");
    extern __shared__ __align__(128) uint8_t smem_raw[];
    constexpr int LIST = NT == PF_CAP0 ? 0 : 1;      // which tile list this shape serves
    constexpr int NCW = 16;                            // decode warps
    constexpr int TEAM = NCW / 2;                      // warps of a team
    constexpr int TW = 8 * KB;                         // words per 16x16 tile (KB bits per weight)
    constexpr int KSTRIDE = NPROJ * 8 * TW;            // words per k-tile in one block's code stream
    constexpr int RAW_BLK = PF_KT * KSTRIDE * 4;       // bytes of one block's k-tiles of a stage
    constexpr int RAW_BYTES = CB * RAW_BLK;
    constexpr int B_TILE = NT * PF_KST * 2;            // one projection's rows of a stage (at the shape's row cap)
    constexpr int B_SLOT = NPROJ * B_TILE;
    __shared__ __align__(8) uint64_t raw_full[PF_RAW_STAGES], raw_empty[PF_RAW_STAGES];
    __shared__ __align__(8) uint64_t b_full[PF_B_MAX], b_empty[PF_B_MAX], a_full[A_STAGES], a_empty[A_STAGES];
    __shared__ __align__(8) uint64_t acc_full, acc_empty, epi_bar;
    __shared__ uint32_t s_tmem;
    __shared__ volatile int s_abort;
    const uint32_t B_STAGES = P.b_stages;
    constexpr uint32_t RAW_STAGES = PF_RAW_STAGES;
    // carve: [B ring][raw ring][epilogue staging zs]
    uint8_t* b_ring = smem_raw;
    uint8_t* raw_ring = b_ring + B_STAGES * B_SLOT;
    float* zs = reinterpret_cast<float*>(raw_ring + RAW_STAGES * RAW_BYTES);
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t nbg = P.n_blocks / CB;              // column-block groups per row tile
    const uint32_t n_items = P.tiles[LIST] * nbg;
    // a CTA without work leaves before it takes tensor memory (the whole CTA reads the same count)
    if (blockIdx.x >= n_items) return;

    if (threadIdx.x == 0) {
        // a code slot and an operand slot belong to one team: the stage count of an item is even, so stage parity = team
        for (uint32_t s = 0; s < RAW_STAGES; ++s) { mbar_init(&raw_full[s], 1); mbar_init(&raw_empty[s], TEAM); }
        for (int s = 0; s < A_STAGES; ++s) { mbar_init(&a_full[s], TEAM); mbar_init(&a_empty[s], 1); }
        for (uint32_t s = 0; s < B_STAGES; ++s) { mbar_init(&b_full[s], 1); mbar_init(&b_empty[s], 1); }
        mbar_init(&acc_full, 1);
        mbar_init(&acc_empty, NCW);
        mbar_init(&epi_bar, NCW);
        s_abort = 0;
        mbar_fence_init();
    }
    if (warp == 0) tmem_alloc(&s_tmem, TCOLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = s_tmem, tmem_a = tmem + NG * NT;
    const uint32_t nstage = P.nkt / PF_KT, width = P.nkt * 16;
    auto give_up = [&](uint32_t code) { if (!s_abort) atomicMax(P.status, code); s_abort = 1; };

    if (warp == NCW) {
        // ---------------- producer: raw code + rows ----------------
        if (lane == 0) {
            uint32_t rs = 0, rph = 0, bs = 0, bph = 0;
            for (uint32_t item = blockIdx.x; item < n_items && !s_abort; item += gridDim.x) {
                const uint32_t nb0 = (item % nbg) * CB;
                const uint32_t* te = prefill_tile(P.tiles, LIST, P.max_tiles, item / nbg);
                const uint32_t expert = te[0], rows16 = (te[2] + 15) / 16 * 16, b_bytes = rows16 * PF_KST * 2;
                const uint32_t* wsrc = P.code + (size_t)expert * P.expert_stride_words + (size_t)nb0 * P.nkt * KSTRIDE;
                const __half* xsrc = P.xa + (size_t)te[3] * width;
                bool ok = true;
                for (uint32_t ks = 0; ks < nstage; ++ks) {
                    if (!mbar_wait_bounded(&raw_empty[rs], rph ^ 1u, &s_abort, 64)) { give_up(ST_WAIT_EMPTY); ok = false; break; }
                    mbar_expect_tx(&raw_full[rs], RAW_BYTES);
                    for (int cb = 0; cb < CB; ++cb)
                        bulk_g2s(raw_ring + rs * RAW_BYTES + cb * RAW_BLK,
                                 wsrc + (size_t)cb * P.nkt * KSTRIDE + (size_t)ks * PF_KT * KSTRIDE, RAW_BLK, &raw_full[rs]);
                    if (++rs == RAW_STAGES) { rs = 0; rph ^= 1u; }
                    if (!mbar_wait_bounded(&b_empty[bs], bph ^ 1u, &s_abort, 64)) { give_up(ST_WAIT_EMPTY); ok = false; break; }
                    mbar_expect_tx(&b_full[bs], NPROJ * b_bytes);
                    for (int p = 0; p < NPROJ; ++p)
                        bulk_g2s(b_ring + bs * B_SLOT + p * B_TILE, xsrc + p * P.xa_proj_stride + (size_t)ks * (rows16 * PF_KST), b_bytes, &b_full[bs]);
                    if (++bs == B_STAGES) { bs = 0; bph ^= 1u; }
                }
                if (!ok) break;
            }
            if (s_abort) for (int i = 0; i < 2000; ++i) __nanosleep(1000);
        }
    } else if (warp == NCW + 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            uint32_t as = 0, aph = 0, bs = 0, nitem = 0;
            LC(long long m_wait = 0, m_issue = 0; uint32_t m_n = 0;)
            const uint32_t b_ring_s = smem_u32(b_ring);
            for (uint32_t item = blockIdx.x; item < n_items && !s_abort; item += gridDim.x, ++nitem) {
                const uint32_t rows16 = (prefill_tile(P.tiles, LIST, P.max_tiles, item / nbg)[2] + 15) / 16 * 16;
                const uint32_t idesc = umma_idesc(UMMA_F16, rows16), lbo_b = rows16 * 16;
                const uint64_t bdesc0 = umma_smem_desc(b_ring_s, lbo_b, PF_SBO);   // + byte offset >> 4 in the low word
                if (!mbar_wait_bounded(&acc_empty, (nitem & 1u) ^ 1u, &s_abort, 64)) { give_up(ST_WAIT_EMPTY); break; }
                tc_fence_after();
                bool ok = true;
                for (uint32_t kk = 0; kk < nstage; ++kk) {
                    LC(const long long w0 = clock64();)
                    if (!mbar_wait_bounded(&a_full[as], aph, &s_abort)) { give_up(ST_WAIT_FULL); ok = false; break; }
                    tc_fence_after();
                    LC(const long long w1 = clock64(); m_wait += w1 - w0; ++m_n;)
                    const uint32_t ta = tmem_a + as * (NG * PF_A_COLS);
#pragma unroll
                    for (int gq = 0; gq < NG; ++gq) {
                        const int p = gq / CB;
                        const uint64_t bd = bdesc0 + ((bs * B_SLOT + p * B_TILE) >> 4);
#pragma unroll
                        for (int i = 0; i < PF_KT; ++i)
                            umma_f16_ts(tmem + gq * NT, ta + gq * PF_A_COLS + i * 8, bd + ((i * 2 * lbo_b) >> 4), idesc,
                                        (kk | (uint32_t)i) ? 1u : 0u);
                    }
                    // one commit per stage: it frees the operand slot, and the decode team that sees it frees the rows' slot
                    umma_commit(&a_empty[as]);
                    if (++as == A_STAGES) { as = 0; aph ^= 1u; }
                    if (++bs == B_STAGES) bs = 0;
                    LC(m_issue += clock64() - w1;)
                }
                if (!ok) break;
                umma_commit(&acc_full);
            }
            LC(if (blockIdx.x == 3 && m_n) printf("LANE<%d,%d,%d> mma thread: items %u stages %u, cycles per stage: wait %lld issue %lld\n", NPROJ, CB,
                                                  NT, nitem, m_n, m_wait / m_n, m_issue / m_n);)
        }
    } else {
        // ---------------- decode warps + epilogue ----------------
        // warp = (lane quarter q, team, sub): its tensor-memory lanes hold the 16-column tiles 2q and 2q + 1 of every
        // group; it decodes them for half of the groups (sub) in the stages of its team.
        const uint32_t q = warp & 3u, slot = warp >> 2, team = slot >> 1, sub2 = slot & 1u;
        constexpr int GPW = NG / 2;                     // groups per warp
        uint32_t wi, wj, lp;
        exl3_lane_plan_kb<KB>(lane, wi, wj, lp);
        const float S = __uint_as_float(SCALE_BITS);
        uint32_t gs0 = 0, nitem = 0, epi_ph = 0;        // gs0: stages of the items before this one
        auto epi_sync = [&]() -> bool {
            __syncwarp();
            if (lane == 0) mbar_arrive(&epi_bar);
            const bool ok = mbar_wait_bounded(&epi_bar, epi_ph, &s_abort);
            epi_ph ^= 1u;
            if (!ok) give_up(ST_WAIT_FULL);
            return ok;
        };
        LC(long long t_wait = 0, t_dec = 0, t_arr = 0, t_epi = 0; uint32_t n_st = 0;)
        for (uint32_t item = blockIdx.x; item < n_items && !s_abort; item += gridDim.x, ++nitem, gs0 += nstage) {
            const uint32_t nb0 = (item % nbg) * CB;
            const uint32_t* te = prefill_tile(P.tiles, LIST, P.max_tiles, item / nbg);
            const uint32_t expert = te[0], row0 = te[1], rows = te[2], srow0 = te[3];
            bool ok = true;
            for (uint32_t ks = team; ks < nstage; ks += 2) {
                LC(const long long c0 = clock64();)
                const uint32_t gs = gs0 + ks;           // stage number since the kernel started (gs0 is even)
                const uint32_t rs = gs % RAW_STAGES, rph = (gs / RAW_STAGES) & 1u, aph = (gs >> 1) & 1u;
                if (!mbar_wait_bounded(&raw_full[rs], rph, &s_abort) || !mbar_wait_bounded(&a_empty[team], aph ^ 1u, &s_abort)) {
                    give_up(ST_WAIT_FULL); ok = false; break;
                }
                // the operand slot is free: the MMAs of this team's last stage (two stages back) are done with their rows too
                if (q == 0 && sub2 == 0 && lane == 0 && gs >= 2) mbar_arrive(&b_empty[(gs - 2) % B_STAGES]);
                LC(const long long c1 = clock64(); t_wait += c1 - c0; ++n_st;)
#pragma unroll
                for (int gi = 0; gi < GPW; ++gi) {
                    const uint32_t gq = sub2 * GPW + gi;
                    const uint32_t p = NPROJ == 2 ? gq / CB : 0u, cb = NPROJ == 2 ? gq % CB : gq;
                    // the group's code of this stage: [k-tile][projection][tile j][TW words]
                    const uint32_t* wt = reinterpret_cast<const uint32_t*>(raw_ring + rs * RAW_BYTES + cb * RAW_BLK) + p * (8u * TW) + (2u * q) * TW;
                    const uint32_t ta = tmem_a + ((q * 32u) << 16) + (team * NG + gq) * PF_A_COLS;
#pragma unroll
                    for (int kt = 0; kt < PF_KT; ++kt) {
#pragma unroll
                        for (int jj = 0; jj < 2; ++jj) {
                            const uint32_t* tw = wt + kt * KSTRIDE + jj * TW;
                            uint32_t bq[4];
                            exl3_decode_lane_kb<KB>(tw[wi], tw[wj], lp, bq);
                            // thread (g, c): lanes g / g + 8 of the tile's 16, columns 2c, 2c + 1 of the k-tile's 8
                            tmem_st_16x256(ta + ((jj * 16u) << 16) + kt * 8, bq);
                        }
                    }
                }
                tmem_wait_st();
                tc_fence_before();
                LC(const long long c2 = clock64(); t_dec += c2 - c1;)
                if (q == 0 && sub2 == 0) {  // the stage's rows have landed too: the issuer then waits on one barrier only
                    const uint32_t bsl = gs % B_STAGES, bph = (gs / B_STAGES) & 1u;
                    if (!mbar_wait_bounded(&b_full[bsl], bph, &s_abort)) { give_up(ST_WAIT_FULL); ok = false; break; }
                }
                __syncwarp();
                if (lane == 0) { mbar_arrive(&a_full[team]); mbar_arrive(&raw_empty[rs]); }
                LC(t_arr += clock64() - c2;)
            }
            if (!ok) break;
            LC(const long long e0 = clock64();)
            // ---- epilogue: per column block, 32 rows at a time ----
            if (!mbar_wait_bounded(&acc_full, nitem & 1u, &s_abort)) { give_up(ST_WAIT_FULL); break; }
            tc_fence_after();
            const uint32_t sub = warp >> 2;
            const uint32_t rows16 = (rows + 15) / 16 * 16;
            for (uint32_t ecb = 0; ecb < (uint32_t)CB && ok; ++ecb) {
                // this lane's four columns of the block and their sign / scale vectors: the same for every row
                const uint32_t col = (nb0 + ecb) * 128 + lane * 4;
                float svg[4], svu[4], shd[4];
                {
                    const __half* sc = P.scales + (size_t)expert * P.scales_stride + 2 * (size_t)P.H;
                    const uint2 s0 = *reinterpret_cast<const uint2*>(NPROJ == 2 ? sc + col : sc + 3 * (size_t)P.I + col);
                    const uint2 s1 = *reinterpret_cast<const uint2*>(NPROJ == 2 ? sc + P.I + col : sc + 3 * (size_t)P.I + col);
                    const uint2 s2 = *reinterpret_cast<const uint2*>(NPROJ == 2 ? sc + 2 * (size_t)P.I + col : sc + 3 * (size_t)P.I + col);
                    const float2 a01 = __half22float2(*reinterpret_cast<const __half2*>(&s0.x)), a23 = __half22float2(*reinterpret_cast<const __half2*>(&s0.y));
                    const float2 b01 = __half22float2(*reinterpret_cast<const __half2*>(&s1.x)), b23 = __half22float2(*reinterpret_cast<const __half2*>(&s1.y));
                    const float2 c01 = __half22float2(*reinterpret_cast<const __half2*>(&s2.x)), c23 = __half22float2(*reinterpret_cast<const __half2*>(&s2.y));
                    svg[0] = a01.x; svg[1] = a01.y; svg[2] = a23.x; svg[3] = a23.y;     // gate's svh, or down's svh_d
                    svu[0] = b01.x; svu[1] = b01.y; svu[2] = b23.x; svu[3] = b23.y;     // up's svh
                    shd[0] = c01.x; shd[1] = c01.y; shd[2] = c23.x; shd[3] = c23.y;     // down's suh
                }
                for (uint32_t rb = 0; rb < rows16 && ok; rb += PF_EPI_ROWS) {
                    // 16 warps: lane quarter q, then (projection, 16-row half) for gate/up; down uses warps 0..7
                    if (sub < 2u * NPROJ) {
                        const uint32_t ep = sub % NPROJ, half = sub / NPROJ;
                        if (rb + half * 16 < rows16) {
                            uint32_t v[16];
                            tmem_ld16(tmem + ((q * 32u) << 16) + (ep * CB + ecb) * NT + rb + half * 16, v);
#pragma unroll
                            for (int i = 0; i < 16; ++i) zs[(ep * PF_EPI_ROWS + half * 16 + i) * PF_ZS_STRIDE + q * 32 + lane] = __uint_as_float(v[i]);
                        }
                    }
                    if (!epi_sync()) { ok = false; break; }
                    for (uint32_t rr = warp; rr < PF_EPI_ROWS; rr += NCW) {
                        const uint32_t r = rb + rr;
                        if (r >= rows16) continue;
                        const bool valid = r < rows;
                        if (NPROJ == 2) {
                            float vv[4] = {0.f, 0.f, 0.f, 0.f};
                            if (valid) {
                                const float4 zg = *reinterpret_cast<const float4*>(zs + (0 * PF_EPI_ROWS + rr) * PF_ZS_STRIDE + lane * 4);
                                const float4 zu = *reinterpret_cast<const float4*>(zs + (1 * PF_EPI_ROWS + rr) * PF_ZS_STRIDE + lane * 4);
                                float gq4[4] = {zg.x, zg.y, zg.z, zg.w}, uq4[4] = {zu.x, zu.y, zu.z, zu.w};
                                hadamard128_warp(gq4, lane);
                                hadamard128_warp(uq4, lane);
#pragma unroll
                                for (int qq = 0; qq < 4; ++qq) {
                                    const float gm = (gq4[qq] * S) * svg[qq], um = (uq4[qq] * S) * svu[qq];
                                    float gate = gm, up = um;
                                    if (P.limit > 0.f) {
                                        gate = (gm != gm) ? gm : (gm < P.limit ? gm : P.limit);
                                        const float u0 = (um != um) ? um : (um > -P.limit ? um : -P.limit);
                                        up = (u0 != u0) ? u0 : (u0 < P.limit ? u0 : P.limit);
                                    }
                                    const float yv = sigmoid_tail_fast(gate);
                                    const float sgm = gate < 0.f ? yv : 1.0f - yv;
                                    vv[qq] = ((gate * sgm) * up) * shd[qq];
                                }
                                hadamard128_warp(vv, lane);
                            }
                            // src/kernels/exl3/header_dig2_x.metal:104: the down input is rounded to f16
                            pf_store4(P.xd + (size_t)srow0 * P.I, rows16, r, col, vv[0] * S, vv[1] * S, vv[2] * S, vv[3] * S);
                        } else if (valid) {
                            const float4 z4 = *reinterpret_cast<const float4*>(zs + rr * PF_ZS_STRIDE + lane * 4);
                            float vv[4] = {z4.x, z4.y, z4.z, z4.w};
                            hadamard128_warp(vv, lane);
                            const uint32_t assign = P.t.order[row0 + r];
                            *reinterpret_cast<float4*>(P.ro + (size_t)assign * P.H + col) =
                                make_float4((vv[0] * S) * svg[0], (vv[1] * S) * svg[1], (vv[2] * S) * svg[2], (vv[3] * S) * svg[3]);
                        }
                    }
                    if (!epi_sync()) { ok = false; break; }
                }
            }
            if (!ok) break;
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty);
            LC(t_epi += clock64() - e0;)
        }
        LC(if (blockIdx.x == 3 && lane == 0 && warp == 9 && n_st) printf(
               "LANE<%d,%d,%d> decode warp 9: items %u of %u stages, cycles per stage of the team: wait %lld decode+store %lld arrive %lld; per item: epilogue %lld\n",
               NPROJ, CB, NT, nitem, n_st, t_wait / n_st, t_dec / n_st, t_arr / n_st, t_epi / (nitem ? nitem : 1));)
    }
    // every thread comes here, also after a give-up: the tensor memory is always released
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (warp == 0) tmem_free(tmem, TCOLS);
}

bool exl3_prefill_supported(Exl3Dims d) { return (d.I / 128) % 2 == 0 && (d.H / 128) % 4 == 0 && d.H % PF_KST == 0 && d.I % PF_KST == 0; }

cudaError_t launch_prefill_plan(DispatchTables t, uint32_t n_experts, const uint8_t* lane_flags, uint32_t min_rows,
                                uint32_t cap0, uint32_t cap1, uint32_t max_tiles, uint32_t* tiles, uint32_t* status,
                                cudaStream_t st) {
    pf_plan_kernel<<<1, 256, 0, st>>>(t, n_experts, lane_flags, min_rows, cap0, cap1, max_tiles, tiles, status);
    return cudaGetLastError();
}

template <int NPROJ, int CB, int NT, int KB, int PER_SM>
static cudaError_t pf_launch(PfParams P, int sm_count, cudaStream_t st) {
    // ring depths: the code ring first (HBM latency), the rest of the budget to the rows
    const size_t raw_bytes = (size_t)CB * PF_KT * NPROJ * 8 * 8 * KB * 4, b_slot = (size_t)NPROJ * NT * PF_KST * 2;
    const size_t zs_bytes = (size_t)NPROJ * PF_EPI_ROWS * PF_ZS_STRIDE * sizeof(float);
    const size_t budget = (PER_SM == 1 ? 222 * 1024 : 110 * 1024) - zs_bytes;
    if (PF_RAW_STAGES * raw_bytes + 2 * b_slot > budget) return cudaErrorInvalidValue;
    size_t nb = (budget - PF_RAW_STAGES * raw_bytes) / b_slot;
    P.b_stages = (uint32_t)(nb > (size_t)PF_B_MAX ? (size_t)PF_B_MAX : nb);
    const size_t smem = P.b_stages * b_slot + PF_RAW_STAGES * raw_bytes + zs_bytes;
    cudaError_t e = cudaFuncSetAttribute(exl3_prefill_kernel<NPROJ, CB, NT, KB, PER_SM>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    exl3_prefill_kernel<NPROJ, CB, NT, KB, PER_SM><<<PER_SM * sm_count, 512 + 64, smem, st>>>(P);
    return cudaGetLastError();
}

template <int KB>
static cudaError_t pf_launch_all(const Exl3PrefillArgs& a, cudaStream_t st) {
    PfParams P{};
    P.tiles = a.tiles; P.max_tiles = a.max_tiles; P.t = a.t; P.scales = a.L.scales; P.scales_stride = exl3_scales_per_expert(a.d);
    P.H = a.d.H; P.I = a.d.I; P.limit = a.limit; P.status = a.status;
    // gate / up: both projections of one column block, tiles up to 64 rows (two CTAs per SM) or up to 192 rows
    P.code = a.L.gu_code; P.expert_stride_words = 2 * exl3_code_words(a.d); P.n_blocks = a.d.I / 128; P.nkt = a.d.H / 16;
    P.xa = a.xa; P.xa_proj_stride = exl3_prefill_staging_rows(a.rows_cap, a.max_tiles) * a.d.H; P.xd = a.xd; P.ro = nullptr;
    PfParams D = P;
    // down: two adjacent column blocks per CTA
    D.code = a.L.d_code; D.expert_stride_words = exl3_code_words(a.d); D.n_blocks = a.d.H / 128; D.nkt = a.d.I / 16;
    D.xa = a.xd; D.xa_proj_stride = 0; D.xd = nullptr; D.ro = a.ro;
    // The two tile lists hold different experts and rows: with a side stream the large tiles' gate/up and down run
    // beside the small tiles' (a few hot experts keep few CTAs busy for long; the other list fills the SMs meanwhile)
    return prefill_lists_side_by_side(st, a.side, a.side_fork, a.side_join, [&](cudaStream_t s1) {
        cudaError_t r = pf_launch<2, 1, PF_CAP1, KB, 1>(P, a.sm_count, s1);
        if (r == cudaSuccess && a.side) r = pf_launch<1, 2, PF_CAP1, KB, 1>(D, a.sm_count, s1);
        if (r == cudaSuccess) r = pf_launch<2, 1, PF_CAP0, KB, 2>(P, a.sm_count, st);
        if (r == cudaSuccess) r = pf_launch<1, 2, PF_CAP0, KB, 2>(D, a.sm_count, st);
        if (r == cudaSuccess && !a.side) r = pf_launch<1, 2, PF_CAP1, KB, 1>(D, a.sm_count, st);
        return r;
    });
}

cudaError_t launch_exl3_prefill(const Exl3PrefillArgs& a, cudaStream_t st) {
    cudaError_t e = launch_prefill_plan(a.t, a.n_experts, nullptr, a.min_rows, PF_CAP0, PF_CAP1, a.max_tiles, a.tiles, a.status, st);
    if (e != cudaSuccess) return e;
    pf_prep_kernel<<<dim3(2 * a.max_tiles, a.d.H / 128), 256, 0, st>>>(a.x, a.top_k, a.d.H, a.L.scales, exl3_scales_per_expert(a.d), a.t,
                                                                      a.tiles, a.max_tiles,
                                                                      exl3_prefill_staging_rows(a.rows_cap, a.max_tiles) * a.d.H, a.xa);
    if ((e = cudaGetLastError()) != cudaSuccess) return e;
    return a.d.K == 3 ? pf_launch_all<3>(a, st) : pf_launch_all<2>(a, st);
}

}  // namespace mlxs
