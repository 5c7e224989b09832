// MXFP4 / NVFP4 expert kernels for experts with many rows: tcgen05 tensor cores, weights decoded into tensor memory.
//
// The reference sends prefill-sized FP4 work to a grouped quantised GEMM over rows sorted by expert
// (src/arch/mimo_v2/math.zig:426-447, src/arch/glm5_next/nvfp4.zig:36-56): bf16 rows times dequantised weights, f32
// accumulate.  Here a CTA owns (expert, a tile of its rows, a group of 128-column blocks).  W^T is the MMA's A operand
// (M = 128 output columns per accumulator group) and is written by the decode warps straight into tensor memory; the
// rows are the B operand in shared memory (N = rows rounded to 16).  Shared memory carries only the packed codes and
// the rows, which is what bounds a one-SM MMA fed from decoded operands: a decoded A tile in shared memory would be
// written once and read once per use, as many bytes as the rows themselves.
//   * tensor memory holds the f32 accumulators and a ring of two decoded A stages of 64 inputs.  Two shapes, each 2
//     groups (gate and up of one column block, or two column blocks of down): 64 rows (experts with up to 64 rows;
//     128 + 128 columns, two CTAs per SM: one CTA's waits and epilogue run under the other's work) and 192 rows (the
//     others; 384 + 128 columns), where a decoded operand serves three times the rows;
//   * a producer thread streams the same repacked code/scale stream the decode-batch kernel reads (bulk copies, one
//     stage = 128 inputs of a 128-column block) and the rows, which a prep kernel laid out in core-matrix order;
//   * 16 decode warps: a thread owns one output column of one group, loads 32 of its codes as one 16-byte word, turns
//     them into 16-bit values two per integer op
//     (src/arch/mimo_v2/kernels/header_mimo_moe_k1.metal:7-12), applies the block scale and stores 16 tensor-memory
//     columns (tcgen05.st).  The k order inside a group of 8 is the decode's (0,4,1,5,2,6,3,7); the prep kernel stores
//     the rows in the same order;
//   * MXFP4: operands are bf16.  The code's 3 magnitude bits placed at bits 6..8 are e2m1 x 2^-126 as bf16 (the 0.5
//     code is a bf16 subnormal); one bf16x2 multiply by 2^(b-1) gives e2m1 x 2^(b-127) exactly, and the rows stay the
//     bf16 they arrived as, so every product is exact.  This needs 2^(b-1) to be a bf16, b <= 128 (block scale <= 2):
//     an expert with a larger scale byte is marked at load and always takes the streaming lane;
//   * NVFP4: operands are f16, weights the exact e2m1 values (one e2m1x2 conversion per two codes) times the block's
//     E4M3 scale (exact in f16, as in the streaming lane), rows rounded bf16 -> f16, the global g/2688 applied in the
//     epilogue (decode_kernels_ref.zig:13-65);
//   * one thread issues tcgen05.mma.kind::f16 (K = 16, A from tensor memory) and commits to mbarriers.  The tensor
//     pipe queues only about two MMAs behind the running one, so this thread's time between two stages shows: a
//     stage therefore carries 64 inputs (8 or 16 MMAs), and the thread waits on one barrier per stage (decode warp 0
//     arrives only after it has seen the rows of the stage land).  Measured per stage of 8 MMAs x 88 cycles: about
//     150 cycles in the wait and 160 in fences, commits and loop;
//   * the decode warps run the epilogue straight from tensor memory (a thread owns one output column of 16 rows):
//     the reference's bf16 rounding chain for gate/up (mimo_moe_k1_gateup.metal:115-128,
//     glm5n_nvfp4_gateup.metal:109-129), stores for down.
// Every wait is bounded; on a give-up the CTA sets the status word, skips work and still frees its tensor memory.
#include <cstdlib>

#include "common.cuh"
#include "kernels.h"
#include "umma.cuh"

namespace mlxs {

constexpr int Q_KS = 128;                     // inputs per raw stage (the stream's stage)
constexpr int Q_SB = 32;                      // inputs per block of the staged rows' layout (one scale block of MXFP4)
constexpr int Q_B_MAX = 12, Q_RAW_MAX = 6;   // most stages of the row ring and of the code ring
constexpr int Q_SBO = 128;
constexpr int Q_KST = 64;                     // inputs per operand stage
constexpr int Q_CAP0 = 64, Q_CAP1 = 192;      // rows per tile of the two shapes (64: two CTAs per SM)
                                              // (256 / 384 accumulator columns; the other columns hold decoded A stages)
constexpr int Q_W_STAGE = 8192;               // code bytes per projection per raw stage (fp4.cu F4_W_STAGE)

__host__ __device__ inline uint32_t q_scale_stage_bytes(bool nv) { return nv ? 1024u : 512u; }
// position of input k % 8 inside its 16-byte group: the order the decode produces.  MXFP4 (two codes per integer op into
// bf16): 0,4,1,5,2,6,3,7; NVFP4 (the e2m1x2 -> f16x2 conversion instruction): natural order
__host__ __device__ inline uint32_t q_pos8(uint32_t j, bool nv) { return nv ? j : (j & 3u) * 2u + (j >> 2); }
// Staged rows of a tile with rows16 rows (its rows padded to 16) over `width` inputs, as K-major core matrices:
// [k/32][(k%32)/8][row/8][row%8][pos], so a block of 32 inputs is rows16 x 64 contiguous bytes, consecutive blocks
// follow each other, and the K-direction distance of two core matrices is rows16 x 16 bytes throughout.  Element offset of (row, k):
__device__ __forceinline__ size_t q_b_off(uint32_t rows16, uint32_t row, uint32_t k, bool nv) {
    return (size_t)(k / Q_SB) * (rows16 * Q_SB) + ((k % Q_SB) / 8) * (rows16 * 8) + (row / 8) * 64 + (row % 8) * 8 + q_pos8(k % 8, nv);
}

// ------------------------------------------------------------------------------------------------------------
// prep: gather the tile's rows into the B-operand order (bf16 kept for MXFP4, rounded to f16 for NVFP4)
// ------------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) q_prep_kernel(const __nv_bfloat16* __restrict__ x, uint32_t top_k, uint32_t H, int nv,
                                                     DispatchTables t, const uint32_t* __restrict__ tiles, uint32_t max_tiles,
                                                     uint16_t* __restrict__ xa) {
    const int list = blockIdx.x >= max_tiles;
    const uint32_t tile = blockIdx.x - (list ? max_tiles : 0u);
    if (tile >= tiles[list]) return;
    const uint32_t* te = prefill_tile(tiles, list, max_tiles, tile);
    const uint32_t row0 = te[1], rows = te[2];
    const uint32_t rows16 = (rows + 15) / 16 * 16, groups = H / 8;
    uint16_t* dst = xa + (size_t)te[3] * H;
    // a thread moves 8 consecutive inputs of one row; consecutive threads take consecutive rows (one core matrix = 128 B)
    for (uint32_t i = blockIdx.y * blockDim.x + threadIdx.x; i < rows16 * groups; i += gridDim.y * blockDim.x) {
        const uint32_t r = i % rows16, kg = i / rows16;
        uint4 raw = make_uint4(0, 0, 0, 0);
        if (r < rows) raw = *reinterpret_cast<const uint4*>(x + (size_t)x_row_of(t, t.order[row0 + r], top_k) * H + (size_t)kg * 8);
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
        // stored order 0,4,1,5,2,6,3,7 (MXFP4) or natural (NVFP4): q_pos8
        const uint4 o = nv ? make_uint4(e[0] | ((uint32_t)e[1] << 16), e[2] | ((uint32_t)e[3] << 16), e[4] | ((uint32_t)e[5] << 16),
                                        e[6] | ((uint32_t)e[7] << 16))
                           : make_uint4(e[0] | ((uint32_t)e[4] << 16), e[1] | ((uint32_t)e[5] << 16), e[2] | ((uint32_t)e[6] << 16),
                                        e[3] | ((uint32_t)e[7] << 16));
        *reinterpret_cast<uint4*>(dst + q_b_off(rows16, r, kg * 8, nv != 0)) = o;
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
    const uint16_t* xa;          // B operand: staged rows over this projection's inputs
    const uint32_t* tiles;
    uint32_t max_tiles;
    DispatchTables t;
    uint32_t H, I;
    uint16_t* xd;                // gate/up output = down's B operand
    void* out;                   // down: ro [A, H] bf16 (chain) or f32
    int out_bf16;
    float limit;
    uint32_t* status;
    uint32_t b_stages, raw_stages;   // ring depths (the launcher fits them to the shared-memory budget)
};

// MXFP4: 8 codes of a word -> 4 bf16x2 of e2m1 x 2^-126 (pairs (0,4), (1,5), (2,6), (3,7))
__device__ __forceinline__ void q_decode8_bf16(uint32_t w, uint32_t (&h)[4]) {
    h[0] = ((w << 6) & 0x01C001C0u) | ((w << 12) & 0x80008000u);
    h[1] = ((w << 2) & 0x01C001C0u) | ((w << 8) & 0x80008000u);
    h[2] = ((w >> 2) & 0x01C001C0u) | ((w << 4) & 0x80008000u);
    h[3] = ((w >> 6) & 0x01C001C0u) | (w & 0x80008000u);
}
// NVFP4: 8 codes of a word -> 4 f16x2 of the exact e2m1 values through the conversion instruction (pairs (0,1), (2,3),
// (4,5), (6,7))
__device__ __forceinline__ void q_decode8_f16(uint32_t w, uint32_t (&h)[4]) {
    asm("{\n\t.reg .b8 b0, b1, b2, b3;\n\t"
        "mov.b32 {b0, b1, b2, b3}, %4;\n\t"
        "cvt.rn.f16x2.e2m1x2 %0, b0;\n\t"
        "cvt.rn.f16x2.e2m1x2 %1, b1;\n\t"
        "cvt.rn.f16x2.e2m1x2 %2, b2;\n\t"
        "cvt.rn.f16x2.e2m1x2 %3, b3;\n\t}"
        : "=r"(h[0]), "=r"(h[1]), "=r"(h[2]), "=r"(h[3])
        : "r"(w));
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
    const float y = sigmoid_tail_fast(x);
    return x < 0.f ? y : 1.0f - y;
}

// NPROJ projections x CB adjacent 128-column blocks = NG accumulator groups of NT tensor-memory columns each; an
// operand stage holds KST inputs (KST / 2 tensor-memory columns per group).  One synchronisation round trip (decode ->
// MMA -> stage free) costs several hundred cycles whatever the stage holds, so a stage carries NG x KST / 16 MMAs.
template <int NPROJ, int CB, int NT, int KST, bool NV, int PER_SM>
__global__ void __launch_bounds__(512 + 64, PER_SM) fp4_prefill_kernel(const QParams P) {
    constexpr int NG = NPROJ * CB;
    constexpr int KB = KST / Q_SB;                                   // 32-input blocks per operand stage
    constexpr int A_COLS = KST / 2;                                  // tensor-memory columns of one group's stage
    constexpr int TCOLS = 512 / PER_SM;                              // tensor-memory columns of this CTA (PER_SM CTAs share an SM)
    constexpr int A_STAGES = (TCOLS - NG * NT) / (NG * A_COLS);
    constexpr int TASKS = NG * KB / 4;                               // (group, block) tasks of a warp per stage
    static_assert((NG == 2 || NG == 4) && A_STAGES >= 2 && TASKS >= 1 && Q_KS % KST == 0, "shape");
    extern __shared__ __align__(128) uint8_t smem_raw[];
    constexpr int LIST = NT == Q_CAP0 ? 0 : 1;
    constexpr int NCW = 16;
    constexpr int B_SLOT = NT * KST * 2;
    constexpr uint32_t SSTAGE = NV ? 1024u : 512u;
    constexpr uint32_t W_BYTES = NPROJ * (Q_W_STAGE + SSTAGE);   // one block's stage of the stream
    constexpr uint32_t RAW_BYTES = CB * W_BYTES;
    __shared__ __align__(8) uint64_t raw_full[Q_RAW_MAX], raw_empty[Q_RAW_MAX];
    __shared__ __align__(8) uint64_t b_full[Q_B_MAX], b_empty[Q_B_MAX], a_full[A_STAGES], a_empty[A_STAGES];
    __shared__ __align__(8) uint64_t acc_full, acc_empty;
    __shared__ uint32_t s_tmem;
    __shared__ volatile int s_abort;
    __shared__ uint32_t s_lut[NV ? 256 : 1];                           // E4M3 byte -> f16x2 of its value
    uint8_t* b_ring = smem_raw;                                        // [stage][B_SLOT]
    const uint32_t B_STAGES = P.b_stages, RAW_STAGES = P.raw_stages;
    uint8_t* raw_ring = b_ring + B_STAGES * B_SLOT;                    // [stage][CB][W_BYTES]
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t nbg = P.n_blocks / CB;
    const uint32_t n_items = P.tiles[LIST] * nbg;
    // a CTA without work leaves before it takes tensor memory (the whole CTA reads the same count)
    if (blockIdx.x >= n_items) return;

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < RAW_STAGES; ++s) { mbar_init(&raw_full[s], 1); mbar_init(&raw_empty[s], NCW); }
        for (int s = 0; s < A_STAGES; ++s) { mbar_init(&a_full[s], NCW); mbar_init(&a_empty[s], 1); }
        for (uint32_t s = 0; s < B_STAGES; ++s) { mbar_init(&b_full[s], 1); mbar_init(&b_empty[s], 1); }
        mbar_init(&acc_full, 1);
        mbar_init(&acc_empty, NCW);
        s_abort = 0;
        mbar_fence_init();
    }
    if (NV && threadIdx.x < 256) s_lut[threadIdx.x] = q_e4m3_f16x2(threadIdx.x);
    if (warp == 0) tmem_alloc(&s_tmem, TCOLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = s_tmem, tmem_a = tmem + NG * NT;
    const uint32_t nstage = P.n_stages_k, width = nstage * Q_KS;
    auto give_up = [&](uint32_t code) { if (!s_abort) atomicMax(P.status, code); s_abort = 1; };

    if (warp == NCW) {
        // ---------------- producer: code/scale stream + rows ----------------
        if (lane == 0) {
            uint32_t rs = 0, rph = 0, bs = 0, bph = 0;   // ring positions and phases
            for (uint32_t item = blockIdx.x; item < n_items && !s_abort; item += gridDim.x) {
                const uint32_t nb0 = (item % nbg) * CB;
                const uint32_t* te = prefill_tile(P.tiles, LIST, P.max_tiles, item / nbg);
                const uint32_t expert = te[0], rows16 = (te[2] + 15) / 16 * 16, b_bytes = rows16 * KST * 2;
                const uint8_t* wsrc = P.w + (size_t)expert * P.expert_stride + (size_t)nb0 * nstage * W_BYTES;
                const uint16_t* xsrc = P.xa + (size_t)te[3] * width;
                bool ok = true;
                for (uint32_t ks = 0; ks < nstage && ok; ++ks) {
                    if (!mbar_wait_bounded(&raw_empty[rs], rph ^ 1u, &s_abort, 64)) { give_up(ST_WAIT_EMPTY); ok = false; break; }
                    mbar_expect_tx(&raw_full[rs], RAW_BYTES);
                    for (int cb = 0; cb < CB; ++cb)
                        bulk_g2s(raw_ring + rs * RAW_BYTES + cb * W_BYTES, wsrc + ((size_t)cb * nstage + ks) * W_BYTES, W_BYTES,
                                 &raw_full[rs]);
                    if (++rs == RAW_STAGES) { rs = 0; rph ^= 1u; }
                    for (uint32_t os = 0; os < Q_KS / KST; ++os) {
                        if (!mbar_wait_bounded(&b_empty[bs], bph ^ 1u, &s_abort, 64)) { give_up(ST_WAIT_EMPTY); ok = false; break; }
                        mbar_expect_tx(&b_full[bs], b_bytes);
                        bulk_g2s(b_ring + bs * B_SLOT, xsrc, b_bytes, &b_full[bs]);
                        xsrc += b_bytes / 2;
                        if (++bs == B_STAGES) { bs = 0; bph ^= 1u; }
                    }
                }
                if (!ok) break;
            }
            if (s_abort) for (int i = 0; i < 2000; ++i) __nanosleep(1000);
        }
    } else if (warp == NCW + 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            // The issue loop is the pipeline's critical path: the tensor pipe queues only about two MMAs behind the one
            // that runs, so every cycle this thread spends between two stages shows.  Per stage: one barrier wait (a
            // ready mbarrier costs about 130 cycles to test), the MMAs, two commits.  The rows' barrier is waited on by
            // decode warp 0 before it arrives.
            uint32_t as = 0, aph = 0, bs = 0, nitem = 0;
            const uint32_t b_ring_s = smem_u32(b_ring);
            for (uint32_t item = blockIdx.x; item < n_items && !s_abort; item += gridDim.x, ++nitem) {
                const uint32_t rows16 = (prefill_tile(P.tiles, LIST, P.max_tiles, item / nbg)[2] + 15) / 16 * 16;
                const uint32_t idesc = umma_idesc(NV ? UMMA_F16 : UMMA_BF16, rows16), lbo_b = rows16 * 16;
                const uint64_t bdesc0 = umma_smem_desc(b_ring_s, lbo_b, Q_SBO);   // + byte offset >> 4 in the low word
                if (!mbar_wait_bounded(&acc_empty, (nitem & 1u) ^ 1u, &s_abort, 64)) { give_up(ST_WAIT_EMPTY); break; }
                tc_fence_after();
                bool ok = true;
                const uint32_t nk = nstage * (Q_KS / KST);
                for (uint32_t kk = 0; kk < nk; ++kk) {
                    if (!mbar_wait_bounded(&a_full[as], aph, &s_abort)) { give_up(ST_WAIT_FULL); ok = false; break; }
                    tc_fence_after();
                    const uint64_t bd = bdesc0 + ((bs * B_SLOT) >> 4);
                    const uint32_t ta = tmem_a + as * (NG * A_COLS);
#pragma unroll
                    for (int gq = 0; gq < NG; ++gq) {
#pragma unroll
                        for (int i = 0; i < KST / 16; ++i)
                            umma_f16_ts(tmem + gq * NT, ta + gq * A_COLS + i * 8, bd + ((i * 2 * lbo_b) >> 4), idesc,
                                        (kk | (uint32_t)i) ? 1u : 0u);
                    }
                    // one commit per stage (a commit costs the issuing thread about as much as an MMA): it frees the
                    // operand slot, and decode warp 0, when it sees that, frees the rows' slot of the same stage
                    umma_commit(&a_empty[as]);
                    if (++as == A_STAGES) { as = 0; aph ^= 1u; }
                    if (++bs == B_STAGES) bs = 0;
                }
                if (!ok) break;
                umma_commit(&acc_full);
            }
        }
    } else {
        // ---------------- decode warps + epilogue ----------------
        // Warp = (lane quarter q = warp % 4, slot = warp / 4): a thread owns output column m = 32 q + lane of group
        // slot % NG and decodes, per operand stage, the 32-input blocks slot / NG, slot / NG + 4 / NG, ...
        const uint32_t q = warp & 3u, slot = warp >> 2;
        const uint32_t gq = slot % NG, kb0 = slot / NG;
        const uint32_t p = NPROJ == 2 ? gq / CB : 0u, cb = NPROJ == 2 ? gq % CB : gq;
        const uint32_t m = q * 32u + lane, wr = m >> 4, r = (m >> 3) & 1u, g = m & 7u;
        uint32_t rs = 0, rph = 0, as = 0, aph = 0, bs = 0, bph = 0, nitem = 0;
        uint32_t n_stage = 0, rel_bs = 0;   // operand stages so far; the rows' slot to free next (A_STAGES stages behind)
        for (uint32_t item = blockIdx.x; item < n_items && !s_abort; item += gridDim.x, ++nitem) {
            const uint32_t nb0 = (item % nbg) * CB;
            const uint32_t* te = prefill_tile(P.tiles, LIST, P.max_tiles, item / nbg);
            const uint32_t expert = te[0], row0 = te[1], rows = te[2], srow0 = te[3];
            bool ok = true;
            for (uint32_t ks = 0; ks < nstage && ok; ++ks) {
                if (!mbar_wait_bounded(&raw_full[rs], rph, &s_abort)) { give_up(ST_WAIT_FULL); ok = false; break; }
                const uint8_t* blk = raw_ring + rs * RAW_BYTES + cb * W_BYTES;
                const uint8_t* sc = blk + NPROJ * Q_W_STAGE + p * SSTAGE;
#pragma unroll
                for (int os = 0; os < Q_KS / KST; ++os) {
                    if (!mbar_wait_bounded(&a_empty[as], aph ^ 1u, &s_abort)) { give_up(ST_WAIT_FULL); ok = false; break; }
                    // the slot is free: the MMAs of the stage that used it (A_STAGES stages back) are done with their rows too
                    if (warp == 0) {
                        if (n_stage >= (uint32_t)A_STAGES) {
                            if (lane == 0) mbar_arrive(&b_empty[rel_bs]);
                            if (++rel_bs == B_STAGES) rel_bs = 0;
                        }
                        ++n_stage;
                    }
#pragma unroll
                    for (int n = 0; n < TASKS; ++n) {
                        const uint32_t kb = kb0 + n * (4 / NG), sb = os * KB + kb;   // block of the stage, of the raw stage
                        // the row's 32 codes of this block: words c = 0..3 of [wr][sb][r][g][c]
                        const uint4 ww = *reinterpret_cast<const uint4*>(blk + p * Q_W_STAGE + (((wr * 4 + sb) * 2 + r) * 32 + g * 4) * 4);
                        const uint32_t wds[4] = {ww.x, ww.y, ww.z, ww.w};
                        uint32_t v[16];
                        if (NV) {
                            const uint32_t s0 = s_lut[sc[(((wr * 4 + sb) * 2 + 0) * 8 + g) * 2 + r]];
                            const uint32_t s1 = s_lut[sc[(((wr * 4 + sb) * 2 + 1) * 8 + g) * 2 + r]];
#pragma unroll
                            for (int c = 0; c < 4; ++c) {
                                uint32_t h[4];
                                q_decode8_f16(wds[c], h);
#pragma unroll
                                for (int i = 0; i < 4; ++i) v[4 * c + i] = q_mul_f16x2(h[i], c < 2 ? s0 : s1);
                            }
                        } else {
                            const uint32_t bb = sc[((wr * 4 + sb) * 8 + g) * 2 + r];
                            const uint32_t s0 = ((bb + 126u) << 7) * 0x00010001u;   // 2^(b - 1) in both halves
#pragma unroll
                            for (int c = 0; c < 4; ++c) {
                                uint32_t h[4];
                                q_decode8_bf16(wds[c], h);
#pragma unroll
                                for (int i = 0; i < 4; ++i) v[4 * c + i] = q_mul_bf16x2(h[i], s0);
                            }
                        }
                        tmem_st16(tmem_a + ((q * 32u) << 16) + (as * NG + gq) * A_COLS + kb * 16, v);
                    }
                    tc_fence_before();
                    if (warp == 0) {  // the stage's rows have landed too: the issuer then waits on one barrier only
                        if (!mbar_wait_bounded(&b_full[bs], bph, &s_abort)) { give_up(ST_WAIT_FULL); ok = false; break; }
                        if (++bs == B_STAGES) { bs = 0; bph ^= 1u; }
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&a_full[as]);
                    if (++as == A_STAGES) { as = 0; aph ^= 1u; }
                }
                if (!ok) break;
                __syncwarp();
                if (lane == 0) mbar_arrive(&raw_empty[rs]);
                if (++rs == RAW_STAGES) { rs = 0; rph ^= 1u; }
            }
            if (!ok) break;
            // ---- epilogue: a thread owns output column 32 q + lane of a group, 16 rows per tensor-memory load ----
            if (!mbar_wait_bounded(&acc_full, nitem & 1u, &s_abort)) { give_up(ST_WAIT_FULL); break; }
            tc_fence_after();
            const uint32_t rows16 = (rows + 15) / 16 * 16, nrb = rows16 / 16;
            if (NPROJ == 2) {
                float gs_g = 1.f, gs_u = 1.f;
                if (NV) {
                    gs_g = P.gscale[expert * 3 + 0] / 2688.0f;
                    gs_u = P.gscale[expert * 3 + 1] / 2688.0f;
                }
                uint16_t* xd_tile = P.xd + (size_t)srow0 * P.I;
                for (uint32_t unit = slot; unit < CB * nrb; unit += 4) {
                    const uint32_t ecb = unit / nrb, rb = (unit % nrb) * 16;
                    uint32_t vg[16], vu[16];
                    tmem_ld16(tmem + ((q * 32u) << 16) + (0 * CB + ecb) * NT + rb, vg);
                    tmem_ld16(tmem + ((q * 32u) << 16) + (1 * CB + ecb) * NT + rb, vu);
                    const uint32_t col = (nb0 + ecb) * 128 + m;
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        // mimo_moe_k1_gateup.metal:115-128 / glm5n_nvfp4_gateup.metal:109-129
                        float gf = bf16_round_f(__uint_as_float(vg[i]) * gs_g), uf = bf16_round_f(__uint_as_float(vu[i]) * gs_u);
                        if (P.limit > 0.f) {
                            gf = gf > P.limit ? P.limit : gf;
                            uf = uf > P.limit ? P.limit : (uf < -P.limit ? -P.limit : uf);
                        }
                        const float hq = bf16_round_f(bf16_round_f(gf * q_sigmoid(gf)) * uf);
                        const uint32_t rr = rb + i;
                        uint16_t bits = 0;
                        if (rr < rows) bits = NV ? __half_as_ushort(__float2half_rn(hq)) : (uint16_t)(__float_as_uint(hq) >> 16);
                        xd_tile[q_b_off(rows16, rr, col, NV)] = bits;
                    }
                }
            } else {
                float gs = 1.f;
                if (NV) gs = P.gscale[expert * 3 + 2] / 2688.0f;
                for (uint32_t unit = slot; unit < CB * nrb; unit += 4) {
                    const uint32_t ecb = unit / nrb, rb = (unit % nrb) * 16;
                    uint32_t v[16];
                    tmem_ld16(tmem + ((q * 32u) << 16) + ecb * NT + rb, v);
                    const uint32_t col = (nb0 + ecb) * 128 + m;
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        const uint32_t rr = rb + i;
                        if (rr >= rows) continue;
                        const uint32_t assign = P.t.order[row0 + rr];
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
    if (warp == 0) tmem_free(tmem, TCOLS);
}

static int q_env(const char* name, int dflt, int lo, int hi) {
    const char* v = getenv(name);
    const int x = v ? atoi(v) : dflt;
    return x < lo ? lo : (x > hi ? hi : x);
}

bool fp4_prefill_supported(uint32_t H, uint32_t I) { return H % 128 == 0 && I % 128 == 0 && (I / 128) % 2 == 0 && (H / 128) % 4 == 0; }

template <int NPROJ, int CB, int NT, int KST, bool NV, int PER_SM>
static cudaError_t q_launch(QParams P, int sm_count, cudaStream_t st) {
    // ring depths: the code ring first (HBM latency), the rest of the budget to the rows
    const size_t raw_bytes = (size_t)CB * NPROJ * (Q_W_STAGE + q_scale_stage_bytes(NV)), b_slot = (size_t)NT * KST * 2;
    const size_t budget = PER_SM == 1 ? 224 * 1024 : 110 * 1024;
    static const int raw_want = q_env("MLXS_Q_RAW_STAGES", 4, 2, Q_RAW_MAX), b_want = q_env("MLXS_Q_B_STAGES", Q_B_MAX, 2, Q_B_MAX);
    P.raw_stages = (uint32_t)raw_want;
    while (P.raw_stages > 2 && P.raw_stages * raw_bytes + 3 * b_slot > budget) --P.raw_stages;
    size_t nb = (budget - P.raw_stages * raw_bytes) / b_slot;
    P.b_stages = (uint32_t)(nb > (size_t)b_want ? (size_t)b_want : nb);
    const size_t smem = P.b_stages * b_slot + P.raw_stages * raw_bytes;
    cudaError_t e = cudaFuncSetAttribute(fp4_prefill_kernel<NPROJ, CB, NT, KST, NV, PER_SM>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    fp4_prefill_kernel<NPROJ, CB, NT, KST, NV, PER_SM><<<PER_SM * sm_count, 512 + 64, smem, st>>>(P);
    return cudaGetLastError();
}

cudaError_t launch_fp4_prefill(const Fp4PrefillArgs& a, cudaStream_t st) {
    cudaError_t e = launch_prefill_plan(a.t, a.n_experts, a.lane_flags, a.min_rows, Q_CAP0, Q_CAP1, a.max_tiles, a.tiles, a.status, st);
    if (e != cudaSuccess) return e;
    q_prep_kernel<<<dim3(2 * a.max_tiles, 8), 256, 0, st>>>(a.x, a.top_k, a.H, a.nv, a.t, a.tiles, a.max_tiles, a.xa);
    if ((e = cudaGetLastError()) != cudaSuccess) return e;
    const uint32_t sstage = q_scale_stage_bytes(a.nv != 0);
    QParams P{};
    P.gscale = a.gscale; P.tiles = a.tiles; P.max_tiles = a.max_tiles; P.t = a.t; P.H = a.H; P.I = a.I; P.limit = a.limit;
    P.status = a.status;
    // gate / up: both projections of one column block, tiles up to 64 rows (two CTAs per SM) or up to 192 rows
    P.w = a.gu; P.w_bytes = 2 * (Q_W_STAGE + sstage); P.n_blocks = a.I / 128; P.n_stages_k = a.H / Q_KS;
    P.expert_stride = (size_t)P.n_blocks * P.n_stages_k * P.w_bytes;
    P.xa = a.xa; P.xd = a.xd; P.out = nullptr; P.out_bf16 = 0;
    QParams D = P;
    // down: two adjacent column blocks per CTA
    D.w = a.dn; D.w_bytes = Q_W_STAGE + sstage; D.n_blocks = a.H / 128; D.n_stages_k = a.I / Q_KS;
    D.expert_stride = (size_t)D.n_blocks * D.n_stages_k * D.w_bytes;
    D.xa = a.xd; D.xd = nullptr; D.out = a.ro; D.out_bf16 = a.ro_bf16;
    // the two tile lists hold different experts and rows: the large tiles' kernels run beside the small tiles' when the
    // call has a side stream for them
    return prefill_lists_side_by_side(st, a.side, a.side_fork, a.side_join, [&](cudaStream_t s1) {
        cudaError_t r = a.nv ? q_launch<2, 1, Q_CAP1, Q_KST, true, 1>(P, a.sm_count, s1) : q_launch<2, 1, Q_CAP1, Q_KST, false, 1>(P, a.sm_count, s1);
        if (r == cudaSuccess && a.side) r = a.nv ? q_launch<1, 2, Q_CAP1, Q_KST, true, 1>(D, a.sm_count, s1) : q_launch<1, 2, Q_CAP1, Q_KST, false, 1>(D, a.sm_count, s1);
        if (r == cudaSuccess) r = a.nv ? q_launch<2, 1, Q_CAP0, Q_KST, true, 2>(P, a.sm_count, st) : q_launch<2, 1, Q_CAP0, Q_KST, false, 2>(P, a.sm_count, st);
        if (r == cudaSuccess) r = a.nv ? q_launch<1, 2, Q_CAP0, Q_KST, true, 2>(D, a.sm_count, st) : q_launch<1, 2, Q_CAP0, Q_KST, false, 2>(D, a.sm_count, st);
        if (r == cudaSuccess && !a.side) r = a.nv ? q_launch<1, 2, Q_CAP1, Q_KST, true, 1>(D, a.sm_count, st) : q_launch<1, 2, Q_CAP1, Q_KST, false, 1>(D, a.sm_count, st);
        return r;
    });
}

}  // namespace mlxs
