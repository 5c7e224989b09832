// MXFP4 experts with many rows on the block-scaled tensor-core kind: tcgen05.mma.kind::mxf8f6f4.block_scale consumes
// the bank's e2m1 codes and E8M0 32-block scales as they are stored; nothing is decoded on the SM.
//
// The reference's MXFP4 prefill is a grouped quantised GEMM over rows sorted by expert that reads the packed weights
// directly (src/arch/mimo_v2/math.zig:426-447): bf16 rows x dequantised weights, f32 accumulate.  Here:
//   * A = W^T (M = 128 output columns per accumulator group): the codes go from the streamed stage (the same repacked
//     stream the decode-batch kernel reads) into the operand's shared-memory geometry by a plain copy: a 16-byte
//     core-matrix row holds 16 codes in its low 8 bytes.  The weight's scale bytes go to tensor memory (row m: lane m,
//     column + m / 32, one byte per 32-input block);
//   * B = the rows.  A bf16 row value is split into an E4M3 high part and an E4M3 low part, each with a power-of-two
//     scale per 32 inputs (UE8M0): v = hi 2^eh + lo 2^(eh - 4) exactly for every element within 2^-13 of its block's
//     largest (smaller ones keep the bits that matter at the block's scale), so with two MMAs per 32 inputs every
//     e2m1 x e4m3 product is exact in the f32 accumulator and the rows keep bf16's precision.  Measured against the
//     bf16-row product: 2e-8 of its rms (one FP8 value per row element instead: 2.7e-2).  Rows with infinities are not
//     representable (E4M3 has none): an infinity becomes the largest finite value of its block scale, a NaN stays NaN;
//   * the pair of 8-bit-rate MMAs takes the tensor time of one 16-bit-rate MMA over the same 32 inputs, so the lane's
//     tensor time is that of the kind::f16 lane; what goes away is its 20 decode instructions per 8 weights;
//   * the rest is the decoded-operand lane's pipeline (fp4_prefill.cu): a producer thread streams codes and rows by
//     bulk copies, 16 warps prepare an operand stage of 64 inputs (copy codes, scale words to tensor memory), one
//     thread issues the MMAs and commits to mbarriers, the 16 warps run the epilogue from tensor memory.  The gate/up
//     epilogue applies the reference's bf16 rounding chain (mimo_moe_k1_gateup.metal:115-128) and writes h already
//     split into high and low parts for the down product (a warp holds one 32-input block of a row: one warp-wide
//     maximum per row gives the block scale).
// Every wait is bounded; on a give-up the CTA sets the status word, skips work and still frees its tensor memory.
#include <cstdlib>

#include "common.cuh"
#include "kernels.h"
#include "umma.cuh"

namespace mlxs {

constexpr int NF_KS = 128;                     // inputs per streamed stage
constexpr int NF_KST = 64;                     // inputs per operand stage: two 32-input blocks
constexpr int NF_W_STAGE = 8192;               // code bytes per projection per streamed stage
constexpr int NF_S_STAGE = 512;                // scale bytes per projection per streamed stage
constexpr int NF_CAP0 = 64, NF_CAP1 = 192;     // rows per tile of the two shapes
constexpr int NF_B_MAX = 8, NF_RAW_MAX = 4, NF_A_MAX = 4;
constexpr int NF_ROW_BYTES = 132;              // staged bytes per row per operand stage: 64 high, 64 low, 4 scale bytes

// Staged rows of a tile (rows16 = rows padded to 16) per operand stage of 64 inputs:
//   [high parts: 4 x (16 inputs) x rows16 x 16 B as K-major core matrices][low parts: the same][rows16 x 4 scale bytes:
//   high block 0, high block 1, low block 0, low block 1]
__host__ __device__ inline size_t nf_stage_bytes(uint32_t rows16) { return (size_t)rows16 * NF_ROW_BYTES; }
__device__ __forceinline__ size_t nf_elem_off(uint32_t rows16, uint32_t row, uint32_t k) {   // high part of (row, input k)
    const uint32_t kk = k % NF_KST;
    return (size_t)(k / NF_KST) * nf_stage_bytes(rows16) + (kk / 16) * (rows16 * 16) + (row / 8) * 128 + (row % 8) * 16 + kk % 16;
}
__device__ __forceinline__ size_t nf_scale_off(uint32_t rows16, uint32_t row, uint32_t k) {  // high scale byte; low: + 2
    return (size_t)(k / NF_KST) * nf_stage_bytes(rows16) + (size_t)rows16 * 128 + row * 4 + (k % NF_KST) / 32;
}

// Block scale from the largest magnitude of a 32-input block (its f32 bits without the sign): the high part's UE8M0 byte
// puts the largest element in [128, 256); the low part's byte is 4 less
__device__ __forceinline__ uint32_t nf_scale_byte(uint32_t amax_bits) {
    const uint32_t ea = amax_bits >> 23;
    return (ea > 11u ? ea : 11u) - 7u;                       // 4 .. 248
}
__device__ __forceinline__ float nf_inv_scale(uint32_t byte_h) { return __uint_as_float((254u - byte_h) << 23); }
// two scaled values -> their E4M3 high and low bytes (element 0 in the low byte)
__device__ __forceinline__ void nf_split2(float q0, float q1, uint32_t& hi2, uint32_t& lo2) {
    uint16_t h, l;
    uint32_t hf;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(h) : "f"(q1), "f"(q0));
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(hf) : "h"(h));
    const float h0 = __half2float(__ushort_as_half((unsigned short)(hf & 0xFFFFu)));
    const float h1 = __half2float(__ushort_as_half((unsigned short)(hf >> 16)));
    const float r0 = (q0 - h0) * 16.0f, r1 = (q1 - h1) * 16.0f;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(l) : "f"(r1), "f"(r0));
    hi2 = h;
    lo2 = l;
}

// ------------------------------------------------------------------------------------------------------------
// prep: gather a tile's rows, split them and lay them out as the B operand.  A thread takes one 32-input block of one
// row (64 bytes in, no exchange between threads); consecutive threads take consecutive rows, so a warp's 16-byte stores
// fill whole core matrices.
// ------------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) nf_prep_kernel(const __nv_bfloat16* __restrict__ x, uint32_t top_k, uint32_t H,
                                                      DispatchTables t, const uint32_t* __restrict__ tiles, uint32_t max_tiles,
                                                      uint8_t* __restrict__ xa) {
    const int list = blockIdx.x >= max_tiles;
    const uint32_t tile = blockIdx.x - (list ? max_tiles : 0u);
    if (tile >= tiles[list]) return;
    const uint32_t* te = prefill_tile(tiles, list, max_tiles, tile);
    const uint32_t row0 = te[1], rows = te[2];
    const uint32_t rows16 = (rows + 15) / 16 * 16, nblk = H / 32;
    uint8_t* dst = xa + (size_t)te[3] * (H / NF_KST) * NF_ROW_BYTES;
    for (uint32_t i = blockIdx.y * blockDim.x + threadIdx.x; i < rows16 * nblk; i += gridDim.y * blockDim.x) {
        const uint32_t r = i % rows16, k = (i / rows16) * 32;
        uint32_t w[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) w[j] = 0u;
        if (r < rows) {
            const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)x_row_of(t, t.order[row0 + r], top_k) * H + k);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint4 v = src[j];
                w[4 * j] = v.x; w[4 * j + 1] = v.y; w[4 * j + 2] = v.z; w[4 * j + 3] = v.w;
            }
        }
        // the largest magnitude of the block: bf16 magnitudes compare as integers
        uint32_t amax = 0;
#pragma unroll
        for (int j = 0; j < 16; ++j) amax = max(amax, max(w[j] & 0x7FFFu, (w[j] >> 16) & 0x7FFFu));
        const uint32_t bh = nf_scale_byte(amax << 16);
        const float inv = nf_inv_scale(bh);
        uint32_t hi[8], lo[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            uint32_t h0, l0, h1, l1;
            nf_split2(__uint_as_float(w[2 * j] << 16) * inv, __uint_as_float(w[2 * j] & 0xFFFF0000u) * inv, h0, l0);
            nf_split2(__uint_as_float(w[2 * j + 1] << 16) * inv, __uint_as_float(w[2 * j + 1] & 0xFFFF0000u) * inv, h1, l1);
            hi[j] = h0 | (h1 << 16);
            lo[j] = l0 | (l1 << 16);
        }
        uint8_t* hp = dst + nf_elem_off(rows16, r, k);
        uint8_t* lp = hp + (size_t)rows16 * 64;
        *reinterpret_cast<uint4*>(hp) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
        *reinterpret_cast<uint4*>(hp + rows16 * 16) = make_uint4(hi[4], hi[5], hi[6], hi[7]);
        *reinterpret_cast<uint4*>(lp) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
        *reinterpret_cast<uint4*>(lp + rows16 * 16) = make_uint4(lo[4], lo[5], lo[6], lo[7]);
        uint8_t* sp = dst + nf_scale_off(rows16, r, k);
        sp[0] = (uint8_t)bh;
        sp[2] = (uint8_t)(bh - 4u);
    }
}

// ------------------------------------------------------------------------------------------------------------
// the kernel
// ------------------------------------------------------------------------------------------------------------
struct NfParams {
    const uint8_t* w;            // layer base of the gate/up or down stream
    size_t expert_stride;
    uint32_t n_blocks, n_stages_k;  // out / 128, in / 128
    const uint8_t* xa;           // B operand: staged rows over this projection's inputs
    const uint32_t* tiles;
    uint32_t max_tiles;
    DispatchTables t;
    uint32_t H, I;
    uint8_t* xd;                 // gate/up output = down's B operand
    void* out;                   // down: ro [A, H] bf16 (chain) or f32
    int out_bf16;
    float limit;
    uint32_t* status;
    uint32_t b_stages, raw_stages, a_stages;
};

__device__ __forceinline__ void umma_mxf8(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t sfa, uint32_t sfb,
                                          uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %6, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale.scale_vec::1X [%0], %1, %2, %3, [%4], [%5], p;\n\t}"
        ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(sfa), "r"(sfb), "r"(accumulate)
        : "memory");
}
// instruction descriptor of the block-scaled kind: b scale byte [4,6), A format [7,10) (E2M1 = 5), B format [10,13)
// (E4M3 = 0), N >> 3 [17,23), scale format [23] (1 = UE8M0), M >> 4 [24,29), a scale byte [29,31)
__device__ __forceinline__ uint32_t nf_idesc(uint32_t n, uint32_t a_sf, uint32_t b_sf) {
    return (b_sf << 4) | (5u << 7) | ((n >> 3) << 17) | (1u << 23) | ((128u >> 4) << 24) | (a_sf << 29);
}
__device__ __forceinline__ void tmem_st1_nowait(uint32_t taddr, uint32_t v) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x1.b32 [%0], {%1};" ::"r"(taddr), "r"(v) : "memory");
}
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ float nf_sigmoid(float x) {  // src/arch/mimo_v2/moe.zig:341-344
    const float y = sigmoid_tail_fast(x);
    return x < 0.f ? y : 1.0f - y;
}

// NPROJ projections x CB adjacent 128-column blocks = NG accumulator groups of NT tensor-memory columns each.  Tensor
// memory after the accumulators: per operand stage NG x 8 columns of weight scales (4 used: column + lane quarter) and 8
// columns of row scales (row n: lane n % 32 of every quarter, column + n / 32; bytes 0, 1 high part, 2, 3 low part).
template <int NPROJ, int CB, int NT, int PER_SM>
__global__ void __launch_bounds__(512 + 64, PER_SM) mxfp4_native_kernel(const NfParams P) {
    constexpr int NG = NPROJ * CB;
    constexpr int SFC = NG * 8 + 8;
    constexpr int TCOLS = 512 / PER_SM;                               // tensor-memory columns of this CTA (PER_SM CTAs share an SM)
    constexpr int LIST = NT == NF_CAP0 ? 0 : 1;
    constexpr int NCW = 16;
    constexpr uint32_t B_SLOT = NT * NF_ROW_BYTES;
    constexpr uint32_t A_SLOT = NG * 8192;                            // an operand stage of codes in operand geometry
    constexpr uint32_t W_BYTES = NPROJ * (NF_W_STAGE + NF_S_STAGE);   // one block's stage of the stream
    constexpr uint32_t RAW_BYTES = CB * W_BYTES;
    static_assert((NG == 2 || NG == 4) && NG * NT + 2 * SFC <= TCOLS, "shape");
    extern __shared__ __align__(128) uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t raw_full[NF_RAW_MAX], raw_empty[NF_RAW_MAX];
    __shared__ __align__(8) uint64_t b_full[NF_B_MAX], b_empty[NF_B_MAX], a_full[NF_A_MAX], a_empty[NF_A_MAX];
    __shared__ __align__(8) uint64_t acc_full, acc_empty;
    __shared__ uint32_t s_tmem;
    __shared__ volatile int s_abort;
    const uint32_t B_STAGES = P.b_stages, RAW_STAGES = P.raw_stages, A_STAGES = P.a_stages;
    uint8_t* a_ring = smem_raw;                                        // [stage][NG][2 blocks][2 x 2048]
    uint8_t* b_ring = a_ring + A_STAGES * A_SLOT;                      // [stage][B_SLOT]
    uint8_t* raw_ring = b_ring + B_STAGES * B_SLOT;                    // [stage][CB][W_BYTES]
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t nbg = P.n_blocks / CB;
    const uint32_t n_items = P.tiles[LIST] * nbg;
    if (blockIdx.x >= n_items) return;   // before any tensor memory is taken (the whole CTA reads the same count)

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < RAW_STAGES; ++s) { mbar_init(&raw_full[s], 1); mbar_init(&raw_empty[s], NCW); }
        for (uint32_t s = 0; s < A_STAGES; ++s) { mbar_init(&a_full[s], NCW); mbar_init(&a_empty[s], 1); }
        for (uint32_t s = 0; s < B_STAGES; ++s) { mbar_init(&b_full[s], 1); mbar_init(&b_empty[s], 1); }
        mbar_init(&acc_full, 1);
        mbar_init(&acc_empty, NCW);
        s_abort = 0;
        mbar_fence_init();
    }
    // the unused high halves of the operand rows stay zero for the whole kernel
    for (uint32_t i = threadIdx.x; i < A_STAGES * A_SLOT / 16; i += blockDim.x) reinterpret_cast<uint4*>(a_ring)[i] = make_uint4(0, 0, 0, 0);
    if (warp == 0) tmem_alloc(&s_tmem, TCOLS);
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = s_tmem, tmem_sf = tmem + NG * NT;
    const uint32_t nstage = P.n_stages_k, width = nstage * NF_KS;
    auto give_up = [&](uint32_t code) { if (!s_abort) atomicMax(P.status, code); s_abort = 1; };

    if (warp == NCW) {
        // ---------------- producer: code/scale stream + rows ----------------
        if (lane == 0) {
            uint32_t rs = 0, rph = 0, bs = 0, bph = 0;
            for (uint32_t item = blockIdx.x; item < n_items && !s_abort; item += gridDim.x) {
                const uint32_t nb0 = (item % nbg) * CB;
                const uint32_t* te = prefill_tile(P.tiles, LIST, P.max_tiles, item / nbg);
                const uint32_t expert = te[0], rows16 = (te[2] + 15) / 16 * 16, b_bytes = rows16 * NF_ROW_BYTES;
                const uint8_t* wsrc = P.w + (size_t)expert * P.expert_stride + (size_t)nb0 * nstage * W_BYTES;
                const uint8_t* xsrc = P.xa + (size_t)te[3] * (width / NF_KST) * NF_ROW_BYTES;
                bool ok = true;
                for (uint32_t ks = 0; ks < nstage && ok; ++ks) {
                    if (!mbar_wait_bounded(&raw_empty[rs], rph ^ 1u, &s_abort, 64)) { give_up(ST_WAIT_EMPTY); ok = false; break; }
                    mbar_expect_tx(&raw_full[rs], RAW_BYTES);
                    for (int cb = 0; cb < CB; ++cb)
                        bulk_g2s(raw_ring + rs * RAW_BYTES + cb * W_BYTES, wsrc + ((size_t)cb * nstage + ks) * W_BYTES, W_BYTES,
                                 &raw_full[rs]);
                    if (++rs == RAW_STAGES) { rs = 0; rph ^= 1u; }
                    for (uint32_t os = 0; os < NF_KS / NF_KST; ++os) {
                        if (!mbar_wait_bounded(&b_empty[bs], bph ^ 1u, &s_abort, 64)) { give_up(ST_WAIT_EMPTY); ok = false; break; }
                        mbar_expect_tx(&b_full[bs], b_bytes);
                        bulk_g2s(b_ring + bs * B_SLOT, xsrc, b_bytes, &b_full[bs]);
                        xsrc += b_bytes;
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
            uint32_t as = 0, aph = 0, bs = 0, nitem = 0;
            const uint32_t a_ring_s = smem_u32(a_ring), b_ring_s = smem_u32(b_ring);
            for (uint32_t item = blockIdx.x; item < n_items && !s_abort; item += gridDim.x, ++nitem) {
                const uint32_t rows16 = (prefill_tile(P.tiles, LIST, P.max_tiles, item / nbg)[2] + 15) / 16 * 16;
                const uint32_t lbo_b = rows16 * 16;
                if (!mbar_wait_bounded(&acc_empty, (nitem & 1u) ^ 1u, &s_abort, 64)) { give_up(ST_WAIT_EMPTY); break; }
                tc_fence_after();
                bool ok = true;
                const uint32_t nk = nstage * (NF_KS / NF_KST);
                for (uint32_t kk = 0; kk < nk; ++kk) {
                    if (!mbar_wait_bounded(&a_full[as], aph, &s_abort)) { give_up(ST_WAIT_FULL); ok = false; break; }
                    tc_fence_after();
                    const uint32_t os = kk & 1u;                       // which half of the streamed stage: weight scale bytes 2 os, 2 os + 1
                    const uint32_t b_s = b_ring_s + bs * B_SLOT, sf = tmem_sf + as * SFC, sfb = sf + NG * 8;
#pragma unroll
                    for (int gq = 0; gq < NG; ++gq) {
#pragma unroll
                        for (int j = 0; j < 2; ++j) {
                            const uint64_t da = umma_smem_desc(a_ring_s + as * A_SLOT + gq * 8192 + j * 4096, 2048, 128);
                            const uint64_t dh = umma_smem_desc(b_s + j * 2 * lbo_b, lbo_b, 128);
                            const uint64_t dl = umma_smem_desc(b_s + rows16 * 64 + j * 2 * lbo_b, lbo_b, 128);
                            umma_mxf8(tmem + gq * NT, da, dh, nf_idesc(rows16, os * 2 + j, j), sf + gq * 8, sfb, (kk | (uint32_t)j) ? 1u : 0u);
                            umma_mxf8(tmem + gq * NT, da, dl, nf_idesc(rows16, os * 2 + j, 2 + j), sf + gq * 8, sfb, 1u);
                        }
                    }
                    // A commit costs the issuing thread about as much as an MMA.  The large shape commits once per
                    // stage (the operand slot; operand warp 0, when it sees that slot free, frees the rows' slot of the
                    // same stage); the two-CTA shape, whose rows' ring is short, commits both
                    umma_commit(&a_empty[as]);
                    if (PER_SM != 1) umma_commit(&b_empty[bs]);
                    if (++as == A_STAGES) { as = 0; aph ^= 1u; }
                    if (++bs == B_STAGES) bs = 0;
                }
                if (!ok) break;
                umma_commit(&acc_full);
            }
        }
    } else {
        // ---------------- operand warps + epilogue ----------------
        // Warp = (lane quarter q = warp % 4, slot = warp / 4).  Codes: the 16 warps share the stage's 16-byte chunks.
        // Weight scales: the warps of slot gq < NG own group gq (a thread owns output column m = 32 q + lane).  Row
        // scales: the warps of slot 3, each into its own lane quarter.
        const uint32_t q = warp & 3u, slot = warp >> 2;
        const uint32_t m = q * 32u + lane, wr = m >> 4, r = (m >> 3) & 1u, g = m & 7u;
        const bool sf_warp = slot < (uint32_t)NG, b_warp = slot == 3u;
        const uint32_t sgq = sf_warp ? slot : 0u, sp = NPROJ == 2 ? sgq / CB : 0u, scb = NPROJ == 2 ? sgq % CB : sgq;
        uint32_t rs = 0, rph = 0, as = 0, aph = 0, bs = 0, bph = 0, nitem = 0;
        uint32_t n_stage = 0, rel_bs = 0;   // operand stages so far; the rows' slot to free next (A_STAGES stages behind)
        for (uint32_t item = blockIdx.x; item < n_items && !s_abort; item += gridDim.x, ++nitem) {
            const uint32_t nb0 = (item % nbg) * CB;
            const uint32_t* te = prefill_tile(P.tiles, LIST, P.max_tiles, item / nbg);
            const uint32_t row0 = te[1], rows = te[2], srow0 = te[3];
            const uint32_t rows16 = (rows + 15) / 16 * 16;
            bool ok = true;
            for (uint32_t ks = 0; ks < nstage && ok; ++ks) {
                if (!mbar_wait_bounded(&raw_full[rs], rph, &s_abort)) { give_up(ST_WAIT_FULL); ok = false; break; }
                const uint8_t* stage = raw_ring + rs * RAW_BYTES;
                uint32_t sword = 0;
                if (sf_warp) {
                    // this column's four block scales of the streamed stage: [wr][block][g][r] bytes
                    const uint8_t* sc = stage + scb * W_BYTES + NPROJ * NF_W_STAGE + sp * NF_S_STAGE;
#pragma unroll
                    for (uint32_t sb = 0; sb < 4; ++sb) sword |= (uint32_t)sc[((wr * 4 + sb) * 8 + g) * 2 + r] << (8 * sb);
                }
#pragma unroll
                for (int os = 0; os < NF_KS / NF_KST; ++os) {
                    if (!mbar_wait_bounded(&a_empty[as], aph ^ 1u, &s_abort)) { give_up(ST_WAIT_FULL); ok = false; break; }
                    tc_fence_after();
                    // the slot is free: the MMAs of the stage that used it (A_STAGES stages back) are done with their rows too
                    if (PER_SM == 1 && warp == 0) {
                        if (n_stage >= A_STAGES) {
                            if (lane == 0) mbar_arrive(&b_empty[rel_bs]);
                            if (++rel_bs == B_STAGES) rel_bs = 0;
                        }
                        ++n_stage;
                    }
                    // codes: chunk c of group gq = (wr, block of the stage, r, g): 32 codes of one column and block ->
                    // the low halves of two operand rows, 2048 bytes apart along K
                    uint8_t* a_slot = a_ring + as * A_SLOT;
#pragma unroll
                    for (uint32_t n = 0; n < NG * 256 / 512; ++n) {
                        const uint32_t id = n * 512 + warp * 32 + lane, gq = id >> 8, c = id & 255u;
                        const uint32_t cwr = c >> 5, sbl = (c >> 4) & 1u, cr = (c >> 3) & 1u, cg = c & 7u;
                        const uint32_t p = NPROJ == 2 ? gq / CB : 0u, cb = NPROJ == 2 ? gq % CB : gq;
                        const uint4 ww = *reinterpret_cast<const uint4*>(stage + cb * W_BYTES + p * NF_W_STAGE +
                                                                         ((((cwr * 4 + (os * 2 + sbl)) * 2 + cr) * 8 + cg) * 16));
                        uint8_t* d = a_slot + gq * 8192 + sbl * 4096 + (cwr * 2 + cr) * 128 + cg * 16;
                        *reinterpret_cast<uint2*>(d) = make_uint2(ww.x, ww.y);
                        *reinterpret_cast<uint2*>(d + 2048) = make_uint2(ww.z, ww.w);
                    }
                    const uint32_t sf = tmem_sf + as * SFC + ((q * 32u) << 16);
                    if (sf_warp) tmem_st1_nowait(sf + sgq * 8 + q, sword);
                    if (b_warp) {
                        if (!mbar_wait_bounded(&b_full[bs], bph, &s_abort)) { give_up(ST_WAIT_FULL); ok = false; break; }
                        const uint32_t* bsc = reinterpret_cast<const uint32_t*>(b_ring + bs * B_SLOT + rows16 * 128);
#pragma unroll
                        for (uint32_t c = 0; c < NT / 32; ++c)
                            if (c * 32 < rows16) tmem_st1_nowait(sf + NG * 8 + c, bsc[c * 32 + lane < rows16 ? c * 32 + lane : 0]);
                        if (++bs == B_STAGES) { bs = 0; bph ^= 1u; }
                    }
                    tmem_wait_st();
                    tc_fence_before();
                    fence_async_smem();
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
            const uint32_t nrb = rows16 / 16;
            if (NPROJ == 2) {
                uint8_t* xd_tile = P.xd + (size_t)srow0 * (P.I / NF_KST) * NF_ROW_BYTES;
                for (uint32_t unit = slot; unit < CB * nrb; unit += 4) {
                    const uint32_t ecb = unit / nrb, rb = (unit % nrb) * 16;
                    uint32_t vg[16], vu[16];
                    tmem_ld16(tmem + ((q * 32u) << 16) + (0 * CB + ecb) * NT + rb, vg);
                    tmem_ld16(tmem + ((q * 32u) << 16) + (1 * CB + ecb) * NT + rb, vu);
                    const uint32_t col = (nb0 + ecb) * 128 + m;         // this warp's 32 columns are one 32-input block of down
                    float hq[16];
                    uint32_t my_byte = 0;
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        // mimo_moe_k1_gateup.metal:115-128
                        float gf = bf16_round_f(__uint_as_float(vg[i])), uf = bf16_round_f(__uint_as_float(vu[i]));
                        if (P.limit > 0.f) {
                            gf = gf > P.limit ? P.limit : gf;
                            uf = uf > P.limit ? P.limit : (uf < -P.limit ? -P.limit : uf);
                        }
                        float hv = bf16_round_f(bf16_round_f(gf * nf_sigmoid(gf)) * uf);
                        if (rb + i >= rows) hv = 0.f;
                        const uint32_t bh = nf_scale_byte(__reduce_max_sync(0xFFFFFFFFu, __float_as_uint(hv) & 0x7FFFFFFFu));
                        hq[i] = hv * nf_inv_scale(bh);
                        if ((lane & 15u) == (uint32_t)i) my_byte = lane < 16u ? bh : bh - 4u;
                    }
                    uint8_t* hi_p = xd_tile + nf_elem_off(rows16, rb, col);
                    uint8_t* lo_p = hi_p + (size_t)rows16 * 64;
#pragma unroll
                    for (int i = 0; i < 16; i += 2) {
                        uint32_t hi2, lo2;
                        nf_split2(hq[i], hq[i + 1], hi2, lo2);
                        hi_p[i * 16] = (uint8_t)(hi2 & 0xFFu);
                        hi_p[i * 16 + 16] = (uint8_t)(hi2 >> 8);
                        lo_p[i * 16] = (uint8_t)(lo2 & 0xFFu);
                        lo_p[i * 16 + 16] = (uint8_t)(lo2 >> 8);
                    }
                    // lanes 0..15: the high scale byte of row rb + lane; lanes 16..31: the low scale byte of row rb + lane - 16
                    xd_tile[nf_scale_off(rows16, rb + (lane & 15u), col) + (lane < 16u ? 0u : 2u)] = (uint8_t)my_byte;
                }
            } else {
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
                        const float z = __uint_as_float(v[i]);
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

template <int NPROJ, int CB, int NT, int PER_SM>
static cudaError_t nf_launch(NfParams P, int sm_count, cudaStream_t st) {
    constexpr int NG = NPROJ * CB;
    const size_t raw_bytes = (size_t)CB * NPROJ * (NF_W_STAGE + NF_S_STAGE), b_slot = (size_t)NT * NF_ROW_BYTES, a_slot = (size_t)NG * 8192;
    const size_t budget = PER_SM == 1 ? 222 * 1024 : 110 * 1024;
    // the large shape has two operand slots: a rows' slot is freed two stages after its use, and the rows' ring wants to
    // be deeper than that
    const uint32_t a_max = (512 / PER_SM - NG * NT) / (NG * 8 + 8);
    const uint32_t a_want = PER_SM == 1 ? 2u : 3u;
    P.a_stages = a_max < a_want ? a_max : a_want;
    P.raw_stages = 3;
    while (P.raw_stages > 2 && P.a_stages * a_slot + P.raw_stages * raw_bytes + 3 * b_slot > budget) --P.raw_stages;
    while (P.a_stages > 2 && P.a_stages * a_slot + P.raw_stages * raw_bytes + 3 * b_slot > budget) --P.a_stages;
    size_t nb = (budget - P.a_stages * a_slot - P.raw_stages * raw_bytes) / b_slot;
    P.b_stages = (uint32_t)(nb > (size_t)NF_B_MAX ? (size_t)NF_B_MAX : nb);
    if (P.b_stages < 2) return cudaErrorInvalidConfiguration;
    if (P.a_stages > P.b_stages) P.a_stages = P.b_stages;
    const size_t smem = P.a_stages * a_slot + P.b_stages * b_slot + P.raw_stages * raw_bytes;
    cudaError_t e = cudaFuncSetAttribute(mxfp4_native_kernel<NPROJ, CB, NT, PER_SM>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    mxfp4_native_kernel<NPROJ, CB, NT, PER_SM><<<PER_SM * sm_count, 512 + 64, smem, st>>>(P);
    return cudaGetLastError();
}

cudaError_t launch_mxfp4_native(const Fp4PrefillArgs& a, cudaStream_t st) {
    cudaError_t e = launch_prefill_plan(a.t, a.n_experts, a.lane_flags, a.min_rows, NF_CAP0, NF_CAP1, a.max_tiles, a.tiles, a.status, st);
    if (e != cudaSuccess) return e;
    uint8_t* xa = reinterpret_cast<uint8_t*>(a.xa);
    uint8_t* xd = reinterpret_cast<uint8_t*>(a.xd);
    nf_prep_kernel<<<dim3(2 * a.max_tiles, 8), 256, 0, st>>>(a.x, a.top_k, a.H, a.t, a.tiles, a.max_tiles, xa);
    if ((e = cudaGetLastError()) != cudaSuccess) return e;
    NfParams P{};
    P.tiles = a.tiles; P.max_tiles = a.max_tiles; P.t = a.t; P.H = a.H; P.I = a.I; P.limit = a.limit; P.status = a.status;
    P.w = a.gu; P.n_blocks = a.I / 128; P.n_stages_k = a.H / NF_KS;
    P.expert_stride = (size_t)P.n_blocks * P.n_stages_k * 2 * (NF_W_STAGE + NF_S_STAGE);
    P.xa = xa; P.xd = xd; P.out = nullptr; P.out_bf16 = 0;
    NfParams D = P;
    D.w = a.dn; D.n_blocks = a.H / 128; D.n_stages_k = a.I / NF_KS;
    D.expert_stride = (size_t)D.n_blocks * D.n_stages_k * (NF_W_STAGE + NF_S_STAGE);
    D.xa = xd; D.xd = nullptr; D.out = a.ro; D.out_bf16 = a.ro_bf16;
    // the two tile lists hold different experts and rows: the large tiles' kernels run beside the small tiles' when the
    // call has a side stream for them
    return prefill_lists_side_by_side(st, a.side, a.side_fork, a.side_join, [&](cudaStream_t s1) {
        cudaError_t r = nf_launch<2, 1, NF_CAP1, 1>(P, a.sm_count, s1);
        if (r == cudaSuccess && a.side) r = nf_launch<1, 2, NF_CAP1, 1>(D, a.sm_count, s1);
        if (r == cudaSuccess) r = nf_launch<2, 1, NF_CAP0, 2>(P, a.sm_count, st);
        if (r == cudaSuccess) r = nf_launch<1, 2, NF_CAP0, 2>(D, a.sm_count, st);
        if (r == cudaSuccess && !a.side) r = nf_launch<1, 2, NF_CAP1, 1>(D, a.sm_count, st);
        return r;
    });
}

}  // namespace mlxs
