// MXFP4 / NVFP4 expert kernels for decode-sized batches.
//
// Weight formats (the reference's own records): codes U32 [out, in/8] (code j of a word at bits 4j), MXFP4 block scale
// U8 E8M0 [out, in/32] (src/arch/mimo_v2/moe.zig:379-416), NVFP4 block scale U8 E4M3 [out, in/16] plus one f32 global
// scale per projection, w = (e4m3 * g/2688) * e2m1 (src/arch/glm5_next/decode_kernels_ref.zig:13-65).
//
// Same streaming structure as the EXL3 kernels: a CTA owns 128 output rows of one expert for up to 16 token rows,
// a producer warp streams the block's bytes through a bulk-copy ring, a consumer warp owns 16 output rows and turns
// its codes into f16 with the e2m1x2 conversion instruction (two codes per instruction, exact values; the reference
// places the code bits with integer ops, src/arch/mimo_v2/kernels/header_mimo_moe_k1.metal:7-12) straight into the mma
// A fragment.  MXFP4: the two mma of a 32-block accumulate into a fresh fragment that is folded with the block's
// power-of-two scale in f32 (exact).  NVFP4: the decoded halves are multiplied by the block's E4M3 scale in f16, which
// is exact (a 2-bit by 4-bit significand product of at most 6 x 448); the global g/2688 is applied once per output in f32.
#include <cstdlib>

#include "common.cuh"
#include "kernels.h"
#include "fp4_prep_body.cuh"

namespace mlxs {

constexpr int F4_KS = 128;           // inputs per pipeline stage (4 sub-blocks of 32)
constexpr int F4_CHUNK = 8;          // token rows per mma n-tile
constexpr int F4_GROUP = 2;          // chunks per work item
constexpr int F4_W_STAGE = 8192;     // bytes of codes per projection per stage: 128 rows x 128 inputs / 2
constexpr int F4_ZS_STRIDE = 132;

__host__ __device__ inline uint32_t f4_scale_stage_bytes(bool nv) { return nv ? 1024u : 512u; }

// ------------------------------------------------------------------------------------------------------------
// load-time repack (bit-preserving)
// ------------------------------------------------------------------------------------------------------------
// dst per (128-row block nb, stage ks): [proj][warp 8][sb 4][r 2][lane 32] codes, then [proj][warp 8][sb 4][...] scales:
//   MXFP4 scales [g 8][r 2] bytes; NVFP4 scales [blk 2][g 8][r 2] bytes.  lane = (g, c): word c of the 32-block for
//   rows 16 warp + g (r = 0) and 16 warp + g + 8 (r = 1).  A warp of the streaming lane reads two runs of 32 words;
//   a thread of the tensor-core lane reads the four words of one output row (r, g) as one 16-byte load.
__global__ void fp4_repack_kernel(const uint8_t* __restrict__ rec, uint32_t H, uint32_t I, int nv,
                                  uint8_t* __restrict__ gu, uint8_t* __restrict__ dn, float* __restrict__ gscale,
                                  uint8_t* lane_flag) {
    const size_t wbytes = (size_t)H * I / 2, sbytes = (size_t)H * I / (nv ? 16 : 32), tail = nv ? 4 : 0;
    const size_t part = wbytes + sbytes + tail;
    const uint32_t sstage = f4_scale_stage_bytes(nv != 0);
    const size_t stride = (size_t)gridDim.x * blockDim.x, tid0 = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (nv && tid0 < 3) gscale[tid0] = *reinterpret_cast<const float*>(rec + tid0 * part + wbytes + sbytes);
    for (int proj = 0; proj < 3; ++proj) {
        const uint32_t rows = proj == 2 ? H : I, cols = proj == 2 ? I : H;
        const uint32_t* w = reinterpret_cast<const uint32_t*>(rec + proj * part);
        const uint8_t* s = rec + proj * part + wbytes;
        const uint32_t nstage = cols / F4_KS, np = proj == 2 ? 1 : 2, pp = proj == 2 ? 0 : proj;
        uint8_t* dst = proj == 2 ? dn : gu;
        const size_t stage_bytes = (size_t)np * (F4_W_STAGE + sstage);
        // codes
        for (size_t i = tid0; i < (size_t)rows * cols / 8; i += stride) {
            const uint32_t row = (uint32_t)(i / (cols / 8)), wi = (uint32_t)(i % (cols / 8));
            const uint32_t nb = row / 128, wr = (row % 128) / 16, rr = row % 16, g = rr % 8, r = rr / 8;
            const uint32_t ks = wi / 16, sb = (wi % 16) / 4, c = wi % 4;
            uint32_t* d = reinterpret_cast<uint32_t*>(dst + ((size_t)nb * nstage + ks) * stage_bytes + (size_t)pp * F4_W_STAGE);
            d[((wr * 4 + sb) * 2 + r) * 32 + g * 4 + c] = w[i];
        }
        // scales
        const uint32_t per_row = cols / (nv ? 16 : 32);
        for (size_t i = tid0; i < (size_t)rows * per_row; i += stride) {
            const uint32_t row = (uint32_t)(i / per_row), bi = (uint32_t)(i % per_row);
            const uint32_t nb = row / 128, wr = (row % 128) / 16, rr = row % 16, g = rr % 8, r = rr / 8;
            const uint32_t blk32 = nv ? bi / 2 : bi, half = nv ? bi % 2 : 0;
            const uint32_t ks = blk32 / 4, sb = blk32 % 4;
            uint8_t* d = dst + ((size_t)nb * nstage + ks) * stage_bytes + (size_t)np * F4_W_STAGE + (size_t)pp * sstage;
            if (nv) d[(((wr * 4 + sb) * 2 + half) * 8 + g) * 2 + r] = s[i];
            else {
                d[((wr * 4 + sb) * 8 + g) * 2 + r] = s[i];
                // the tensor-core lane forms 2^(b-1) as a bf16: b > 128 keeps this expert in the streaming lane
                if (lane_flag && s[i] > 128u) *lane_flag = 3;
            }
        }
    }
}

cudaError_t launch_fp4_repack(const uint8_t* record_dev, uint32_t H, uint32_t I, int nv, uint8_t* gu_e, uint8_t* dn_e,
                              float* gscale_e, uint8_t* lane_flag, cudaStream_t st) {
    fp4_repack_kernel<<<592, 256, 0, st>>>(record_dev, H, I, nv, gu_e, dn_e, gscale_e, lane_flag);
    return cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------------------
// activation staging: bf16 rows -> f16 in the kernels' B-fragment order
// ------------------------------------------------------------------------------------------------------------
// per (chunk of 8 rows, 32-block): lane (g = row slot, c) holds 4 u32: {x[8c+0],x[8c+1]}, {x[8c+2],x[8c+3]},
// {x[8c+4],x[8c+5]}, {x[8c+6],x[8c+7]} (the first two feed the block's first mma, the others the second): the order in
// which the conversion instruction hands out a word's eight codes
__global__ void __launch_bounds__(256) fp4_prep_kernel(const __nv_bfloat16* __restrict__ x, uint32_t top_k, uint32_t H,
                                                       DispatchTables t, uint32_t* __restrict__ xa) {
    const uint32_t chunk = blockIdx.x;
    if (chunk >= t.header[HDR_NCHUNKS]) return;
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;  // warp = row slot
    const bool valid = warp < t.chunk_rows[chunk];
    const uint32_t tok = valid ? x_row_of(t, t.order[t.chunk_row0[chunk] + warp], top_k) : 0u;
    fp4_prep_row(x, tok, valid, H, chunk, warp, blockIdx.y * 32 + lane, gridDim.y * 32, xa);
}

cudaError_t launch_fp4_prep(const __nv_bfloat16* x, uint32_t top_k, uint32_t H, DispatchTables t, uint32_t* xa,
                            cudaStream_t st) {
    fp4_prep_kernel<<<dim3(t.max_chunks, 4), 256, 0, st>>>(x, top_k, H, t, xa);
    return cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------------------
// the streaming kernel
// ------------------------------------------------------------------------------------------------------------
struct Fp4Params {
    const uint8_t* w;            // layer base of the gate/up or down stream
    size_t expert_stride;        // bytes per expert in that stream
    const float* gscale;         // NVFP4: [E][3] global scales, else null
    uint32_t n_blocks, n_stages_k;  // out / 128, in / 128
    uint32_t max_parts;          // cap on the parts of the sum (4; a tuning knob for measurements, MLXS_K_PARTS)
    uint32_t sub;                // 128-input sub-stages per ring stage (one barrier round trip serves `sub` of them)
    const uint32_t* xa;          // [chunk][in/32][128] u32
    DispatchTables t;
    uint32_t counter_idx;
    uint32_t H, I;
    uint32_t* xa_d;              // gate/up epilogue output: [chunk][I/32][128] u32
    void* out;                   // down: ro [A, H] bf16 (chain) or f32
    int out_bf16;
    float limit;                 // > 0: clamped epilogue (glm5n_nvfp4_gateup.metal:109-129), else MiMo's
    uint32_t* status;
    uint32_t n_ring, stage_bytes, w_bytes;
    // The sum over the inputs is taken in `parts` equal parts folded left in part order (a function of the shape only, so
    // a row's bits do not depend on the batch); calls with fewer items than CTAs spread an item's parts over 2 or 4
    // CTAs, as the EXL3 streaming kernel does
    float* ks_scratch;           // [items][parts][zs words] or null
    uint32_t* ks_count;          // [ks_cap_items or more], zero between launches
    uint32_t n_sm, ks_cap_items; // SMs of the device; items the workspace and the counters hold
};

// flags: 1 = first stage of a part of the sum, 2 = last stage of a part, 4 = last stage of this CTA's share of the item
// Only `item` and `flags` (with the chunk count in bits 8..) are read every stage, the rest at the end of a part.
struct F4Meta { int32_t item; uint32_t flags, mc, ks, chunk0, expert, nb, part; };

// Eight e2m1 codes of a word -> four f16x2 through sm_100a's e2m1x2 conversion (one instruction per two codes, exact
// values): h[i] = codes (2i, 2i + 1).  Measured against placing the code bits with shifts and masks (two logic ops per
// weight on the half-rate pipe): the gate/up stream went from 0.57 to 0.77 of the measured HBM rate.
__device__ __forceinline__ void fp4_decode8(uint32_t w, uint32_t (&h)[4]) {
    asm("{\n\t.reg .b8 b0, b1, b2, b3;\n\t"
        "mov.b32 {b0, b1, b2, b3}, %4;\n\t"
        "cvt.rn.f16x2.e2m1x2 %0, b0;\n\t"
        "cvt.rn.f16x2.e2m1x2 %1, b1;\n\t"
        "cvt.rn.f16x2.e2m1x2 %2, b2;\n\t"
        "cvt.rn.f16x2.e2m1x2 %3, b3;\n\t}"
        : "=r"(h[0]), "=r"(h[1]), "=r"(h[2]), "=r"(h[3])
        : "r"(w));
}
// E4M3 byte -> half2 (both halves) of its value (glm5n_e4m3: bits << 7 is the value x 2^-8 as f16; x 256 is exact)
__device__ __forceinline__ __half2 e4m3_half2(uint32_t b) {
    const uint32_t v = b & 127u;
    const uint32_t u = (v << 7) | (((v + 1u) >> 7) << 14) | ((b & 128u) << 8);
    const uint32_t uu = u * 0x00010001u;
    const uint32_t k256 = 0x5C005C00u;
    return __hmul2(*reinterpret_cast<const __half2*>(&uu), *reinterpret_cast<const __half2*>(&k256));
}
__device__ __forceinline__ uint32_t hmul2_u32(uint32_t a, __half2 s) {
    __half2 r = __hmul2(*reinterpret_cast<__half2*>(&a), s);
    return *reinterpret_cast<uint32_t*>(&r);
}

template <int NPROJ, bool NV, int MC>
__device__ __forceinline__ void fp4_stage(const uint8_t* __restrict__ st, const uint8_t* __restrict__ xs, uint32_t x_mt_stride,
                                          uint32_t p, uint32_t j, uint32_t lane, const uint32_t* __restrict__ lut,
                                          float (&acc)[F4_GROUP][4]) {
    // st: one 128-input sub-stage of codes and scales; xs: the same sub-stage of the first chunk's rows, the next
    // chunk's x_mt_stride uint4 further
    const uint32_t* wv = reinterpret_cast<const uint32_t*>(st + (size_t)p * F4_W_STAGE) + (j * 4) * 64 + lane;
    const uint8_t* sc = st + (size_t)NPROJ * F4_W_STAGE + (size_t)p * f4_scale_stage_bytes(NV);
    const uint4* xv = reinterpret_cast<const uint4*>(xs) + lane;
    const uint32_t g = lane >> 2, c = lane & 3u;
#pragma unroll
    for (int sb = 0; sb < 4; ++sb) {
        const uint2 ww = make_uint2(wv[sb * 64], wv[sb * 64 + 32]);
        uint32_t hx[4], hy[4];
        fp4_decode8(ww.x, hx);
        fp4_decode8(ww.y, hy);
        float s_lo = 1.f, s_hi = 1.f;
        if (NV) {
            const uint32_t bb = *reinterpret_cast<const uint16_t*>(sc + (((j * 4 + sb) * 2 + (c >> 1)) * 8 + g) * 2);
            const uint32_t u0 = lut[bb & 0xFFu], u1 = lut[bb >> 8];  // E4M3 byte -> f16x2 of its value
            const __half2 sg = *reinterpret_cast<const __half2*>(&u0), sg8 = *reinterpret_cast<const __half2*>(&u1);
#pragma unroll
            for (int i = 0; i < 4; ++i) { hx[i] = hmul2_u32(hx[i], sg); hy[i] = hmul2_u32(hy[i], sg8); }
        } else {
            const uint32_t bb = *reinterpret_cast<const uint16_t*>(sc + ((j * 4 + sb) * 8 + g) * 2);
            // 2^(b - 127); b = 0 is the subnormal 2^-127 (src/arch/mimo_v2/moe.zig:410-413)
            const uint32_t b0 = bb & 0xFFu, b1 = bb >> 8;
            s_lo = __uint_as_float(b0 ? b0 << 23 : 0x00400000u);
            s_hi = __uint_as_float(b1 ? b1 << 23 : 0x00400000u);
        }
        const uint32_t a1[4] = {hx[0], hy[0], hx[1], hy[1]}, a2[4] = {hx[2], hy[2], hx[3], hy[3]};
#pragma unroll
        for (int mt = 0; mt < MC; ++mt) {
            const uint4 xq = xv[mt * x_mt_stride + sb * 32];
            if (NV) {
                mma_f16(acc[mt], a1, xq.x, xq.y);
                mma_f16(acc[mt], a2, xq.z, xq.w);
            } else {
                float tmp[4] = {0.f, 0.f, 0.f, 0.f};
                mma_f16(tmp, a1, xq.x, xq.y);
                mma_f16(tmp, a2, xq.z, xq.w);
                acc[mt][0] = fmaf(tmp[0], s_lo, acc[mt][0]); acc[mt][1] = fmaf(tmp[1], s_lo, acc[mt][1]);
                acc[mt][2] = fmaf(tmp[2], s_hi, acc[mt][2]); acc[mt][3] = fmaf(tmp[3], s_hi, acc[mt][3]);
            }
        }
    }
}

// SUB sub-stages of one ring slot, unrolled
template <int NPROJ, bool NV, int MC, int SUB>
__device__ __forceinline__ void fp4_slot(const uint8_t* __restrict__ st, const uint8_t* __restrict__ xs, uint32_t w_bytes,
                                         uint32_t x_mt_stride, uint32_t p, uint32_t j, uint32_t lane,
                                         const uint32_t* __restrict__ lut, float (&acc)[F4_GROUP][4]) {
#pragma unroll
    for (int u = 0; u < SUB; ++u)
        fp4_stage<NPROJ, NV, MC>(st + u * w_bytes, xs + u * (4 * F4_XA_SB_WORDS * 4), x_mt_stride, p, j, lane, lut, acc);
}

__device__ __forceinline__ float sigmoid_ref(float x) {  // src/arch/mimo_v2/moe.zig:341-344 (MLX's f32 sigmoid)
    const float y = 1.0f / (1.0f + expf(fabsf(x)));
    return x < 0.f ? y : 1.0f - y;
}

template <int NPROJ, bool NV>
__global__ void __launch_bounds__(NPROJ * 256 + 32, NPROJ == 1 ? 3 : 2) fp4_gemv_kernel(const Fp4Params P) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    constexpr int NCW = NPROJ * 8;
    constexpr int MAXS = 8;
    __shared__ __align__(8) uint64_t full_bar[MAXS], empty_bar[MAXS], epi_bar;
    __shared__ __align__(8) F4Meta meta[MAXS];
    __shared__ volatile int s_abort;
    __shared__ volatile int s_last_part;
    __shared__ uint32_t s_lut[NV ? 256 : 1];
    float* zs = reinterpret_cast<float*>(smem_raw);  // [NPROJ][F4_GROUP][8 rows][F4_ZS_STRIDE]
    uint8_t* ring = smem_raw + (size_t)NPROJ * F4_GROUP * F4_CHUNK * F4_ZS_STRIDE * sizeof(float);
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t NS = P.n_ring;
    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < NS; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], NCW); }
        mbar_init(&epi_bar, NCW);
        s_abort = 0;
        mbar_fence_init();
    }
    if (NV && threadIdx.x < 256) {
        const __half2 hv = e4m3_half2(threadIdx.x);
        s_lut[threadIdx.x] = *reinterpret_cast<const uint32_t*>(&hv);
    }
    __syncthreads();
    const uint32_t n_items = P.t.header[HDR_NGROUPS] * P.n_blocks;
    const uint32_t xa_chunk_words = (NPROJ == 2 ? P.H : P.I) / 32 * F4_XA_SB_WORDS;
    uint32_t LP = P.n_stages_k % 4 == 0 ? 4u : (P.n_stages_k % 2 == 0 ? 2u : 1u);   // parts of the sum (shape only)
    LP = LP < P.max_parts ? LP : P.max_parts;
    const uint32_t part_stages = P.n_stages_k / LP;
    // CTAs an item's parts are spread over (this call's item count)
    const uint32_t NP = P.ks_scratch ? ksplit_ctas(n_items, LP, gridDim.x, P.ks_cap_items) : 1u;
    const uint32_t share_stages = P.n_stages_k / NP;

    if (warp == NCW) {
        if (lane == 0) {
            uint32_t s = 0, ph = 0;     // ring slot and phase
            const uint32_t np_mask = NP - 1, np_shift = NP == 4 ? 2u : (NP == 2 ? 1u : 0u);
            bool ok = true;
            while (ok) {
                const uint32_t unit = atomicAdd(&P.t.header[P.counter_idx], 1u);
                const bool last = unit >= n_items * NP;
                const uint32_t item = unit >> np_shift, share = unit & np_mask;
                uint32_t g = 0, nb = 0, chunk0 = 0, mc = 0, expert = 0;
                if (!last) {
                    g = item / P.n_blocks; nb = item % P.n_blocks;
                    chunk0 = P.t.group_chunk0[g]; mc = P.t.group_mc[g]; expert = P.t.chunk_expert[chunk0];
                }
                const uint8_t* wsrc = P.w + (size_t)expert * P.expert_stride + (size_t)nb * P.n_stages_k * P.w_bytes;
                const uint32_t ks_begin = share * share_stages, ks_end = last ? ks_begin + 1 : ks_begin + share_stages;
                uint32_t part = share * (LP / NP), in_part = 0;
                const uint32_t sub = P.sub, xa_sub_bytes = sub * (4 * F4_XA_SB_WORDS * 4);
                for (uint32_t ks = ks_begin; ks < ks_end; ks += sub, s = (s + 1 == NS) ? (ph ^= 1u, 0u) : s + 1) {
                    if (!mbar_wait_bounded(&empty_bar[s], ph ^ 1u, &s_abort, 128)) {
                        if (!s_abort) atomicMax(P.status, (uint32_t)ST_WAIT_EMPTY);
                        s_abort = 1; ok = false; break;
                    }
                    meta[s].item = last ? -1 : (int32_t)item;
                    meta[s].ks = ks; meta[s].chunk0 = chunk0; meta[s].mc = mc; meta[s].expert = expert; meta[s].nb = nb;
                    meta[s].part = part;
                    const bool part_ends = in_part + sub == part_stages;
                    meta[s].flags = (in_part == 0 ? 1u : 0u) | (part_ends ? 2u : 0u) | (ks + sub >= ks_end ? 4u : 0u) | (mc << 8);
                    in_part = part_ends ? 0u : in_part + sub;
                    part += part_ends ? 1u : 0u;
                    if (last) { mbar_arrive(&full_bar[s]); ok = false; break; }
                    uint8_t* dst = ring + (size_t)s * P.stage_bytes;
                    mbar_expect_tx(&full_bar[s], sub * P.w_bytes + mc * xa_sub_bytes);
                    bulk_g2s(dst, wsrc + (size_t)ks * P.w_bytes, sub * P.w_bytes, &full_bar[s]);
                    for (uint32_t m = 0; m < mc; ++m)
                        bulk_g2s(dst + sub * P.w_bytes + m * xa_sub_bytes,
                                 P.xa + (size_t)(chunk0 + m) * xa_chunk_words + (size_t)ks * 4 * F4_XA_SB_WORDS,
                                 xa_sub_bytes, &full_bar[s]);
                }
            }
            if (s_abort) for (int i = 0; i < 2000; ++i) __nanosleep(1000);
        }
        return;
    }

    const uint32_t p = warp >> 3, j = warp & 7u;
    float acc[F4_GROUP][4];
    uint32_t epi_ph = 0;
    auto epi_sync = [&]() -> bool {
        __syncwarp();
        if (lane == 0) mbar_arrive(&epi_bar);
        const bool ok = mbar_wait_bounded(&epi_bar, epi_ph, &s_abort);
        epi_ph ^= 1u;
        if (!ok) { if (!s_abort) atomicMax(P.status, (uint32_t)ST_WAIT_FULL); s_abort = 1; }
        return ok;
    };
    // ring slot and its phase advance by increment-and-wrap (the ring depth is a run-time value: no division per stage)
    for (uint32_t s = 0, ph = 0;; s = (s + 1 == NS) ? (ph ^= 1u, 0u) : s + 1) {
        if (!mbar_wait_bounded(&full_bar[s], ph, &s_abort)) {
            if (!s_abort) atomicMax(P.status, (uint32_t)ST_WAIT_FULL);
            s_abort = 1;
            break;
        }
        const uint2 hot = *reinterpret_cast<const uint2*>(&meta[s]);   // item, flags | chunk count << 8
        if ((int32_t)hot.x < 0) break;
        const uint32_t flags = hot.y, stage_mc = hot.y >> 8;
        if (flags & 1u) {
#pragma unroll
            for (int a = 0; a < F4_GROUP; ++a)
#pragma unroll
                for (int q = 0; q < 4; ++q) acc[a][q] = 0.f;
        }
        const uint8_t* st = ring + (size_t)s * P.stage_bytes;
        const uint8_t* xs = st + P.sub * P.w_bytes;
        const uint32_t x_mt_stride = P.sub * (4 * F4_XA_SB_WORDS / 4);
        if (P.sub == 2) {
            if (stage_mc == 1) fp4_slot<NPROJ, NV, 1, 2>(st, xs, P.w_bytes, x_mt_stride, p, j, lane, s_lut, acc);
            else fp4_slot<NPROJ, NV, 2, 2>(st, xs, P.w_bytes, x_mt_stride, p, j, lane, s_lut, acc);
        } else {
            for (uint32_t u = 0; u < P.sub; ++u, st += P.w_bytes, xs += 4 * F4_XA_SB_WORDS * 4) {
                if (stage_mc == 1) fp4_stage<NPROJ, NV, 1>(st, xs, x_mt_stride, p, j, lane, s_lut, acc);
                else fp4_stage<NPROJ, NV, 2>(st, xs, x_mt_stride, p, j, lane, s_lut, acc);
            }
        }
        F4Meta m;
        if (flags & 2u) m = meta[s];       // the slot may be refilled once this warp has arrived below
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty_bar[s]);
        if (!(flags & 2u)) continue;

        // ---- end of a part of the sum: D fragment = (output row g | g+8) x (token slots 2c, 2c+1) ----
        // One CTA per item: the parts are folded left in the staging array.  Several CTAs: every part goes to its slot.
        const uint32_t g = lane >> 2, c = lane & 3u;
        float gs = 1.f;
        if (NV) gs = P.gscale[m.expert * 3 + (NPROJ == 2 ? p : 2)] / 2688.0f;
        const bool fold = NP == 1 && m.part != 0;
        constexpr uint32_t ZS_VEC = NPROJ * F4_GROUP * F4_CHUNK * F4_ZS_STRIDE / 4;
        // several CTAs per item: a part goes from the registers straight to its slot of the workspace
        float* zdst = NP > 1 ? P.ks_scratch + ((size_t)m.item * LP + m.part) * (ZS_VEC * 4) : zs;
#pragma unroll
        for (int mt = 0; mt < F4_GROUP; ++mt) {
            if (mt < (int)m.mc) {
                float* zr = zdst + ((p * F4_GROUP + mt) * F4_CHUNK + 2 * c) * F4_ZS_STRIDE + j * 16 + g;
                if (fold) {
                    zr[0] += acc[mt][0] * gs; zr[F4_ZS_STRIDE] += acc[mt][1] * gs;
                    zr[8] += acc[mt][2] * gs; zr[F4_ZS_STRIDE + 8] += acc[mt][3] * gs;
                } else {
                    zr[0] = acc[mt][0] * gs; zr[F4_ZS_STRIDE] = acc[mt][1] * gs;
                    zr[8] = acc[mt][2] * gs; zr[F4_ZS_STRIDE + 8] = acc[mt][3] * gs;
                }
            }
        }
        if (!(flags & 4u)) continue;
        if (NP == 1) {
            if (!epi_sync()) break;
        } else {
            // every thread's parts are out before thread 0 counts this CTA in
            __threadfence();
            if (!epi_sync()) break;
            if (threadIdx.x == 0) {
                const uint32_t seen = atomicAdd(&P.ks_count[m.item], 1u);
                s_last_part = seen == NP - 1 ? 1 : 0;
                if (seen == NP - 1) P.ks_count[m.item] = 0;
            }
            if (!epi_sync()) break;
            if (!s_last_part) continue;
            __threadfence();
            // only the chunks that hold rows: [projection][chunk < mc][row][stride]
            const float4* base = reinterpret_cast<const float4*>(P.ks_scratch) + (size_t)m.item * LP * ZS_VEC;
            const uint32_t per_p = m.mc * (F4_CHUNK * F4_ZS_STRIDE / 4);
            for (uint32_t i0 = threadIdx.x; i0 < NPROJ * per_p; i0 += NCW * 32) {
                const uint32_t i = (i0 / per_p) * (F4_GROUP * F4_CHUNK * F4_ZS_STRIDE / 4) + i0 % per_p;
                float4 a = __ldcg(base + i);
                for (uint32_t q = 1; q < LP; ++q) {
                    const float4 b = __ldcg(base + (size_t)q * ZS_VEC + i);
                    a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
                }
                reinterpret_cast<float4*>(zs)[i] = a;
            }
            if (!epi_sync()) break;
        }
        // ---- epilogue of the item ----
        for (uint32_t combo = warp; combo < (uint32_t)F4_GROUP * F4_CHUNK; combo += NCW) {
            const uint32_t mt = combo / F4_CHUNK, row = combo % F4_CHUNK;
            if (mt >= m.mc) continue;
            const uint32_t chunk = m.chunk0 + mt;
            const bool valid = row < P.t.chunk_rows[chunk];
            const uint32_t col = m.nb * 128 + lane * 4;
            if (NPROJ == 2) {
                __half hv[4];
#pragma unroll
                for (int q = 0; q < 4; ++q) hv[q] = __float2half_rn(0.f);
                if (valid) {
                    const float4 zg = *reinterpret_cast<const float4*>(zs + ((0 * F4_GROUP + mt) * F4_CHUNK + row) * F4_ZS_STRIDE + lane * 4);
                    const float4 zu = *reinterpret_cast<const float4*>(zs + ((1 * F4_GROUP + mt) * F4_CHUNK + row) * F4_ZS_STRIDE + lane * 4);
                    const float gq[4] = {zg.x, zg.y, zg.z, zg.w}, uq[4] = {zu.x, zu.y, zu.z, zu.w};
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        // mimo_moe_k1_gateup.metal:115-128 / glm5n_nvfp4_gateup.metal:109-129
                        float gf = bf16_round_f(gq[q]), uf = bf16_round_f(uq[q]);
                        if (P.limit > 0.f) {
                            gf = gf > P.limit ? P.limit : gf;
                            uf = uf > P.limit ? P.limit : (uf < -P.limit ? -P.limit : uf);
                        }
                        const float hq = bf16_round_f(bf16_round_f(gf * sigmoid_ref(gf)) * uf);
                        hv[q] = __float2half_rn(hq);
                    }
                }
                // the down kernel's B-fragment order: 32-block lane/8 of this 128 block, word c = (lane % 8) / 2,
                // inputs 4 (lane % 2) + q in natural order
                __half* dsth = reinterpret_cast<__half*>(
                    P.xa_d + ((size_t)chunk * (P.I / 32) + m.nb * 4 + (lane >> 3)) * F4_XA_SB_WORDS + (row * 4 + ((lane & 7u) >> 1)) * 4);
#pragma unroll
                for (int q = 0; q < 4; ++q) dsth[4 * (lane & 1u) + q] = hv[q];
            } else if (valid) {
                const float4 z4 = *reinterpret_cast<const float4*>(zs + ((size_t)mt * F4_CHUNK + row) * F4_ZS_STRIDE + lane * 4);
                const uint32_t assign = P.t.order[P.t.chunk_row0[chunk] + row];
                if (P.out_bf16) {
                    __nv_bfloat162 lo = __floats2bfloat162_rn(z4.x, z4.y), hi = __floats2bfloat162_rn(z4.z, z4.w);
                    *reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(P.out) + (size_t)assign * P.H + col) =
                        make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
                } else {
                    *reinterpret_cast<float4*>(static_cast<float*>(P.out) + (size_t)assign * P.H + col) = z4;
                }
            }
        }
        if (!epi_sync()) break;
    }
}

static int f4_tune_env(const char* name, int dflt, int lo, int hi) {
    const char* v = getenv(name);
    if (!v) return dflt;
    int x = atoi(v);
    return x < lo ? lo : (x > hi ? hi : x);
}

cudaError_t launch_fp4_gemv(const Fp4GemvArgs& a, int down, cudaStream_t st) {
    Fp4Params P{};
    const int nproj = down ? 1 : 2;
    const uint32_t sstage = f4_scale_stage_bytes(a.nv != 0);
    P.w = down ? a.dn : a.gu;
    P.w_bytes = nproj * (F4_W_STAGE + sstage);
    P.n_blocks = (down ? a.H : a.I) / 128;
    P.n_stages_k = (down ? a.I : a.H) / F4_KS;
    P.expert_stride = (size_t)P.n_blocks * P.n_stages_k * P.w_bytes;
    P.gscale = a.gscale;
    P.xa = down ? a.xa_d : a.xa;
    P.t = a.t;
    P.counter_idx = down ? HDR_CTR_DOWN : HDR_CTR_GU;
    P.H = a.H; P.I = a.I; P.xa_d = a.xa_d; P.out = a.ro; P.out_bf16 = a.ro_bf16; P.limit = a.limit; P.status = a.status;
    P.ks_scratch = a.ks_scratch; P.ks_count = a.ks_count;
    static const int k_parts = f4_tune_env("MLXS_K_PARTS", 4, 1, 4);
    P.max_parts = (uint32_t)k_parts;
    static const int gu_ctas = f4_tune_env("MLXS_F4_GU_CTAS", 2, 1, 2), dn_ctas = f4_tune_env("MLXS_F4_DN_CTAS", 3, 1, 3);
    const int per_sm = down ? dn_ctas : gu_ctas;
    const uint32_t zs_bytes = (uint32_t)(nproj * F4_GROUP * F4_CHUNK * F4_ZS_STRIDE * sizeof(float));
    P.n_sm = (uint32_t)a.sm_count; P.ks_cap_items = ksplit_cap_items(a.sm_count, zs_bytes);
    const uint32_t budget = (uint32_t)(225 * 1024 / per_sm) - 2048u;
    // One barrier round trip of the ring serves `sub` 128-input sub-stages: the largest of 4, 2, 1 that divides a part
    // of the sum and still leaves a ring of two slots.
    static const int sub_max = f4_tune_env("MLXS_F4_SUB", 2, 1, 4);
    uint32_t lp = P.n_stages_k % 4 == 0 ? 4u : (P.n_stages_k % 2 == 0 ? 2u : 1u);
    lp = lp < P.max_parts ? lp : P.max_parts;
    const uint32_t one = P.w_bytes + F4_GROUP * 4 * F4_XA_SB_WORDS * 4;
    uint32_t sub = (uint32_t)sub_max;
    while (sub > 1 && ((P.n_stages_k / lp) % sub != 0 || (budget - zs_bytes) / (sub * one) < 2)) sub >>= 1;
    P.sub = sub;
    P.stage_bytes = sub * one;
    uint32_t ns = (budget - zs_bytes) / P.stage_bytes;
    if (ns > 8) ns = 8;
    if (ns < 2) return cudaErrorInvalidValue;
    P.n_ring = ns;
    const size_t smem = zs_bytes + (size_t)ns * P.stage_bytes;
    const int ctas = per_sm * a.sm_count;
    cudaError_t e;
#define MLXS_F4_LAUNCH(NP, NVV)                                                                               \
    do {                                                                                                      \
        e = cudaFuncSetAttribute(fp4_gemv_kernel<NP, NVV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        if (e != cudaSuccess) return e;                                                                       \
        fp4_gemv_kernel<NP, NVV><<<ctas, NP * 256 + 32, smem, st>>>(P);                                       \
    } while (0)
    if (!down && a.nv) MLXS_F4_LAUNCH(2, true);
    else if (!down) MLXS_F4_LAUNCH(2, false);
    else if (a.nv) MLXS_F4_LAUNCH(1, true);
    else MLXS_F4_LAUNCH(1, false);
#undef MLXS_F4_LAUNCH
    return cudaGetLastError();
}

}  // namespace mlxs
