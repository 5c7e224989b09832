// EXL3 (K=3, mul1 trellis, 128-wide Hadamard with suh/svh) expert kernels for decode-sized batches.
//
// One projection is y = H128( H128(x * suh) . W_hat ) * svh (src/arch/glm5_next/exl3_forms_ref.zig:137-152; op order
// of the decode chain: src/arch/deepseek_v41/experts.zig:449-467).  The weight stream is the bound: a CTA owns one
// 128-wide output block of one expert for up to 16 of its rows, streams that block's code once through a ring of
// bulk-copied (TMA 1-D) shared-memory stages, decodes each 16x16 tile in registers straight into one mma A fragment
// (the trellis' tensor-core order makes a lane's 8 code positions exactly its fragment of W^T: 16 output columns x 16
// inputs) and multiplies with the rows' rotated activations as the B operand: 8 token slots = 4 rows as f16 hi + the
// same rows as f16 lo, so the f32 precision of the reference's decode chain is kept while the FMAs run on the tensor
// pipe, one mma per tile for up to 4 rows.  The output-side Hadamard, svh, the clamped SwiGLU and the down
// projection's input rotation are fused into the gate/up epilogue; H128 . svh into the down epilogue.
#include <cstdlib>

#include "common.cuh"
#include "kernels.h"
#include "exl3_prep_body.cuh"

namespace mlxs {

constexpr int KT = 8;             // k-tiles (16 inputs each) per pipeline stage = one 128-block of the input
constexpr int ZS_STRIDE = 132;    // padded row stride of the epilogue's f32 staging

// ------------------------------------------------------------------------------------------------------------
// load-time repack: reference record -> kernel layout (bit-preserving: words move, no bit changes)
// ------------------------------------------------------------------------------------------------------------
__global__ void exl3_repack_kernel(const uint8_t* __restrict__ rec, uint32_t H, uint32_t I, uint32_t TW,
                                   uint32_t* __restrict__ gu, uint32_t* __restrict__ dn, __half* __restrict__ sc) {
    const size_t code_bytes = (size_t)(H / 16) * (I / 16) * TW * 4;   // TW words per 16x16 tile (24 at K = 3, 16 at K = 2)
    // record offsets (src/expert/bank.zig:116-141): per projection code, rout [out], rin [in]
    const size_t off_g = 0, off_g_rout = code_bytes, off_g_rin = off_g_rout + 2 * (size_t)I;
    const size_t off_u = off_g_rin + 2 * (size_t)H, off_u_rout = off_u + code_bytes, off_u_rin = off_u_rout + 2 * (size_t)I;
    const size_t off_d = off_u_rin + 2 * (size_t)H, off_d_rout = off_d + code_bytes, off_d_rin = off_d_rout + 2 * (size_t)H;
    const size_t words = code_bytes / 4;
    const size_t n_gu = 2 * words, n_all = 3 * words, n_sc = (size_t)3 * H + 3 * I;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_all + n_sc; i += stride) {
        if (i < n_gu) {
            // destination index -> (nb, kt, p, j, w)
            size_t r = i;
            const uint32_t w = r % TW; r /= TW;
            const uint32_t j = r % 8; r /= 8;
            const uint32_t p = r % 2; r /= 2;
            const uint32_t kt = r % (H / 16); r /= (H / 16);
            const uint32_t nb = (uint32_t)r;
            const uint32_t* src = reinterpret_cast<const uint32_t*>(rec + (p ? off_u : off_g));
            gu[i] = src[((size_t)kt * (I / 16) + nb * 8 + j) * TW + w];
        } else if (i < n_all) {
            size_t r = i - n_gu;
            const uint32_t w = r % TW; r /= TW;
            const uint32_t j = r % 8; r /= 8;
            const uint32_t kt = r % (I / 16); r /= (I / 16);
            const uint32_t nb = (uint32_t)r;
            const uint32_t* src = reinterpret_cast<const uint32_t*>(rec + off_d);
            dn[i - n_gu] = src[((size_t)kt * (H / 16) + nb * 8 + j) * TW + w];
        } else {
            const size_t s = i - n_all;
            const __half* h;
            if (s < H) h = reinterpret_cast<const __half*>(rec + off_g_rin) + s;                        // suh_g
            else if (s < 2 * (size_t)H) h = reinterpret_cast<const __half*>(rec + off_u_rin) + (s - H);  // suh_u
            else if (s < 2 * (size_t)H + I) h = reinterpret_cast<const __half*>(rec + off_g_rout) + (s - 2 * (size_t)H);
            else if (s < 2 * (size_t)H + 2 * (size_t)I)
                h = reinterpret_cast<const __half*>(rec + off_u_rout) + (s - 2 * (size_t)H - I);
            else if (s < 2 * (size_t)H + 3 * (size_t)I)
                h = reinterpret_cast<const __half*>(rec + off_d_rin) + (s - 2 * (size_t)H - 2 * (size_t)I);  // suh_d
            else h = reinterpret_cast<const __half*>(rec + off_d_rout) + (s - 2 * (size_t)H - 3 * (size_t)I);  // svh_d
            sc[s] = *h;
        }
    }
}

cudaError_t launch_exl3_repack(const uint8_t* record_dev, Exl3Dims d, uint32_t* gu_code_e, uint32_t* d_code_e,
                               __half* scales_e, cudaStream_t st) {
    exl3_repack_kernel<<<592, 256, 0, st>>>(record_dev, d.H, d.I, exl3_tile_words(d), gu_code_e, d_code_e, scales_e);
    return cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------------------
// activation staging: rows -> mma A-fragment order, f16 hi / lo
// ------------------------------------------------------------------------------------------------------------
template <bool RAW>
__global__ void __launch_bounds__(CHUNK_ROWS * 32) exl3_prep_kernel(const void* __restrict__ xin, uint32_t top_k, uint32_t in_dim,
                                                        const __half* __restrict__ scales, size_t scales_stride,
                                                        DispatchTables t, uint32_t* __restrict__ xa) {
    const uint32_t chunk = blockIdx.x;
    if (chunk >= t.header[HDR_NCHUNKS]) return;
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;  // warp = row of the chunk
    const uint32_t e = t.chunk_expert[chunk], rows = t.chunk_rows[chunk];
    const bool valid = warp < rows;
    const uint32_t assign = valid ? t.order[t.chunk_row0[chunk] + warp] : 0u;
    const uint32_t tok = x_row_of(t, assign, top_k);
    for (uint32_t b = blockIdx.y; b < in_dim / 128; b += gridDim.y)
        exl3_prep_row_block<RAW>(xin, tok, valid, e, in_dim, scales, scales_stride, chunk, warp, b, lane, xa);
}

cudaError_t launch_exl3_prep_in(const __nv_bfloat16* x, uint32_t top_k, Exl3Layer L, Exl3Dims d, DispatchTables t,
                                uint32_t* xa_gu, cudaStream_t st) {
    exl3_prep_kernel<false><<<dim3(t.max_chunks, 8), CHUNK_ROWS * 32, 0, st>>>(x, top_k, d.H, L.scales, exl3_scales_per_expert(d), t, xa_gu);
    return cudaGetLastError();
}
cudaError_t launch_exl3_prep_raw(const float* xh, uint32_t in_dim, DispatchTables t, uint32_t* xa, cudaStream_t st) {
    exl3_prep_kernel<true><<<dim3(t.max_chunks, 8), CHUNK_ROWS * 32, 0, st>>>(xh, 1, in_dim, nullptr, 0, t, xa);
    return cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------------------
// the streaming GEMV
// ------------------------------------------------------------------------------------------------------------
enum { EPI_GATE_UP = 0, EPI_DOWN = 1, EPI_RAW = 2 };

struct GemvParams {
    const uint32_t* code;        // layer base (or the expert's base when expert_stride_words == 0)
    size_t expert_stride_words;
    uint32_t n_blocks;           // out / 128
    uint32_t nkt;                // in / 16
    uint32_t kt_stride_words;    // words per k-tile in the block stream (192 per projection present)
    uint32_t proj_off_words;     // where this kernel's (first) projection sits inside a k-tile
    const uint32_t* xa;          // [chunk][NPROJ][nkt][128]
    DispatchTables t;
    uint32_t counter_idx;
    const __half* scales;        // layer base
    size_t scales_stride;
    uint32_t H, I;
    uint32_t* xa_d;              // gate/up epilogue output
    float* out;                  // down: ro [A, H]; raw: z [rows, out_dim]
    uint32_t out_dim;
    float limit;
    uint32_t* status;
    uint32_t n_stages;
    uint32_t stage_bytes, w_bytes;
    uint32_t max_parts;          // cap on the parts of the sum (4; a tuning knob for measurements, MLXS_K_PARTS)
    // The sum over the inputs is always taken in `parts` equal parts, folded left in part order: a fixed function of the
    // shape, so a row's bits do not depend on the batch around it.  Calls with fewer work items than CTAs spread an
    // item's parts over 2 or 4 CTAs: each leaves its parts here and the last to arrive folds them and runs the epilogue.
    float* ks_scratch;           // [items][parts][zs words] or null (one CTA per item always)
    uint32_t* ks_count;          // [ks_cap_items] arrivals per item, zero between launches
    uint32_t n_sm, ks_cap_items; // SMs of the device; items the workspace and the counters hold
    // Every wait gives up after poll_limit polls.  Self-test only (mlxs_moe_debug_wait): withhold = n makes every
    // producer leave out the copies of its n-th ring stage, so the consumers' wait for that stage runs out, the CTA
    // records ST_WAIT_FULL and returns with nothing in flight.
    uint32_t poll_limit, withhold;
};

// flags: 1 = first stage of a part of the sum, 2 = last stage of a part, 4 = last stage of this CTA's share of the item;
// bits 16.. = sub-stages (of KT k-tiles each) this ring slot carries
struct StageMeta { int32_t item; uint32_t flags, mc, kt0, chunk0, expert, nb, part; };

// one pipeline stage (KT k-tiles) of one warp's 16-column tile, MC chunks of activations
template <int NPROJ, int KSTRIDE, int KB, int MC>
__device__ __forceinline__ void gemv_stage(const uint32_t* __restrict__ wt, const uint2* __restrict__ at, uint32_t mt_stride,
                                           uint32_t wi, uint32_t wj, uint32_t lp, float (&acc)[GROUP_CHUNKS][4]) {
    // at: this projection's KT activation tiles of the first chunk (B-fragment order), the next chunk's mt_stride uint2 on
#pragma unroll
    for (int kt = 0; kt < KT; ++kt) {
        const uint32_t lo = wt[kt * KSTRIDE + wi], hi = wt[kt * KSTRIDE + wj];
        uint32_t b[4];
        exl3_decode_lane_kb<KB>(lo, hi, lp, b);
        // W^T as the A operand: rows = the tile's 16 output columns
        const uint32_t a[4] = {b[0], b[2], b[1], b[3]};
#pragma unroll
        for (int mt = 0; mt < MC; ++mt) {
            const uint2 xv = at[mt * mt_stride + kt * 32];
            mma_f16(acc[mt], a, xv.x, xv.y);
        }
    }
}

// SUB sub-stages of one ring slot, unrolled
template <int NPROJ, int KSTRIDE, int KB, int MC, int SUB>
__device__ __forceinline__ void gemv_slot(const uint32_t* __restrict__ wt, const uint2* __restrict__ at, uint32_t mt_stride,
                                          uint32_t wi, uint32_t wj, uint32_t lp, float (&acc)[GROUP_CHUNKS][4]) {
#pragma unroll
    for (int u = 0; u < SUB; ++u)
        gemv_stage<NPROJ, KSTRIDE, KB, MC>(wt + u * KT * KSTRIDE, at + u * KT * 32, mt_stride, wi, wj, lp, acc);
}

// KSTRIDE = words per k-tile of the block stream (8 tiles x 8 KB words per projection present), KB = bits per weight
template <int NPROJ, int EPI, int KSTRIDE, int KB>
__global__ void __launch_bounds__(NPROJ * 256 + 32, NPROJ == 1 ? 3 : 2) exl3_gemv_kernel(const GemvParams P) {
    constexpr uint32_t TW = 8 * KB;        // words per 16x16 tile
    extern __shared__ __align__(128) uint8_t smem_raw[];
    constexpr int NCW = NPROJ * 8;         // consumer warps: projection x 16-column tile of the 128 block
    constexpr int MAXS = 8;
    __shared__ __align__(8) uint64_t full_bar[MAXS], empty_bar[MAXS], epi_bar;
    __shared__ __align__(8) StageMeta meta[MAXS];
    __shared__ volatile int s_abort;
    __shared__ volatile int s_last_part;
    // epilogue staging: [NPROJ][GROUP_CHUNKS][CHUNK_ROWS][ZS_STRIDE]
    float* zs = reinterpret_cast<float*>(smem_raw);
    uint8_t* ring = smem_raw + (size_t)NPROJ * GROUP_CHUNKS * CHUNK_ROWS * ZS_STRIDE * sizeof(float);
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t NS = P.n_stages;

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < NS; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], NCW); }
        mbar_init(&epi_bar, NCW);
        s_abort = 0;
        mbar_fence_init();
    }
    __syncthreads();
    const uint32_t n_items = P.t.header[HDR_NGROUPS] * P.n_blocks;
    // parts of the sum (shape only), and over how many CTAs an item's parts are spread (this call's item count)
    uint32_t LP = P.nkt % (4 * KT) == 0 ? 4u : (P.nkt % (2 * KT) == 0 ? 2u : 1u);
    LP = LP < P.max_parts ? LP : P.max_parts;
    const uint32_t part_kt = P.nkt / LP;
    const uint32_t NP = P.ks_scratch ? ksplit_ctas(n_items, LP, gridDim.x, P.ks_cap_items) : 1u;
    const uint32_t share_kt = P.nkt / NP;

    if (warp == NCW) {
        // ---------------- producer warp: one lane issues every copy ----------------
        if (lane == 0) {
            uint32_t s = 0, ph = 0;     // ring slot and phase
            uint32_t n_stage = 0;       // stages this producer has filled (self-test: the withheld one)
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
                const uint32_t* wsrc = P.code + (size_t)expert * P.expert_stride_words +
                                       (size_t)nb * P.nkt * P.kt_stride_words;
                const uint32_t k_begin = share * share_kt, k_end = last ? k_begin + 1 : k_begin + share_kt;
                // One barrier round trip serves `sub` sub-stages of KT k-tiles: the most (up to 3; 1 for rows in 3 or 4 chunks) that divide a part of
                // the sum and fit the ring slot with this item's chunks of rows.
                uint32_t sub = 1;
                if (!last)
                    for (uint32_t c = mc > 2 ? 1u : 3u; c > 1; --c)
                        if ((part_kt / KT) % c == 0 && c * (P.w_bytes + mc * NPROJ * KT * A_TILE_WORDS * 4) <= P.stage_bytes) { sub = c; break; }
                const uint32_t step = sub * KT, xa_bytes = step * A_TILE_WORDS * 4;
                // k_begin is a multiple of the part length: the place inside a part advances with the stages
                uint32_t part = share * (LP / NP), in_part = 0;
                for (uint32_t kt0 = k_begin; kt0 < k_end; kt0 += step, s = (s + 1 == NS) ? (ph ^= 1u, 0u) : s + 1) {
                    if (!mbar_wait_bounded(&empty_bar[s], ph ^ 1u, &s_abort, 128, P.poll_limit)) {
                        if (!s_abort) atomicMax(P.status, (uint32_t)ST_WAIT_EMPTY);
                        s_abort = 1; ok = false; break;
                    }
                    meta[s].item = last ? -1 : (int32_t)item;
                    meta[s].kt0 = kt0; meta[s].chunk0 = chunk0; meta[s].mc = mc; meta[s].expert = expert; meta[s].nb = nb;
                    meta[s].part = part;
                    const bool part_ends = in_part + step == part_kt;
                    meta[s].flags = (in_part == 0 ? 1u : 0u) | (part_ends ? 2u : 0u) | (kt0 + step >= k_end ? 4u : 0u) | (sub << 16);
                    in_part = part_ends ? 0u : in_part + step;
                    part += part_ends ? 1u : 0u;
                    if (last) { mbar_arrive(&full_bar[s]); ok = false; break; }
                    if (P.withhold && ++n_stage == P.withhold) continue;   // self-test: this stage never arrives
                    uint8_t* dst = ring + (size_t)s * P.stage_bytes;
                    mbar_expect_tx(&full_bar[s], sub * P.w_bytes + mc * NPROJ * xa_bytes);
                    bulk_g2s(dst, wsrc + (size_t)kt0 * P.kt_stride_words, sub * P.w_bytes, &full_bar[s]);
                    for (uint32_t m = 0; m < mc; ++m)
                        for (int p = 0; p < NPROJ; ++p)
                            bulk_g2s(dst + sub * P.w_bytes + (m * NPROJ + p) * xa_bytes,
                                     P.xa + (((size_t)(chunk0 + m) * NPROJ + p) * P.nkt + kt0) * A_TILE_WORDS, xa_bytes,
                                     &full_bar[s]);
                }
            }
            // after a give-up: let copies already issued land before the CTA's shared memory is released
            if (s_abort) for (int i = 0; i < 2000; ++i) __nanosleep(1000);
        }
        return;
    }

    // ---------------- consumer warps ----------------
    const uint32_t p = warp >> 3, j = warp & 7u;  // projection, 16-column tile
    uint32_t wi, wj, lp;
    exl3_lane_plan_kb<KB>(lane, wi, wj, lp);
    float acc[GROUP_CHUNKS][4];
    const float S = __uint_as_float(SCALE_BITS);
    uint32_t epi_ph = 0;
    // every wait in this kernel is a bounded mbarrier wait: the epilogue's two rendezvous of the consumer warps too
    auto epi_sync = [&]() -> bool {
        __syncwarp();
        if (lane == 0) mbar_arrive(&epi_bar);
        const bool ok = mbar_wait_bounded(&epi_bar, epi_ph, &s_abort, 0, P.poll_limit);
        epi_ph ^= 1u;
        if (!ok) { if (!s_abort) atomicMax(P.status, (uint32_t)ST_WAIT_FULL); s_abort = 1; }
        return ok;
    };
    // ring slot and its phase advance by increment-and-wrap (the ring depth is a run-time value: no division per stage)
    for (uint32_t s = 0, ph = 0;; s = (s + 1 == NS) ? (ph ^= 1u, 0u) : s + 1) {
        if (!mbar_wait_bounded(&full_bar[s], ph, &s_abort, 0, P.poll_limit)) {
            if (!s_abort) atomicMax(P.status, (uint32_t)ST_WAIT_FULL);
            s_abort = 1;
            break;
        }
        const StageMeta m = meta[s];
        if (m.item < 0) break;
        const uint32_t flags = m.flags, stage_mc = m.mc;
        if (flags & 1u) {
#pragma unroll
            for (int a = 0; a < GROUP_CHUNKS; ++a)
#pragma unroll
                for (int c = 0; c < 4; ++c) acc[a][c] = 0.f;
        }
        // slot: [sub x KT k-tiles of codes][chunk][projection][sub x KT activation tiles]
        const uint32_t sub = flags >> 16;
        const uint8_t* st = ring + (size_t)s * P.stage_bytes;
        const uint32_t* wt = reinterpret_cast<const uint32_t*>(st) + P.proj_off_words + p * (8u * TW) + j * TW;
        const uint2* at = reinterpret_cast<const uint2*>(st + sub * P.w_bytes) + p * (sub * KT * 32) + lane;
        const uint32_t mt_stride = NPROJ * sub * KT * 32;
        static_assert(GROUP_CHUNKS * CHUNK_ROWS == 16, "the K-split workspace is sized for 16 rows per item");
        static_assert(GROUP_CHUNKS == 4, "the stage dispatch below enumerates the chunk counts");
        // straight-line code per (chunks, sub-stages): rows in 3 or 4 chunks always come one sub-stage per slot
        if (stage_mc == 1) {
            if (sub == 2) gemv_slot<NPROJ, KSTRIDE, KB, 1, 2>(wt, at, mt_stride, wi, wj, lp, acc);
            else if (sub == 3) gemv_slot<NPROJ, KSTRIDE, KB, 1, 3>(wt, at, mt_stride, wi, wj, lp, acc);
            else gemv_slot<NPROJ, KSTRIDE, KB, 1, 1>(wt, at, mt_stride, wi, wj, lp, acc);
        } else if (stage_mc == 2) {
            if (sub == 2) gemv_slot<NPROJ, KSTRIDE, KB, 2, 2>(wt, at, mt_stride, wi, wj, lp, acc);
            else if (sub == 3) gemv_slot<NPROJ, KSTRIDE, KB, 2, 3>(wt, at, mt_stride, wi, wj, lp, acc);
            else gemv_slot<NPROJ, KSTRIDE, KB, 2, 1>(wt, at, mt_stride, wi, wj, lp, acc);
        } else if (stage_mc == 3) {
            gemv_slot<NPROJ, KSTRIDE, KB, 3, 1>(wt, at, mt_stride, wi, wj, lp, acc);
        } else {
            gemv_slot<NPROJ, KSTRIDE, KB, 4, 1>(wt, at, mt_stride, wi, wj, lp, acc);
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty_bar[s]);
        if (!(flags & 2u)) continue;

        // ---------------- end of a part of the sum ----------------
        // the D fragment holds (column g | g+8) x (token slots 2c, 2c+1); z[row] = hi slot + lo slot = lane c + lane c+2.
        // One CTA per item: the parts are folded left in the staging array.  Several CTAs: every part goes to its slot.
        const uint32_t g = lane >> 2, c = lane & 3u;
        const bool fold = NP == 1 && m.part != 0;
        constexpr uint32_t ZS_VEC = NPROJ * GROUP_CHUNKS * CHUNK_ROWS * ZS_STRIDE / 4;
        // several CTAs per item: a part goes from the registers straight to its slot of the workspace
        float* zdst = NP > 1 ? P.ks_scratch + ((size_t)m.item * LP + m.part) * (ZS_VEC * 4) : zs;
#pragma unroll
        for (int mt = 0; mt < GROUP_CHUNKS; ++mt) {
            if (mt < (int)m.mc) {
                float v[4];
#pragma unroll
                for (int q = 0; q < 4; ++q) v[q] = acc[mt][q] + __shfl_xor_sync(0xFFFFFFFFu, acc[mt][q], 2);
                if (c < 2) {
                    float* zr = zdst + ((p * GROUP_CHUNKS + mt) * CHUNK_ROWS + 2 * c) * ZS_STRIDE + j * 16 + g;
                    if (fold) { zr[0] += v[0]; zr[ZS_STRIDE] += v[1]; zr[8] += v[2]; zr[ZS_STRIDE + 8] += v[3]; }
                    else { zr[0] = v[0]; zr[ZS_STRIDE] = v[1]; zr[8] = v[2]; zr[ZS_STRIDE + 8] = v[3]; }
                }
            }
        }
        if (!(flags & 4u)) continue;
        if (NP == 1) {
            if (!epi_sync()) break;
        } else {
            // every thread's parts are out before thread 0 counts this CTA in; the last CTA of the item to arrive folds
            // the parts in part order (whoever it is) and goes on to the epilogue; the others take the next unit
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
            const uint32_t per_p = m.mc * (CHUNK_ROWS * ZS_STRIDE / 4);
            for (uint32_t i0 = threadIdx.x; i0 < NPROJ * per_p; i0 += NCW * 32) {
                const uint32_t i = (i0 / per_p) * (GROUP_CHUNKS * CHUNK_ROWS * ZS_STRIDE / 4) + i0 % per_p;
                float4 a = __ldcg(base + i);
                for (uint32_t q = 1; q < LP; ++q) {
                    const float4 b = __ldcg(base + (size_t)q * ZS_VEC + i);
                    a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
                }
                reinterpret_cast<float4*>(zs)[i] = a;
            }
            if (!epi_sync()) break;
        }
        // ---------------- epilogue of the item ----------------
        for (uint32_t combo = warp; combo < (uint32_t)GROUP_CHUNKS * CHUNK_ROWS; combo += NCW) {
            const uint32_t mt = combo / CHUNK_ROWS, row = combo % CHUNK_ROWS;
            if (mt >= m.mc) continue;
            const uint32_t chunk = m.chunk0 + mt;
            const bool valid = row < P.t.chunk_rows[chunk];
            const uint32_t col = m.nb * 128 + lane * 4;
            if (EPI == EPI_GATE_UP) {
                float v[4] = {0.f, 0.f, 0.f, 0.f};
                if (valid) {
                    const float4 zg = *reinterpret_cast<const float4*>(zs + ((0 * GROUP_CHUNKS + mt) * CHUNK_ROWS + row) * ZS_STRIDE + lane * 4);
                    const float4 zu = *reinterpret_cast<const float4*>(zs + ((1 * GROUP_CHUNKS + mt) * CHUNK_ROWS + row) * ZS_STRIDE + lane * 4);
                    float gq[4] = {zg.x, zg.y, zg.z, zg.w}, uq[4] = {zu.x, zu.y, zu.z, zu.w};
                    hadamard128_warp(gq, lane);
                    hadamard128_warp(uq, lane);
                    const __half* sc = P.scales + (size_t)m.expert * P.scales_stride;
                    const uint2 sg = *reinterpret_cast<const uint2*>(sc + 2 * (size_t)P.H + col);               // svh_g
                    const uint2 su = *reinterpret_cast<const uint2*>(sc + 2 * (size_t)P.H + P.I + col);         // svh_u
                    const uint2 sd = *reinterpret_cast<const uint2*>(sc + 2 * (size_t)P.H + 2 * (size_t)P.I + col);  // suh_d
                    const float2 sg01 = __half22float2(*reinterpret_cast<const __half2*>(&sg.x));
                    const float2 sg23 = __half22float2(*reinterpret_cast<const __half2*>(&sg.y));
                    const float2 su01 = __half22float2(*reinterpret_cast<const __half2*>(&su.x));
                    const float2 su23 = __half22float2(*reinterpret_cast<const __half2*>(&su.y));
                    const float2 sd01 = __half22float2(*reinterpret_cast<const __half2*>(&sd.x));
                    const float2 sd23 = __half22float2(*reinterpret_cast<const __half2*>(&sd.y));
                    const float svg[4] = {sg01.x, sg01.y, sg23.x, sg23.y}, svu[4] = {su01.x, su01.y, su23.x, su23.y};
                    const float shd[4] = {sd01.x, sd01.y, sd23.x, sd23.y};
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        // src/kernels/exl3/q3_exl3_prep_gu_epi.metal:42-74
                        const float gm = (gq[q] * S) * svg[q], um = (uq[q] * S) * svu[q];
                        float gate = gm, up = um;
                        if (P.limit > 0.f) {
                            gate = (gm != gm) ? gm : (gm < P.limit ? gm : P.limit);
                            const float u0 = (um != um) ? um : (um > -P.limit ? um : -P.limit);
                            up = (u0 != u0) ? u0 : (u0 < P.limit ? u0 : P.limit);
                        }
                        const float yv = 1.0f / (1.0f + expf(fabsf(gate)));
                        const float sgm = gate < 0.f ? yv : 1.0f - yv;
                        v[q] = ((gate * sgm) * up) * shd[q];
                    }
                    hadamard128_warp(v, lane);
#pragma unroll
                    for (int q = 0; q < 4; ++q) v[q] *= S;
                }
                store_frag4(P.xa_d + ((size_t)chunk * (P.I / 16) + m.nb * 8) * A_TILE_WORDS, row, lane, v);
            } else if (valid) {
                const float4 z4 = *reinterpret_cast<const float4*>(zs + ((size_t)mt * CHUNK_ROWS + row) * ZS_STRIDE + lane * 4);
                float v[4] = {z4.x, z4.y, z4.z, z4.w};
                const uint32_t assign = P.t.order[P.t.chunk_row0[chunk] + row];
                if (EPI == EPI_DOWN) {
                    hadamard128_warp(v, lane);
                    const __half* sc = P.scales + (size_t)m.expert * P.scales_stride + 2 * (size_t)P.H + 3 * (size_t)P.I;  // svh_d
                    const uint2 so = *reinterpret_cast<const uint2*>(sc + col);
                    const float2 s01 = __half22float2(*reinterpret_cast<const __half2*>(&so.x));
                    const float2 s23 = __half22float2(*reinterpret_cast<const __half2*>(&so.y));
                    v[0] = (v[0] * S) * s01.x; v[1] = (v[1] * S) * s01.y; v[2] = (v[2] * S) * s23.x; v[3] = (v[3] * S) * s23.y;
                }
                *reinterpret_cast<float4*>(P.out + (size_t)assign * P.out_dim + col) = make_float4(v[0], v[1], v[2], v[3]);
            }
        }
        if (!epi_sync()) break;
    }
}

static int tune_env(const char* name, int dflt, int lo, int hi) {
    const char* v = getenv(name);
    if (!v) return dflt;
    int x = atoi(v);
    return x < lo ? lo : (x > hi ? hi : x);
}

static cudaError_t launch_gemv(int nproj, int epi, int kbits, GemvParams& P, int sm_count, cudaStream_t st) {
    const uint32_t zs_bytes = (uint32_t)(nproj * GROUP_CHUNKS * CHUNK_ROWS * ZS_STRIDE * sizeof(float));
    P.w_bytes = KT * P.kt_stride_words * 4;
    const uint32_t stage_one = P.w_bytes + GROUP_CHUNKS * nproj * KT * A_TILE_WORDS * 4;   // one sub-stage, 4 chunks of rows
    // resident CTAs per SM (tunable for experiments: MLXS_GU_CTAS 1..2, MLXS_DN_CTAS 1..3); the shared-memory ring
    // takes what the SM's 227 KB leave per CTA
    static const int gu_ctas = tune_env("MLXS_GU_CTAS", 2, 1, 2), dn_ctas = tune_env("MLXS_DN_CTAS", 3, 1, 3);
    const int per_sm = nproj == 2 ? gu_ctas : dn_ctas;
    const uint32_t budget = (uint32_t)(225 * 1024 / per_sm) - 2048u;
    // Ring: two large slots (each carries as many sub-stages of an item as fit, see the producer) rather than many
    // small ones: the barrier round trip per slot is what the consumers pay for.  MLXS_EXL3_RING = n forces n slots of
    // the largest size that fits.
    static const int ring_slots = tune_env("MLXS_EXL3_RING", 2, 2, 8);
    uint32_t ns = (uint32_t)ring_slots;
    P.stage_bytes = ((budget - zs_bytes) / ns) & ~127u;
    if (P.stage_bytes < stage_one) { ns = (budget - zs_bytes) / stage_one; P.stage_bytes = stage_one; }
    if (ns < 2) return cudaErrorInvalidValue;
    if (ns > 8) ns = 8;
    P.n_stages = ns;
    const size_t smem = zs_bytes + (size_t)ns * P.stage_bytes;
    cudaError_t e;
    const int ctas = per_sm * sm_count;
    static const int k_parts = tune_env("MLXS_K_PARTS", 4, 1, 4);
    P.max_parts = (uint32_t)k_parts;
#define MLXS_LAUNCH(NP, EP, KS, KBITS)                                                                            \
    do {                                                                                                         \
        e = cudaFuncSetAttribute(exl3_gemv_kernel<NP, EP, KS, KBITS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        if (e != cudaSuccess) return e;                                                                          \
        exl3_gemv_kernel<NP, EP, KS, KBITS><<<ctas, NP * 256 + 32, smem, st>>>(P);                               \
    } while (0)
    if (kbits == 3) {
        if (nproj == 2) MLXS_LAUNCH(2, EPI_GATE_UP, 384, 3);
        else if (epi == EPI_DOWN) MLXS_LAUNCH(1, EPI_DOWN, 192, 3);
        else if (P.kt_stride_words == 192) MLXS_LAUNCH(1, EPI_RAW, 192, 3);
        else MLXS_LAUNCH(1, EPI_RAW, 384, 3);
    } else if (kbits == 2) {
        if (nproj == 2) MLXS_LAUNCH(2, EPI_GATE_UP, 256, 2);
        else if (epi == EPI_DOWN) MLXS_LAUNCH(1, EPI_DOWN, 128, 2);
        else if (P.kt_stride_words == 128) MLXS_LAUNCH(1, EPI_RAW, 128, 2);
        else MLXS_LAUNCH(1, EPI_RAW, 256, 2);
    } else {
        return cudaErrorInvalidValue;
    }
#undef MLXS_LAUNCH
    return cudaGetLastError();
}

cudaError_t launch_exl3_gate_up(const Exl3GemvArgs& a, cudaStream_t st) {
    GemvParams P{};
    P.code = a.L.gu_code;
    P.expert_stride_words = 2 * exl3_code_words(a.d);
    P.n_blocks = a.d.I / 128; P.nkt = a.d.H / 16; P.kt_stride_words = 16 * exl3_tile_words(a.d); P.proj_off_words = 0;
    P.xa = a.xa_gu; P.t = a.t; P.counter_idx = HDR_CTR_GU;
    P.scales = a.L.scales; P.scales_stride = exl3_scales_per_expert(a.d);
    P.H = a.d.H; P.I = a.d.I; P.xa_d = a.xa_d; P.out = nullptr; P.out_dim = a.d.I; P.limit = a.limit; P.status = a.status;
    P.ks_scratch = a.ks_scratch; P.ks_count = a.ks_count; P.n_sm = (uint32_t)a.sm_count;
    P.ks_cap_items = ksplit_cap_items(a.sm_count, (size_t)2 * GROUP_CHUNKS * CHUNK_ROWS * ZS_STRIDE * sizeof(float));
    P.poll_limit = a.poll_limit ? a.poll_limit : (1u << 20); P.withhold = a.withhold;
    return launch_gemv(2, EPI_GATE_UP, (int)a.d.K, P, a.sm_count, st);
}
cudaError_t launch_exl3_down(const Exl3GemvArgs& a, cudaStream_t st) {
    GemvParams P{};
    P.code = a.L.d_code;
    P.expert_stride_words = exl3_code_words(a.d);
    P.n_blocks = a.d.H / 128; P.nkt = a.d.I / 16; P.kt_stride_words = 8 * exl3_tile_words(a.d); P.proj_off_words = 0;
    P.xa = a.xa_d; P.t = a.t; P.counter_idx = HDR_CTR_DOWN;
    P.scales = a.L.scales; P.scales_stride = exl3_scales_per_expert(a.d);
    P.H = a.d.H; P.I = a.d.I; P.xa_d = nullptr; P.out = a.ro; P.out_dim = a.d.H; P.limit = a.limit; P.status = a.status;
    P.ks_scratch = a.ks_scratch; P.ks_count = a.ks_count; P.n_sm = (uint32_t)a.sm_count;
    P.ks_cap_items = ksplit_cap_items(a.sm_count, (size_t)GROUP_CHUNKS * CHUNK_ROWS * ZS_STRIDE * sizeof(float));
    P.poll_limit = a.poll_limit ? a.poll_limit : (1u << 20); P.withhold = 0;
    return launch_gemv(1, EPI_DOWN, (int)a.d.K, P, a.sm_count, st);
}
cudaError_t launch_exl3_raw(const uint32_t* code_e, uint32_t in_dim, uint32_t out_dim, uint32_t ktile_stride_words,
                            uint32_t proj_off_words, int kbits, DispatchTables t, const uint32_t* xa, float* z,
                            uint32_t* status, int sm_count, cudaStream_t st) {
    GemvParams P{};
    P.code = code_e; P.expert_stride_words = 0;
    P.n_blocks = out_dim / 128; P.nkt = in_dim / 16; P.kt_stride_words = ktile_stride_words; P.proj_off_words = proj_off_words;
    P.xa = xa; P.t = t; P.counter_idx = HDR_CTR_AUX;
    P.scales = nullptr; P.scales_stride = 0; P.H = 0; P.I = 0; P.xa_d = nullptr; P.out = z; P.out_dim = out_dim;
    P.limit = 0.f; P.status = status; P.poll_limit = 1u << 20; P.withhold = 0;
    return launch_gemv(1, EPI_RAW, kbits, P, sm_count, st);
}

}  // namespace mlxs
