// Dense bf16 products on the tcgen05 tensor cores: the shared expert's three linears and the router's logits.
//
// The shared expert (src/arch/deepseek_v41/graph.zig:2162-2172) is h = silu(min(w1 x, lim)) * clip(w3 x, +-lim),
// out = w2 h; the router's logits are f32(x) . W_g^T (graph.zig:2033).  All of them are C[T, N] = X[T, K] . W[N, K]^T
// with bf16 operands and f32 accumulation.  As in the expert lanes W is the MMA's A operand (M = 128 output features per
// accumulator group) and the token rows are the B operand (N = up to 256 rows, rounded to 16): a ragged last tile pads
// to 16 rows, and the epilogue's stores run along the feature dimension.
//   * weights are re-tiled once at load into K-major core matrices, [feature block of 128][k stage of 64][8-row group]
//     ([projection] for gate / up) [8-k group][8 rows x 8 k]: one (block, stage) is one contiguous run for a bulk copy,
//     gate and up of the same block travel together;
//   * rows are staged once per call in the same core-matrix order (dense_rows_kernel); the gate/up epilogue writes h
//     straight into that order for the down product;
//   * a CTA owns (token tile, feature block) with two accumulator groups in tensor memory (gate and up of one block,
//     or two adjacent blocks of a single projection): 2 x 256 columns = all 512;
//   * one producer thread (bulk copies into a 3-stage ring, mbarriers), one MMA thread (tcgen05.mma.kind::f16 on bf16,
//     K = 16 per instruction, commits free the stage), eight epilogue warps (tcgen05.ld, activation, stores);
//   * small batches split the reduction dimension over several CTAs so that every SM streams weights: each CTA leaves
//     its f32 partial tile in a scratch slot, the last to arrive folds the parts in part order (a fixed order, so the
//     bits do not depend on which CTA came last) and runs the epilogue.
// Every wait is bounded; on a give-up the CTA records the status word, skips its work and still frees tensor memory.
#include <cstdlib>

#include "common.cuh"
#include "kernels.h"
#include "umma.cuh"

namespace mlxs {

constexpr int DG_KS = 64;                         // inputs per stage
constexpr int DG_NT = 256;                        // rows per token tile (MMA N)
constexpr int DG_STAGES = 3;
constexpr int DG_A_TILE = 128 * DG_KS * 2;        // one projection's (block, stage): 16 KB
constexpr int DG_A_STAGE = 2 * DG_A_TILE;         // two accumulator groups' weights
constexpr int DG_B_STAGE = DG_NT * DG_KS * 2;     // rows of a stage: 32 KB at 256 rows
constexpr int DG_EPI_WARPS = 8;

// ---- load-time re-tiling of a weight matrix W[n_out, K] (row-major bf16) ----
// np = 2: w0 and w1 interleaved per 8-row group ([rc][p][kc][8][8]); np = 1: w0 alone ([rc][kc][8][8])
__global__ void dense_retile_kernel(const __nv_bfloat16* __restrict__ w0, const __nv_bfloat16* __restrict__ w1, uint32_t n_out,
                                    uint32_t K, int np, uint4* __restrict__ dst) {
    const size_t n_vec = (size_t)np * n_out * K / 8;
    const uint32_t nks = K / DG_KS;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_vec; i += (size_t)gridDim.x * blockDim.x) {
        size_t r = i;
        const uint32_t r8 = r % 8; r /= 8;
        const uint32_t kc = r % 8; r /= 8;
        const uint32_t p = np == 2 ? (uint32_t)(r % 2) : 0u; if (np == 2) r /= 2;
        const uint32_t rc = r % 16; r /= 16;
        const uint32_t ks = r % nks; r /= nks;
        const uint32_t nb = (uint32_t)r;
        const __nv_bfloat16* src = (p ? w1 : w0) + (size_t)(nb * 128 + rc * 8 + r8) * K + (size_t)ks * DG_KS + kc * 8;
        dst[i] = *reinterpret_cast<const uint4*>(src);
    }
}

cudaError_t launch_dense_retile(const __nv_bfloat16* w0, const __nv_bfloat16* w1, uint32_t n_out, uint32_t K, void* dst,
                                cudaStream_t st) {
    if (n_out % 128 || K % DG_KS) return cudaErrorInvalidValue;
    dense_retile_kernel<<<592, 256, 0, st>>>(w0, w1, n_out, K, w1 ? 2 : 1, static_cast<uint4*>(dst));
    return cudaGetLastError();
}

// ---- rows -> B-operand order ----
// element offset of (row r of tile tt, input k): tiles before tt are full
__host__ __device__ inline size_t dg_b_off(uint32_t K, uint32_t tt, uint32_t rows16, uint32_t r, uint32_t k) {
    return (size_t)tt * DG_NT * K + (size_t)(k / DG_KS) * (rows16 * DG_KS) + (size_t)((k % DG_KS) / 8) * (rows16 * 8) +
           (r / 8) * 64 + (r % 8) * 8 + k % 8;
}
__global__ void __launch_bounds__(256) dense_rows_kernel(const __nv_bfloat16* __restrict__ x, uint32_t T, uint32_t K,
                                                         uint16_t* __restrict__ xb) {
    const uint32_t tt = blockIdx.x;
    const uint32_t rows = min((uint32_t)DG_NT, T - tt * DG_NT), rows16 = (rows + 15) / 16 * 16, groups = K / 8;
    // a thread moves 8 consecutive inputs of one row; consecutive threads take consecutive rows (one core matrix = 128 B)
    for (uint32_t i = blockIdx.y * blockDim.x + threadIdx.x; i < rows16 * groups; i += gridDim.y * blockDim.x) {
        const uint32_t r = i % rows16, kg = i / rows16;
        uint4 raw = make_uint4(0, 0, 0, 0);
        if (r < rows) raw = *reinterpret_cast<const uint4*>(x + (size_t)(tt * DG_NT + r) * K + (size_t)kg * 8);
        *reinterpret_cast<uint4*>(xb + dg_b_off(K, tt, rows16, r, kg * 8)) = raw;
    }
}

struct DenseParams {
    const uint8_t* w;          // re-tiled weights
    uint32_t n_blocks;         // output features / 128
    uint32_t n_ks;             // K / 64
    const uint16_t* xb;        // rows in B-operand order
    uint32_t T, K;
    float limit;
    uint16_t* hb;              // gate/up: h in B-operand order over n_out inputs
    float* out;                // plain: [T, n_out] f32
    uint32_t n_out;
    uint32_t k_parts;          // CTAs that share one item's reduction dimension (1: none)
    float* part_scratch;       // [item][part][2 groups][rows16][128] f32
    uint32_t* part_count;      // [item] arrivals, zero between launches
    uint32_t* status;
    uint32_t poll_limit;
};

// NPROJ = 2: gate and up of one feature block (activation epilogue -> hb); NPROJ = 1: two adjacent blocks -> out
template <int NPROJ>
__global__ void __launch_bounds__(64 + DG_EPI_WARPS * 32, 1) dense_gemm_kernel(const DenseParams P) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t full_bar[DG_STAGES], empty_bar[DG_STAGES], acc_full, acc_empty, epi_bar;
    __shared__ uint32_t s_tmem;
    __shared__ volatile int s_abort;
    __shared__ volatile int s_last;
    uint8_t* a_ring = smem_raw;                              // [stage][2 groups' tiles]
    uint8_t* b_ring = smem_raw + DG_STAGES * DG_A_STAGE;     // [stage][rows16 x 64]
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t n_tt = (P.T + DG_NT - 1) / DG_NT;
    const uint32_t n_fb = NPROJ == 2 ? P.n_blocks : P.n_blocks / 2;     // feature-block groups
    const uint32_t KP = P.k_parts;
    const uint32_t n_units = n_tt * n_fb * KP;
    if (blockIdx.x >= n_units) return;   // before any tensor memory is taken (the whole CTA reads the same count)

    if (threadIdx.x == 0) {
        for (int s = 0; s < DG_STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
        mbar_init(&acc_full, 1);
        mbar_init(&acc_empty, DG_EPI_WARPS);
        mbar_init(&epi_bar, DG_EPI_WARPS);
        s_abort = 0;
        mbar_fence_init();
    }
    if (warp == 0) tmem_alloc(&s_tmem, 512);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = s_tmem;
    // part p of the reduction covers stages [p n_ks / KP, (p + 1) n_ks / KP): a function of the shape and the part count
    auto part_begin = [&](uint32_t part) { return (uint32_t)(((uint64_t)part * P.n_ks) / KP); };
    auto give_up = [&](uint32_t code) { if (!s_abort) atomicMax(P.status, code); s_abort = 1; };
    // unit -> (token tile, feature-block group, part of the reduction); feature blocks vary fastest so that the CTAs
    // running together share the rows of a few token tiles and the weights in L2
    auto decode_unit = [&](uint32_t unit, uint32_t& tt, uint32_t& fb, uint32_t& part) {
        part = unit % KP;
        const uint32_t item = unit / KP;
        fb = item % n_fb;
        tt = item / n_fb;
    };

    if (warp == 0) {
        // ---------------- producer ----------------
        if (lane == 0) {
            uint32_t s = 0, ph = 0;
            for (uint32_t unit = blockIdx.x; unit < n_units && !s_abort; unit += gridDim.x) {
                uint32_t tt, fb, part;
                decode_unit(unit, tt, fb, part);
                const uint32_t rows = min((uint32_t)DG_NT, P.T - tt * DG_NT), rows16 = (rows + 15) / 16 * 16;
                const uint32_t b_bytes = rows16 * DG_KS * 2;
                const uint16_t* xsrc = P.xb + (size_t)tt * DG_NT * P.K;
                bool ok = true;
                for (uint32_t ks = part_begin(part); ks < part_begin(part + 1); ++ks) {
                    if (!mbar_wait_bounded(&empty_bar[s], ph ^ 1u, &s_abort, 64, P.poll_limit)) { give_up(ST_WAIT_EMPTY); ok = false; break; }
                    mbar_expect_tx(&full_bar[s], DG_A_STAGE + b_bytes);
                    if (NPROJ == 2) {
                        bulk_g2s(a_ring + s * DG_A_STAGE, P.w + ((size_t)fb * P.n_ks + ks) * DG_A_STAGE, DG_A_STAGE, &full_bar[s]);
                    } else {
                        bulk_g2s(a_ring + s * DG_A_STAGE, P.w + ((size_t)(2 * fb) * P.n_ks + ks) * DG_A_TILE, DG_A_TILE, &full_bar[s]);
                        bulk_g2s(a_ring + s * DG_A_STAGE + DG_A_TILE, P.w + ((size_t)(2 * fb + 1) * P.n_ks + ks) * DG_A_TILE, DG_A_TILE, &full_bar[s]);
                    }
                    bulk_g2s(b_ring + s * DG_B_STAGE, xsrc + (size_t)ks * (rows16 * DG_KS), b_bytes, &full_bar[s]);
                    if (++s == DG_STAGES) { s = 0; ph ^= 1u; }
                }
                if (!ok) break;
            }
            if (s_abort) for (int i = 0; i < 2000; ++i) __nanosleep(1000);
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            uint32_t s = 0, ph = 0, n_done = 0;
            const uint32_t a_s = smem_u32(a_ring), b_s = smem_u32(b_ring);
            // gate / up interleave per 8-row group: a projection's core matrices of one K group are 2 KB apart
            constexpr uint32_t A_SBO = NPROJ == 2 ? 2048u : 1024u, A_LBO = 128u, A_GROUP = NPROJ == 2 ? 1024u : (uint32_t)DG_A_TILE;
            for (uint32_t unit = blockIdx.x; unit < n_units && !s_abort; unit += gridDim.x, ++n_done) {
                uint32_t tt, fb, part;
                decode_unit(unit, tt, fb, part);
                const uint32_t rows = min((uint32_t)DG_NT, P.T - tt * DG_NT), rows16 = (rows + 15) / 16 * 16;
                const uint32_t idesc = umma_idesc(UMMA_BF16, rows16), lbo_b = rows16 * 16;
                if (!mbar_wait_bounded(&acc_empty, (n_done & 1u) ^ 1u, &s_abort, 64, P.poll_limit)) { give_up(ST_WAIT_EMPTY); break; }
                tc_fence_after();
                bool ok = true;
                const uint32_t nk = part_begin(part + 1) - part_begin(part);
                for (uint32_t kk = 0; kk < nk; ++kk) {
                    if (!mbar_wait_bounded(&full_bar[s], ph, &s_abort, 0, P.poll_limit)) { give_up(ST_WAIT_FULL); ok = false; break; }
                    tc_fence_after();
                    const uint32_t a0 = a_s + s * DG_A_STAGE, b0 = b_s + s * DG_B_STAGE;
#pragma unroll
                    for (int gq = 0; gq < 2; ++gq) {
#pragma unroll
                        for (int i = 0; i < DG_KS / 16; ++i)
                            umma_f16(tmem + gq * DG_NT, umma_smem_desc(a0 + gq * A_GROUP + i * 2 * A_LBO, A_LBO, A_SBO),
                                     umma_smem_desc(b0 + i * 2 * lbo_b, lbo_b, 128), idesc, (kk | (uint32_t)i) ? 1u : 0u);
                    }
                    umma_commit(&empty_bar[s]);
                    if (++s == DG_STAGES) { s = 0; ph ^= 1u; }
                }
                if (!ok) break;
                umma_commit(&acc_full);
            }
        }
    } else {
        // ---------------- epilogue warps ----------------
        // warp = (lane quarter q, half): a thread owns output feature 32 q + lane of both groups; the 16-row chunks of
        // the tile alternate between the two halves
        const uint32_t ew = warp - 2, q = warp & 3u, half = ew >> 2;
        uint32_t n_done = 0, epi_ph = 0;
        // rendezvous of the epilogue warps: a bounded mbarrier wait like every other wait of the kernel
        auto epi_sync = [&]() -> bool {
            __syncwarp();
            if (lane == 0) mbar_arrive(&epi_bar);
            const bool ok = mbar_wait_bounded(&epi_bar, epi_ph, &s_abort, 0, P.poll_limit);
            epi_ph ^= 1u;
            if (!ok) give_up(ST_WAIT_FULL);
            return ok;
        };
        for (uint32_t unit = blockIdx.x; unit < n_units && !s_abort; unit += gridDim.x, ++n_done) {
            uint32_t tt, fb, part;
            decode_unit(unit, tt, fb, part);
            const uint32_t item = unit / KP;
            const uint32_t rows = min((uint32_t)DG_NT, P.T - tt * DG_NT), rows16 = (rows + 15) / 16 * 16, nch = rows16 / 16;
            if (!mbar_wait_bounded(&acc_full, n_done & 1u, &s_abort, 0, P.poll_limit)) { give_up(ST_WAIT_FULL); break; }
            tc_fence_after();
            const uint32_t fl = q * 32u + lane;                 // feature inside the block
            bool last = true;
            if (KP > 1) {
                // leave this part's tile in its slot: [item][part][group][chunk row][feature]
                float* slot = P.part_scratch + ((size_t)item * KP + part) * (2 * DG_NT * 128);
                for (uint32_t c = half; c < nch; c += 2) {
#pragma unroll
                    for (int gq = 0; gq < 2; ++gq) {
                        uint32_t v[16];
                        tmem_ld16(tmem + ((q * 32u) << 16) + gq * DG_NT + c * 16, v);
#pragma unroll
                        for (int i = 0; i < 16; ++i) slot[((size_t)gq * DG_NT + c * 16 + i) * 128 + fl] = __uint_as_float(v[i]);
                    }
                }
                __threadfence();
                // every epilogue warp has left its share; one thread then counts the CTA in
                if (!epi_sync()) break;
                if (ew == 0 && lane == 0) {
                    const uint32_t seen = atomicAdd(&P.part_count[item], 1u);
                    s_last = seen == KP - 1 ? 1 : 0;
                    if (seen == KP - 1) P.part_count[item] = 0;
                }
                if (!epi_sync()) break;
                last = s_last != 0;
                if (last) __threadfence();
            }
            if (last) {
                const float* base = P.part_scratch + (size_t)item * KP * (2 * DG_NT * 128);
                for (uint32_t c = half; c < nch; c += 2) {
                    float vg[16], vu[16];
                    if (KP > 1) {
#pragma unroll
                        for (int i = 0; i < 16; ++i) {
                            float a = 0.f, b = 0.f;
                            for (uint32_t pp = 0; pp < KP; ++pp) {
                                const float* sl = base + (size_t)pp * (2 * DG_NT * 128);
                                const float x0 = __ldcg(sl + ((size_t)c * 16 + i) * 128 + fl);
                                const float x1 = __ldcg(sl + ((size_t)DG_NT + c * 16 + i) * 128 + fl);
                                a = pp == 0 ? x0 : a + x0;
                                b = pp == 0 ? x1 : b + x1;
                            }
                            vg[i] = a; vu[i] = b;
                        }
                    } else {
                        uint32_t r0[16], r1[16];
                        tmem_ld16(tmem + ((q * 32u) << 16) + 0 * DG_NT + c * 16, r0);
                        tmem_ld16(tmem + ((q * 32u) << 16) + 1 * DG_NT + c * 16, r1);
#pragma unroll
                        for (int i = 0; i < 16; ++i) { vg[i] = __uint_as_float(r0[i]); vu[i] = __uint_as_float(r1[i]); }
                    }
                    if (NPROJ == 2) {
                        const uint32_t f = fb * 128 + fl;
#pragma unroll
                        for (int i = 0; i < 16; ++i) {
                            const uint32_t r = c * 16 + i;
                            float gate = vg[i], up = vu[i];
                            if (P.limit > 0.f) {
                                gate = (gate != gate) ? gate : (gate < P.limit ? gate : P.limit);
                                up = (up != up) ? up : (up > P.limit ? P.limit : (up < -P.limit ? -P.limit : up));
                            }
                            const float yv = sigmoid_tail_fast(gate);
                            const float sg = gate < 0.f ? yv : 1.0f - yv;
                            const __nv_bfloat16 hv = __float2bfloat16_rn((gate * sg) * up);
                            // padding rows of the tile are written as zeros: the down product reads whole 16-row groups
                            P.hb[dg_b_off(P.n_out, tt, rows16, r, f)] = r < rows ? __bfloat16_as_ushort(hv) : (uint16_t)0;
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < 16; ++i) {
                            const uint32_t r = c * 16 + i;
                            if (r < rows) {
                                float* o = P.out + (size_t)(tt * DG_NT + r) * P.n_out + (size_t)(2 * fb) * 128 + fl;
                                o[0] = vg[i];
                                o[128] = vu[i];
                            }
                        }
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
    if (warp == 0) tmem_free(tmem, 512);
}

// Parts of the reduction per item: as many as give every SM a weight stream, each part at least 4 stages long.  A
// function of the item count (token tiles x feature blocks) and the SM count, so calls of up to 256 tokens always split
// the same way and a row's bits do not depend on the batch around it.
static uint32_t dg_pick_parts(uint32_t n_items, uint32_t n_ks, int sm_count) {
    uint32_t kp = (uint32_t)sm_count / (n_items ? n_items : 1u);
    if (kp > n_ks / 4) kp = n_ks / 4;
    if (kp > 16) kp = 16;
    return kp ? kp : 1u;
}

size_t dense_gemm_scratch_bytes(int sm_count) { return (size_t)sm_count * 2 * DG_NT * 128 * sizeof(float); }

template <int NPROJ>
static cudaError_t dg_launch(DenseParams P, int sm_count, cudaStream_t st) {
    const size_t smem = (size_t)DG_STAGES * (DG_A_STAGE + DG_B_STAGE);
    cudaError_t e = cudaFuncSetAttribute(dense_gemm_kernel<NPROJ>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    const uint32_t n_tt = (P.T + DG_NT - 1) / DG_NT, n_fb = NPROJ == 2 ? P.n_blocks : P.n_blocks / 2;
    const uint32_t n_items = n_tt * n_fb;
    P.k_parts = P.part_scratch ? dg_pick_parts(n_items, P.n_ks, sm_count) : 1;
    // the scratch holds one slot per (item, part): items x parts <= SMs by construction
    const uint32_t n_units = n_items * P.k_parts;
    const uint32_t grid = n_units < (uint32_t)sm_count ? n_units : (uint32_t)sm_count;
    dense_gemm_kernel<NPROJ><<<grid, 64 + DG_EPI_WARPS * 32, smem, st>>>(P);
    return cudaGetLastError();
}

// Units of one item must run concurrently-or-in-order for the last-arriver fold; they do: a CTA takes units blockIdx,
// blockIdx + grid, ..., nobody waits for another CTA, and the fold happens in whichever CTA arrives last.
cudaError_t launch_dense_shared_expert(const DenseSharedArgs& a, cudaStream_t st) {
    if (a.T == 0) return cudaSuccess;
    const uint32_t n_tt = (a.T + DG_NT - 1) / DG_NT;
    dense_rows_kernel<<<dim3(n_tt, 16), 256, 0, st>>>(a.x, a.T, a.H, a.xb);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    DenseParams P{};
    P.status = a.status; P.poll_limit = 1u << 20; P.limit = a.limit; P.T = a.T;
    P.part_scratch = a.part_scratch; P.part_count = a.part_count;
    // gate / up -> h (B-operand order over I inputs)
    P.w = static_cast<const uint8_t*>(a.w_gu); P.n_blocks = a.I / 128; P.n_ks = a.H / DG_KS; P.xb = a.xb; P.K = a.H; P.hb = a.hb; P.out = nullptr; P.n_out = a.I;
    if ((e = dg_launch<2>(P, a.sm_count, st)) != cudaSuccess) return e;
    // down -> out f32 [T, H]
    P.w = static_cast<const uint8_t*>(a.w_d); P.n_blocks = a.H / 128; P.n_ks = a.I / DG_KS; P.xb = a.hb; P.K = a.I; P.hb = nullptr; P.out = a.out; P.n_out = a.H;
    return dg_launch<1>(P, a.sm_count, st);
}

cudaError_t launch_dense_logits(const __nv_bfloat16* x, const void* w_tiled, uint32_t T, uint32_t E, uint32_t H, uint16_t* xb,
                                float* logits, float* part_scratch, uint32_t* part_count, uint32_t* status, int sm_count,
                                cudaStream_t st) {
    if (T == 0) return cudaSuccess;
    const uint32_t n_tt = (T + DG_NT - 1) / DG_NT;
    dense_rows_kernel<<<dim3(n_tt, 16), 256, 0, st>>>(x, T, H, xb);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    DenseParams P{};
    P.status = status; P.poll_limit = 1u << 20; P.limit = 0.f; P.T = T;
    P.part_scratch = part_scratch; P.part_count = part_count;
    P.w = static_cast<const uint8_t*>(w_tiled); P.n_blocks = E / 128; P.n_ks = H / DG_KS; P.xb = xb; P.K = H; P.hb = nullptr;
    P.out = logits; P.n_out = E;
    return dg_launch<1>(P, sm_count, st);
}

bool dense_gemm_supported(uint32_t n_out, uint32_t K, int two_blocks) {
    return K % DG_KS == 0 && n_out % (two_blocks ? 256 : 128) == 0;
}

}  // namespace mlxs
