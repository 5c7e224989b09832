// Shared device helpers for the routed-MoE kernels (sm_100a).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace mlxs {

// Error words kernels may write into the handle's status word (never trap, never spin without a bound).
enum : uint32_t {
    ST_OK = 0,
    ST_BAD_EXPERT_ID = 1,    // a routed id outside [0, n_experts)
    ST_WAIT_FULL = 2,        // a consumer's bounded wait for a staged copy ran out
    ST_WAIT_EMPTY = 3,       // the producer's bounded wait for a free stage ran out
    ST_WORKLIST_OVERFLOW = 4,
    ST_NOT_LOADED = 5,       // a routed expert has no resident record
    ST_EP_OVERFLOW = 6,      // expert parallel: a rank received more rows than its workspace holds
    ST_EP_TIMEOUT = 7        // expert parallel: a peer's epoch word did not arrive within the bound
};

constexpr uint32_t SCALE_BITS = 0x3DB504F3u;  // 128^-0.5 (src/arch/deepseek_v41/experts.zig:428-429)
constexpr uint32_t MUL1 = 0x83DCD12Du;        // src/expert/bank.zig:109

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// ---- mbarrier + bulk copy (TMA 1-D) ----
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait: gives up after `limit` polls (each poll itself blocks for a hardware-defined slice) or as soon as
// *abort_flag is set by another thread of the CTA.  Returns false when it gave up.
// sleep_ns > 0: back off between polls (the single-lane producer / MMA-issuer roles wait most of the time; polling
// flat out would take issue slots from the warps that do the arithmetic).
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                                  uint32_t sleep_ns = 0, uint32_t limit = (1u << 20)) {
    for (uint32_t i = 0; i < limit; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if (sleep_ns) __nanosleep(sleep_ns);
        if ((i & 63u) == 63u && *abort_flag) return false;
    }
    return false;
}
// global -> this CTA's shared memory, completion counted in bytes on `bar`; 16-byte aligned addresses and size
__device__ __forceinline__ void bulk_g2s(void* dst_smem, const void* src_gmem, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(dst_smem)),
                 "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void named_bar_sync(int id, int nthreads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

// ---- tensor-core fragment op: D(16x8 f32) += A(16x16 f16, row) x B(16x8 f16, col) ----
__device__ __forceinline__ void mma_f16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// ---- EXL3 mul1: two 16-bit trellis states -> half2 (lo = a, hi = b) ----
// value = f16( (1024 + bytesum(state * 0x83DCD12D)) * h(0x1EEE) + h(0xC931) ), one rounding
// (src/exl3/kernels.zig:963-971; src/kernels/exl3/dsv41_exl3_mul1h_k3_2304.metal:27-31)
__device__ __forceinline__ uint32_t mul1_pair(uint32_t sa, uint32_t sb) {
    uint32_t xa = sa * MUL1, xb = sb * MUL1;
    uint32_t ha = __dp4a(xa, 0x01010101u, 0x6400u);  // 0x6400 + byte sum = the half bits of 1024 + s
    uint32_t hb = __dp4a(xb, 0x01010101u, 0x6400u);
    uint32_t pk = hb * 65536u + ha;
    const uint32_t kinv = 0x1EEE1EEEu, kbias = 0xC931C931u;
    __half2 r = __hfma2(*reinterpret_cast<__half2*>(&pk), *reinterpret_cast<const __half2*>(&kinv),
                        *reinterpret_cast<const __half2*>(&kbias));
    return *reinterpret_cast<uint32_t*>(&r);
}

// One lane's share of a 16x16 K=3 tile: lane L owns code positions 8L..8L+7, i.e. the 37 stream bits ending at
// stream bit 24(L+1); `lo` is the tile word holding that last bit, `hi` the word before it (circular), lp the
// distance of the last bit from the word's bit 0.  Returns the two B fragments (k16 x n8) of the tile's column
// halves for mma m16n8k16: b[0], b[1] = columns 0..7, b[2], b[3] = columns 8..15 (the exllamav3 tensor-core order,
// src/exl3/kernels.zig:978-986).
__device__ __forceinline__ void exl3_decode_lane(uint32_t lo, uint32_t hi, uint32_t lp, uint32_t (&b)[4]) {
    uint32_t v0 = __funnelshift_r(lo, hi, lp);  // stream bits, window m at bits [3m, 3m+16)
    uint32_t vh = hi >> lp;
    uint32_t v1 = __funnelshift_r(v0, vh, 18);  // windows 6, 7 at bits 0 and 3
    uint32_t w0 = v0 & 0xFFFFu;
    uint32_t w1 = (v0 >> 3) & 0xFFFFu;
    uint32_t w2 = (v0 >> 6) & 0xFFFFu;
    uint32_t w3 = (v0 >> 9) & 0xFFFFu;
    uint32_t w4 = (v0 >> 12) & 0xFFFFu;
    uint32_t w5 = (v0 >> 15) & 0xFFFFu;
    uint32_t w6 = v1 & 0xFFFFu;
    uint32_t w7 = (v1 >> 3) & 0xFFFFu;
    // code position j = 7 - m; positions (0,1),(2,3) -> columns 0..7 rows (r0,r0+1),(r0+8,r0+9); (4,5),(6,7) -> 8..15
    b[0] = mul1_pair(w7, w6);
    b[1] = mul1_pair(w5, w4);
    b[2] = mul1_pair(w3, w2);
    b[3] = mul1_pair(w1, w0);
}
__device__ __forceinline__ void exl3_lane_plan(uint32_t lane, uint32_t& wi, uint32_t& wj, uint32_t& lp) {
    wi = (3u * lane + 2u) >> 2;        // word of the lane's last stream bit
    wj = (wi + 23u) % 24u;             // the word before it, circular
    lp = 8u * ((lane + 1u) & 3u);
}
// The same for K = 2 (a tile is 16 words): lane L's 8 states end at stream bits 16 L + 2 .. 16 L + 16, i.e. they live in
// the 30 bits ending with halfword L.  `lo` = the word holding halfword L, `hi` = the word before it (circular),
// lp = 0 when halfword L is the word's low half, 16 when it is the high half; window m at bits [2m, 2m + 16).
// Bit-level definition: src/exl3/kernels.zig:988-1020 (tileStates at K = 2), generic window formulas
// scripts/dsv41_exl3_k2_gen.py:96-112.
__device__ __forceinline__ void exl3_decode_lane_k2(uint32_t lo, uint32_t hi, uint32_t lp, uint32_t (&b)[4]) {
    const uint32_t v0 = __funnelshift_r(lo, hi, lp);
    const uint32_t w0 = v0 & 0xFFFFu, w1 = (v0 >> 2) & 0xFFFFu, w2 = (v0 >> 4) & 0xFFFFu, w3 = (v0 >> 6) & 0xFFFFu;
    const uint32_t w4 = (v0 >> 8) & 0xFFFFu, w5 = (v0 >> 10) & 0xFFFFu, w6 = (v0 >> 12) & 0xFFFFu, w7 = (v0 >> 14) & 0xFFFFu;
    b[0] = mul1_pair(w7, w6);
    b[1] = mul1_pair(w5, w4);
    b[2] = mul1_pair(w3, w2);
    b[3] = mul1_pair(w1, w0);
}
__device__ __forceinline__ void exl3_lane_plan_k2(uint32_t lane, uint32_t& wi, uint32_t& wj, uint32_t& lp) {
    wi = lane >> 1;
    wj = (wi + 15u) % 16u;
    lp = (lane & 1u) ? 0u : 16u;
}
// by code width
template <int KB>
__device__ __forceinline__ void exl3_decode_lane_kb(uint32_t lo, uint32_t hi, uint32_t lp, uint32_t (&b)[4]) {
    if (KB == 3) exl3_decode_lane(lo, hi, lp, b);
    else exl3_decode_lane_k2(lo, hi, lp, b);
}
template <int KB>
__device__ __forceinline__ void exl3_lane_plan_kb(uint32_t lane, uint32_t& wi, uint32_t& wj, uint32_t& lp) {
    if (KB == 3) exl3_lane_plan(lane, wi, wj, lp);
    else exl3_lane_plan_k2(lane, wi, wj, lp);
}

// ---- 128-point Sylvester-natural Hadamard over a warp: lane holds elements 4*lane .. 4*lane+3 ----
// (unnormalised; src/arch/glm5_next/exl3_forms_ref.zig:116-135)
__device__ __forceinline__ void hadamard128_warp(float (&v)[4], uint32_t lane) {
    float a0 = v[0] + v[1], a1 = v[0] - v[1], a2 = v[2] + v[3], a3 = v[2] - v[3];
    v[0] = a0 + a2; v[1] = a1 + a3; v[2] = a0 - a2; v[3] = a1 - a3;
#pragma unroll
    for (uint32_t m = 1; m < 32; m <<= 1) {
        bool up = (lane & m) != 0;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            float o = __shfl_xor_sync(0xFFFFFFFFu, v[q], m);
            v[q] = up ? (o - v[q]) : (v[q] + o);
        }
    }
}

// split an f32 into f16 hi + f16 lo (hi + lo carries ~22 significant bits)
__device__ __forceinline__ void split_hi_lo(float x, __half& hi, __half& lo) {
    hi = __float2half_rn(x);
    lo = __float2half_rn(x - __half2float(hi));
}
__device__ __forceinline__ uint32_t pack_h2(__half a, __half b) {
    return (uint32_t)__half_as_ushort(a) | ((uint32_t)__half_as_ushort(b) << 16);
}
__device__ __forceinline__ float bf16_round_f(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }
// 1 / (1 + e^|x|) through the special-function unit (ex2.approx, rcp.approx: a few ulp) for the tensor-core lanes, whose
// results are rounded to 16 bits right after; the streaming lanes keep expf and the IEEE division
__device__ __forceinline__ float sigmoid_tail_fast(float x) { return __fdividef(1.0f, 1.0f + __expf(fabsf(x))); }

// Over how many CTAs (1, 2 or 4, at most lp) the parts of an item's sum are spread in one call of a streaming kernel:
// as many as still give every unit a CTA of its own.  (Splitting further to even out the SMs' shares was measured: the
// extra folds cost more than the balance gains, 0.165 against 0.156 ms at one token.)  cap_items: the items the fold's
// workspace holds.
__device__ __forceinline__ uint32_t ksplit_ctas(uint32_t n_items, uint32_t lp, uint32_t grid, uint32_t cap_items) {
    if (!n_items || n_items > cap_items) return 1u;
    uint32_t np = 1;
    while (np < lp && n_items * (np * 2) <= grid) np *= 2;
    return np;
}

// ---- fixed-sequence exp / log for the router: IEEE +, *, fma, / only, so the host restatement of the same
// statements gives the same bits ----
__device__ __forceinline__ float det_expf(float x) {
    if (x != x) return x;
    if (x > 88.75f) return __int_as_float(0x7F800000);
    if (x < -104.0f) return 0.0f;
    const float magic = 12582912.0f;
    float t = __fmul_rn(x, 1.44269504f);
    float n = __fsub_rn(__fadd_rn(t, magic), magic);
    float r = __fmaf_rn(n, -0.693145752f, x);
    r = __fmaf_rn(n, -1.42860677e-06f, r);
    float p = 1.98412701e-04f;
    p = __fmaf_rn(p, r, 1.38888892e-03f);
    p = __fmaf_rn(p, r, 8.33333377e-03f);
    p = __fmaf_rn(p, r, 4.16666679e-02f);
    p = __fmaf_rn(p, r, 1.66666672e-01f);
    p = __fmaf_rn(p, r, 0.5f);
    p = __fmaf_rn(p, r, 1.0f);
    p = __fmaf_rn(p, r, 1.0f);
    int ni = (int)n;
    int n1 = ni / 2, n2 = ni - n1;
    float s1 = __int_as_float((n1 + 127) << 23), s2 = __int_as_float((n2 + 127) << 23);
    return __fmul_rn(__fmul_rn(p, s1), s2);
}
__device__ __forceinline__ float det_logf(float x) {
    uint32_t b = __float_as_uint(x);
    int e = (int)(b >> 23) - 127;
    float m = __uint_as_float((b & 0x007FFFFFu) | 0x3F800000u);
    if (m > 1.41421354f) { m = __fmul_rn(m, 0.5f); e += 1; }
    float f = __fsub_rn(m, 1.0f);
    float s = __fdiv_rn(f, __fadd_rn(2.0f, f));
    float z = __fmul_rn(s, s);
    float R = 9.09090936e-02f;
    R = __fmaf_rn(R, z, 1.11111112e-01f);
    R = __fmaf_rn(R, z, 1.42857149e-01f);
    R = __fmaf_rn(R, z, 0.2f);
    R = __fmaf_rn(R, z, 3.33333343e-01f);
    R = __fmul_rn(R, z);
    float s2 = __fadd_rn(s, s);
    float lo = __fmaf_rn(s2, R, s2);
    float ef = (float)e;
    lo = __fmaf_rn(ef, 1.42860677e-06f, lo);
    return __fmaf_rn(ef, 0.693145752f, lo);
}

}  // namespace mlxs
