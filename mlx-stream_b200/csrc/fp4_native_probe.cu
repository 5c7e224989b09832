// Measured answer to "why not the native block-scaled FP4 tensor-core path?": tcgen05.mma.kind::mxf8f6f4.block_scale
// with A = the MXFP4 codes and E8M0 block scales exactly as the bank stores them, B = the bf16 rows split into an E4M3
// high part and an E4M3 low part, each with its own UE8M0 block scale (two MMAs per 32 inputs).
//   * numerics: every e2m1 x e4m3 product is exact in the f32 accumulator, and hi + lo carries bf16's 8 significant
//     bits, so the result matches the bf16-row product to ~1e-3 of its rms (hi alone: a few percent);
//   * throughput: kind::mxf8f6f4 runs at the 8-bit rate, twice the 16-bit rate, and the hi / lo pair needs two MMAs per
//     32 inputs, so the pair delivers the 16-bit rate: what the native kind takes off the SM is the decode, not tensor
//     time.  The probe times both instruction streams on operands resident in shared memory.
// What was learned about the instruction on the way (sm_100a, no swizzle, K-major):
//   * shared memory holds 4-bit A elements in 8-bit containers' geometry: a 16-byte core-matrix row = 16 elements in its
//     low 8 bytes (two code words of the bank as they are), the high 8 bytes unused;
//   * instruction descriptor: b_sf_id [4,6), a_format [7,10) (E2M1 = 5), b_format [10,13) (E4M3 = 0), N >> 3 [17,23),
//     scale format [23] (1 = UE8M0), M >> 4 [24,29), a_sf_id [29,31);
//   * scale bytes live in tensor memory: row m of A reads lane m, column (scale address) + m / 32, byte a_sf_id; row n of
//     B reads lane n % 32 (quarter 0 suffices, the probe replicates), column + n / 32, byte b_sf_id.
#include <cuda_runtime.h>

#include <cmath>
#include <cstring>
#include <vector>

#include "../../include/mlxs_moe.h"
#include "common.cuh"
#include "umma.cuh"

int mlxs_fail(int rc, const char* fmt, ...);

namespace mlxs {

constexpr int NP_M = 128, NP_N = 64, NP_K = 128;   // one numerics tile: 4 blocks of 32 inputs

__device__ __forceinline__ void umma_mxf8(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t sfa, uint32_t sfb,
                                          uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %6, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale.scale_vec::1X [%0], %1, %2, %3, [%4], [%5], p;\n\t}"
        ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(sfa), "r"(sfb), "r"(accumulate)
        : "memory");
}
__host__ __device__ inline uint32_t mxf8_idesc(uint32_t n, uint32_t a_sf, uint32_t b_sf) {
    return (b_sf << 4) | (5u << 7) | (0u << 10) | ((n >> 3) << 17) | (1u << 23) | ((128u >> 4) << 24) | (a_sf << 29);
}
__device__ __forceinline__ void tmem_st1(uint32_t taddr, uint32_t v) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x1.b32 [%0], {%1};" ::"r"(taddr), "r"(v) : "memory");
}

// D[128, N] = sum_k A[m][k] 2^(sa[m][k/32] - 127) (Bhi[n][k] 2^(shi[n][k/32] - 127) + Blo[n][k] 2^(slo[n][k/32] - 127))
// a_codes: [128][K/8] u32 (code j of a word at bits 4j); sa: [128][K/32] bytes; bhi / blo: [N][K] e4m3 bytes;
// shi / slo: [N][K/32] bytes; use_lo: 0 = hi alone.  One CTA of 128 threads.
__global__ void __launch_bounds__(128) mxf8_numerics_kernel(const uint32_t* __restrict__ a_codes, const uint8_t* __restrict__ sa,
                                                            const uint8_t* __restrict__ bhi, const uint8_t* __restrict__ blo,
                                                            const uint8_t* __restrict__ shi, const uint8_t* __restrict__ slo,
                                                            int use_lo, float* __restrict__ d_out, uint32_t* status) {
    __shared__ __align__(128) uint8_t sA[NP_M * NP_K];          // [k16][m8][8][16 B], 16 elements in the low 8 bytes of a row
    __shared__ __align__(128) uint8_t sBh[NP_N * NP_K], sBl[NP_N * NP_K];   // [k16][n8][8][16 B]
    __shared__ __align__(8) uint64_t bar;
    __shared__ uint32_t s_tmem;
    __shared__ volatile int s_abort;
    const uint32_t tid = threadIdx.x, warp = tid >> 5;
    for (uint32_t i = tid; i < NP_M * (NP_K / 16); i += blockDim.x) {
        const uint32_t m = i % NP_M, k16 = i / NP_M;
        uint2* row = reinterpret_cast<uint2*>(sA + k16 * (NP_M / 8) * 128 + (m / 8) * 128 + (m % 8) * 16);
        row[0] = make_uint2(a_codes[m * (NP_K / 8) + 2 * k16], a_codes[m * (NP_K / 8) + 2 * k16 + 1]);
        row[1] = make_uint2(0u, 0u);
    }
    for (uint32_t i = tid; i < NP_N * (NP_K / 16); i += blockDim.x) {
        const uint32_t n = i % NP_N, k16 = i / NP_N;
        const uint32_t off = k16 * (NP_N / 8) * 128 + (n / 8) * 128 + (n % 8) * 16;
        *reinterpret_cast<uint4*>(sBh + off) = *reinterpret_cast<const uint4*>(bhi + n * NP_K + k16 * 16);
        *reinterpret_cast<uint4*>(sBl + off) = *reinterpret_cast<const uint4*>(blo + n * NP_K + k16 * 16);
    }
    if (tid == 0) { mbar_init(&bar, 1); s_abort = 0; mbar_fence_init(); }
    if (warp == 0) tmem_alloc(&s_tmem, 128);
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = s_tmem, sfa = tmem + 64, sfh = tmem + 72, sfl = tmem + 80;
    // scale words: A row m = this thread's lane, column + warp; B row n at lane n % 32 of every quarter, column + n / 32
    tmem_st1(sfa + ((warp * 32u) << 16) + warp, *reinterpret_cast<const uint32_t*>(sa + tid * 4));
    for (uint32_t c = 0; c < NP_N / 32; ++c) {
        const uint32_t n = c * 32 + (tid & 31u);
        tmem_st1(sfh + ((warp * 32u) << 16) + c, *reinterpret_cast<const uint32_t*>(shi + n * 4));
        tmem_st1(sfl + ((warp * 32u) << 16) + c, *reinterpret_cast<const uint32_t*>(slo + n * 4));
    }
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (tid == 0) {
        const uint32_t lbo_a = (NP_M / 8) * 128, lbo_b = (NP_N / 8) * 128;
        for (uint32_t kb = 0; kb < NP_K / 32; ++kb) {
            const uint32_t id = mxf8_idesc(NP_N, kb, kb);
            const uint64_t da = umma_smem_desc(smem_u32(sA) + kb * 2 * lbo_a, lbo_a, 128);
            umma_mxf8(tmem, da, umma_smem_desc(smem_u32(sBh) + kb * 2 * lbo_b, lbo_b, 128), id, sfa, sfh, kb ? 1u : 0u);
            if (use_lo) umma_mxf8(tmem, da, umma_smem_desc(smem_u32(sBl) + kb * 2 * lbo_b, lbo_b, 128), id, sfa, sfl, 1u);
        }
        umma_commit(&bar);
    }
    if (!mbar_wait_bounded(&bar, 0, &s_abort)) {
        if (tid == 0) atomicMax(status, (uint32_t)ST_WAIT_FULL);
    } else {
        tc_fence_after();
        for (uint32_t c0 = 0; c0 < NP_N; c0 += 16) {
            uint32_t v[16];
            tmem_ld16(tmem + ((warp * 32u) << 16) + c0, v);
            for (int i = 0; i < 16; ++i) d_out[tid * NP_N + c0 + i] = __uint_as_float(v[i]);
        }
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (warp == 0) tmem_free(tmem, 128);
}

// Issue-rate loop on operands that stay in shared memory (contents irrelevant): mode 0 = kind::f16 (bf16, K = 16 per MMA),
// mode 1 = kind::mxf8f6f4.block_scale (K = 32 per MMA), mode 2 = kind::f16 with the A operand in tensor memory.  M = 128,
// N = nn, `mmas` instructions per CTA, one CTA per SM.
__global__ void __launch_bounds__(128) mxf8_rate_kernel(int mode, uint32_t mmas, uint32_t* status, uint32_t nn) {
    extern __shared__ __align__(128) uint8_t smem_raw[];   // A 128 x 64 B, B 256 x 64 B
    __shared__ __align__(8) uint64_t bar;
    __shared__ uint32_t s_tmem;
    __shared__ volatile int s_abort;
    const uint32_t tid = threadIdx.x, warp = tid >> 5;
    for (uint32_t i = tid; i < (128 + 256) * 64 / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(smem_raw)[i] = 0x38383838u;
    if (tid == 0) { mbar_init(&bar, 1); s_abort = 0; mbar_fence_init(); }
    if (warp == 0) tmem_alloc(&s_tmem, 512);
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = s_tmem;
    for (uint32_t c = 256; c < 272; ++c) tmem_st1(tmem + ((warp * 32u) << 16) + c, 0x7F7F7F7Fu);
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (tid == 0) {
        const uint32_t a_s = smem_u32(smem_raw), b_s = a_s + 128 * 64;
        if (mode == 0 || mode == 2) {
            // 16-bit elements: a core matrix is 8 rows x 8 elements; K = 16 is two of them
            const uint64_t da = umma_smem_desc(a_s, 16 * 128, 128), db = umma_smem_desc(b_s, 32 * 128, 128);
            const uint32_t id = umma_idesc(UMMA_BF16, nn);
            if (mode == 0) for (uint32_t i = 0; i < mmas; ++i) umma_f16(tmem, da, db, id, i ? 1u : 0u);
            else for (uint32_t i = 0; i < mmas; ++i) umma_f16_ts(tmem, tmem + 300, db, id, i ? 1u : 0u);
        } else {
            const uint64_t da = umma_smem_desc(a_s, 16 * 128, 128), db = umma_smem_desc(b_s, 32 * 128, 128);
            const uint32_t id = mxf8_idesc(nn, 0, 0);
            for (uint32_t i = 0; i < mmas; ++i) umma_mxf8(tmem, da, db, id, tmem + 256, tmem + 264, i ? 1u : 0u);
        }
        umma_commit(&bar);
    }
    if (!mbar_wait_bounded(&bar, 0, &s_abort, 64, 1u << 22) && tid == 0) atomicMax(status, (uint32_t)ST_WAIT_FULL);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (warp == 0) tmem_free(tmem, 512);
}

}  // namespace mlxs

namespace {

// f32 -> E4M3 (OCP FP8, no infinities, max 448), round to nearest even, saturating
uint8_t e4m3_from_float(float x) {
    const uint8_t sign = std::signbit(x) ? 0x80 : 0;
    float a = std::fabs(x);
    if (!(a == a)) return 0x7F;
    if (a >= 464.0f) return sign | 0x7E;                 // above the last rounding boundary: saturate to 448
    if (a < 0.0009765625f) return sign;                  // below half of the smallest subnormal (2^-9 / 2)... rounds to 0
    int e;
    std::frexp(a, &e);                                   // a = m 2^e, m in [0.5, 1)
    int ex = e - 1;                                      // a = 1.f x 2^ex
    if (ex < -6) ex = -6;                                // subnormals share the exponent 2^-6
    const float q = std::ldexp(a, 3 - ex);               // in units of 2^(ex - 3)
    float r = std::nearbyint(q);                         // ties to even (default rounding mode)
    int mant = (int)r;
    if (mant >= 16) { mant >>= 1; ex += 1; }
    if (ex == -6 && mant < 8) return sign | (uint8_t)mant;               // subnormal
    if (ex > 8 || (ex == 8 && mant > 14)) return sign | 0x7E;
    return sign | (uint8_t)(((ex + 7) << 3) | (mant - 8));
}
float e4m3_to_float(uint8_t b) {
    const int e = (b >> 3) & 15, m = b & 7;
    const float v = e == 0 ? std::ldexp((float)m, -9) : std::ldexp((float)(8 + m), e - 10);
    return (b & 0x80) ? -v : v;
}
float e2m1_value(uint32_t c) {
    static const float t[8] = {0.f, 0.5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f};
    return (c & 8) ? -t[c & 7] : t[c & 7];
}
uint64_t splitmix(uint64_t& s) {
    s += 0x9E3779B97F4A7C15ull;
    uint64_t z = s;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

}  // namespace

extern "C" int mlxs_moe_fp4_native_probe(int32_t device, uint32_t rate_mmas, mlxs_fp4_native_result* out) {
    using namespace mlxs;
    if (!out) return mlxs_fail(MLXS_E_ARG, "fp4_native_probe: null argument");
    memset(out, 0, sizeof *out);
    cudaError_t e = cudaSetDevice(device);
    if (e != cudaSuccess) return mlxs_fail(MLXS_E_CUDA, "fp4_native_probe: cudaSetDevice: %s", cudaGetErrorString(e));
    cudaDeviceProp prop;
    if ((e = cudaGetDeviceProperties(&prop, device)) != cudaSuccess || prop.major != 10)
        return mlxs_fail(MLXS_E_CUDA, "fp4_native_probe: needs an sm_100 device");
    // ---- numerics: random codes and block scales, bf16 rows ~ N(0,1) split into hi + lo ----
    uint64_t seed = 0xF4F4F4;
    std::vector<uint32_t> codes(NP_M * NP_K / 8);
    std::vector<uint8_t> sa(NP_M * NP_K / 32), bhi(NP_N * NP_K), blo(NP_N * NP_K), shi(NP_N * NP_K / 32), slo(NP_N * NP_K / 32);
    std::vector<float> x(NP_N * NP_K);
    for (auto& w : codes) w = (uint32_t)splitmix(seed);
    for (auto& s : sa) s = (uint8_t)(118 + splitmix(seed) % 6);          // 2^-9 .. 2^-4: the range an N(0, 0.02) bank uses
    for (auto& v : x) {
        const double u1 = ((splitmix(seed) >> 11) + 1.0) / 9007199254740993.0, u2 = (splitmix(seed) >> 11) / 9007199254740992.0;
        const float g = (float)(std::sqrt(-2.0 * std::log(u1)) * std::cos(6.283185307179586 * u2));
        uint32_t b;
        memcpy(&b, &g, 4);
        b = (b + 0x7FFF + ((b >> 16) & 1)) & 0xFFFF0000u;                // round to bf16
        memcpy(&v, &b, 4);
    }
    for (int n = 0; n < NP_N; ++n)
        for (int kb = 0; kb < NP_K / 32; ++kb) {
            float amax = 0.f;
            for (int k = 0; k < 32; ++k) amax = std::fmax(amax, std::fabs(x[n * NP_K + kb * 32 + k]));
            int ea = 0;
            if (amax > 0.f) { std::frexp(amax, &ea); ea -= 1; }         // amax = 1.f x 2^ea
            const int eh = ea - 8 + (std::ldexp(amax, -ea) > 1.75f ? 1 : 0), el = eh - 4;   // amax / 2^eh <= 448; the residual fits 2^el x 448
            shi[n * 4 + kb] = (uint8_t)(eh + 127);
            slo[n * 4 + kb] = (uint8_t)(el + 127);
            for (int k = 0; k < 32; ++k) {
                const float v = x[n * NP_K + kb * 32 + k];
                const uint8_t h = e4m3_from_float(std::ldexp(v, -eh));
                const float r = v - std::ldexp(e4m3_to_float(h), eh);
                bhi[n * NP_K + kb * 32 + k] = h;
                blo[n * NP_K + kb * 32 + k] = e4m3_from_float(std::ldexp(r, -el));
            }
        }
    std::vector<double> ref((size_t)NP_M * NP_N);
    double ref_sq = 0;
    for (int m = 0; m < NP_M; ++m)
        for (int n = 0; n < NP_N; ++n) {
            double acc = 0;
            for (int k = 0; k < NP_K; ++k)
                acc += (double)e2m1_value((codes[m * (NP_K / 8) + k / 8] >> (4 * (k % 8))) & 15) * std::ldexp(1.0, (int)sa[m * 4 + k / 32] - 127) *
                       (double)x[n * NP_K + k];
            ref[(size_t)m * NP_N + n] = acc;
            ref_sq += acc * acc;
        }
    uint8_t* dbuf = nullptr;
    const size_t bytes = codes.size() * 4 + sa.size() + bhi.size() + blo.size() + shi.size() + slo.size() + (size_t)NP_M * NP_N * 4 + 256;
    if ((e = cudaMalloc(&dbuf, bytes + 1024)) != cudaSuccess) return mlxs_fail(MLXS_E_CUDA, "fp4_native_probe: cudaMalloc: %s", cudaGetErrorString(e));
    size_t off = 0;
    auto put = [&](const void* p, size_t n) { uint8_t* d = dbuf + off; cudaMemcpy(d, p, n, cudaMemcpyHostToDevice); off += (n + 255) / 256 * 256; return d; };
    const uint32_t* d_codes = reinterpret_cast<const uint32_t*>(put(codes.data(), codes.size() * 4));
    const uint8_t *d_sa = put(sa.data(), sa.size()), *d_bhi = put(bhi.data(), bhi.size()), *d_blo = put(blo.data(), blo.size());
    const uint8_t *d_shi = put(shi.data(), shi.size()), *d_slo = put(slo.data(), slo.size());
    float* d_out = reinterpret_cast<float*>(dbuf + off);
    off += (size_t)NP_M * NP_N * 4;
    uint32_t* d_status = reinterpret_cast<uint32_t*>(dbuf + ((off + 255) / 256 * 256));
    cudaMemset(d_status, 0, 4);
    std::vector<float> got((size_t)NP_M * NP_N);
    double errs[2] = {0, 0};
    for (int use_lo = 1; use_lo >= 0 && e == cudaSuccess; --use_lo) {
        mxf8_numerics_kernel<<<1, 128>>>(d_codes, d_sa, d_bhi, d_blo, d_shi, d_slo, use_lo, d_out, d_status);
        if ((e = cudaDeviceSynchronize()) != cudaSuccess) break;
        cudaMemcpy(got.data(), d_out, got.size() * 4, cudaMemcpyDeviceToHost);
        double sq = 0;
        for (size_t i = 0; i < got.size(); ++i) sq += ((double)got[i] - ref[i]) * ((double)got[i] - ref[i]);
        errs[use_lo] = std::sqrt(sq / (ref_sq + 1e-300));
    }
    // ---- issue rates ----
    double tf[2] = {0, 0};
    if (e == cudaSuccess && rate_mmas) {
        const size_t smem = (128 + 256) * 64;
        cudaEvent_t a, b;
        cudaEventCreate(&a);
        cudaEventCreate(&b);
        for (int mode = 0; mode < 2 && e == cudaSuccess; ++mode) {
            mxf8_rate_kernel<<<prop.multiProcessorCount, 128, smem>>>(mode, rate_mmas / 8 + 1, d_status, 256u);   // warm-up
            cudaEventRecord(a, 0);
            mxf8_rate_kernel<<<prop.multiProcessorCount, 128, smem>>>(mode, rate_mmas, d_status, 256u);
            cudaEventRecord(b, 0);
            if ((e = cudaEventSynchronize(b)) != cudaSuccess) break;
            float ms = 0.f;
            cudaEventElapsedTime(&ms, a, b);
            const double flops = 2.0 * 128 * 256 * (mode ? 32 : 16) * (double)rate_mmas * prop.multiProcessorCount;
            tf[mode] = flops / (ms * 1e-3) / 1e12;
        }
        cudaEventDestroy(a);
        cudaEventDestroy(b);
    }
    uint32_t st = 0;
    if (e == cudaSuccess) cudaMemcpy(&st, d_status, 4, cudaMemcpyDeviceToHost);
    cudaFree(dbuf);
    if (e != cudaSuccess) return mlxs_fail(MLXS_E_CUDA, "fp4_native_probe: %s", cudaGetErrorString(e));
    if (st) return mlxs_fail(MLXS_E_DEVICE_STATUS, "fp4_native_probe: a bounded wait ran out (status %u)", st);
    out->rel_l2_hi_lo = errs[1];
    out->rel_l2_hi_only = errs[0];
    out->tflops_f16 = tf[0];
    out->tflops_mxf8f6f4 = tf[1];
    out->tflops_hi_lo_effective = tf[1] / 2.0;
    return MLXS_OK;
}

extern "C" int mlxs_moe_mma_rate(int32_t device, uint32_t n, int a_from_tmem, uint32_t mmas, double* ns_per_mma) {
    using namespace mlxs;
    if (!ns_per_mma || !mmas) return mlxs_fail(MLXS_E_ARG, "mma_rate: null or zero argument");
    if (n < 16 || n > 256 || n % 16) return mlxs_fail(MLXS_E_ARG, "mma_rate: n = %u is not a multiple of 16 in 16 .. 256", n);
    cudaError_t e = cudaSetDevice(device);
    if (e != cudaSuccess) return mlxs_fail(MLXS_E_CUDA, "mma_rate: cudaSetDevice: %s", cudaGetErrorString(e));
    cudaDeviceProp prop;
    if ((e = cudaGetDeviceProperties(&prop, device)) != cudaSuccess || prop.major != 10)
        return mlxs_fail(MLXS_E_CUDA, "mma_rate: needs an sm_100 device");
    uint32_t* d_status = nullptr;
    if ((e = cudaMalloc(&d_status, 16)) != cudaSuccess) return mlxs_fail(MLXS_E_CUDA, "mma_rate: cudaMalloc: %s", cudaGetErrorString(e));
    cudaMemset(d_status, 0, 16);
    const size_t smem = (128 + 256) * 64;
    const int mode = a_from_tmem ? 2 : 0;
    cudaEvent_t a, b;
    cudaEventCreate(&a);
    cudaEventCreate(&b);
    mxf8_rate_kernel<<<prop.multiProcessorCount, 128, smem>>>(mode, mmas / 8 + 1, d_status, n);   // warm-up
    cudaEventRecord(a, 0);
    mxf8_rate_kernel<<<prop.multiProcessorCount, 128, smem>>>(mode, mmas, d_status, n);
    cudaEventRecord(b, 0);
    e = cudaEventSynchronize(b);
    float ms = 0.f;
    if (e == cudaSuccess) cudaEventElapsedTime(&ms, a, b);
    uint32_t st = 0;
    if (e == cudaSuccess) cudaMemcpy(&st, d_status, 4, cudaMemcpyDeviceToHost);
    cudaEventDestroy(a);
    cudaEventDestroy(b);
    cudaFree(d_status);
    if (e != cudaSuccess) return mlxs_fail(MLXS_E_CUDA, "mma_rate: %s", cudaGetErrorString(e));
    if (st) return mlxs_fail(MLXS_E_DEVICE_STATUS, "mma_rate: a bounded wait ran out (status %u)", st);
    *ns_per_mma = (double)ms * 1e6 / (double)mmas;
    return MLXS_OK;
}
