/*
 * CPU oracle for the routed-MoE hot path.  TEST INFRASTRUCTURE ONLY: the tests, the smoke check and the
 * benchmark's CPU-baseline leg load this; the product library never links, loads or calls it.
 *
 * Every function restates one piece of the reference's CPU reference math; the citation beside each
 * declaration is the reference file:line it follows (paths relative to the reference project).
 *
 * Parity pins (checked by the CPU test-suite): the mul1 table digest and the four plane digests of
 * src/kernels/exl3/manifest.json, the two GLM-shape plane digests of src/arch/glm5_next/exl3_parity.zig:19-23,
 * the expert-forward fixture of src/arch/glm5_next/testdata/exl3-ref (W_hat digests, h_mul1.f32, y_mul1.f32),
 * the E4M3 / E2M1 / E8M0 known answers of src/arch/glm5_next/decode_kernels_ref.zig:170-218 and
 * src/arch/mimo_v2/moe.zig:1059-1064, the router known answer of src/arch/mimo_v2/config.zig:503-514 and the
 * permutation known answer of src/sdk_ext/quant.zig:692-699.
 * Unpinned (no golden in the reference): softmax routing, the FP4 prefill accumulation order (lives in MLX).
 */
#ifndef MLXS_ORACLE_H
#define MLXS_ORACLE_H
#include <stddef.h>
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif

/* ---- seeded streams: src/exl3/kernels.zig:1022-1041, src/arch/glm5_next/exl3_forms_ref.zig:41-93 ---- */
uint64_t orc_splitmix64(uint64_t *state);
void orc_fill_code(uint64_t seed, int16_t *out, size_t n);
void orc_fill_scales(uint64_t seed, double scale, uint16_t *out_f16, size_t n);
void orc_fill_x_bf16(uint64_t seed, float *out, size_t n);
float orc_bf16_round(float x);
float orc_h2f(uint16_t h);
uint16_t orc_f2h(double v);

/* ---- EXL3 trellis decode: src/exl3/kernels.zig:960-1020 ---- */
uint16_t orc_mul1_decode(uint32_t state);
void orc_mul1_table(uint16_t *out65536);
void orc_tile_perm(uint8_t *out256);
void orc_tile_states(const int16_t *words, int K, uint16_t *out256);
void orc_reconstruct(const int16_t *code, size_t n_i, size_t n_j, int K, const uint16_t *table, uint16_t *w,
                     uint16_t *states_or_null);

/* ---- EXL3 record geometry: src/expert/bank.zig:116-141 (nine segments, gate/up/down x code/rout/rin) ---- */
typedef struct {
    uint64_t off[9];
    uint64_t len[9];
    uint64_t logical_bytes;
    uint64_t record_bytes; /* logical rounded up to 4096 */
} orc_exl3_geom;
int orc_exl3_geometry(int K, uint64_t hidden, uint64_t inter, orc_exl3_geom *g);
/* a record image from one seed: code seeds seed+1,4,7; rin (suh) seeds seed+2,5,8; rout (svh) seeds seed+3,6,9
 * (src/arch/glm5_next/exl3_forms_ref.zig:81-93, at any shape and with the two scales as arguments) */
void orc_exl3_synth_record(uint64_t seed, uint64_t hidden, uint64_t inter, double suh_scale, double svh_scale,
                           uint8_t *rec);
void orc_exl3_synth_record_k(int K, uint64_t seed, uint64_t hidden, uint64_t inter, double suh_scale, double svh_scale,
                             uint8_t *rec);

/* ---- EXL3 f64 forward: src/arch/glm5_next/exl3_forms_ref.zig:116-195 ---- */
void orc_fwht128(double *v, size_t n);
void orc_exl3_forward(const double *x, size_t in, const uint16_t *w, const uint16_t *suh, const uint16_t *svh,
                      double *y, size_t out);
double orc_swiglu_clamped(double g, double u, double limit); /* limit <= 0: plain silu(g)*u */
/* one expert on `rows` input rows (f64): h [rows, inter], y [rows, hidden] (either may be NULL) */
int orc_exl3_expert_f64(const uint8_t *rec, uint64_t hidden, uint64_t inter, double limit, const double *x,
                        size_t rows, double *h, double *y);
int orc_exl3_expert_f64_k(int K, const uint8_t *rec, uint64_t hidden, uint64_t inter, double limit, const double *x,
                          size_t rows, double *h_out, double *y_out);
/* the f32 seam chain per output word: src/arch/glm5_next/exl3_forms_ref.zig:231-343 */
int orc_exl3_expert_f32chain(const uint8_t *rec, uint64_t hidden, uint64_t inter, const float *x, size_t rows,
                             float *h, float *y);

/* ---- FP4 formats ---- */
float orc_e2m1_value(uint32_t c);                /* src/arch/glm5_next/decode_kernels_ref.zig:79-83 */
uint16_t orc_e2m1_halfbits(uint32_t c);          /* decode_kernels_ref.zig:13-16 */
void orc_fp4_decode8(uint32_t w, uint32_t out[4]); /* decode_kernels_ref.zig:22-29 */
float orc_e4m3_kernel(uint8_t b);                /* decode_kernels_ref.zig:32-36 (the texts' decode) */
float orc_e4m3_value(uint8_t b);                 /* decode_kernels_ref.zig:71-76 (the format's definition) */
float orc_nvfp4_weight(uint8_t scale, uint32_t code, float g); /* decode_kernels_ref.zig:86-88 */
float orc_nvfp4_kernel_weight(uint8_t scale, uint32_t code, float g); /* :39-47, 59-63 */
float orc_e8m0_value(uint32_t b);                /* src/arch/mimo_v2/moe.zig:408-413 without the 2^-8 */
float orc_mxfp4_scale_ref(uint32_t b);           /* moe.zig:410-413, as written (x 2^-8, subnormals flushed) */
float orc_silu_mul_ref(float gate, float up);    /* moe.zig:355-360 */
float orc_silu_mul_clamped_ref(float gate, float up, float limit); /* glm5n_nvfp4_gateup.metal:109-129 */
/* dequantised row-major [rows, cols] f32 of a projection */
void orc_mxfp4_decode(const uint32_t *words, const uint8_t *scales, size_t rows, size_t cols, float *out);
void orc_nvfp4_decode(const uint32_t *words, const uint8_t *scales, float g, size_t rows, size_t cols, float *out);

/* ---- router ---- */
enum { ORC_SCORE_SQRTSOFTPLUS = 0, ORC_SCORE_SIGMOID = 1, ORC_SCORE_SOFTMAX = 2 };
/* libm arithmetic (src/arch/mimo_v2/config.zig:427-446; src/kernels/exl3/q3rc_router_tail.metal:12-40).
 * ids in rank order (score+bias descending, ties to the lower index, NaN last); weights from the unbiased score,
 * / (sum + 1e-20) when norm, x scale. */
int orc_route_libm(const float *logits, const float *bias_or_null, size_t T, size_t E, size_t k, int scoring,
                   int norm, float scale, int32_t *ids, float *weights);
/* the same with the fixed-sequence exp / log the device kernels also evaluate: bit-exact target for ids */
int orc_route_det(const float *logits, const float *bias_or_null, size_t T, size_t E, size_t k, int scoring,
                  int norm, float scale, int32_t *ids, float *weights);
float orc_det_expf(float x);
float orc_det_logf(float x);

/* ---- dispatch: stable counting sort by slot (src/sdk_ext/quant.zig:269-290) ---- */
void orc_dispatch(const int32_t *slot, size_t n, size_t n_slots, uint32_t *order, uint32_t *sorted_slot,
                  uint32_t *inv, uint32_t *offsets /* [n_slots+1] */);

/* ---- layer (router outputs given): per expert decode once, run its rows, weighted combine ---- */
enum { ORC_BANK_EXL3 = 0, ORC_BANK_MXFP4 = 1, ORC_BANK_NVFP4 = 2, ORC_BANK_EXL3_K2 = 3 };
typedef struct {
    int bank;
    uint64_t hidden, inter, n_experts, top_k;
    double limit;        /* swiglu clamp; <= 0 none */
    int chain_rounding;  /* FP4 banks: apply the reference decode texts' bf16 rounding points */
    int shared_bf16_add; /* GLM-Flash: routed rounded to bf16, then bf16 add of the shared row */
} orc_layer_cfg;
/* records[e]: that expert's record image in the bank's reference layout (NULL for experts never routed).
 * x: bf16 values as f32 [T, hidden]; ids [T, k]; weights [T, k]; shared: bf16 bits w1 [I,H], w3 [I,H], w2 [H,I] or
 * NULL.  y [T, hidden] f64 (before the final bf16 store); ro (optional) [T, k, hidden] f64 unweighted. */
int orc_layer(const orc_layer_cfg *cfg, const uint8_t *const *records, const float *x, size_t T, const int32_t *ids,
              const float *weights, const uint16_t *sh_w1, const uint16_t *sh_w3, const uint16_t *sh_w2, double *y,
              double *ro);
/* the f32 fast form used as the timed CPU baseline (EXL3: on-the-fly decode + f32 FMA, OpenMP over
 * (expert, 16-column tile): src/arch/glm5_next/exl3_forms_ref.zig:299-343) */
int orc_layer_fast(const orc_layer_cfg *cfg, const uint8_t *const *records, const float *x, size_t T,
                   const int32_t *ids, const float *weights, const uint16_t *sh_w1, const uint16_t *sh_w3,
                   const uint16_t *sh_w2, float *y, int threads);
int orc_max_threads(void);

/* FP4 record geometry: src/arch/mimo_v2/bank.zig:341-345 (six parts), src/arch/glm5_next/bank.zig:5-13 (nine) */
uint64_t orc_mxfp4_record_bytes(uint64_t hidden, uint64_t inter, uint64_t off[6]);
uint64_t orc_nvfp4_record_bytes(uint64_t hidden, uint64_t inter, uint64_t off[9]);
/* our synthetic FP4 quantiser (the reference has none): N(0, sigma) weights by Box-Muller over splitmix64, block
 * scale from the block amax, codes by round-to-nearest-even onto the e2m1 grid */
void orc_mxfp4_synth_record(uint64_t seed, uint64_t hidden, uint64_t inter, double sigma, uint8_t *rec);
void orc_nvfp4_synth_record(uint64_t seed, uint64_t hidden, uint64_t inter, double sigma, uint8_t *rec);

#ifdef __cplusplus
}
#endif
#endif
