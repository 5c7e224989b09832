/*
 * CPU oracle for the routed-MoE hot path (see mlxs_oracle.h).  TEST INFRASTRUCTURE ONLY.
 * Plain C11 + OpenMP; compiled with -ffp-contract=off so every product and sum below rounds where it is written.
 */
#include "mlxs_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

/* ------------------------------------------------------------------------------------------------ */
/* scalar helpers                                                                                    */
/* ------------------------------------------------------------------------------------------------ */

static inline uint32_t f2u(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static inline float u2f(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }

float orc_h2f(uint16_t h) {
    uint32_t s = (uint32_t)(h & 0x8000) << 16, e = (h >> 10) & 31, m = h & 1023;
    if (e == 0) {
        if (m == 0) return u2f(s);
        float v = ldexpf((float)m, -24);
        return s ? -v : v;
    }
    if (e == 31) return u2f(s | 0x7F800000u | (m << 13));
    return u2f(s | ((e + 112) << 23) | (m << 13));
}

/* double -> binary16 bits, one round-to-nearest-even */
uint16_t orc_f2h(double v) {
    uint64_t b; memcpy(&b, &v, 8);
    uint16_t s = (uint16_t)((b >> 48) & 0x8000);
    double a = fabs(v);
    if (a != a) return (uint16_t)(s | 0x7E00);
    if (a >= 65520.0) return (uint16_t)(s | 0x7C00);
    if (a < 6.103515625e-05) { /* subnormal half: multiples of 2^-24 */
        double q = nearbyint(a * 16777216.0); /* ties to even under the default mode */
        return (uint16_t)(s | (uint16_t)q);
    }
    int ex; double fr = frexp(a, &ex); /* a = fr 2^ex, fr in [0.5,1) */
    double m = nearbyint(fr * 2048.0); /* 11 significant bits */
    if (m == 2048.0) { m = 1024.0; ex += 1; }
    int e = ex - 1 + 15;
    if (e >= 31) return (uint16_t)(s | 0x7C00);
    return (uint16_t)(s | (e << 10) | ((int)m - 1024));
}

/* src/arch/glm5_next/exl3_forms_ref.zig:68-72 */
float orc_bf16_round(float x) {
    uint32_t b = f2u(x);
    uint32_t r = ((b + 0x7FFFu + ((b >> 16) & 1u)) >> 16) << 16;
    return u2f(r);
}
static inline float bf16_bits_f32(uint16_t b) { return u2f((uint32_t)b << 16); }

/* ------------------------------------------------------------------------------------------------ */
/* seeded streams                                                                                    */
/* ------------------------------------------------------------------------------------------------ */

/* src/exl3/kernels.zig:1022-1028 */
uint64_t orc_splitmix64(uint64_t *state) {
    *state += 0x9E3779B97F4A7C15ull;
    uint64_t z = *state;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

static inline double unit53(uint64_t z) { return (double)(z >> 11) / 9007199254740992.0; }

/* src/arch/glm5_next/exl3_forms_ref.zig:45-55: the little-endian int16 view of the splitmix64 words */
void orc_fill_code(uint64_t seed, int16_t *out, size_t n) {
    uint64_t s = seed;
    for (size_t i = 0; i < n; i += 4) {
        uint64_t z = orc_splitmix64(&s);
        for (size_t j = 0; j < 4 && i + j < n; ++j) out[i + j] = (int16_t)(uint16_t)(z >> (16 * j));
    }
}

/* exl3_forms_ref.zig:57-66: f16(sign (0.5 + u) scale), sign = -1 when bit 0 of the word is set */
void orc_fill_scales(uint64_t seed, double scale, uint16_t *out, size_t n) {
    uint64_t s = seed;
    for (size_t i = 0; i < n; ++i) {
        uint64_t z = orc_splitmix64(&s);
        double sign = (z & 1) ? -1.0 : 1.0;
        out[i] = orc_f2h(sign * (0.5 + unit53(z)) * scale);
    }
}

/* exl3_forms_ref.zig:74-78: bf16 values of f32(2u - 1) */
void orc_fill_x_bf16(uint64_t seed, float *out, size_t n) {
    uint64_t s = seed;
    for (size_t i = 0; i < n; ++i) out[i] = orc_bf16_round((float)(2.0 * unit53(orc_splitmix64(&s)) - 1.0));
}

/* ------------------------------------------------------------------------------------------------ */
/* EXL3 trellis decode                                                                               */
/* ------------------------------------------------------------------------------------------------ */

/* src/exl3/kernels.zig:963-971 */
uint16_t orc_mul1_decode(uint32_t state) {
    uint32_t x = state * 0x83DCD12Du;
    uint32_t s = (x & 0xFF) + ((x >> 8) & 0xFF) + ((x >> 16) & 0xFF) + (x >> 24);
    double k_inv = (double)orc_h2f(0x1EEE), k_bias = (double)orc_h2f(0xC931);
    return orc_f2h((double)(1024 + s) * k_inv + k_bias); /* exact in f64, one rounding to f16 */
}

void orc_mul1_table(uint16_t *out) {
    for (uint32_t s = 0; s < 65536; ++s) out[s] = orc_mul1_decode(s);
}

/* src/exl3/kernels.zig:978-986 */
void orc_tile_perm(uint8_t *perm) {
    for (int t = 0; t < 32; ++t) {
        int r0 = (t % 4) * 2;
        int rows[4] = {r0, r0 + 1, r0 + 8, r0 + 9};
        for (int j = 0; j < 8; ++j) perm[t * 8 + j] = (uint8_t)(rows[j % 4] * 16 + t / 4 + (j < 4 ? 0 : 8));
    }
}

/* src/exl3/kernels.zig:990-1002 */
void orc_tile_states(const int16_t *words, int K, uint16_t *out) {
    size_t nw = 8 * (size_t)K;
    uint64_t u[64];
    for (size_t m = 0; m < nw; ++m)
        u[m] = (uint64_t)(uint16_t)words[2 * m] | ((uint64_t)(uint16_t)words[2 * m + 1] << 16);
    for (size_t p = 0; p < 256; ++p) {
        size_t b1 = (p + 1) * K + 256 * (size_t)K;
        size_t hi_word = (b1 - 16) / 32, lo_word = (b1 - 1) / 32;
        unsigned s0 = (unsigned)((lo_word + 1) * 32 - b1);
        out[p] = (uint16_t)(((u[hi_word % nw] << 32) | u[lo_word % nw]) >> s0);
    }
}

/* src/exl3/kernels.zig:1006-1020 */
void orc_reconstruct(const int16_t *code, size_t n_i, size_t n_j, int K, const uint16_t *table, uint16_t *w,
                     uint16_t *states) {
    size_t tw = 16 * (size_t)K, cols = n_j * 16;
    uint8_t perm[256];
    orc_tile_perm(perm);
#pragma omp parallel for schedule(static)
    for (size_t ti = 0; ti < n_i; ++ti) {
        uint16_t st[256];
        for (size_t tj = 0; tj < n_j; ++tj) {
            orc_tile_states(code + (ti * n_j + tj) * tw, K, st);
            for (size_t p = 0; p < 256; ++p) {
                size_t pos = perm[p];
                size_t at = (ti * 16 + pos / 16) * cols + tj * 16 + pos % 16;
                w[at] = table[st[p]];
                if (states) states[at] = st[p];
            }
        }
    }
}

/* src/expert/bank.zig:116-141 */
int orc_exl3_geometry(int K, uint64_t hidden, uint64_t inter, orc_exl3_geom *g) {
    if (K <= 0 || K > 8 || hidden == 0 || inter == 0 || hidden % 16 || inter % 16) return -1;
    uint64_t off = 0;
    for (int p = 0; p < 3; ++p) {
        uint64_t in = p == 2 ? inter : hidden, out = p == 2 ? hidden : inter;
        uint64_t lens[3] = {(in / 16) * (out / 16) * 16 * (uint64_t)K * 2, out * 2, in * 2};
        for (int j = 0; j < 3; ++j) {
            g->off[p * 3 + j] = off;
            g->len[p * 3 + j] = lens[j];
            off += lens[j];
        }
    }
    g->logical_bytes = off;
    g->record_bytes = (off + 4095) / 4096 * 4096;
    return 0;
}

void orc_exl3_synth_record_k(int K, uint64_t seed, uint64_t hidden, uint64_t inter, double suh_scale, double svh_scale,
                             uint8_t *rec) {
    orc_exl3_geom g;
    orc_exl3_geometry(K, hidden, inter, &g);
    for (int p = 0; p < 3; ++p) {
        orc_fill_code(seed + 1 + 3 * p, (int16_t *)(rec + g.off[3 * p]), g.len[3 * p] / 2);
        orc_fill_scales(seed + 2 + 3 * p, suh_scale, (uint16_t *)(rec + g.off[3 * p + 2]), g.len[3 * p + 2] / 2);
        orc_fill_scales(seed + 3 + 3 * p, svh_scale, (uint16_t *)(rec + g.off[3 * p + 1]), g.len[3 * p + 1] / 2);
    }
}

void orc_exl3_synth_record(uint64_t seed, uint64_t hidden, uint64_t inter, double suh_scale, double svh_scale,
                           uint8_t *rec) {
    orc_exl3_synth_record_k(3, seed, hidden, inter, suh_scale, svh_scale, rec);
}

/* ------------------------------------------------------------------------------------------------ */
/* EXL3 f64 forward                                                                                  */
/* ------------------------------------------------------------------------------------------------ */

/* src/arch/glm5_next/exl3_forms_ref.zig:116-135 */
void orc_fwht128(double *v, size_t n) {
    const double rs = sqrt(128.0);
    for (size_t b = 0; b < n; b += 128) {
        double *x = v + b;
        for (size_t h = 1; h < 128; h <<= 1)
            for (size_t i = 0; i < 128; i += 2 * h)
                for (size_t j = i; j < i + h; ++j) {
                    double a = x[j], c = x[j + h];
                    x[j] = a + c;
                    x[j + h] = a - c;
                }
        for (size_t j = 0; j < 128; ++j) x[j] /= rs;
    }
}

/* exl3_forms_ref.zig:137-152 */
void orc_exl3_forward(const double *x, size_t in, const uint16_t *w, const uint16_t *suh, const uint16_t *svh,
                      double *y, size_t out) {
    double *xh = (double *)malloc(in * sizeof(double));
    for (size_t i = 0; i < in; ++i) xh[i] = x[i] * (double)orc_h2f(suh[i]);
    orc_fwht128(xh, in);
    memset(y, 0, out * sizeof(double));
    for (size_t i = 0; i < in; ++i) {
        double xi = xh[i];
        const uint16_t *row = w + i * out;
        for (size_t o = 0; o < out; ++o) y[o] += xi * (double)orc_h2f(row[o]);
    }
    orc_fwht128(y, out);
    for (size_t o = 0; o < out; ++o) y[o] *= (double)orc_h2f(svh[o]);
    free(xh);
}

/* exl3_forms_ref.zig:154-157 (limit 10 there); src/sdk_ext/quant.zig:56-61 */
double orc_swiglu_clamped(double g, double u, double limit) {
    if (limit > 0) {
        double gc = g < limit ? g : limit;
        if (g != g) gc = g;
        double uc = u;
        if (u == u) uc = u > limit ? limit : (u < -limit ? -limit : u);
        return gc / (1.0 + exp(-gc)) * uc;
    }
    return g / (1.0 + exp(-g)) * u;
}

typedef struct {
    uint16_t *wg, *wu, *wd; /* decoded f16 bits, row-major [in, out] */
    float *fg, *fu, *fd;    /* the same as f32 (optional) */
} exl3_dec;

static int exl3_decode_record(int K, const uint8_t *rec, uint64_t hidden, uint64_t inter, const uint16_t *table,
                              exl3_dec *d) {
    orc_exl3_geom g;
    if (orc_exl3_geometry(K, hidden, inter, &g)) return -1;
    size_t n = (size_t)hidden * inter;
    d->wg = (uint16_t *)malloc(n * 2);
    d->wu = (uint16_t *)malloc(n * 2);
    d->wd = (uint16_t *)malloc(n * 2);
    if (!d->wg || !d->wu || !d->wd) return -2;
    orc_reconstruct((const int16_t *)(rec + g.off[0]), hidden / 16, inter / 16, K, table, d->wg, NULL);
    orc_reconstruct((const int16_t *)(rec + g.off[3]), hidden / 16, inter / 16, K, table, d->wu, NULL);
    orc_reconstruct((const int16_t *)(rec + g.off[6]), inter / 16, hidden / 16, K, table, d->wd, NULL);
    return 0;
}
static void exl3_dec_free(exl3_dec *d) { free(d->wg); free(d->wu); free(d->wd); }

static const uint16_t *table_once(void) {
    static uint16_t *t = NULL;
#pragma omp critical(orc_table)
    {
        if (!t) {
            uint16_t *n = (uint16_t *)malloc(65536 * 2);
            orc_mul1_table(n);
            t = n;
        }
    }
    return t;
}

/* y = t128(t128(x suh) W) svh for `rows` rows at once; W f16 bits [in, out]; parallel over output columns */
static void exl3_forward_rows(const double *x, size_t rows, size_t in, const uint16_t *w, const uint16_t *suh,
                              const uint16_t *svh, double *y, size_t out) {
    double *xh = (double *)malloc(rows * in * sizeof(double));
    for (size_t r = 0; r < rows; ++r) {
        for (size_t i = 0; i < in; ++i) xh[r * in + i] = x[r * in + i] * (double)orc_h2f(suh[i]);
        orc_fwht128(xh + r * in, in);
    }
    memset(y, 0, rows * out * sizeof(double));
#pragma omp parallel for schedule(static)
    for (size_t ob = 0; ob < out; ob += 64) {
        for (size_t i = 0; i < in; ++i) {
            const uint16_t *row = w + i * out + ob;
            float wf[64];
            for (size_t o = 0; o < 64; ++o) wf[o] = orc_h2f(row[o]);
            for (size_t r = 0; r < rows; ++r) {
                double xi = xh[r * in + i];
                double *yr = y + r * out + ob;
                for (size_t o = 0; o < 64; ++o) yr[o] += xi * (double)wf[o];
            }
        }
    }
    for (size_t r = 0; r < rows; ++r) {
        orc_fwht128(y + r * out, out);
        for (size_t o = 0; o < out; ++o) y[r * out + o] *= (double)orc_h2f(svh[o]);
    }
    free(xh);
}

/* src/arch/glm5_next/exl3_forms_ref.zig:159-195 */
int orc_exl3_expert_f64(const uint8_t *rec, uint64_t hidden, uint64_t inter, double limit, const double *x,
                        size_t rows, double *h_out, double *y_out) {
    return orc_exl3_expert_f64_k(3, rec, hidden, inter, limit, x, rows, h_out, y_out);
}
/* the same at any K (the record's code segments shrink to 16 K int16 per tile, src/exl3/kernels.zig:163-177) */
int orc_exl3_expert_f64_k(int K, const uint8_t *rec, uint64_t hidden, uint64_t inter, double limit, const double *x,
                          size_t rows, double *h_out, double *y_out) {
    orc_exl3_geom g;
    if (orc_exl3_geometry(K, hidden, inter, &g)) return -1;
    if (hidden % 128 || inter % 128) return -1;
    exl3_dec d;
    int rc = exl3_decode_record(K, rec, hidden, inter, table_once(), &d);
    if (rc) return rc;
    const uint16_t *g_rout = (const uint16_t *)(rec + g.off[1]), *g_rin = (const uint16_t *)(rec + g.off[2]);
    const uint16_t *u_rout = (const uint16_t *)(rec + g.off[4]), *u_rin = (const uint16_t *)(rec + g.off[5]);
    const uint16_t *d_rout = (const uint16_t *)(rec + g.off[7]), *d_rin = (const uint16_t *)(rec + g.off[8]);
    double *gg = (double *)malloc(rows * inter * sizeof(double));
    double *uu = (double *)malloc(rows * inter * sizeof(double));
    double *hh = (double *)malloc(rows * inter * sizeof(double));
    exl3_forward_rows(x, rows, hidden, d.wg, g_rin, g_rout, gg, inter);
    exl3_forward_rows(x, rows, hidden, d.wu, u_rin, u_rout, uu, inter);
    for (size_t i = 0; i < rows * inter; ++i) hh[i] = orc_swiglu_clamped(gg[i], uu[i], limit);
    if (h_out) memcpy(h_out, hh, rows * inter * sizeof(double));
    if (y_out) exl3_forward_rows(hh, rows, inter, d.wd, d_rin, d_rout, y_out, hidden);
    free(gg); free(uu); free(hh);
    exl3_dec_free(&d);
    return 0;
}

/* ---- the f32 seam chain (exl3_forms_ref.zig:231-343) ---- */

static const uint32_t SCALE_BITS = 1035273459u; /* 128^-0.5 as the texts write it */

/* exl3_forms_ref.zig:246-259: stage h, thread t: k = t & (h-1), j = ((t-k) << 1) + k */
static void emu_butterfly(float *B) {
    for (uint32_t h = 1; h < 128; h <<= 1)
        for (uint32_t t = 0; t < 64; ++t) {
            uint32_t k = t & (h - 1), j = ((t - k) << 1) + k;
            float a = B[j], c = B[j + h];
            B[j] = a + c;
            B[j + h] = a - c;
        }
}

/* exl3_forms_ref.zig:236-243 */
static void emu_rot_in(const float *x, const uint16_t *r, float *out, size_t n) {
    const float S = u2f(SCALE_BITS);
    for (size_t i = 0; i < n; ++i) out[i] = x[i] * orc_h2f(r[i]);
    for (size_t b = 0; b < n; b += 128) {
        emu_butterfly(out + b);
        for (size_t i = 0; i < 128; ++i) out[b + i] = out[b + i] * S;
    }
}

/* exl3_forms_ref.zig:263-297: the stock GEMV of output tile tn with its lane plan and column sums */
static void emu_gemv_tile(const float *xh, const uint16_t *w, uint32_t in, uint32_t out, uint32_t tn, float *z) {
    float accs[32][8];
    for (uint32_t l = 0; l < 32; ++l) {
        float acc[8] = {0};
        for (uint32_t tk = 0; tk < in / 16; ++tk)
            for (uint32_t m = 0; m < 8; ++m) {
                uint32_t q = m & 3;
                uint32_t dr = 2 * (l & 3) + (q < 2 ? 9u : 3u) - q;
                uint32_t col = (l >> 2) + (m < 4 ? 8u : 0u);
                float wv = orc_h2f(w[(size_t)(tk * 16 + dr) * out + tn * 16 + col]);
                acc[m] = fmaf(xh[tk * 16 + dr], wv, acc[m]);
            }
        memcpy(accs[l], acc, sizeof acc);
    }
    float red[16][32];
    memset(red, 0, sizeof red);
    for (uint32_t l = 0; l < 32; ++l)
        for (uint32_t m = 0; m < 8; ++m) {
            uint32_t c = (l >> 2) + (m < 4 ? 8u : 0u);
            red[c][l] += accs[l][m];
        }
    for (uint32_t c = 0; c < 16; ++c) {
        float s = 0;
        for (uint32_t l = 0; l < 32; ++l) s += red[c][l];
        z[c] = s;
    }
}

/* exl3_forms_ref.zig:299-343 */
int orc_exl3_expert_f32chain(const uint8_t *rec, uint64_t hidden, uint64_t inter, const float *x, size_t rows,
                             float *h_out, float *y_out) {
    orc_exl3_geom g;
    if (orc_exl3_geometry(3, hidden, inter, &g) || hidden % 128 || inter % 128) return -1;
    exl3_dec d;
    int rc = exl3_decode_record(3, rec, hidden, inter, table_once(), &d);
    if (rc) return rc;
    const uint16_t *og = (const uint16_t *)(rec + g.off[1]), *rg = (const uint16_t *)(rec + g.off[2]);
    const uint16_t *ou = (const uint16_t *)(rec + g.off[4]), *ru = (const uint16_t *)(rec + g.off[5]);
    const uint16_t *od = (const uint16_t *)(rec + g.off[7]), *rd = (const uint16_t *)(rec + g.off[8]);
    const float S = u2f(SCALE_BITS);
    for (size_t r = 0; r < rows; ++r) {
        float *xg = (float *)malloc(hidden * 4), *xu = (float *)malloc(hidden * 4);
        float *h = (float *)malloc(inter * 4), *xd = (float *)malloc(inter * 4);
        emu_rot_in(x + r * hidden, rg, xg, hidden);
        emu_rot_in(x + r * hidden, ru, xu, hidden);
#pragma omp parallel for schedule(static)
        for (uint32_t blk = 0; blk < inter / 128; ++blk) {
            float bg[128], bu[128];
            for (uint32_t t = 0; t < 8; ++t) {
                emu_gemv_tile(xg, d.wg, (uint32_t)hidden, (uint32_t)inter, blk * 8 + t, bg + t * 16);
                emu_gemv_tile(xu, d.wu, (uint32_t)hidden, (uint32_t)inter, blk * 8 + t, bu + t * 16);
            }
            emu_butterfly(bg);
            emu_butterfly(bu);
            for (uint32_t e = 0; e < 128; ++e) {
                uint32_t col = blk * 128 + e;
                float gv = bg[e] * S;
                float gm = gv * orc_h2f(og[col]);
                float gate = isnan(gm) ? gm : (gm < 10.0f ? gm : 10.0f);
                float uv = bu[e] * S;
                float um = uv * orc_h2f(ou[col]);
                float up0 = isnan(um) ? um : (um > -10.0f ? um : -10.0f);
                float up = isnan(up0) ? up0 : (up0 < 10.0f ? up0 : 10.0f);
                float yv = 1.0f / (1.0f + expf(fabsf(gate)));
                float sg = gate < 0 ? yv : 1.0f - yv;
                h[col] = (gate * sg) * up;
            }
        }
        if (h_out) memcpy(h_out + r * inter, h, inter * 4);
        if (y_out) {
            emu_rot_in(h, rd, xd, inter);
#pragma omp parallel for schedule(static)
            for (uint32_t hb = 0; hb < hidden / 128; ++hb) {
                float bd[128];
                for (uint32_t t = 0; t < 8; ++t)
                    emu_gemv_tile(xd, d.wd, (uint32_t)inter, (uint32_t)hidden, hb * 8 + t, bd + t * 16);
                emu_butterfly(bd);
                for (uint32_t c = 0; c < 128; ++c)
                    y_out[r * hidden + hb * 128 + c] = (bd[c] * S) * orc_h2f(od[hb * 128 + c]);
            }
        }
        free(xg); free(xu); free(h); free(xd);
    }
    exl3_dec_free(&d);
    return 0;
}

/* ------------------------------------------------------------------------------------------------ */
/* FP4 formats                                                                                       */
/* ------------------------------------------------------------------------------------------------ */

/* src/arch/glm5_next/decode_kernels_ref.zig:79-83 */
float orc_e2m1_value(uint32_t c) {
    static const float mag[8] = {0, 0.5f, 1, 1.5f, 2, 3, 4, 6};
    float v = mag[c & 7];
    return (c & 8) ? -v : v;
}
/* decode_kernels_ref.zig:13-16 */
uint16_t orc_e2m1_halfbits(uint32_t c) { return (uint16_t)(((c & 7) << 9) | ((c & 8) << 12)); }
/* decode_kernels_ref.zig:22-29 */
void orc_fp4_decode8(uint32_t w, uint32_t out[4]) {
    out[0] = ((w << 9) & 0x0E000E00u) | ((w << 12) & 0x80008000u);
    out[1] = ((w << 5) & 0x0E000E00u) | ((w << 8) & 0x80008000u);
    out[2] = ((w << 1) & 0x0E000E00u) | ((w << 4) & 0x80008000u);
    out[3] = ((w >> 3) & 0x0E000E00u) | (w & 0x80008000u);
}
/* decode_kernels_ref.zig:32-36 */
float orc_e4m3_kernel(uint8_t b) {
    uint32_t v = b & 127;
    uint16_t u = (uint16_t)((v << 7) | (((v + 1) >> 7) << 14) | (((uint32_t)b & 128) << 8));
    return orc_h2f(u) * 256.0f;
}
/* decode_kernels_ref.zig:71-76 */
float orc_e4m3_value(uint8_t b) {
    int e = (b >> 3) & 0xF;
    int m = b & 7;
    float mag;
    if (e == 15 && m == 7) mag = NAN;
    else if (e == 0) mag = ldexpf((float)m, -9);
    else mag = ldexpf((float)(8 + m), e - 10);
    return (b & 0x80) ? -mag : mag;
}
/* decode_kernels_ref.zig:86-88: s = e4m3 * (g / 2688), then s * e2m1, f32 */
float orc_nvfp4_weight(uint8_t scale, uint32_t code, float g) {
    float inv = g / 2688.0f;
    float s = orc_e4m3_value(scale) * inv;
    return s * orc_e2m1_value(code);
}
/* decode_kernels_ref.zig:39-47 + 59-63: the texts' (scale x 2^14) times the code's half */
float orc_nvfp4_kernel_weight(uint8_t scale, uint32_t code, float g) {
    float inv = g / 2688.0f;
    float s = (orc_e4m3_kernel(scale) * inv) * 16384.0f;
    return s * orc_h2f(orc_e2m1_halfbits(code));
}
float orc_e8m0_value(uint32_t b) { return ldexpf(1.0f, (int)(b & 255) - 127); }
static inline float ftz(float v) { return fabsf(v) < 1.17549435e-38f ? copysignf(0.0f, v) : v; }
/* src/arch/mimo_v2/moe.zig:410-413 */
float orc_mxfp4_scale_ref(uint32_t b) {
    float v = u2f(b == 0 ? 0x400000u : b << 23);
    return ftz(ftz(v) * 0.00390625f);
}
/* moe.zig:341-344 */
static float sigmoid_ref(float x) {
    float y = ftz(1.0f / (1.0f + expf(fabsf(x))));
    return x < 0 ? y : 1.0f - y;
}
/* moe.zig:355-360 */
float orc_silu_mul_ref(float gate, float up) {
    float gf = orc_bf16_round(gate);
    return orc_bf16_round(orc_bf16_round(ftz(gf * sigmoid_ref(gf))) * orc_bf16_round(up));
}
/* src/kernels/glm5_next_nvfp4/glm5n_nvfp4_gateup.metal:109-129 */
float orc_silu_mul_clamped_ref(float gate, float up, float lim) {
    float gf = orc_bf16_round(gate);
    float gc = gf > lim ? lim : gf;
    float uf = orc_bf16_round(up);
    float uc = uf > lim ? lim : (uf < -lim ? -lim : uf);
    return orc_bf16_round(orc_bf16_round(ftz(gc * sigmoid_ref(gc))) * orc_bf16_round(uc));
}

/* weight [rows, cols/8] u32 (code j of a word at bits 4j), scales [rows, cols/32] E8M0: mimo_v2/moe.zig:379-416 */
void orc_mxfp4_decode(const uint32_t *words, const uint8_t *scales, size_t rows, size_t cols, float *out) {
#pragma omp parallel for schedule(static)
    for (size_t r = 0; r < rows; ++r)
        for (size_t c = 0; c < cols; ++c) {
            uint32_t w = words[r * (cols / 8) + c / 8];
            float s = orc_e8m0_value(scales[r * (cols / 32) + c / 32]);
            out[r * cols + c] = orc_e2m1_value((w >> (4 * (c % 8))) & 15) * s;
        }
}
/* decode_kernels_ref.zig:51-65 */
void orc_nvfp4_decode(const uint32_t *words, const uint8_t *scales, float g, size_t rows, size_t cols, float *out) {
#pragma omp parallel for schedule(static)
    for (size_t r = 0; r < rows; ++r)
        for (size_t c = 0; c < cols; ++c) {
            uint32_t w = words[r * (cols / 8) + c / 8];
            out[r * cols + c] = orc_nvfp4_weight(scales[r * (cols / 16) + c / 16], (w >> (4 * (c % 8))) & 15, g);
        }
}

uint64_t orc_mxfp4_record_bytes(uint64_t hidden, uint64_t inter, uint64_t off[6]) {
    uint64_t lens[6] = {inter * hidden / 2, inter * hidden / 32, inter * hidden / 2,
                        inter * hidden / 32, hidden * inter / 2, hidden * inter / 32};
    uint64_t at = 0;
    for (int i = 0; i < 6; ++i) { if (off) off[i] = at; at += lens[i]; }
    return at;
}
uint64_t orc_nvfp4_record_bytes(uint64_t hidden, uint64_t inter, uint64_t off[9]) {
    uint64_t lens[9] = {inter * hidden / 2, inter * hidden / 16, 4, inter * hidden / 2, inter * hidden / 16, 4,
                        hidden * inter / 2, hidden * inter / 16, 4};
    uint64_t at = 0;
    for (int i = 0; i < 9; ++i) { if (off) off[i] = at; at += lens[i]; }
    return at;
}

/* ---- our synthetic FP4 quantiser (the reference ships none; its converters copy release bytes) ---- */

static double gauss(uint64_t *s) {
    double u1 = unit53(orc_splitmix64(s)), u2 = unit53(orc_splitmix64(s));
    if (u1 < 1e-300) u1 = 1e-300;
    return sqrt(-2.0 * log(u1)) * cos(6.283185307179586 * u2);
}
static uint32_t e2m1_encode(double v) { /* round to nearest, ties to the even code, saturate at 6 */
    static const double mag[8] = {0, 0.5, 1, 1.5, 2, 3, 4, 6};
    double a = fabs(v);
    int best = 0;
    double bd = 1e300;
    for (int i = 0; i < 8; ++i) {
        double dd = fabs(a - mag[i]);
        if (dd < bd || (dd == bd && (i & 1) == 0)) { bd = dd; best = i; }
    }
    return (uint32_t)best | (v < 0 ? 8u : 0u);
}
static void fp4_quant_proj_mx(uint64_t *s, size_t rows, size_t cols, double sigma, uint32_t *words, uint8_t *scales) {
    double blk[32];
    for (size_t r = 0; r < rows; ++r)
        for (size_t b = 0; b < cols / 32; ++b) {
            double amax = 0;
            for (int i = 0; i < 32; ++i) { blk[i] = gauss(s) * sigma; amax = fmax(amax, fabs(blk[i])); }
            int ex = amax > 0 ? (int)floor(log2(amax)) - 2 : -127; /* OCP MX: shared exponent = floor(log2 amax) - emax */
            if (ex < -127) ex = -127;
            if (ex > 127) ex = 127;
            scales[r * (cols / 32) + b] = (uint8_t)(ex + 127);
            double inv = ldexp(1.0, -ex);
            for (int wi = 0; wi < 4; ++wi) {
                uint32_t w = 0;
                for (int j = 0; j < 8; ++j) w |= e2m1_encode(blk[wi * 8 + j] * inv) << (4 * j);
                words[r * (cols / 8) + b * 4 + wi] = w;
            }
        }
}
void orc_mxfp4_synth_record(uint64_t seed, uint64_t hidden, uint64_t inter, double sigma, uint8_t *rec) {
    uint64_t off[6];
    orc_mxfp4_record_bytes(hidden, inter, off);
    for (int p = 0; p < 3; ++p) {
        uint64_t s = seed * 3 + p + 1;
        size_t rows = p == 2 ? hidden : inter, cols = p == 2 ? inter : hidden;
        fp4_quant_proj_mx(&s, rows, cols, sigma, (uint32_t *)(rec + off[2 * p]), rec + off[2 * p + 1]);
    }
}
static uint8_t e4m3_encode_pos(double v) { /* nearest non-negative finite E4M3, ties to the even byte */
    if (!(v > 0)) return 0;
    if (v >= 448.0) return 0x7E;
    int ex;
    frexp(v, &ex);            /* v = f 2^ex, f in [0.5, 1) -> binade exponent ex - 1 */
    int e = ex - 1;
    if (e < -6) e = -6;       /* subnormals share the 2^-6 binade: steps of 2^-9 */
    double step = ldexp(1.0, e - 3);
    double q = nearbyint(v / step); /* ties to even; consecutive bytes alternate parity */
    double r = q * step;
    int best = 0;
    /* r is exactly representable: find its byte by the format's definition */
    if (r >= 448.0) return 0x7E;
    if (r < 0.015625) return (uint8_t)nearbyint(r * 512.0);
    frexp(r, &ex);
    e = ex - 1;
    best = ((e + 7) << 3) | ((int)nearbyint(r / ldexp(1.0, e - 3)) - 8);
    return (uint8_t)best;
}
void orc_nvfp4_synth_record(uint64_t seed, uint64_t hidden, uint64_t inter, double sigma, uint8_t *rec) {
    uint64_t off[9];
    orc_nvfp4_record_bytes(hidden, inter, off);
    for (int p = 0; p < 3; ++p) {
        uint64_t s = seed * 3 + p + 1;
        size_t rows = p == 2 ? hidden : inter, cols = p == 2 ? inter : hidden;
        size_t n = rows * cols;
        double *w = (double *)malloc(n * sizeof(double));
        double amax = 0;
        for (size_t i = 0; i < n; ++i) { w[i] = gauss(&s) * sigma; amax = fmax(amax, fabs(w[i])); }
        float g = (float)amax; /* the tensor amax: g / 2688 = amax / (448 * 6) */
        float inv = g / 2688.0f;
        memcpy(rec + off[3 * p + 2], &g, 4);
        uint32_t *words = (uint32_t *)(rec + off[3 * p]);
        uint8_t *scales = rec + off[3 * p + 1];
        for (size_t r = 0; r < rows; ++r)
            for (size_t b = 0; b < cols / 16; ++b) {
                const double *blk = w + r * cols + b * 16;
                double bm = 0;
                for (int i = 0; i < 16; ++i) bm = fmax(bm, fabs(blk[i]));
                uint8_t sb = e4m3_encode_pos(bm / (6.0 * (double)inv));
                scales[r * (cols / 16) + b] = sb;
                double sc = (double)(orc_e4m3_value(sb) * inv);
                for (int wi = 0; wi < 2; ++wi) {
                    uint32_t word = 0;
                    for (int j = 0; j < 8; ++j)
                        word |= e2m1_encode(sc > 0 ? blk[wi * 8 + j] / sc : 0.0) << (4 * j);
                    words[r * (cols / 8) + b * 2 + wi] = word;
                }
            }
        free(w);
    }
}

/* ------------------------------------------------------------------------------------------------ */
/* router                                                                                            */
/* ------------------------------------------------------------------------------------------------ */

/* Fixed-sequence exp and log: IEEE single +, *, fma and / only, written so that a device kernel evaluating the
 * same statements gives the same bits (the reference's own CPU and GPU exps differ in the last place, so bit-exact
 * ids need one definition on both sides). */
float orc_det_expf(float x) {
    if (x != x) return x;
    if (x > 88.75f) return INFINITY;
    if (x < -104.0f) return 0.0f;
    const float magic = 12582912.0f; /* 1.5 * 2^23: rounds to the nearest integer, ties to even */
    float t = x * 1.44269504f;
    float n = (t + magic) - magic;
    float r = fmaf(n, -0.693145752f, x);
    r = fmaf(n, -1.42860677e-06f, r);
    float p = 1.98412701e-04f;
    p = fmaf(p, r, 1.38888892e-03f);
    p = fmaf(p, r, 8.33333377e-03f);
    p = fmaf(p, r, 4.16666679e-02f);
    p = fmaf(p, r, 1.66666672e-01f);
    p = fmaf(p, r, 0.5f);
    p = fmaf(p, r, 1.0f);
    p = fmaf(p, r, 1.0f);
    int ni = (int)n;
    int n1 = ni / 2, n2 = ni - n1;
    float s1 = u2f((uint32_t)(n1 + 127) << 23), s2 = u2f((uint32_t)(n2 + 127) << 23);
    return (p * s1) * s2;
}
float orc_det_logf(float x) { /* x normal and positive */
    uint32_t b = f2u(x);
    int e = (int)(b >> 23) - 127;
    uint32_t mb = (b & 0x007FFFFFu) | 0x3F800000u;
    float m = u2f(mb);
    if (m > 1.41421354f) { m = m * 0.5f; e += 1; }
    float f = m - 1.0f;
    float s = f / (2.0f + f);
    float z = s * s;
    float R = 9.09090936e-02f;
    R = fmaf(R, z, 1.11111112e-01f);
    R = fmaf(R, z, 1.42857149e-01f);
    R = fmaf(R, z, 0.2f);
    R = fmaf(R, z, 3.33333343e-01f);
    R = R * z;
    float s2 = s + s;
    float lo = fmaf(s2, R, s2);
    float ef = (float)e;
    lo = fmaf(ef, 1.42860677e-06f, lo);
    return fmaf(ef, 0.693145752f, lo);
}

typedef float (*fn1)(float);
static float libm_exp(float x) { return expf(x); }
static float libm_log(float x) { return logf(x); }

/* src/kernels/exl3/header_router_tail.metal: log1p and logaddexp(x, 0), statement for statement */
static float rt_log1p(float x, fn1 lg) {
    float xp1 = 1.0f + x;
    if (xp1 == INFINITY) return INFINITY;
    if (xp1 == 1.0f) return x;
    return x * (lg(xp1) / (xp1 - 1.0f));
}
static float rt_softplus(float g, fn1 ex, fn1 lg) {
    if (g != g) return NAN;
    float maxval = g > 0.0f ? g : 0.0f, minval = g > 0.0f ? 0.0f : g;
    if (minval == -INFINITY || maxval == INFINITY) return maxval;
    return maxval + rt_log1p(ex(minval - maxval), lg);
}
/* rank order of q3rc_router_tail.metal:17-26 / mimo_glue_top8.metal:19-27: score descending, ties to the lower
 * index, NaN last */
static int before(float o, size_t j, float v, size_t n) {
    int on = o != o, vn = v != v;
    if (vn) return (!on) || j < n;
    return !on && (o > v || (o == v && j < n));
}

static int route_impl(const float *logits, const float *bias, size_t T, size_t E, size_t k, int scoring, int norm,
                      float scale, int32_t *ids, float *weights, fn1 ex, fn1 lg) {
    if (k == 0 || k > E || E == 0) return -1;
    if (scoring < 0 || scoring > 2) return -1;
#pragma omp parallel for schedule(static)
    for (size_t t = 0; t < T; ++t) {
        const float *x = logits + t * E;
        float *score = (float *)malloc(E * 4), *key = (float *)malloc(E * 4);
        unsigned char *taken = (unsigned char *)calloc(E, 1);
        if (scoring == ORC_SCORE_SIGMOID) {
            for (size_t e = 0; e < E; ++e) {
                float y = 1.0f / (1.0f + ex(fabsf(x[e])));
                score[e] = x[e] < 0 ? y : 1.0f - y;
            }
        } else if (scoring == ORC_SCORE_SQRTSOFTPLUS) {
            for (size_t e = 0; e < E; ++e) score[e] = sqrtf(rt_softplus(x[e], ex, lg));
        } else {
            float m = -INFINITY;
            int has_nan = 0;
            for (size_t e = 0; e < E; ++e) { if (x[e] != x[e]) has_nan = 1; else if (x[e] > m) m = x[e]; }
            float part[32] = {0};
            for (size_t e = 0; e < E; ++e) {
                score[e] = has_nan ? NAN : ex(x[e] - m);
                part[e & 31] += score[e];
            }
            for (int off = 16; off >= 1; off >>= 1) {
                float nx[32];
                for (int l = 0; l < 32; ++l) nx[l] = part[l] + part[l ^ off];
                memcpy(part, nx, sizeof nx);
            }
            for (size_t e = 0; e < E; ++e) score[e] = score[e] / part[0];
        }
        for (size_t e = 0; e < E; ++e) key[e] = bias ? score[e] + bias[e] : score[e];
        float picked[64];
        for (size_t j = 0; j < k; ++j) {
            size_t best = E;
            for (size_t e = 0; e < E; ++e) {
                if (taken[e]) continue;
                if (best == E || before(key[e], e, key[best], best)) best = e;
            }
            taken[best] = 1;
            ids[t * k + j] = (int32_t)best;
            picked[j] = score[best];
        }
        float total = 0;
        for (size_t j = 0; j < k; ++j) total = picked[j] + total;
        float den = total + 1e-20f;
        for (size_t j = 0; j < k; ++j) {
            float q = norm ? picked[j] / den : picked[j];
            weights[t * k + j] = q * scale;
        }
        free(score); free(key); free(taken);
    }
    return 0;
}
int orc_route_libm(const float *logits, const float *bias, size_t T, size_t E, size_t k, int scoring, int norm,
                   float scale, int32_t *ids, float *weights) {
    if (k > 64) return -1;
    return route_impl(logits, bias, T, E, k, scoring, norm, scale, ids, weights, libm_exp, libm_log);
}
int orc_route_det(const float *logits, const float *bias, size_t T, size_t E, size_t k, int scoring, int norm,
                  float scale, int32_t *ids, float *weights) {
    if (k > 64) return -1;
    return route_impl(logits, bias, T, E, k, scoring, norm, scale, ids, weights, orc_det_expf, orc_det_logf);
}

/* ------------------------------------------------------------------------------------------------ */
/* dispatch                                                                                          */
/* ------------------------------------------------------------------------------------------------ */

/* src/sdk_ext/quant.zig:269-290: stable by slot, as a counting sort */
void orc_dispatch(const int32_t *slot, size_t n, size_t n_slots, uint32_t *order, uint32_t *sorted_slot,
                  uint32_t *inv, uint32_t *offsets) {
    uint32_t *cnt = (uint32_t *)calloc(n_slots + 1, 4);
    for (size_t i = 0; i < n; ++i) cnt[slot[i] + 1] += 1;
    for (size_t i = 1; i <= n_slots; ++i) cnt[i] += cnt[i - 1];
    if (offsets) memcpy(offsets, cnt, (n_slots + 1) * 4);
    for (size_t i = 0; i < n; ++i) {
        order[cnt[slot[i]]] = (uint32_t)i;
        cnt[slot[i]] += 1;
    }
    for (size_t i = 0; i < n; ++i) {
        if (sorted_slot) sorted_slot[i] = (uint32_t)slot[order[i]];
        if (inv) inv[order[i]] = (uint32_t)i;
    }
    free(cnt);
}

/* ------------------------------------------------------------------------------------------------ */
/* layer                                                                                             */
/* ------------------------------------------------------------------------------------------------ */

int orc_max_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* bf16 dense shared expert (src/arch/deepseek_v41/graph.zig:2162-2172 over bf16 linears): gate/up in f32 class
 * precision (f64 here), clamped SwiGLU, h rounded to the activation dtype (bf16), down. */
static void shared_expert_f64(const orc_layer_cfg *c, const uint16_t *w1, const uint16_t *w3, const uint16_t *w2,
                              const float *x, size_t T, double *out) {
    size_t H = c->hidden, I = c->inter;
    double *h = (double *)malloc(T * I * sizeof(double));
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < I; ++i)
        for (size_t t = 0; t < T; ++t) {
            double g = 0, u = 0;
            for (size_t j = 0; j < H; ++j) {
                double xv = x[t * H + j];
                g += xv * (double)bf16_bits_f32(w1[i * H + j]);
                u += xv * (double)bf16_bits_f32(w3[i * H + j]);
            }
            h[t * I + i] = (double)orc_bf16_round((float)orc_swiglu_clamped(g, u, c->limit));
        }
#pragma omp parallel for schedule(static)
    for (size_t o = 0; o < H; ++o)
        for (size_t t = 0; t < T; ++t) {
            double s = 0;
            for (size_t i = 0; i < I; ++i) s += h[t * I + i] * (double)bf16_bits_f32(w2[o * I + i]);
            out[t * H + o] = s;
        }
    free(h);
}

/* FP4 expert on `rows` rows: wg, wu [I, H] and wd [H, I] dequantised f32; sums in f64, the reference decode
 * texts' rounding points when chain is set (mimo_moe_k1_gateup.metal:115-128, glm5n_nvfp4_gateup.metal:109-129,
 * the down texts' bf16 store). */
static void fp4_expert_rows(const orc_layer_cfg *c, const float *wg, const float *wu, const float *wd,
                            const double *x, size_t rows, double *y) {
    size_t H = c->hidden, I = c->inter;
    double *h = (double *)malloc(rows * I * sizeof(double));
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < I; ++i)
        for (size_t r = 0; r < rows; ++r) {
            double g = 0, u = 0;
            for (size_t j = 0; j < H; ++j) {
                g += x[r * H + j] * (double)wg[i * H + j];
                u += x[r * H + j] * (double)wu[i * H + j];
            }
            if (c->chain_rounding) {
                if (c->limit > 0) h[r * I + i] = orc_silu_mul_clamped_ref((float)g, (float)u, (float)c->limit);
                else h[r * I + i] = orc_silu_mul_ref((float)g, (float)u);
            } else {
                h[r * I + i] = orc_swiglu_clamped(g, u, c->limit);
            }
        }
#pragma omp parallel for schedule(static)
    for (size_t o = 0; o < H; ++o)
        for (size_t r = 0; r < rows; ++r) {
            double s = 0;
            for (size_t i = 0; i < I; ++i) s += h[r * I + i] * (double)wd[o * I + i];
            y[r * H + o] = c->chain_rounding ? (double)orc_bf16_round((float)s) : s;
        }
    free(h);
}

int orc_layer(const orc_layer_cfg *c, const uint8_t *const *records, const float *x, size_t T, const int32_t *ids,
              const float *weights, const uint16_t *sh_w1, const uint16_t *sh_w3, const uint16_t *sh_w2, double *y,
              double *ro_out) {
    size_t H = c->hidden, I = c->inter, E = c->n_experts, k = c->top_k, A = T * k;
    if (H % 128 || I % 128) return -1;
    for (size_t a = 0; a < A; ++a)
        if (ids[a] < 0 || (size_t)ids[a] >= E) return -3;
    uint32_t *order = (uint32_t *)malloc(A * 4 + 4), *offs = (uint32_t *)malloc((E + 1) * 4);
    orc_dispatch(ids, A, E, order, NULL, NULL, offs);
    double *ro = ro_out ? ro_out : (double *)malloc(A * H * sizeof(double));
    int rc = 0;
    for (size_t e = 0; e < E && !rc; ++e) {
        size_t n = offs[e + 1] - offs[e];
        if (!n) continue;
        if (!records[e]) { rc = -4; break; }
        double *xe = (double *)malloc(n * H * sizeof(double)), *ye = (double *)malloc(n * H * sizeof(double));
        for (size_t r = 0; r < n; ++r) {
            size_t tok = order[offs[e] + r] / k;
            for (size_t j = 0; j < H; ++j) xe[r * H + j] = x[tok * H + j];
        }
        if (c->bank == ORC_BANK_EXL3 || c->bank == ORC_BANK_EXL3_K2) {
            rc = orc_exl3_expert_f64_k(c->bank == ORC_BANK_EXL3 ? 3 : 2, records[e], H, I, c->limit, xe, n, NULL, ye);
        } else {
            size_t nw = H * I;
            float *wg = (float *)malloc(nw * 4), *wu = (float *)malloc(nw * 4), *wd = (float *)malloc(nw * 4);
            const uint8_t *rec = records[e];
            if (c->bank == ORC_BANK_MXFP4) {
                uint64_t off[6];
                orc_mxfp4_record_bytes(H, I, off);
                orc_mxfp4_decode((const uint32_t *)(rec + off[0]), rec + off[1], I, H, wg);
                orc_mxfp4_decode((const uint32_t *)(rec + off[2]), rec + off[3], I, H, wu);
                orc_mxfp4_decode((const uint32_t *)(rec + off[4]), rec + off[5], H, I, wd);
            } else {
                uint64_t off[9];
                orc_nvfp4_record_bytes(H, I, off);
                float gg, gu, gd;
                memcpy(&gg, rec + off[2], 4); memcpy(&gu, rec + off[5], 4); memcpy(&gd, rec + off[8], 4);
                orc_nvfp4_decode((const uint32_t *)(rec + off[0]), rec + off[1], gg, I, H, wg);
                orc_nvfp4_decode((const uint32_t *)(rec + off[3]), rec + off[4], gu, I, H, wu);
                orc_nvfp4_decode((const uint32_t *)(rec + off[6]), rec + off[7], gd, H, I, wd);
            }
            fp4_expert_rows(c, wg, wu, wd, xe, n, ye);
            free(wg); free(wu); free(wd);
        }
        for (size_t r = 0; r < n; ++r) memcpy(ro + (size_t)order[offs[e] + r] * H, ye + r * H, H * sizeof(double));
        free(xe); free(ye);
    }
    if (!rc) {
        double *sh = NULL;
        if (sh_w1) {
            sh = (double *)malloc(T * H * sizeof(double));
            shared_expert_f64(c, sh_w1, sh_w3, sh_w2, x, T, sh);
        }
        for (size_t t = 0; t < T; ++t)
            for (size_t j = 0; j < H; ++j) {
                if (c->bank != ORC_BANK_EXL3 && c->bank != ORC_BANK_EXL3_K2 && c->chain_rounding) {
                    /* mimo_v2/moe.zig:363-372: products added to 0, folded k = 0..top_k-1, bf16 once */
                    float acc = (float)ro[(t * k) * H + j] * weights[t * k] + 0.0f;
                    for (size_t q = 1; q < k; ++q) {
                        float p = (float)ro[(t * k + q) * H + j] * weights[t * k + q] + 0.0f;
                        acc = p + acc;
                    }
                    float routed = orc_bf16_round(acc);
                    /* glm5n_moe_combine.metal:6-16: bf16 add of the shared row */
                    if (sh) routed = orc_bf16_round(routed + orc_bf16_round((float)sh[t * H + j]));
                    y[t * H + j] = routed;
                } else {
                    /* deepseek_v41/graph.zig:2182-2184: sum_k f32(ro) w + shared */
                    double acc = 0;
                    for (size_t q = 0; q < k; ++q) acc += ro[(t * k + q) * H + j] * (double)weights[t * k + q];
                    if (sh) acc += sh[t * H + j];
                    y[t * H + j] = acc;
                }
            }
        free(sh);
    }
    if (!ro_out) free(ro);
    free(order); free(offs);
    return rc;
}

/* ---- the timed CPU baseline: f32, weights decoded on the fly, OpenMP over (expert, output tile) ---- */

static void hadamard128_f32(float *B) {
    for (uint32_t h = 1; h < 128; h <<= 1)
        for (uint32_t i = 0; i < 128; i += 2 * h)
            for (uint32_t j = i; j < i + h; ++j) {
                float a = B[j], c = B[j + h];
                B[j] = a + c;
                B[j + h] = a - c;
            }
}

/* z [rows, out] = xh [rows, in] . W_hat, W_hat decoded tile by tile from `code` [in/16, out/16, 48] */
static void exl3_gemm_fast(const int16_t *code, size_t in, size_t out, const float *tablef, const uint8_t *perm,
                           const float *xh, size_t rows, float *z) {
    size_t n_i = in / 16, n_j = out / 16;
#pragma omp for schedule(static) nowait
    for (size_t tj = 0; tj < n_j; ++tj) {
        float acc[64][16];
        for (size_t r0 = 0; r0 < rows; r0 += 64) {
            size_t nr = rows - r0 < 64 ? rows - r0 : 64;
            memset(acc, 0, sizeof acc);
            for (size_t ti = 0; ti < n_i; ++ti) {
                uint16_t st[256];
                float wt[16][16];
                orc_tile_states(code + (ti * n_j + tj) * 48, 3, st);
                for (int p = 0; p < 256; ++p) wt[perm[p] / 16][perm[p] % 16] = tablef[st[p]];
                for (size_t r = 0; r < nr; ++r) {
                    const float *xr = xh + (r0 + r) * in + ti * 16;
                    for (int dr = 0; dr < 16; ++dr) {
                        float xv = xr[dr];
                        for (int cc = 0; cc < 16; ++cc) acc[r][cc] = fmaf(xv, wt[dr][cc], acc[r][cc]);
                    }
                }
            }
            for (size_t r = 0; r < nr; ++r) memcpy(z + (r0 + r) * out + tj * 16, acc[r], 64);
        }
    }
}

int orc_layer_fast(const orc_layer_cfg *c, const uint8_t *const *records, const float *x, size_t T,
                   const int32_t *ids, const float *weights, const uint16_t *sh_w1, const uint16_t *sh_w3,
                   const uint16_t *sh_w2, float *y, int threads) {
    size_t H = c->hidden, I = c->inter, E = c->n_experts, k = c->top_k, A = T * k;
    if (c->bank != ORC_BANK_EXL3 || H % 128 || I % 128) return -1;
#ifdef _OPENMP
    if (threads > 0) omp_set_num_threads(threads);
#endif
    const uint16_t *tab = table_once();
    float *tablef = (float *)malloc(65536 * 4);
    for (int i = 0; i < 65536; ++i) tablef[i] = orc_h2f(tab[i]);
    uint8_t perm[256];
    orc_tile_perm(perm);
    uint32_t *order = (uint32_t *)malloc(A * 4 + 4), *offs = (uint32_t *)malloc((E + 1) * 4);
    orc_dispatch(ids, A, E, order, NULL, NULL, offs);
    float *ro = (float *)malloc(A * H * 4);
    const float S = u2f(SCALE_BITS);
    orc_exl3_geom g;
    orc_exl3_geometry(3, H, I, &g);
    float lim = (float)c->limit;
    for (size_t e = 0; e < E; ++e) {
        size_t n = offs[e + 1] - offs[e];
        if (!n) continue;
        const uint8_t *rec = records[e];
        if (!rec) return -4;
        const uint16_t *og = (const uint16_t *)(rec + g.off[1]), *rg = (const uint16_t *)(rec + g.off[2]);
        const uint16_t *ou = (const uint16_t *)(rec + g.off[4]), *ru = (const uint16_t *)(rec + g.off[5]);
        const uint16_t *od = (const uint16_t *)(rec + g.off[7]), *rd = (const uint16_t *)(rec + g.off[8]);
        float *xg = (float *)malloc(n * H * 4), *xu = (float *)malloc(n * H * 4);
        float *zg = (float *)malloc(n * I * 4), *zu = (float *)malloc(n * I * 4);
        float *xd = (float *)malloc(n * I * 4), *zd = (float *)malloc(n * H * 4);
#pragma omp parallel
        {
#pragma omp for schedule(static)
            for (size_t r = 0; r < n; ++r) {
                const float *xr = x + (size_t)(order[offs[e] + r] / k) * H;
                for (size_t j = 0; j < H; ++j) {
                    xg[r * H + j] = xr[j] * orc_h2f(rg[j]);
                    xu[r * H + j] = xr[j] * orc_h2f(ru[j]);
                }
                for (size_t b = 0; b < H; b += 128) {
                    hadamard128_f32(xg + r * H + b);
                    hadamard128_f32(xu + r * H + b);
                    for (size_t j = 0; j < 128; ++j) { xg[r * H + b + j] *= S; xu[r * H + b + j] *= S; }
                }
            }
            exl3_gemm_fast((const int16_t *)(rec + g.off[0]), H, I, tablef, perm, xg, n, zg);
            exl3_gemm_fast((const int16_t *)(rec + g.off[3]), H, I, tablef, perm, xu, n, zu);
#pragma omp barrier
#pragma omp for schedule(static)
            for (size_t r = 0; r < n; ++r) {
                for (size_t b = 0; b < I; b += 128) {
                    hadamard128_f32(zg + r * I + b);
                    hadamard128_f32(zu + r * I + b);
                    for (size_t j = 0; j < 128; ++j) {
                        size_t col = b + j;
                        float gm = (zg[r * I + col] * S) * orc_h2f(og[col]);
                        float um = (zu[r * I + col] * S) * orc_h2f(ou[col]);
                        float gate = gm, up = um;
                        if (lim > 0) {
                            gate = isnan(gm) ? gm : (gm < lim ? gm : lim);
                            up = isnan(um) ? um : (um > -lim ? (um < lim ? um : lim) : -lim);
                        }
                        float yv = 1.0f / (1.0f + expf(fabsf(gate)));
                        float sg = gate < 0 ? yv : 1.0f - yv;
                        xd[r * I + col] = ((gate * sg) * up) * orc_h2f(rd[col]);
                    }
                    hadamard128_f32(xd + r * I + b);
                    for (size_t j = 0; j < 128; ++j) xd[r * I + b + j] *= S;
                }
            }
            exl3_gemm_fast((const int16_t *)(rec + g.off[6]), I, H, tablef, perm, xd, n, zd);
#pragma omp barrier
#pragma omp for schedule(static)
            for (size_t r = 0; r < n; ++r) {
                float *dst = ro + (size_t)order[offs[e] + r] * H;
                for (size_t b = 0; b < H; b += 128) {
                    hadamard128_f32(zd + r * H + b);
                    for (size_t j = 0; j < 128; ++j) dst[b + j] = (zd[r * H + b + j] * S) * orc_h2f(od[b + j]);
                }
            }
        }
        free(xg); free(xu); free(zg); free(zu); free(xd); free(zd);
    }
    /* shared expert (bf16 dense), f32 */
    float *sh = NULL;
    if (sh_w1) {
        sh = (float *)calloc(T * H, 4);
        float *hh = (float *)malloc(T * I * 4);
#pragma omp parallel for schedule(static)
        for (size_t i = 0; i < I; ++i)
            for (size_t t = 0; t < T; ++t) {
                float gg = 0, uu = 0;
                for (size_t j = 0; j < H; ++j) {
                    gg = fmaf(x[t * H + j], bf16_bits_f32(sh_w1[i * H + j]), gg);
                    uu = fmaf(x[t * H + j], bf16_bits_f32(sh_w3[i * H + j]), uu);
                }
                hh[t * I + i] = orc_bf16_round((float)orc_swiglu_clamped(gg, uu, c->limit));
            }
#pragma omp parallel for schedule(static)
        for (size_t o = 0; o < H; ++o)
            for (size_t t = 0; t < T; ++t) {
                float s = 0;
                for (size_t i = 0; i < I; ++i) s = fmaf(hh[t * I + i], bf16_bits_f32(sh_w2[o * I + i]), s);
                sh[t * H + o] = s;
            }
        free(hh);
    }
#pragma omp parallel for schedule(static)
    for (size_t t = 0; t < T; ++t)
        for (size_t j = 0; j < H; ++j) {
            float acc = 0;
            for (size_t q = 0; q < k; ++q) acc += ro[(t * k + q) * H + j] * weights[t * k + q];
            if (sh) acc += sh[t * H + j];
            y[t * H + j] = orc_bf16_round(acc);
        }
    free(sh); free(ro); free(order); free(offs); free(tablef);
    return 0;
}
