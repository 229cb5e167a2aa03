/* TEST INFRASTRUCTURE - not a product path. See btb_oracle.h.
 *
 * Build: gcc -O2 -ffp-contract=off -fopenmp -fPIC -shared (Makefile beside this file). -ffp-contract=off matters:
 * every fused multiply-add below is an explicit fmaf and nothing else may be contracted.
 */
#include "btb_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif
#if defined(__x86_64__)
#include <immintrin.h>
#endif

/* ------------------------------------------------------------------------------------------------------- */
/* scalar helpers                                                                                          */
/* ------------------------------------------------------------------------------------------------------- */

static inline float bits_f32(uint32_t b) {
    float f;
    memcpy(&f, &b, 4);
    return f;
}
static inline uint32_t f32_bits(float f) {
    uint32_t b;
    memcpy(&b, &f, 4);
    return b;
}
static inline float bf2f(uint16_t v) { return bits_f32((uint32_t)v << 16); }
/* round to nearest even as the card's __float2bfloat16_rn: a NaN becomes the canonical 0x7FFF */
static inline uint16_t f2bf(float f) {
    uint32_t b = f32_bits(f);
    if ((b & 0x7FFFFFFFu) > 0x7F800000u) return 0x7FFF;
    return (uint16_t)((b + 0x7FFFu + ((b >> 16) & 1u)) >> 16);
}
static inline float bfround(float f) { return bf2f(f2bf(f)); }

/* ------------------------------------------------------------------------------------------------------- */
/* widens                                                                                                  */
/* ------------------------------------------------------------------------------------------------------- */

static inline uint16_t p12_bits(const uint8_t* lo, const uint8_t* hi4, const uint8_t* table, size_t i) {
    const uint8_t byte = hi4[i >> 1];
    const uint8_t code = (i & 1) ? (uint8_t)(byte >> 4) : (uint8_t)(byte & 0x0F);
    return (uint16_t)(((uint16_t)table[code] << 8) | lo[i]);
}

static int p12_check(const int32_t* esc_idx, size_t n_esc, size_t n) {
    /* strictly ascending and in range, native/src/gemv.rs:4178-4193 */
    for (size_t k = 0; k < n_esc; ++k) {
        if (esc_idx[k] < 0 || (size_t)esc_idx[k] >= n) return BTB_ERR_DOMAIN;
        if (k && esc_idx[k] <= esc_idx[k - 1]) return BTB_ERR_DOMAIN;
    }
    return BTB_OK;
}

int orc_widen_p12(const uint8_t* lo, const uint8_t* hi4, const uint8_t* table, const int32_t* esc_idx,
                  const uint8_t* esc_val, size_t n_esc, size_t n, uint16_t* out) {
    if (!lo || !hi4 || !table || !out || (n_esc && (!esc_idx || !esc_val))) return BTB_ERR_NULL;
    int rc = p12_check(esc_idx, n_esc, n);
    if (rc) return rc;
    for (size_t i = 0; i < n; ++i) out[i] = p12_bits(lo, hi4, table, i);
    for (size_t k = 0; k < n_esc; ++k) {
        const size_t i = (size_t)esc_idx[k];
        out[i] = (uint16_t)(((uint16_t)esc_val[k] << 8) | lo[i]);
    }
    return BTB_OK;
}

static const float FP4[16] = {0.0f,  0.5f,  1.0f,  1.5f,  2.0f,  3.0f,  4.0f,  6.0f,
                              -0.0f, -0.5f, -1.0f, -1.5f, -2.0f, -3.0f, -4.0f, -6.0f};

static inline float mx_scale(uint8_t s) {
    const float f = bits_f32((uint32_t)(s == 0 ? 1 : s) << 23);
    return s == 0 ? f * 0.5f : f;
}

int orc_widen_mxfp4(const uint8_t* blocks, const uint8_t* scales, size_t rows, size_t cols, float* out) {
    if (!blocks || !scales || !out) return BTB_ERR_NULL;
    if (!rows || !cols || cols % 32) return BTB_ERR_DOMAIN;
    const size_t g = cols / 32;
    for (size_t r = 0; r < rows; ++r)
        for (size_t b = 0; b < g; ++b) {
            const float sc = mx_scale(scales[r * g + b]);
            const uint8_t* blk = blocks + (r * g + b) * 16;
            float* o = out + r * cols + b * 32;
            for (int j = 0; j < 16; ++j) {
                o[2 * j] = FP4[blk[j] & 15] * sc;
                o[2 * j + 1] = FP4[blk[j] >> 4] * sc;
            }
        }
    return BTB_OK;
}

static inline float f8_value(uint8_t b) {
    const uint32_t a = b & 0x7Fu;
    float mag;
    if (a == 0x7F)
        mag = NAN;
    else if (a < 8)
        mag = (float)a * (1.0f / 512.0f);
    else
        mag = bits_f32((a << 20) + (120u << 23));
    return bits_f32(f32_bits(mag) | ((uint32_t)(b & 0x80u) << 24));
}
/* the reference's integer rounding (a quiet NaN stays one), native/src/gemv.rs:3004-3008 */
static inline float round_bf16_int(float f) {
    const uint32_t b = f32_bits(f);
    return bits_f32((b + 0x7FFFu + ((b >> 16) & 1u)) & 0xFFFF0000u);
}

int orc_widen_fp8(const uint8_t* w, const float* scales, size_t rows, size_t cols, size_t sr, size_t sc,
                  uint16_t* out) {
    if (!w || !scales || !out) return BTB_ERR_NULL;
    if (!rows || !cols || !sr || !sc || rows % sr || cols % sc) return BTB_ERR_DOMAIN;
    const size_t bm = rows / sr, bn = cols / sc;
    for (size_t r = 0; r < rows; ++r)
        for (size_t c = 0; c < cols; ++c) {
            const float v = round_bf16_int(f8_value(w[r * cols + c]) * scales[(r / bm) * sc + c / bn]);
            out[r * cols + c] = (uint16_t)(f32_bits(v) >> 16);
        }
    return BTB_OK;
}

/* ------------------------------------------------------------------------------------------------------- */
/* card-order GEMV                                                                                         */
/* ------------------------------------------------------------------------------------------------------- */

/* the 32 lane chains of one (m, r), then the butterfly xor 16, 8, 4, 2, 1; lane 0's value.
 * wrow: the row's C weights as f32 (already widened); xrow: the vector's C values as f32. */
static float card_row(const float* wrow, const float* xrow, int C) {
    float acc[32];
    const int nchunk = C >> 3;
    for (int l = 0; l < 32; ++l) {
        float a = 0.f;
        for (int c = l; c < nchunk; c += 32)
            for (int e = 0; e < 8; ++e) a = fmaf(wrow[8 * c + e], xrow[8 * c + e], a);
        acc[l] = a;
    }
    for (int off = 16; off > 0; off >>= 1) {
        float nx[32];
        for (int l = 0; l < 32; ++l) nx[l] = acc[l] + acc[l ^ off];
        memcpy(acc, nx, sizeof acc);
    }
    return acc[0];
}

static int card_gemv_f32w(const float* wf, const float* xf, uint16_t* y, int M, int R, int C) {
#pragma omp parallel for schedule(static)
    for (int r = 0; r < R; ++r)
        for (int m = 0; m < M; ++m) y[(size_t)m * R + r] = f2bf(card_row(wf + (size_t)r * C, xf + (size_t)m * C, C));
    return BTB_OK;
}

static float* widen_bf16_vec(const uint16_t* v, size_t n) {
    float* f = (float*)malloc(n * sizeof(float) + 64);
    if (f)
        for (size_t i = 0; i < n; ++i) f[i] = bf2f(v[i]);
    return f;
}

static int card_args(const void* a, const void* b, const void* c, int M, int R, int C) {
    if (!a || !b || !c) return BTB_ERR_NULL;
    if (M <= 0 || R <= 0 || C <= 0 || (C & 7)) return BTB_ERR_DOMAIN;
    return BTB_OK;
}

int orc_gemv_card_bf16(const uint16_t* w, const uint16_t* x, uint16_t* y, int M, int R, int C) {
    int rc = card_args(w, x, y, M, R, C);
    if (rc) return rc;
    float* xf = widen_bf16_vec(x, (size_t)M * C);
#pragma omp parallel
    {
        float* wf = (float*)malloc((size_t)C * sizeof(float));
#pragma omp for schedule(static)
        for (int r = 0; r < R; ++r) {
            for (int c = 0; c < C; ++c) wf[c] = bf2f(w[(size_t)r * C + c]);
            for (int m = 0; m < M; ++m) y[(size_t)m * R + r] = f2bf(card_row(wf, xf + (size_t)m * C, C));
        }
        free(wf);
    }
    free(xf);
    return BTB_OK;
}

static inline float act_silu(float g) { return g / (1.f + expf(-g)); }

int orc_silu_mul(const uint16_t* gu, uint16_t* m, int T, int I) {
    if (!gu || !m) return BTB_ERR_NULL;
    for (int t = 0; t < T; ++t)
        for (int i = 0; i < I; ++i) {
            const float g = bf2f(gu[(size_t)t * 2 * I + i]);
            const float u = bf2f(gu[(size_t)t * 2 * I + I + i]);
            m[(size_t)t * I + i] = f2bf(bfround(act_silu(g)) * u);
        }
    return BTB_OK;
}

int orc_gemv_card_silu_bf16(const uint16_t* w, const uint16_t* gu, uint16_t* y, int M, int R, int C) {
    int rc = card_args(w, gu, y, M, R, C);
    if (rc) return rc;
    uint16_t* xm = (uint16_t*)malloc((size_t)M * C * 2);
    orc_silu_mul(gu, xm, M, C);
    rc = orc_gemv_card_bf16(w, xm, y, M, R, C);
    free(xm);
    return rc;
}

int orc_gemv_card_p12(const uint8_t* lo, const uint8_t* hi4, const uint8_t* table, const int32_t* esc_idx,
                      const uint8_t* esc_val, size_t n_esc, const uint16_t* x, uint16_t* y, int M, int R, int C) {
    int rc = card_args(lo, x, y, M, R, C);
    if (rc) return rc;
    const size_t n = (size_t)R * C;
    uint16_t* wb = (uint16_t*)malloc(n * 2);
    rc = orc_widen_p12(lo, hi4, table, esc_idx, esc_val, n_esc, n, wb);
    if (!rc) rc = orc_gemv_card_bf16(wb, x, y, M, R, C);
    free(wb);
    return rc;
}

int orc_gemv_card_fp8(const uint8_t* w, const float* scales, int sr, int sc, const uint16_t* x, uint16_t* y, int M,
                      int R, int C) {
    int rc = card_args(w, x, y, M, R, C);
    if (rc) return rc;
    uint16_t* wb = (uint16_t*)malloc((size_t)R * C * 2);
    rc = orc_widen_fp8(w, scales, (size_t)R, (size_t)C, (size_t)sr, (size_t)sc, wb);
    if (!rc) rc = orc_gemv_card_bf16(wb, x, y, M, R, C);
    free(wb);
    return rc;
}

int orc_gemv_card_mxfp4(const uint8_t* blocks, const uint8_t* scales, const uint16_t* x, uint16_t* y, int M, int R,
                        int C) {
    int rc = card_args(blocks, x, y, M, R, C);
    if (rc) return rc;
    if (!scales) return BTB_ERR_NULL;
    float* wf = (float*)malloc((size_t)R * C * sizeof(float));
    float* xf = widen_bf16_vec(x, (size_t)M * C);
    rc = orc_widen_mxfp4(blocks, scales, (size_t)R, (size_t)C, wf);
    if (!rc) rc = card_gemv_f32w(wf, xf, y, M, R, C);
    free(wf);
    free(xf);
    return rc;
}

/* ------------------------------------------------------------------------------------------------------- */
/* residual + RMSNorm, norm + rope + cache write                                                           */
/* ------------------------------------------------------------------------------------------------------- */

int orc_add_rmsnorm(uint16_t* h, const uint16_t* y, const uint16_t* w, float eps, uint16_t* x, int T, int H,
                    int centered) {
    if (!h || !w || !x) return BTB_ERR_NULL;
    for (int t = 0; t < T; ++t) {
        uint16_t* hr = h + (size_t)t * H;
        const uint16_t* yr = y ? y + (size_t)t * H : NULL;
        float red[256];
        for (int tid = 0; tid < 256; ++tid) {
            float ss = 0.f;
            for (int i = tid; i < H; i += 256) {
                float hv = bf2f(hr[i]);
                if (yr) {
                    hv = bfround(hv + bf2f(yr[i]));
                    hr[i] = f2bf(hv);
                }
                ss = fmaf(hv, hv, ss);
            }
            red[tid] = ss;
        }
        for (int s = 128; s > 0; s >>= 1)
            for (int tid = 0; tid < s; ++tid) red[tid] += red[tid + s];
        const float rstd = 1.0f / sqrtf(red[0] / (float)H + eps);
        for (int i = 0; i < H; ++i) {
            const float wv = bf2f(w[i]);
            x[(size_t)t * H + i] = f2bf(bf2f(hr[i]) * rstd * (centered ? 1.f + wv : wv));
        }
    }
    return BTB_OK;
}

int orc_norm_rope_kv(const uint16_t* qkv, const uint16_t* wq, const uint16_t* wk, float eps, const uint16_t* cos_t,
                     const uint16_t* sin_t, int n0, const int32_t* depth, uint16_t* K, uint16_t* V, uint16_t* qo,
                     int T, int Hq, int Hk, int D, long hs, long rs, int centered, const int32_t* tbl) {
    if (!qkv || !cos_t || !sin_t || !depth || !K || !V || !qo) return BTB_ERR_NULL;
    if (D % 32 || D > 256) return BTB_ERR_DOMAIN;
    const int E = D / 32;
    const size_t width = (size_t)(Hq + 2 * Hk) * D;
    for (int t = 0; t < T; ++t) {
        int slot = n0 + t;
        const int pos = n0 + depth[t];
        if (tbl) slot = tbl[slot];
        for (int head = 0; head < Hq + 2 * Hk; ++head) {
            const uint16_t* src = qkv + (size_t)t * width + (size_t)head * D;
            if (head >= Hq + Hk) {
                uint16_t* dst = V + (size_t)(head - Hq - Hk) * hs + (size_t)slot * rs;
                memcpy(dst, src, (size_t)D * 2);
                continue;
            }
            const int is_q = head < Hq;
            const uint16_t* wn = is_q ? wq : wk;
            float v[256];
            for (int d = 0; d < D; ++d) v[d] = bf2f(src[d]);
            if (wn) {
                /* lane l holds dims l*E .. l*E+E-1: its own chain, then the butterfly */
                float acc[32];
                for (int l = 0; l < 32; ++l) {
                    float ss = 0.f;
                    for (int e = 0; e < E; ++e) ss = fmaf(v[l * E + e], v[l * E + e], ss);
                    acc[l] = ss;
                }
                for (int off = 16; off > 0; off >>= 1) {
                    float nx[32];
                    for (int l = 0; l < 32; ++l) nx[l] = acc[l] + acc[l ^ off];
                    memcpy(acc, nx, sizeof acc);
                }
                const float rstd = 1.0f / sqrtf(acc[0] / (float)D + eps);
                for (int d = 0; d < D; ++d) {
                    const float wv = bf2f(wn[d]);
                    v[d] = bfround(v[d] * rstd * (centered ? 1.f + wv : wv));
                }
            }
            uint16_t* dst = is_q ? qo + ((size_t)t * Hq + head) * D : K + (size_t)(head - Hq) * hs + (size_t)slot * rs;
            for (int d = 0; d < D; ++d) {
                /* rotate_half: the partner is the dim half a head away (lane ^ 16, same element) */
                const int pd = d < D / 2 ? d + D / 2 : d - D / 2;
                const float sgn = d < D / 2 ? -1.f : 1.f;
                const float qc = bfround(v[d] * bf2f(cos_t[(size_t)pos * D + d]));
                dst[d] = f2bf(fmaf(sgn * v[pd], bf2f(sin_t[(size_t)pos * D + d]), qc));
            }
        }
    }
    return BTB_OK;
}

/* ------------------------------------------------------------------------------------------------------- */
/* decode attention: tile -> group -> row folds                                                            */
/* ------------------------------------------------------------------------------------------------------- */

#define ATT_BN 64
#define ATT_GT 8
#define NEG_INF (-INFINITY)

static void fold_ml(float* M, float* L, float m, float l, float* cO, float* co) {
    const int em = m == NEG_INF, eM = *M == NEG_INF;
    const float hi = fmaxf(*M, m), lo = fminf(*M, m);
    const float e = exp2f(em || eM ? 0.f : lo - hi);
    *cO = em ? 1.f : eM ? 0.f : (*M >= m ? 1.f : e);
    *co = em ? 0.f : eM ? 1.f : (*M > m ? e : 1.f);
    *L = fmaf(l, *co, *L * *cO);
    *M = hi;
}

int orc_attn_decode(const uint16_t* q, const uint16_t* K, const uint16_t* V, uint16_t* out, int n0,
                    const int32_t* par, int T, int Hq, int Hk, int D, long hs, long rs, float scale, int win,
                    const int32_t* tbl, const float* sinks) {
    if (!q || !K || !V || !out || !par) return BTB_ERR_NULL;
    if (T <= 0 || T > 32 || Hk <= 0 || Hq % Hk || D > 256) return BTB_ERR_DOMAIN;
    const int G = Hq / Hk;
    const float scale2 = scale * 1.4426950408889634f;
    for (int t = 0; t < T; ++t) {
        /* the token's path, root first */
        int anc[32], len = 0;
        for (int p = t; p >= 0 && p < T && len < 32; p = par[p]) ++len;
        {
            int k = len;
            for (int p = t; k > 0; p = par[p]) anc[--k] = p;
        }
        const int last = n0 + len - 1;
        const int first = win > 0 ? (last + 1 - win > 0 ? last + 1 - win : 0) : 0;
        for (int hq = 0; hq < Hq; ++hq) {
            const int g = hq / G;
            const uint16_t* qr = q + ((size_t)t * Hq + hq) * D;
            float qf[256];
            for (int d = 0; d < D; ++d) qf[d] = bf2f(qr[d]);
            float RM = NEG_INF, RL = 0.f, RO[256];
            for (int d = 0; d < D; ++d) RO[d] = 0.f;
            const int gk = ATT_BN * ATT_GT;
            for (int grp = first / gk; grp <= last / gk; ++grp) {
                float GM = NEG_INF, GL = 0.f, GO[256];
                for (int d = 0; d < D; ++d) GO[d] = 0.f;
                for (int tile = 0; tile < ATT_GT; ++tile) {
                    const int j0 = grp * gk + tile * ATT_BN;
                    if (j0 > last || j0 + ATT_BN - 1 < first) continue;
                    float s[ATT_BN], m = NEG_INF;
                    const uint16_t* vrow[ATT_BN];
                    for (int i = 0; i < ATT_BN; ++i) {
                        const int j = j0 + i;
                        s[i] = NEG_INF;
                        vrow[i] = NULL;
                        if (j < first || j > last) continue;
                        int sl = j < n0 ? j : n0 + anc[j - n0];
                        if (tbl) sl = tbl[sl];
                        const uint16_t* kr = K + (size_t)g * hs + (size_t)sl * rs;
                        vrow[i] = V + (size_t)g * hs + (size_t)sl * rs;
                        float a = 0.f;
                        for (int d = 0; d < D; ++d) a = fmaf(bf2f(kr[d]), qf[d], a);
                        s[i] = a * scale2;
                        m = fmaxf(m, s[i]);
                    }
                    float l = 0.f, o[256];
                    for (int d = 0; d < D; ++d) o[d] = 0.f;
                    for (int i = 0; i < ATT_BN; ++i) {
                        if (!vrow[i]) continue;
                        const float p = exp2f(s[i] - m);
                        l += p;
                        const float pb = bfround(p);
                        for (int d = 0; d < D; ++d) o[d] = fmaf(pb, bf2f(vrow[i][d]), o[d]);
                    }
                    float cO, co;
                    fold_ml(&GM, &GL, m, l, &cO, &co);
                    for (int d = 0; d < D; ++d) GO[d] = fmaf(o[d], co, GO[d] * cO);
                }
                float cO, co;
                fold_ml(&RM, &RL, GM, GL, &cO, &co);
                for (int d = 0; d < D; ++d) RO[d] = fmaf(GO[d], co, RO[d] * cO);
            }
            if (sinks) {
                /* one more logit in the denominator, no value: the sink in log2 units */
                float cO, co;
                fold_ml(&RM, &RL, sinks[hq] * 1.4426950408889634f, 1.f, &cO, &co);
                for (int d = 0; d < D; ++d) RO[d] = RO[d] * cO;
            }
            const float inv = 1.f / RL;
            for (int d = 0; d < D; ++d) out[((size_t)t * Hq + hq) * D + d] = f2bf(RO[d] * inv);
        }
    }
    return BTB_OK;
}

/* ------------------------------------------------------------------------------------------------------- */
/* router, argmax                                                                                          */
/* ------------------------------------------------------------------------------------------------------- */

int orc_moe_route(const void* logits, int ls, int E, int k, int mode, int f32_logits, int32_t* idx, uint16_t* w,
                  int T) {
    if (!logits || !idx || !w) return BTB_ERR_NULL;
    if (E <= 0 || k <= 0 || k > E || k > 32 || E > 4096) return BTB_ERR_DOMAIN;
    float* pr = (float*)malloc((size_t)E * sizeof(float));
    float* lg = (float*)malloc((size_t)E * sizeof(float));
    for (int t = 0; t < T; ++t) {
        for (int e = 0; e < E; ++e)
            lg[e] = f32_logits ? ((const float*)logits)[(size_t)t * ls + e] : bf2f(((const uint16_t*)logits)[(size_t)t * ls + e]);
        float topv[32];
        int topi[32];
        if (mode == 0) {
            float m = NEG_INF;
            for (int e = 0; e < E; ++e) m = fmaxf(m, lg[e]);
            /* thread tid of 256 sums its strided elements, then the 256 -> 1 tree */
            float red[256];
            for (int tid = 0; tid < 256; ++tid) {
                float s = 0.f;
                for (int e = tid; e < E; e += 256) {
                    const float p = expf(lg[e] - m);
                    pr[e] = p;
                    s += p;
                }
                red[tid] = s;
            }
            for (int s = 128; s > 0; s >>= 1)
                for (int tid = 0; tid < s; ++tid) red[tid] += red[tid + s];
            for (int e = 0; e < E; ++e) pr[e] = pr[e] / red[0];
        } else {
            for (int e = 0; e < E; ++e) pr[e] = lg[e];
        }
        /* k rounds of the total order's maximum (value desc, index asc); a picked one leaves the field */
        unsigned char taken[4096];
        memset(taken, 0, (size_t)E);
        for (int j = 0; j < k; ++j) {
            int bi = -1;
            for (int e = 0; e < E; ++e) {
                if (taken[e]) continue;
                if (bi < 0 || pr[e] > pr[bi]) bi = e;
            }
            taken[bi] = 1;
            topi[j] = bi;
            topv[j] = pr[bi];
        }
        if (mode == 0) {
            float sum = 0.f;
            for (int j = 0; j < k; ++j) sum += topv[j];
            for (int j = 0; j < k; ++j) {
                idx[(size_t)t * k + j] = topi[j];
                w[(size_t)t * k + j] = f2bf(topv[j] / sum);
            }
        } else {
            /* softmax over the k picked logits in f32 (max, exp, sum in rank order), then the hidden dtype */
            float m = topv[0], sum = 0.f, ex[32];
            for (int j = 1; j < k; ++j) m = fmaxf(m, topv[j]);
            for (int j = 0; j < k; ++j) {
                ex[j] = expf(topv[j] - m);
                sum += ex[j];
            }
            for (int j = 0; j < k; ++j) {
                idx[(size_t)t * k + j] = topi[j];
                w[(size_t)t * k + j] = f2bf(ex[j] / sum);
            }
        }
    }
    free(pr);
    free(lg);
    return BTB_OK;
}

int orc_argmax_bf16(const uint16_t* logits, int T, int V, int64_t* out) {
    if (!logits || !out) return BTB_ERR_NULL;
    for (int t = 0; t < T; ++t) {
        const uint16_t* r = logits + (size_t)t * V;
        int best = 0;
        float bv = bf2f(r[0]);
        for (int i = 1; i < V; ++i) {
            const float v = bf2f(r[i]);
            if (v > bv || (isnan(bv) && !isnan(v))) {
                bv = v;
                best = i;
            }
        }
        out[t] = best;
    }
    return BTB_OK;
}

/* ---- the sampled pick: native/src/sample.rs:17-155,255-384 (and native/cuda/btb_kernels.cu:1865-2124) ---------- */

static uint32_t smp_ordered(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
/* exp(t), t <= 0: t = n ln2 + r, e^r a degree-7 series, 0 below -87; each operation rounded on its own */
static float smp_exp(float t) {
    if (t < -87.0f) return 0.0f;
    const float n = roundf(t * 1.4426950408889634f);
    const float r = t - n * 0.69314575f - n * 1.4286068e-6f;
    const float p = 1.0f + r * (1.0f + r * (0.5f + r * (0.16666667f + r * (0.041666668f + r * (0.008333334f +
                    r * (0.001388889f + r * 0.0001984127f))))));
    int e = (int)n + 127;
    e = e < 1 ? 1 : (e > 254 ? 254 : e);
    const uint32_t eb = (uint32_t)e << 23;
    float sc;
    memcpy(&sc, &eb, 4);
    return sc * p;
}
float orc_sample_uniform(uint64_t key, uint32_t i) {
    uint64_t h = key ^ ((uint64_t)i * 0x9E3779B97F4A7C15ull);
    h ^= h >> 32;
    h *= 0xBF58476D1CE4E5B9ull;
    h ^= h >> 29;
    h *= 0x94D049BB133111EBull;
    h ^= h >> 32;
    return ((float)(uint32_t)(h >> 41) + 0.5f) * (1.0f / 8388608.0f);
}
static uint64_t smp_mix_step(uint64_t x, uint64_t p) {
    x = (x ^ p) + 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    x ^= x >> 31;
    return x;
}
uint64_t orc_sample_key(uint64_t seed, uint64_t pos, uint32_t salt) {
    uint64_t x = smp_mix_step(smp_mix_step(0ull, seed), pos);
    if (salt) x = smp_mix_step(x, salt);
    return x & 0x7FFFFFFFFFFFFFFFull;
}
float orc_sample_exp(float t) { return smp_exp(t); }

static uint64_t smp_mass(float a, float m, uint32_t floor) {
    return (smp_ordered(a) >= floor && a - m >= -21.0f) ? (uint64_t)(smp_exp(a - m) * 1073741824.0f) : 0;
}
/* the threshold at which the count (w == NULL) or the mass of tokens with u' >= u first reaches the target, by three
 * radix levels of 11 + 11 + 10 bits over the tokens with u' >= floor */
static uint32_t smp_select(const float* s, const uint64_t* w, int V, uint64_t need, float top_p, uint32_t floor) {
    uint32_t prefix = 0, shift = 32;
    uint64_t* bin = (uint64_t*)malloc(2048 * sizeof(uint64_t));
    for (int level = 0; level < 3; ++level) {
        const uint32_t bits = level < 2 ? 11 : 10;
        shift -= bits;
        const uint32_t hi = shift + bits;
        memset(bin, 0, 2048 * sizeof(uint64_t));
        for (int i = 0; i < V; ++i) {
            const uint32_t u = smp_ordered(s[i]);
            if (u >= floor && (hi >= 32 || (u >> hi) == (prefix >> hi))) bin[(u >> shift) & 2047] += w ? w[i] : 1;
        }
        if (level == 0 && w) {
            uint64_t z = 0;
            for (int b = 0; b < 2048; ++b) z += bin[b];
            need = (uint64_t)((float)z * top_p);
            if (!need) need = 1; /* at least the top token */
        }
        uint64_t acc = 0;
        uint32_t pick = 0;
        for (int b = 2047; b >= 0; --b) {
            acc += bin[b];
            if (acc >= need) {
                pick = (uint32_t)b;
                need -= acc - bin[b];
                break;
            }
        }
        prefix |= pick << shift;
    }
    free(bin);
    return prefix;
}

/* x [R, V] f32 logits, keys [R]; out [R] tokens; floors [R, 2] (may be null) the top-k and top-p thresholds as ordered
 * bits; margin [R] (may be null) the winner's lead over the runner-up in the Gumbel race */
int orc_sample_pick(const float* x, int R, int V, const uint64_t* keys, float inv_t, uint32_t top_k, float top_p,
                    uint32_t* out, uint32_t* floors, float* margin) {
    if (!x || !keys || !out) return BTB_ERR_NULL;
    if (R <= 0 || V <= 0 || !(inv_t > 0.0f)) return BTB_ERR_DOMAIN;
    float* s = (float*)malloc((size_t)V * sizeof(float));
    uint64_t* w = (uint64_t*)malloc((size_t)V * sizeof(uint64_t));
    for (int r = 0; r < R; ++r) {
        const float* row = x + (size_t)r * V;
        float m = -INFINITY;
        for (int i = 0; i < V; ++i) {
            s[i] = row[i] * inv_t;
            m = fmaxf(m, s[i]);
        }
        uint32_t fk = 0, fp = 0;
        if (top_k > 0) fk = smp_select(s, NULL, V, top_k, 0.0f, 0);
        if (top_p < 1.0f) {
            for (int i = 0; i < V; ++i) w[i] = smp_mass(s[i], m, fk);
            fp = smp_select(s, w, V, 0, top_p, fk);
        }
        const uint32_t floor = fk > fp ? fk : fp;
        float best = -INFINITY, second = -INFINITY;
        uint32_t bi = 0;
        for (int i = 0; i < V; ++i) {
            if (smp_ordered(s[i]) < floor || !(s[i] - m >= -21.0f)) continue;
            const float v = s[i] - logf(-logf(orc_sample_uniform(keys[r], (uint32_t)i)));
            if (v > best) {
                second = best;
                best = v;
                bi = (uint32_t)i;
            } else if (v > second) {
                second = v;
            }
        }
        out[r] = bi;
        if (floors) floors[2 * r] = fk, floors[2 * r + 1] = fp;
        if (margin) margin[r] = best - second;
    }
    free(s);
    free(w);
    return BTB_OK;
}

/* ---- the verify pass's pick: native/cuda/btb_kernels.cu:2126-2359 (btb_sample_verify), btb/sampling.py:272-372 ----
 * A row is a tree node with up to 32 drafted children in draw order. hasq 0: the node draws from the target, the child
 * equal to the draw is accepted. hasq 1: child i accepted when u_i * q_i(c) < p_i(c), p_{i+1} = norm(max(0, p_i - q_i));
 * none accepted, a draw from the last residual. The kernel's float sums run as one block of 1024 threads: thread t adds
 * tokens t, t + 1024, ... in order, a warp folds by strides 16, 8, 4, 2, 1, the 32 warps' sums are added in order.
 * That order is restated here so the two agree to the bit. */
#define VRF_THREADS 1024
static float vrf_block_sum(const float* part) {
    float warp[VRF_THREADS / 32];
    for (int w = 0; w < VRF_THREADS / 32; ++w) {
        float v[32], t[32];
        memcpy(v, part + 32 * w, sizeof v);
        for (int o = 16; o > 0; o >>= 1) {
            for (int l = 0; l < 32; ++l) t[l] = v[l] + v[l ^ o];
            memcpy(v, t, sizeof v);
        }
        warp[w] = v[0];
    }
    float z = 0.0f;
    for (int w = 0; w < VRF_THREADS / 32; ++w) z += warp[w];
    return z;
}
static float vrf_left(const float* s, const float* qrow, const int* kid, int x, int k, float m, uint32_t floor, int Vd,
                      const float* zp, const float* zq) {
    float w = smp_ordered(s[x]) >= floor ? smp_exp(s[x] - m) : 0.0f;
    float qx = x < Vd ? qrow[x] : 0.0f;
    for (int j = 0; j < k; ++j) {
        const float a = w / zp[j], b = qx / zq[j];
        w = fmaxf(0.0f, a - b);
        if (kid[j] == x) qx = 0.0f;
    }
    return w;
}
/* x [R, V] f32 logits, q [R, Vd], kids [R, C] (-1 after the last), hasq [R], keys [R]; out [R] packed
 * (accepted slot + 1) << 24 | token */
int orc_sample_verify(const float* x, int R, int V, const float* q, int Vd, const int32_t* kids, int C,
                      const uint32_t* hasq, const uint64_t* keys, float inv_t, uint32_t top_k, float top_p,
                      uint32_t* out) {
    if (!x || !hasq || !keys || !out || (Vd > 0 && !q) || (C > 0 && !kids)) return BTB_ERR_NULL;
    if (R <= 0 || V <= 0 || C < 0 || C > 32 || !(inv_t > 0.0f)) return BTB_ERR_DOMAIN;
    float* s = (float*)malloc((size_t)V * sizeof(float));
    uint64_t* w = (uint64_t*)malloc((size_t)V * sizeof(uint64_t));
    float part[VRF_THREADS];
    for (int r = 0; r < R; ++r) {
        const float* row = x + (size_t)r * V;
        const float* qrow = q + (size_t)r * Vd;
        int kid[32];
        for (int c = 0; c < 32; ++c) kid[c] = c < C ? kids[(size_t)r * C + c] : -1;
        float m = -INFINITY;
        for (int i = 0; i < V; ++i) {
            s[i] = row[i] * inv_t;
            m = fmaxf(m, s[i]);
        }
        uint32_t fk = 0, fp = 0;
        if (top_k > 0) fk = smp_select(s, NULL, V, top_k, 0.0f, 0);
        if (top_p < 1.0f) {
            for (int i = 0; i < V; ++i) w[i] = smp_mass(s[i], m, fk);
            fp = smp_select(s, w, V, 0, top_p, fk);
        }
        const uint32_t floor = fk > fp ? fk : fp;
        const uint64_t key = keys[r];
        if (!hasq[r]) {
            float best = -INFINITY;
            uint32_t bi = 0;
            for (int i = 0; i < V; ++i) {
                if (smp_ordered(s[i]) < floor || !(s[i] - m >= -21.0f)) continue;
                const float v = s[i] - logf(-logf(orc_sample_uniform(key, (uint32_t)i)));
                if (v > best) best = v, bi = (uint32_t)i;
            }
            uint32_t slot = 0;
            for (int c = 0; c < C; ++c)
                if (kid[c] >= 0 && (uint32_t)kid[c] == bi) {
                    slot = (uint32_t)c + 1;
                    break;
                }
            out[r] = (slot << 24) | bi;
            continue;
        }
        float zp[33], zq[33];
        memset(part, 0, sizeof part);
        for (int i = 0; i < V; ++i)
            if (smp_ordered(s[i]) >= floor) part[i % VRF_THREADS] += smp_exp(s[i] - m);
        zp[0] = vrf_block_sum(part);
        memset(part, 0, sizeof part);
        for (int i = 0; i < Vd; ++i) part[i % VRF_THREADS] += qrow[i];
        zq[0] = vrf_block_sum(part);
        int tried = 0;
        uint32_t accepted = 0, token = 0;
        for (int i = 0; i < C; ++i) {
            const int c = kid[i];
            if (c < 0) break;
            const float qc = (c < Vd && zq[i] > 0.0f) ? fminf(qrow[c] / zq[i], 1.0f) : 0.0f;
            if (!(qc > 0.0f)) break;
            const float pc = vrf_left(s, qrow, kid, c, i, m, floor, Vd, zp, zq) / zp[i];
            const float u = orc_sample_uniform(key, 0xF00000u + (uint32_t)i);
            if (u * qc < pc) {
                accepted = (uint32_t)i + 1, token = (uint32_t)c;
                break;
            }
            memset(part, 0, sizeof part);
            for (int t = 0; t < V; ++t) part[t % VRF_THREADS] += vrf_left(s, qrow, kid, t, i + 1, m, floor, Vd, zp, zq);
            const float z = vrf_block_sum(part);
            zp[i + 1] = z;
            zq[i + 1] = zq[i] - qrow[c];
            if (!(z > 0.0f)) {
                accepted = (uint32_t)i + 1, token = (uint32_t)c;
                break;
            }
            tried = i + 1;
        }
        if (accepted) {
            out[r] = (accepted << 24) | token;
            continue;
        }
        float best = -INFINITY;
        uint32_t bi = 0;
        for (int t = 0; t < V; ++t) {
            const float wl = vrf_left(s, qrow, kid, t, tried, m, floor, Vd, zp, zq);
            if (!(wl > 0.0f)) continue;
            const float v = logf(wl) + -logf(-logf(orc_sample_uniform(key, (uint32_t)t)));
            if (v > best) best = v, bi = (uint32_t)t;
        }
        out[r] = bi;
    }
    free(s);
    free(w);
    return BTB_OK;
}

/* ------------------------------------------------------------------------------------------------------- */
/* CPU tier: 16-lane GEMV over bf16 / pack12 / MXFP4 / FP8                                                 */
/* ------------------------------------------------------------------------------------------------------- */

static int g_force_scalar = 0;
void orc_force_scalar(int on) { g_force_scalar = on; }

static int have_avx512(void) {
#if defined(__x86_64__)
    static int cached = -1;
    if (cached < 0) cached = __builtin_cpu_supports("avx512f") && __builtin_cpu_supports("avx512bw");
    return cached && !g_force_scalar;
#else
    return 0;
#endif
}

const char* btb_isa(void) { return have_avx512() ? "avx512" : "scalar"; }

/* native/src/gemv.rs:46-58 */
static inline float reduce16(const float* a) {
    float t[8];
    for (int j = 0; j < 8; ++j) t[j] = a[2 * j] + a[2 * j + 1];
    const float u0 = t[0] + t[1], u1 = t[2] + t[3], u2 = t[4] + t[5], u3 = t[6] + t[7];
    const float v0 = u0 + u1, v1 = u2 + u3;
    return v0 + v1;
}

#define COL_TILE 512
#define ROW_UNROLL 4

enum { W_BF16, W_P12, W_MX4, W_FP8 };
typedef struct {
    int kind;
    size_t rows, cols;
    const uint16_t* bf;
    const uint8_t *lo, *hi4, *table, *esc_val;
    const int32_t* esc_idx;
    size_t n_esc;
    const uint8_t *blocks, *mscales;
    const uint8_t* f8;
    const float* fscales;
    size_t sc, bm, bn;
} Wt;

#if defined(__x86_64__)
__attribute__((target("avx512f,avx512bw"))) static size_t widen_bf16_avx512(const uint16_t* p, size_t n, float* dst) {
    size_t j = 0;
    for (; j + 16 <= n; j += 16) {
        __m512i v = _mm512_cvtepu16_epi32(_mm256_loadu_si256((const __m256i*)(p + j)));
        _mm512_storeu_ps(dst + j, _mm512_castsi512_ps(_mm512_slli_epi32(v, 16)));
    }
    return j;
}
__attribute__((target("avx512f,avx512bw"))) static void accum_tile_avx512(float* acc, const float* wide, size_t R,
                                                                        const float* x, size_t nb) {
    __m512 a[4];
    for (size_t r = 0; r < R; ++r) a[r] = _mm512_loadu_ps(acc + r * 16);
    for (size_t k = 0; k < nb; ++k) {
        const __m512 xv = _mm512_loadu_ps(x + k * 16);
        for (size_t r = 0; r < R; ++r) a[r] = _mm512_fmadd_ps(_mm512_loadu_ps(wide + r * 512 + k * 16), xv, a[r]);
    }
    for (size_t r = 0; r < R; ++r) _mm512_storeu_ps(acc + r * 16, a[r]);
}
#endif

/* columns [c0, c0+n) of row r as f32 into dst */
static void widen_tile(const Wt* w, size_t r, size_t c0, size_t n, float* dst) {
    switch (w->kind) {
    case W_BF16: {
        const uint16_t* p = w->bf + r * w->cols + c0;
        size_t j = 0;
#if defined(__x86_64__)
        if (have_avx512()) j = widen_bf16_avx512(p, n, dst);
#endif
        for (; j < n; ++j) dst[j] = bf2f(p[j]);
        break;
    }
    case W_P12: {
        const size_t s = r * w->cols + c0;
        for (size_t j = 0; j < n; ++j) dst[j] = bf2f(p12_bits(w->lo, w->hi4, w->table, s + j));
        if (w->n_esc) {
            /* the first escape at or past the tile's start (binary search), then the tile's run of them */
            size_t a = 0, b = w->n_esc;
            while (a < b) {
                const size_t mid = (a + b) / 2;
                if ((size_t)w->esc_idx[mid] < s) a = mid + 1;
                else b = mid;
            }
            for (size_t k = a; k < w->n_esc && (size_t)w->esc_idx[k] < s + n; ++k) {
                const size_t i = (size_t)w->esc_idx[k];
                dst[i - s] = bits_f32(((uint32_t)w->esc_val[k] << 24) | ((uint32_t)w->lo[i] << 16));
            }
        }
        break;
    }
    case W_MX4: {
        const size_t g = w->cols / 32;
        for (size_t j = 0; j < n; ++j) {
            const size_t c = c0 + j, b = c / 32, k = c % 32;
            const uint8_t byte = w->blocks[(r * g + b) * 16 + k / 2];
            dst[j] = FP4[(k & 1) ? byte >> 4 : byte & 15] * mx_scale(w->mscales[r * g + b]);
        }
        break;
    }
    case W_FP8: {
        const float* srow = w->fscales + (r / w->bm) * w->sc;
        const uint8_t* src = w->f8 + r * w->cols;
        for (size_t j = 0; j < n; ++j) dst[j] = round_bf16_int(f8_value(src[c0 + j]) * srow[(c0 + j) / w->bn]);
        break;
    }
    }
}

/* lane j of each of R rows takes the tile's columns j, j + 16, .. in order, one fma each */
static void accum_tile(float* acc, const float* wide, size_t R, const float* x, size_t n) {
    const size_t nb = n / 16;
#if defined(__x86_64__)
    if (have_avx512()) {
        accum_tile_avx512(acc, wide, R, x, nb);
    } else
#endif
    {
        for (size_t k = 0; k < nb; ++k)
            for (size_t r = 0; r < R; ++r)
                for (int j = 0; j < 16; ++j)
                    acc[r * 16 + j] = fmaf(wide[r * COL_TILE + k * 16 + j], x[k * 16 + j], acc[r * 16 + j]);
    }
    for (size_t j = 0; j < n - nb * 16; ++j)
        for (size_t r = 0; r < R; ++r)
            acc[r * 16 + j] = fmaf(wide[r * COL_TILE + nb * 16 + j], x[nb * 16 + j], acc[r * 16 + j]);
}

#if defined(__x86_64__)
/* one bf16 vector: straight from the rows, no widened tile (native/src/gemv.rs:272-302, the b == 1 arm) */
__attribute__((target("avx512f,avx512bw"))) static void bf16_rows4_avx512(const uint16_t* w, size_t cols,
                                                                        const float* x, float* y4, size_t R) {
    __m512 a[ROW_UNROLL];
    for (size_t r = 0; r < R; ++r) a[r] = _mm512_setzero_ps();
    const size_t nb = cols / 16;
    for (size_t k = 0; k < nb; ++k) {
        const __m512 xv = _mm512_loadu_ps(x + k * 16);
        for (size_t r = 0; r < R; ++r) {
            __m512i v = _mm512_cvtepu16_epi32(_mm256_loadu_si256((const __m256i*)(w + r * cols + k * 16)));
            a[r] = _mm512_fmadd_ps(_mm512_castsi512_ps(_mm512_slli_epi32(v, 16)), xv, a[r]);
        }
    }
    float acc[ROW_UNROLL * 16];
    for (size_t r = 0; r < R; ++r) _mm512_storeu_ps(acc + r * 16, a[r]);
    for (size_t j = 0; j < cols - nb * 16; ++j)
        for (size_t r = 0; r < R; ++r)
            acc[r * 16 + j] = fmaf(bf2f(w[r * cols + nb * 16 + j]), x[nb * 16 + j], acc[r * 16 + j]);
    for (size_t r = 0; r < R; ++r) y4[r] = reduce16(acc + r * 16);
}
#endif

static void gemv_rows_range(const Wt* w, const float* x, size_t b, float* y, size_t r0, size_t r1) {
    float wide[ROW_UNROLL * COL_TILE];
    float acc[ROW_UNROLL * 16];
    size_t r = r0;
    while (r < r1) {
        const size_t R = r1 - r >= ROW_UNROLL ? ROW_UNROLL : 1;
#if defined(__x86_64__)
        if (w->kind == W_BF16 && b == 1 && have_avx512()) {
            float y4[ROW_UNROLL];
            bf16_rows4_avx512(w->bf + r * w->cols, w->cols, x, y4, R);
            for (size_t rr = 0; rr < R; ++rr) y[r + rr] = y4[rr];
            r += R;
            continue;
        }
#endif
        for (size_t i = 0; i < b; ++i) {
            /* an accumulator meets the tiles in order with a fixed lane mapping: the bits do not depend on b */
            memset(acc, 0, sizeof acc);
            for (size_t c0 = 0; c0 < w->cols; c0 += COL_TILE) {
                const size_t n = w->cols - c0 < COL_TILE ? w->cols - c0 : COL_TILE;
                for (size_t rr = 0; rr < R; ++rr) widen_tile(w, r + rr, c0, n, wide + rr * COL_TILE);
                accum_tile(acc, wide, R, x + i * w->cols + c0, n);
            }
            for (size_t rr = 0; rr < R; ++rr) y[i * w->rows + r + rr] = reduce16(acc + rr * 16);
        }
        r += R;
    }
}

static int32_t gemv_any(const Wt* w, const float* x, size_t b, float* y, size_t threads) {
    if (!x || !y) return BTB_ERR_NULL;
    if (!w->rows || !w->cols || !b || threads > 1024) return BTB_ERR_DOMAIN;
    if (w->rows > (SIZE_MAX / 4) / w->cols) return BTB_ERR_DOMAIN;
    int nt = 1;
#ifdef _OPENMP
    nt = threads ? (int)threads : omp_get_num_procs();
#endif
    /* a few long chunks a thread, never under ROW_UNROLL rows (native/src/gemv.rs:31-35) */
    size_t chunk = (w->rows + (size_t)nt * 4 - 1) / ((size_t)nt * 4);
    if (chunk < ROW_UNROLL) chunk = ROW_UNROLL;
    chunk = (chunk + ROW_UNROLL - 1) / ROW_UNROLL * ROW_UNROLL;
    const long nchunks = (long)((w->rows + chunk - 1) / chunk);
#pragma omp parallel for schedule(dynamic, 1) num_threads(nt)
    for (long c = 0; c < nchunks; ++c) {
        const size_t r0 = (size_t)c * chunk, r1 = r0 + chunk < w->rows ? r0 + chunk : w->rows;
        gemv_rows_range(w, x, b, y, r0, r1);
    }
    return BTB_OK;
}

int32_t btb_gemv_bf16_rows(const uint16_t* w, size_t rows, size_t cols, const float* x, size_t b, float* y,
                           size_t threads) {
    if (!w) return BTB_ERR_NULL;
    Wt t = {.kind = W_BF16, .rows = rows, .cols = cols, .bf = w};
    return gemv_any(&t, x, b, y, threads);
}

int32_t btb_gemv_p12_rows(const uint8_t* lo, const uint8_t* hi4, const uint8_t* table, const int32_t* esc_idx,
                          const uint8_t* esc_val, size_t n_esc, size_t rows, size_t cols, const float* x, size_t b,
                          float* y, size_t threads) {
    if (!lo || !hi4 || !table || (n_esc && (!esc_idx || !esc_val))) return BTB_ERR_NULL;
    if (!rows || !cols) return BTB_ERR_DOMAIN;
    int rc = p12_check(esc_idx, n_esc, rows * cols);
    if (rc) return rc;
    Wt t = {.kind = W_P12, .rows = rows, .cols = cols, .lo = lo, .hi4 = hi4, .table = table,
            .esc_idx = esc_idx, .esc_val = esc_val, .n_esc = n_esc};
    return gemv_any(&t, x, b, y, threads);
}

int32_t btb_gemv_mxfp4_rows(const uint8_t* blocks, const uint8_t* scales, size_t rows, size_t cols, const float* x,
                            size_t b, float* y, size_t threads) {
    if (!blocks || !scales) return BTB_ERR_NULL;
    if (cols % 32) return BTB_ERR_DOMAIN;
    Wt t = {.kind = W_MX4, .rows = rows, .cols = cols, .blocks = blocks, .mscales = scales};
    return gemv_any(&t, x, b, y, threads);
}

int32_t btb_gemv_fp8_rows(const uint8_t* w, const float* scales, size_t rows, size_t cols, size_t sr, size_t sc,
                          const float* x, size_t b, float* y, size_t threads) {
    if (!w || !scales) return BTB_ERR_NULL;
    if (!sr || !sc || !rows || !cols || rows % sr || cols % sc) return BTB_ERR_DOMAIN;
    Wt t = {.kind = W_FP8, .rows = rows, .cols = cols, .f8 = w, .fscales = scales, .sc = sc, .bm = rows / sr,
            .bn = cols / sc};
    return gemv_any(&t, x, b, y, threads);
}

/* f32 online softmax over the cache rows in order, one part (native/src/attn.rs:400-439) */
int32_t btb_attn_decode_bf16(const float* q, const uint16_t* k, const uint16_t* v, size_t n, size_t hq, size_t hk,
                             size_t d, size_t k_head_stride, size_t v_head_stride, float scale, float* out,
                             size_t threads) {
    (void)threads;
    if (!q || !k || !v || !out) return BTB_ERR_NULL;
    if (!n || !hq || !hk || !d || hq % hk || !isfinite(scale)) return BTB_ERR_DOMAIN;
    const size_t group = hq / hk;
    for (size_t h = 0; h < hq; ++h) {
        const size_t g = h / group;
        const float* qr = q + h * d;
        float* acc = out + h * d;
        for (size_t i = 0; i < d; ++i) acc[i] = 0.f;
        float rmax = -INFINITY, rsum = 0.f;
        for (size_t r = 0; r < n; ++r) {
            const uint16_t* kr = k + g * k_head_stride + r * d;
            const uint16_t* vr = v + g * v_head_stride + r * d;
            float s = 0.f;
            for (size_t i = 0; i < d; ++i) s = fmaf(bf2f(kr[i]), qr[i], s);
            s *= scale;
            float p;
            if (s > rmax) {
                const float corr = expf(rmax - s);
                for (size_t i = 0; i < d; ++i) acc[i] *= corr;
                rsum = rsum * corr + 1.0f;
                rmax = s;
                p = 1.0f;
            } else {
                p = expf(s - rmax);
                rsum += p;
            }
            for (size_t i = 0; i < d; ++i) acc[i] = fmaf(p, bf2f(vr[i]), acc[i]);
        }
        const float inv = 1.0f / rsum;
        for (size_t i = 0; i < d; ++i) acc[i] *= inv;
    }
    return BTB_OK;
}
