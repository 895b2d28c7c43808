/*
 * CPU oracle for lloom-tensor's quantized matmul.  TEST INFRASTRUCTURE ONLY:
 * the product (the CUDA library) never links, loads or calls this file.
 *
 * Each function restates the arithmetic of the reference function cited above
 * it (paths are relative to the reference project root).  All float arithmetic
 * is IEEE binary32, sequential, and must not be contracted: build with
 * -ffp-contract=off and without -ffast-math (see the Makefile beside this file).
 *
 * Third-party arithmetic the reference relies on and this file restates:
 *   - crate `half` 2.7.1 (Cargo.lock): f16::from_f32 / to_f32 are IEEE binary16
 *     conversions, round-to-nearest-even, subnormals kept.
 *   - Rust std: f32::round is round-half-away-from-zero; `as i8/u8/i32` from a
 *     float saturates and maps NaN to 0; Iterator::sum::<f32> is a left fold.
 *
 * Parity status: PINNED by the reference's own golden values (quantize ramps,
 * cosine vectors, GEMM == GEMV bit identity); see tests/test_oracle_golden.py.
 */
#include "lloom_oracle.h"

#include <math.h>
#include <string.h>
#include <stdlib.h>
#include <pthread.h>
#include <stdatomic.h>
#if defined(__x86_64__) || defined(__i386__)
#include <immintrin.h>
#define LO_X86 1
#endif

#define QK8_0 32
#define QK_K 256

/* ---- block layouts (lloom-tensor/src/quantized/k_quants.rs:155-159, 217-223, 255-261, 265-270) ---- */
#pragma pack(push, 1)
typedef struct { uint16_t d; int8_t qs[QK8_0]; } blk_q8_0;                          /* 34 B  */
typedef struct { uint16_t d, dmin; uint8_t scales[12]; uint8_t qs[QK_K / 2]; } blk_q4k; /* 144 B */
typedef struct { uint8_t ql[QK_K / 2]; uint8_t qh[QK_K / 4]; int8_t scales[QK_K / 16]; uint16_t d; } blk_q6k; /* 210 B */
typedef struct { float d; int8_t qs[QK_K]; int16_t bsums[QK_K / 16]; } blk_q8k;     /* 292 B */
/* k_quants.rs:84-131 (Q4_0, Q5_0), 184-192 (Q5K) */
typedef struct { uint16_t d; uint8_t qs[16]; } blk_q4_0;                            /* 18 B  */
typedef struct { uint16_t d; uint8_t qh[4]; uint8_t qs[16]; } blk_q5_0;             /* 22 B  */
typedef struct { uint16_t d, dmin; uint8_t scales[12]; uint8_t qh[QK_K / 8]; uint8_t qs[QK_K / 2]; } blk_q5k; /* 176 B */
#pragma pack(pop)

_Static_assert(sizeof(blk_q8_0) == 34, "Q8_0 block");
_Static_assert(sizeof(blk_q4k) == 144, "Q4_K block");
_Static_assert(sizeof(blk_q6k) == 210, "Q6_K block");
_Static_assert(sizeof(blk_q8k) == 292, "Q8_K block");
_Static_assert(sizeof(blk_q4_0) == 18, "Q4_0 block");
_Static_assert(sizeof(blk_q5_0) == 22, "Q5_0 block");
_Static_assert(sizeof(blk_q5k) == 176, "Q5_K block");

int64_t lo_block_elems(int dtype) {
    switch (dtype) {
    case LO_Q8_0: case LO_Q4_0: case LO_Q5_0: return QK8_0;
    case LO_Q4_K: case LO_Q5_K: case LO_Q6_K: case LO_Q8_K: return QK_K;
    default: return 0;
    }
}
int64_t lo_block_bytes(int dtype) {
    switch (dtype) {
    case LO_Q8_0: return sizeof(blk_q8_0);
    case LO_Q4_K: return sizeof(blk_q4k);
    case LO_Q6_K: return sizeof(blk_q6k);
    case LO_Q8_K: return sizeof(blk_q8k);
    case LO_Q4_0: return sizeof(blk_q4_0);
    case LO_Q5_0: return sizeof(blk_q5_0);
    case LO_Q5_K: return sizeof(blk_q5k);
    default: return 0;
    }
}

/* ---- scalar conventions ---- */

/* IEEE binary16 -> binary32, exact. */
float lo_f16_to_f32(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1f;
    uint32_t man = h & 0x3ffu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else { /* subnormal: normalise */
            int shift = 0;
            while (!(man & 0x400u)) { man <<= 1; ++shift; }
            man &= 0x3ffu;
            bits = sign | ((uint32_t)(127 - 15 - shift + 1) << 23) | (man << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7f800000u | (man << 13);
    } else {
        bits = sign | ((exp + 127 - 15) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

/* IEEE binary32 -> binary16, round to nearest even, subnormals kept. */
uint16_t lo_f32_to_f16(float f) {
    uint32_t x;
    memcpy(&x, &f, 4);
    uint16_t sign = (uint16_t)((x >> 16) & 0x8000u);
    uint32_t exp = (x >> 23) & 0xff;
    uint32_t man = x & 0x7fffffu;
    if (exp == 0xff) return (uint16_t)(sign | 0x7c00u | (man ? (0x200u | (man >> 13)) : 0));
    int e = (int)exp - 127 + 15;
    if (e >= 31) return (uint16_t)(sign | 0x7c00u);
    if (e <= 0) {
        if (e < -10) return sign; /* below half the smallest subnormal */
        man |= 0x800000u;
        int shift = 14 - e; /* 14..24 */
        uint32_t half_man = man >> shift;
        uint32_t rem = man & ((1u << shift) - 1);
        uint32_t halfway = 1u << (shift - 1);
        if (rem > halfway || (rem == halfway && (half_man & 1))) ++half_man;
        return (uint16_t)(sign | half_man);
    }
    uint32_t half = ((uint32_t)e << 10) | (man >> 13);
    uint32_t rem = man & 0x1fffu;
    if (rem > 0x1000u || (rem == 0x1000u && (half & 1))) ++half; /* may carry into the exponent: correct */
    return (uint16_t)(sign | half);
}

/* Rust `v as i32` from f32: saturating, NaN -> 0. */
static inline int32_t sat_i32(float v) {
    if (v != v) return 0;
    if (v >= 2147483648.0f) return INT32_MAX;
    if (v <= -2147483648.0f) return INT32_MIN;
    return (int32_t)v;
}
/* Rust `v as i8` from f32. */
static inline int8_t sat_i8(float v) {
    if (v != v) return 0;
    if (v >= 127.0f) return 127;
    if (v <= -128.0f) return -128;
    return (int8_t)v;
}
/* utils.rs:1-3  nearest_int = v.round() as i32; f32::round is half away from zero = roundf. */
static inline int32_t nearest_int(float v) { return sat_i32(roundf(v)); }
static inline int32_t clampi(int32_t v, int32_t lo, int32_t hi) { return v < lo ? lo : (v > hi ? hi : v); }
/* f32::max: returns the other operand if one is NaN. */
static inline float rmaxf(float a, float b) { return (a != a) ? b : ((b != b) ? a : (a > b ? a : b)); }

/* ---- Q8_0 (k_quants.rs:714-819) ---- */

/* BlockQ8_0::from_float, k_quants.rs:738-767 */
static void quantize_row_q8_0(const float *x, blk_q8_0 *y, int64_t k) {
    for (int64_t i = 0; i < k / QK8_0; ++i) {
        const float *xb = x + i * QK8_0;
        float amax = 0.0f;
        for (int j = 0; j < QK8_0; ++j) amax = rmaxf(amax, fabsf(xb[j]));
        float d = amax / 127.0f;
        float id = (d != 0.0f) ? 1.0f / d : 0.0f;
        y[i].d = lo_f32_to_f16(d);
        for (int j = 0; j < QK8_0; ++j) y[i].qs[j] = sat_i8(roundf(xb[j] * id));
    }
}
/* BlockQ8_0::to_float, k_quants.rs:720-736 */
static void dequantize_row_q8_0(const blk_q8_0 *x, float *y, int64_t k) {
    for (int64_t i = 0; i < k / QK8_0; ++i) {
        float d = lo_f16_to_f32(x[i].d);
        for (int j = 0; j < QK8_0; ++j) y[i * QK8_0 + j] = (float)x[i].qs[j] * d;
    }
}

/* ---- Q8_K (k_quants.rs:2361-2452) ---- */

/* BlockQ8K::from_float (non-NEON arm), k_quants.rs:2400-2438.
 * For an all-zero block the reference leaves bsums as they were; here they are
 * set to 0 (they are only ever multiplied by d == 0). */
static void quantize_row_q8k(const float *x, blk_q8k *y, int64_t k) {
    for (int64_t i = 0; i < k / QK_K; ++i) {
        const float *xb = x + i * QK_K;
        float max = 0.0f, amax = 0.0f;
        for (int j = 0; j < QK_K; ++j) {
            float ax = fabsf(xb[j]);
            if (amax < ax) { amax = ax; max = xb[j]; } /* strict: first of equal magnitudes wins */
        }
        if (amax == 0.0f) {
            y[i].d = 0.0f;
            memset(y[i].qs, 0, QK_K);
            memset(y[i].bsums, 0, sizeof(y[i].bsums));
            continue;
        }
        float iscale = -127.0f / max;
        for (int j = 0; j < QK_K; ++j) {
            float v = roundf(iscale * xb[j]);
            if (v < -128.0f) v = -128.0f;
            if (v > 127.0f) v = 127.0f;
            y[i].qs[j] = sat_i8(v);
        }
        for (int j = 0; j < QK_K / 16; ++j) {
            int32_t s = 0;
            for (int t = 0; t < 16; ++t) s += y[i].qs[j * 16 + t];
            y[i].bsums[j] = (int16_t)s;
        }
        y[i].d = 1.0f / iscale;
    }
}
/* BlockQ8K::to_float, k_quants.rs:2440-2452 */
static void dequantize_row_q8k(const blk_q8k *x, float *y, int64_t k) {
    for (int64_t i = 0; i < k / QK_K; ++i)
        for (int j = 0; j < QK_K; ++j) y[i * QK_K + j] = x[i].d * (float)x[i].qs[j];
}

/* ---- Q4_K (k_quants.rs:1504-1775, utils.rs:50-60, 227-284) ---- */

/* utils.rs:50-60 get_scale_min_k4 */
static inline void scale_min_k4(int j, const uint8_t *q, uint8_t *sc, uint8_t *mn) {
    if (j < 4) {
        *sc = q[j] & 63;
        *mn = q[j + 4] & 63;
    } else {
        *sc = (uint8_t)((q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4));
        *mn = (uint8_t)((q[j + 4] >> 4) | ((q[j] >> 6) << 4));
    }
}

/* utils.rs:227-284 make_qkx1_quants(nmax, ntry, x[0..n]) -> (scale, -min) */
static void make_qkx1_quants(int nmax, int ntry, const float *x, int n, float *out_scale, float *out_min) {
    uint8_t L[32];
    memset(L, 0, sizeof(L));
    float min = x[0], max = x[0];
    for (int i = 1; i < n; ++i) {
        if (x[i] < min) min = x[i];
        if (x[i] > max) max = x[i];
    }
    if (max == min) { *out_scale = 0.0f; *out_min = 0.0f; return; }
    if (min > 0.0f) min = 0.0f;
    float iscale = (float)nmax / (max - min);
    float scale = 1.0f / iscale;
    for (int it = 0; it < ntry; ++it) {
        float sumlx = 0.0f;
        int32_t suml2 = 0;
        int changed = 0;
        for (int i = 0; i < n; ++i) {
            int32_t li = clampi(nearest_int(iscale * (x[i] - min)), 0, nmax);
            if ((uint8_t)li != L[i]) { L[i] = (uint8_t)li; changed = 1; }
            sumlx += (x[i] - min) * (float)li;
            suml2 += li * li;
        }
        scale = sumlx / (float)suml2;
        float sum = 0.0f;
        for (int i = 0; i < n; ++i) sum += x[i] - scale * (float)L[i];
        min = sum / (float)n;
        if (min > 0.0f) min = 0.0f;
        iscale = 1.0f / scale;
        if (!changed) break;
    }
    *out_scale = scale;
    *out_min = -min;
}

/* BlockQ4K::from_float, k_quants.rs:1622-1680 */
static void quantize_row_q4k(const float *x, blk_q4k *y, int64_t k) {
    for (int64_t i = 0; i < k / QK_K; ++i) {
        const float *xb = x + i * QK_K;
        blk_q4k *b = &y[i];
        memset(b, 0, sizeof(*b));
        float mins[8], scales[8];
        for (int j = 0; j < 8; ++j) make_qkx1_quants(15, 5, xb + 32 * j, 32, &scales[j], &mins[j]);
        float max_scale = 0.0f, max_min = 0.0f;
        for (int j = 0; j < 8; ++j) { max_scale = rmaxf(scales[j], max_scale); max_min = rmaxf(mins[j], max_min); }
        float inv_scale = max_scale > 0.0f ? 63.0f / max_scale : 0.0f;
        float inv_min = max_min > 0.0f ? 63.0f / max_min : 0.0f;
        for (int j = 0; j < 8; ++j) {
            int32_t lsi = nearest_int(inv_scale * scales[j]);
            int32_t lmi = nearest_int(inv_min * mins[j]);
            uint8_t ls = (uint8_t)(lsi < 63 ? lsi : 63);
            uint8_t lm = (uint8_t)(lmi < 63 ? lmi : 63);
            if (j < 4) {
                b->scales[j] = ls;
                b->scales[j + 4] = lm;
            } else {
                b->scales[j + 4] = (uint8_t)((ls & 0xF) | ((lm & 0xF) << 4));
                b->scales[j - 4] |= (uint8_t)((ls >> 4) << 6);
                b->scales[j] |= (uint8_t)((lm >> 4) << 6);
            }
        }
        b->d = lo_f32_to_f16(max_scale / 63.0f);
        b->dmin = lo_f32_to_f16(max_min / 63.0f);
        uint8_t L[QK_K];
        memset(L, 0, sizeof(L));
        float bd = lo_f16_to_f32(b->d), bdmin = lo_f16_to_f32(b->dmin);
        for (int j = 0; j < 8; ++j) {
            uint8_t sc, m;
            scale_min_k4(j, b->scales, &sc, &m);
            float d = bd * (float)sc;
            if (d != 0.0f) {
                float dm = bdmin * (float)m;
                for (int t = 0; t < 32; ++t)
                    L[32 * j + t] = (uint8_t)clampi(nearest_int((xb[32 * j + t] + dm) / d), 0, 15);
            }
        }
        for (int g = 0; g < 4; ++g)
            for (int t = 0; t < 32; ++t) b->qs[32 * g + t] = (uint8_t)(L[64 * g + t] | (L[64 * g + 32 + t] << 4));
    }
}

/* BlockQ4K::to_float, k_quants.rs:1747-1774 */
static void dequantize_row_q4k(const blk_q4k *x, float *y, int64_t k) {
    for (int64_t i = 0; i < k / QK_K; ++i) {
        const blk_q4k *b = &x[i];
        float d = lo_f16_to_f32(b->d), min = lo_f16_to_f32(b->dmin);
        float *yb = y + i * QK_K;
        for (int g = 0; g < 4; ++g) {
            uint8_t sc, m;
            scale_min_k4(2 * g, b->scales, &sc, &m);
            float d1 = d * (float)sc, m1 = min * (float)m;
            scale_min_k4(2 * g + 1, b->scales, &sc, &m);
            float d2 = d * (float)sc, m2 = min * (float)m;
            const uint8_t *q = b->qs + 32 * g;
            for (int t = 0; t < 32; ++t) yb[64 * g + t] = d1 * (float)(q[t] & 0xF) - m1;
            for (int t = 0; t < 32; ++t) yb[64 * g + 32 + t] = d2 * (float)(q[t] >> 4) - m2;
        }
    }
}

/* ---- Q6_K (k_quants.rs:2079-2359, utils.rs:62-224) ---- */

/* utils.rs:62-224 make_qx_quants(n, nmax, x, ls, rmse_type = 1, qw = null):
 * weights are x*x; the rmse_type >= 3 tail of the reference is unreachable here. */
static float make_qx_quants_w(int n, int nmax, const float *x, int8_t *ls, const float *qw) {
    float max = 0.0f, amax = 0.0f;
    for (int i = 0; i < n; ++i) {
        float ax = fabsf(x[i]);
        if (ax > amax) { amax = ax; max = x[i]; }
    }
    if (amax == 0.0f) {
        for (int i = 0; i < n; ++i) ls[i] = 0;
        return 0.0f;
    }
    float iscale = -(float)nmax / max;
    float sumlx = 0.0f, suml2 = 0.0f;
    for (int i = 0; i < n; ++i) {
        int32_t l = clampi(nearest_int(iscale * x[i]), -nmax, nmax - 1);
        ls[i] = (int8_t)(l + nmax);
        float w = qw ? qw[i] : x[i] * x[i];
        float lf = (float)l;
        sumlx += w * x[i] * lf;
        suml2 += w * lf * lf;
    }
    float scale = sumlx / suml2;
    float best = scale * sumlx;
    for (int itry = 0; itry < 3; ++itry) {
        float is = 1.0f / scale;
        float slx = 0.0f, sl2 = 0.0f;
        int changed = 0;
        for (int i = 0; i < n; ++i) {
            int32_t l = clampi(nearest_int(is * x[i]), -nmax, nmax - 1);
            if (l + nmax != (int32_t)ls[i]) changed = 1;
            float w = qw ? qw[i] : x[i] * x[i];
            float lf = (float)l;
            slx += w * x[i] * lf;
            sl2 += w * lf * lf;
        }
        if (!changed || sl2 == 0.0f || slx * slx <= best * sl2) break;
        for (int i = 0; i < n; ++i) {
            int32_t l = nearest_int(is * x[i]);
            ls[i] = (int8_t)(nmax + clampi(l, -nmax, nmax - 1));
        }
        sumlx = slx;
        suml2 = sl2;
        scale = sumlx / suml2;
        best = scale * sumlx;
    }
    for (int itry = 0; itry < 5; ++itry) {
        int n_changed = 0;
        for (int i = 0; i < n; ++i) {
            float w = qw ? qw[i] : x[i] * x[i];
            int32_t l = (int32_t)ls[i] - nmax;
            float slx = sumlx - w * x[i] * (float)l;
            if (slx > 0.0f) {
                float sl2 = suml2 - w * (float)l * (float)l;
                int32_t new_l = clampi(nearest_int(x[i] * sl2 / slx), -nmax, nmax - 1);
                if (new_l != l) {
                    slx += w * x[i] * (float)new_l;
                    sl2 += w * (float)new_l * (float)new_l;
                    if (sl2 > 0.0f && slx * slx * suml2 > sumlx * sumlx * sl2) {
                        ls[i] = (int8_t)(nmax + new_l);
                        sumlx = slx;
                        suml2 = sl2;
                        scale = sumlx / suml2;
                        best = scale * sumlx;
                        ++n_changed;
                    }
                }
            }
        }
        if (n_changed == 0) break;
    }
    (void)best;
    return scale;
}

/* BlockQ6K::from_float, k_quants.rs:2174-2244.  An all-zero superblock follows
 * the same float path as the reference (iscale = -inf, d = f16(-0), NaN -> 0). */
/* imatrix == NULL: BlockQ6K::from_float (k_quants.rs:2174-2244); else from_float_imatrix (k_quants.rs:2246-2325) on
 * one row: the importance weights of superblock i of the row are imatrix[256 i ..]. */
static void quantize_row_q6k_w(const float *x, blk_q6k *y, int64_t k, const float *imatrix) {
    int8_t L[QK_K];
    float scales[QK_K / 16];
    memset(L, 0, sizeof(L));
    for (int64_t i = 0; i < k / QK_K; ++i) {
        const float *xb = x + i * QK_K;
        blk_q6k *b = &y[i];
        float max_scale = 0.0f, max_abs_scale = 0.0f;
        for (int ib = 0; ib < 16; ++ib) {
            float s = make_qx_quants_w(16, 32, xb + 16 * ib, L + 16 * ib, imatrix ? imatrix + QK_K * i + 16 * ib : 0);
            scales[ib] = s;
            float as = fabsf(s);
            if (as > max_abs_scale) { max_abs_scale = as; max_scale = s; }
        }
        float iscale = -128.0f / max_scale;
        b->d = lo_f32_to_f16(1.0f / iscale);
        for (int ib = 0; ib < 16; ++ib) {
            int32_t v = nearest_int(iscale * scales[ib]);
            b->scales[ib] = (int8_t)(v < 127 ? v : 127);
        }
        float bd = lo_f16_to_f32(b->d);
        for (int j = 0; j < 16; ++j) {
            float d = bd * (float)b->scales[j];
            if (d == 0.0f) continue;
            for (int t = 0; t < 16; ++t) {
                int32_t ll = clampi(nearest_int(xb[16 * j + t] / d), -32, 31);
                L[16 * j + t] = (int8_t)(ll + 32);
            }
        }
        for (int h = 0; h < 2; ++h) {
            const int8_t *Lh = L + 128 * h;
            uint8_t *ql = b->ql + 64 * h;
            uint8_t *qh = b->qh + 32 * h;
            for (int t = 0; t < 32; ++t) {
                int8_t q1 = Lh[t] & 0xF, q2 = Lh[t + 32] & 0xF, q3 = Lh[t + 64] & 0xF, q4 = Lh[t + 96] & 0xF;
                ql[t] = (uint8_t)(q1 | (q3 << 4));
                ql[t + 32] = (uint8_t)(q2 | (q4 << 4));
                qh[t] = (uint8_t)((Lh[t] >> 4) | ((Lh[t + 32] >> 4) << 2) | ((Lh[t + 64] >> 4) << 4) |
                                  ((Lh[t + 96] >> 4) << 6));
            }
        }
    }
}

/* codes of one Q6_K superblock, minus 32, in element order (k_quants.rs:2133-2146, 2339-2353) */
static inline void q6k_codes(const blk_q6k *b, int8_t *out) {
    for (int h = 0; h < 2; ++h) {
        const uint8_t *ql = b->ql + 64 * h;
        const uint8_t *qh = b->qh + 32 * h;
        int8_t *o = out + 128 * h;
        for (int t = 0; t < 32; ++t) {
            o[t] = (int8_t)((int)((ql[t] & 0xF) | ((qh[t] & 3) << 4)) - 32);
            o[t + 32] = (int8_t)((int)((ql[t + 32] & 0xF) | (((qh[t] >> 2) & 3) << 4)) - 32);
            o[t + 64] = (int8_t)((int)((ql[t] >> 4) | (((qh[t] >> 4) & 3) << 4)) - 32);
            o[t + 96] = (int8_t)((int)((ql[t + 32] >> 4) | (((qh[t] >> 6) & 3) << 4)) - 32);
        }
    }
}

/* BlockQ6K::to_float, k_quants.rs:2327-2358: y = d * sc * q evaluated left to right. */
static void dequantize_row_q6k(const blk_q6k *x, float *y, int64_t k) {
    int8_t q[QK_K];
    for (int64_t i = 0; i < k / QK_K; ++i) {
        const blk_q6k *b = &x[i];
        float d = lo_f16_to_f32(b->d);
        q6k_codes(b, q);
        for (int e = 0; e < QK_K; ++e) y[i * QK_K + e] = d * (float)b->scales[e / 16] * (float)q[e];
    }
}

/* ---- Q4_0 (k_quants.rs:293-392), Q5_0 (k_quants.rs:495-600), Q5_K (k_quants.rs:1778-2077) ---- */

/* Rust `f32 as u8`: truncation toward zero, saturating, NaN -> 0 */
static inline uint8_t sat_u8_trunc(float v) {
    if (!(v == v)) return 0;
    if (v <= 0.0f) return 0;
    if (v >= 255.0f) return 255;
    return (uint8_t)v;
}
/* Rust `f32 as i8`: truncation toward zero, saturating, NaN -> 0 */
static inline int8_t sat_i8_trunc(float v) {
    if (!(v == v)) return 0;
    if (v <= -128.0f) return -128;
    if (v >= 127.0f) return 127;
    return (int8_t)v;
}

/* BlockQ4_0::from_float, k_quants.rs:320-352 */
static void quantize_row_q4_0(const float *x, blk_q4_0 *y, int64_t k) {
    for (int64_t i = 0; i < k / QK8_0; ++i) {
        const float *xb = x + i * QK8_0;
        float amax = 0.0f, max = 0.0f;
        for (int j = 0; j < QK8_0; ++j)
            if (amax < fabsf(xb[j])) { amax = fabsf(xb[j]); max = xb[j]; }
        float d = max / -8.0f;
        float id = d != 0.0f ? 1.0f / d : 0.0f;
        y[i].d = lo_f32_to_f16(d);
        for (int j = 0; j < 16; ++j) {
            float x0 = xb[j] * id, x1 = xb[16 + j] * id;
            uint8_t xi0 = sat_u8_trunc(x0 + 8.5f), xi1 = sat_u8_trunc(x1 + 8.5f);
            if (xi0 > 15) xi0 = 15;
            if (xi1 > 15) xi1 = 15;
            y[i].qs[j] = (uint8_t)(xi0 | (xi1 << 4));
        }
    }
}

/* BlockQ4_0::to_float, k_quants.rs:299-318 */
static void dequantize_row_q4_0(const blk_q4_0 *x, float *y, int64_t k) {
    for (int64_t i = 0; i < k / QK8_0; ++i) {
        float d = lo_f16_to_f32(x[i].d);
        for (int j = 0; j < 16; ++j) {
            int x0 = (x[i].qs[j] & 0x0F) - 8, x1 = (x[i].qs[j] >> 4) - 8;
            y[i * QK8_0 + j] = (float)x0 * d;
            y[i * QK8_0 + j + 16] = (float)x1 * d;
        }
    }
}

/* BlockQ5_0::from_float, k_quants.rs:536-575 */
static void quantize_row_q5_0(const float *x, blk_q5_0 *y, int64_t k) {
    for (int64_t i = 0; i < k / QK8_0; ++i) {
        const float *xb = x + i * QK8_0;
        float amax = 0.0f, max = 0.0f;
        for (int j = 0; j < QK8_0; ++j)
            if (amax < fabsf(xb[j])) { amax = fabsf(xb[j]); max = xb[j]; }
        float d = max / -16.0f;
        float id = d != 0.0f ? 1.0f / d : 0.0f;
        y[i].d = lo_f32_to_f16(d);
        uint32_t qh = 0;
        for (int j = 0; j < 16; ++j) {
            float x0 = xb[j] * id, x1 = xb[j + 16] * id;
            int8_t s0 = sat_i8_trunc(x0 + 16.5f), s1 = sat_i8_trunc(x1 + 16.5f);
            uint8_t xi0 = (uint8_t)(s0 < 31 ? s0 : 31), xi1 = (uint8_t)(s1 < 31 ? s1 : 31);
            y[i].qs[j] = (uint8_t)((xi0 & 0x0F) | ((xi1 & 0x0F) << 4));
            qh |= (((uint32_t)xi0 & 0x10u) >> 4) << j;
            qh |= (((uint32_t)xi1 & 0x10u) >> 4) << (j + 16);
        }
        y[i].qh[0] = (uint8_t)qh; y[i].qh[1] = (uint8_t)(qh >> 8); y[i].qh[2] = (uint8_t)(qh >> 16); y[i].qh[3] = (uint8_t)(qh >> 24);
    }
}

static inline uint32_t q5_0_qh(const blk_q5_0 *b) {
    return (uint32_t)b->qh[0] | ((uint32_t)b->qh[1] << 8) | ((uint32_t)b->qh[2] << 16) | ((uint32_t)b->qh[3] << 24);
}

/* BlockQ5_0::to_float, k_quants.rs:578-600 */
static void dequantize_row_q5_0(const blk_q5_0 *x, float *y, int64_t k) {
    for (int64_t i = 0; i < k / QK8_0; ++i) {
        float d = lo_f16_to_f32(x[i].d);
        uint32_t qh = q5_0_qh(&x[i]);
        for (int j = 0; j < 16; ++j) {
            uint8_t xh_0 = (uint8_t)(((qh >> j) << 4) & 0x10), xh_1 = (uint8_t)((qh >> (j + 12)) & 0x10);
            int x0 = (int)((x[i].qs[j] & 0x0F) | xh_0) - 16, x1 = (int)((x[i].qs[j] >> 4) | xh_1) - 16;
            y[i * QK8_0 + j] = (float)x0 * d;
            y[i * QK8_0 + j + 16] = (float)x1 * d;
        }
    }
}

/* the 32 signed codes of a Q4_0 / Q5_0 block in element order */
static inline void q4_0_codes(const blk_q4_0 *b, int8_t *c) {
    for (int j = 0; j < 16; ++j) { c[j] = (int8_t)((b->qs[j] & 0x0F) - 8); c[j + 16] = (int8_t)((b->qs[j] >> 4) - 8); }
}
static inline void q5_0_codes(const blk_q5_0 *b, int8_t *c) {
    uint32_t qh = q5_0_qh(b);
    for (int j = 0; j < 16; ++j) {
        uint8_t xh_0 = (uint8_t)(((qh & (1u << j)) >> j) << 4), xh_1 = (uint8_t)((qh & (1u << (j + 16))) >> (j + 12));
        c[j] = (int8_t)((int)((b->qs[j] & 0x0F) | xh_0) - 16);
        c[j + 16] = (int8_t)((int)((b->qs[j] >> 4) | xh_1) - 16);
    }
}

/* BlockQ5K::from_float, k_quants.rs:1883-1968 */
static void quantize_row_q5k(const float *x, blk_q5k *y, int64_t k) {
    for (int64_t i = 0; i < k / QK_K; ++i) {
        const float *xb = x + i * QK_K;
        blk_q5k *b = &y[i];
        memset(b, 0, sizeof(*b));
        float mins[8], scales[8];
        for (int j = 0; j < 8; ++j) make_qkx1_quants(31, 5, xb + 32 * j, 32, &scales[j], &mins[j]);
        float max_scale = 0.0f, max_min = 0.0f;
        for (int j = 0; j < 8; ++j) { max_scale = rmaxf(scales[j], max_scale); max_min = rmaxf(mins[j], max_min); }
        float inv_scale = max_scale > 0.0f ? 63.0f / max_scale : 0.0f;
        float inv_min = max_min > 0.0f ? 63.0f / max_min : 0.0f;
        for (int j = 0; j < 8; ++j) {
            int32_t lsi = nearest_int(inv_scale * scales[j]);
            int32_t lmi = nearest_int(inv_min * mins[j]);
            uint8_t ls = (uint8_t)(lsi < 63 ? lsi : 63);
            uint8_t lm = (uint8_t)(lmi < 63 ? lmi : 63);
            if (j < 4) {
                b->scales[j] = ls;
                b->scales[j + 4] = lm;
            } else {
                b->scales[j + 4] = (uint8_t)((ls & 0xF) | ((lm & 0xF) << 4));
                b->scales[j - 4] |= (uint8_t)((ls >> 4) << 6);
                b->scales[j] |= (uint8_t)((lm >> 4) << 6);
            }
        }
        b->d = lo_f32_to_f16(max_scale / 63.0f);
        b->dmin = lo_f32_to_f16(max_min / 63.0f);
        uint8_t L[QK_K];
        memset(L, 0, sizeof(L));
        float bd = lo_f16_to_f32(b->d), bdmin = lo_f16_to_f32(b->dmin);
        for (int j = 0; j < 8; ++j) {
            uint8_t sc, m;
            scale_min_k4(j, b->scales, &sc, &m);
            float d = bd * (float)sc;
            if (d == 0.0f) continue;
            float dm = bdmin * (float)m;
            for (int t = 0; t < 32; ++t) L[32 * j + t] = (uint8_t)clampi(nearest_int((xb[32 * j + t] + dm) / d), 0, 31);
        }
        uint8_t m1 = 1, m2 = 2;
        for (int n = 0; n < QK_K; n += 64) {
            int off = (n / 64) * 32;
            for (int j = 0; j < 32; ++j) {
                uint8_t l1 = L[n + j], l2 = L[n + j + 32];
                if (l1 > 15) { l1 -= 16; b->qh[j] |= m1; }
                if (l2 > 15) { l2 -= 16; b->qh[j] |= m2; }
                b->qs[off + j] = (uint8_t)(l1 | (l2 << 4));
            }
            m1 <<= 2;
            m2 <<= 2;
        }
    }
}

/* BlockQ5K::to_float, k_quants.rs:2043-2076 */
static void dequantize_row_q5k(const blk_q5k *x, float *y, int64_t k) {
    for (int64_t i = 0; i < k / QK_K; ++i) {
        const blk_q5k *b = &x[i];
        float d = lo_f16_to_f32(b->d), min = lo_f16_to_f32(b->dmin);
        float *yb = y + i * QK_K;
        uint8_t u1 = 1, u2 = 2;
        for (int g = 0; g < 4; ++g) {
            uint8_t sc, m;
            scale_min_k4(2 * g, b->scales, &sc, &m);
            float d1 = d * (float)sc, m1 = min * (float)m;
            scale_min_k4(2 * g + 1, b->scales, &sc, &m);
            float d2 = d * (float)sc, m2 = min * (float)m;
            const uint8_t *q = b->qs + 32 * g;
            for (int t = 0; t < 32; ++t) yb[64 * g + t] = d1 * ((float)(q[t] & 0xF) + ((b->qh[t] & u1) ? 16.0f : 0.0f)) - m1;
            for (int t = 0; t < 32; ++t) yb[64 * g + 32 + t] = d2 * ((float)(q[t] >> 4) + ((b->qh[t] & u2) ? 16.0f : 0.0f)) - m2;
            u1 <<= 2;
            u2 <<= 2;
        }
    }
}

/* the 256 unsigned 5-bit codes of a Q5_K block in element order, and its (scale, min) pairs */
static inline void q5k_codes(const blk_q5k *b, int8_t *a) {
    uint8_t m = 1;
    for (int g = 0; g < 4; ++g) {
        for (int t = 0; t < 32; ++t) a[64 * g + t] = (int8_t)((b->qs[32 * g + t] & 0xF) + ((b->qh[t] & m) ? 16 : 0));
        m <<= 1;
        for (int t = 0; t < 32; ++t) a[64 * g + 32 + t] = (int8_t)((b->qs[32 * g + t] >> 4) + ((b->qh[t] & m) ? 16 : 0));
        m <<= 1;
    }
}
static inline void q5k_scales_mins(const blk_q5k *b, uint8_t *sc, uint8_t *mn) {
    for (int j = 0; j < 8; ++j) scale_min_k4(j, b->scales, &sc[j], &mn[j]);
}

static void quantize_row_q6k(const float *x, blk_q6k *y, int64_t k) { quantize_row_q6k_w(x, y, k, 0); }

/* ---- importance-matrix quantizers: from_float_imatrix of Q4K (k_quants.rs:1682-1745) and Q5K (:1959-2041), with
 * make_qkx3_quants (utils.rs:372-466) and make_qp_quants (utils.rs:469-560) ---- */

static void make_qkx3_quants(int n, int nmax, const float *x, const float *weights, float rmin, float rdelta, int nstep,
                             int use_mad, float *out_scale, float *out_min) {
    uint8_t L[32], Laux[32];
    memset(L, 0, sizeof(L));
    float min_val = x[0], max_val = x[0];
    float sum_w = weights ? weights[0] : x[0] * x[0];
    float sum_x = sum_w * x[0];
    for (int i = 1; i < n; ++i) {
        if (x[i] < min_val) min_val = x[i];
        if (x[i] > max_val) max_val = x[i];
        float w = weights ? weights[i] : x[i] * x[i];
        sum_w += w;
        sum_x += w * x[i];
    }
    if (min_val > 0.0f) min_val = 0.0f;
    if (max_val <= min_val) { *out_scale = 0.0f; *out_min = -min_val; return; }
    float iscale = (float)nmax / (max_val - min_val);
    float scale = 1.0f / iscale;
    float best_mad = 0.0f;
    for (int i = 0; i < n; ++i) {
        uint8_t l = (uint8_t)clampi(nearest_int(iscale * (x[i] - min_val)), 0, nmax);
        L[i] = l;
        float diff = scale * (float)l + min_val - x[i];
        diff = use_mad ? fabsf(diff) : diff * diff;
        float w = weights ? weights[i] : x[i] * x[i];
        best_mad += w * diff;
    }
    if (nstep < 1) { *out_scale = scale; *out_min = -min_val; return; }
    for (int is = 0; is <= nstep; ++is) {
        iscale = (rmin + rdelta * (float)is + (float)nmax) / (max_val - min_val);
        float sum_l = 0.0f, sum_l2 = 0.0f, sum_xl = 0.0f;
        for (int i = 0; i < n; ++i) {
            uint8_t l = (uint8_t)clampi(nearest_int(iscale * (x[i] - min_val)), 0, nmax);
            Laux[i] = l;
            float w = weights ? weights[i] : x[i] * x[i];
            float lf = (float)l;
            sum_l += w * lf;
            sum_l2 += w * (lf * lf);
            sum_xl += w * lf * x[i];
        }
        float d = sum_w * sum_l2 - sum_l * sum_l;
        if (d > 0.0f) {
            float this_scale = (sum_w * sum_xl - sum_x * sum_l) / d;
            float this_min = (sum_l2 * sum_x - sum_l * sum_xl) / d;
            if (this_min > 0.0f) { this_min = 0.0f; this_scale = sum_xl / sum_l2; }
            float mad = 0.0f;
            for (int i = 0; i < n; ++i) {
                float diff = this_scale * (float)Laux[i] + this_min - x[i];
                diff = use_mad ? fabsf(diff) : diff * diff;
                float w = weights ? weights[i] : x[i] * x[i];
                mad += w * diff;
            }
            if (mad < best_mad) {
                memcpy(L, Laux, sizeof(L));
                best_mad = mad;
                scale = this_scale;
                min_val = this_min;
            }
        }
    }
    *out_scale = scale;
    *out_min = -min_val;
}

static float make_qp_quants(int n, uint8_t nmax, const float *x, uint8_t *L, const float *qw) {
    float max = 0.0f;
    for (int i = 0; i < n; ++i) max = rmaxf(max, x[i]);
    if (max == 0.0f) { for (int i = 0; i < n; ++i) L[i] = 0; return 0.0f; }
    float iscale = (float)nmax / max;
    for (int i = 0; i < n; ++i) L[i] = (uint8_t)nearest_int(iscale * x[i]);  /* i32 -> u8: wrapping, as Rust `as` */
    float scale = 1.0f / iscale;
    float best_mse = 0.0f;
    for (int i = 0; i < n; ++i) { float diff = x[i] - scale * (float)L[i]; best_mse += qw[i] * diff * diff; }
    for (int is = -4; is <= 4; ++is) {
        if (is == 0) continue;
        float iscale_is = (0.1f * (float)is + (float)nmax) / max;
        float scale_is = 1.0f / iscale_is;
        float mse = 0.0f;
        for (int i = 0; i < n; ++i) {
            uint8_t li = (uint8_t)nearest_int(iscale_is * x[i]);
            if (li > nmax) li = nmax;
            float diff = x[i] - scale_is * (float)li;
            mse += qw[i] * diff * diff;
        }
        if (mse < best_mse) { best_mse = mse; iscale = iscale_is; }
    }
    float sumlx = 0.0f, suml2 = 0.0f;
    for (int i = 0; i < n; ++i) {
        uint8_t li = sat_u8_trunc(roundf(iscale * x[i]));  /* f32 -> u8: saturating */
        if (li > nmax) li = nmax;
        L[i] = li;
        sumlx += qw[i] * x[i] * (float)li;
        suml2 += qw[i] * ((float)li * (float)li);
    }
    for (int itry = 0; itry < 5; ++itry) {
        int n_changed = 0;
        for (int i = 0; i < n; ++i) {
            float slx = sumlx - qw[i] * x[i] * (float)L[i];
            float sl2 = suml2 - qw[i] * ((float)L[i] * (float)L[i]);
            if (slx > 0.0f && sl2 > 0.0f) {
                uint8_t new_li = (uint8_t)nearest_int(x[i] * sl2 / slx);
                if (new_li > nmax) new_li = nmax;
                if (new_li != L[i]) {
                    slx += qw[i] * x[i] * (float)new_li;
                    sl2 += qw[i] * ((float)new_li * (float)new_li);
                    if ((slx * slx) * suml2 > (sumlx * sumlx) * sl2) {
                        L[i] = new_li;
                        sumlx = slx;
                        suml2 = sl2;
                        ++n_changed;
                    }
                }
            }
        }
        if (n_changed == 0) break;
    }
    return sumlx / suml2;
}

/* the (d, dmin, scales[12]) header both k-quants with 6-bit (scale, min) pairs share, imatrix form: returns through b */
static void kquant_imatrix_header(const float *xb, const float *iw, int nmax, int clamp63, uint16_t *d_out, uint16_t *dmin_out,
                                  uint8_t *scales12) {
    float mins[8], scales[8], weights[32], sw[8];
    uint8_t ls[8], lm[8];
    memset(ls, 0, sizeof(ls));
    memset(lm, 0, sizeof(lm));
    float sum_x2 = 0.0f;
    for (int t = 0; t < QK_K; ++t) sum_x2 += xb[t] * xb[t];
    float sigma2 = 2.0f * sum_x2 / (float)QK_K;
    for (int j = 0; j < 8; ++j) {
        for (int l = 0; l < 32; ++l) weights[l] = iw[32 * j + l] * sqrtf(sigma2 + xb[32 * j + l] * xb[32 * j + l]);
        float sumw = 0.0f;
        for (int l = 0; l < 32; ++l) sumw += weights[l];
        sw[j] = sumw;
        make_qkx3_quants(32, nmax, xb + 32 * j, weights, -0.9f, 0.05f, 36, 0, &scales[j], &mins[j]);
    }
    float d_block = make_qp_quants(8, 63, scales, ls, sw);
    float m_block = make_qp_quants(8, 63, mins, lm, sw);
    for (int j = 0; j < 8; ++j) {
        uint8_t lsv = ls[j], lmv = lm[j];
        if (clamp63) { if (lsv > 63) lsv = 63; if (lmv > 63) lmv = 63; }
        if (j < 4) {
            scales12[j] = lsv;
            scales12[j + 4] = lmv;
        } else {
            scales12[j + 4] = (uint8_t)((lsv & 0xF) | ((lmv & 0xF) << 4));
            scales12[j - 4] |= (uint8_t)((lsv >> 4) << 6);
            scales12[j] |= (uint8_t)((lmv >> 4) << 6);
        }
    }
    *d_out = lo_f32_to_f16(d_block);
    *dmin_out = lo_f32_to_f16(m_block);
}

static void quantize_row_q4k_imatrix(const float *x, blk_q4k *y, int64_t k, const float *imatrix) {
    for (int64_t i = 0; i < k / QK_K; ++i) {
        const float *xb = x + i * QK_K;
        blk_q4k *b = &y[i];
        memset(b, 0, sizeof(*b));
        kquant_imatrix_header(xb, imatrix + QK_K * i, 15, 0, &b->d, &b->dmin, b->scales);
        uint8_t L[QK_K];
        memset(L, 0, sizeof(L));
        float bd = lo_f16_to_f32(b->d), bdmin = lo_f16_to_f32(b->dmin);
        for (int j = 0; j < 8; ++j) {
            uint8_t sc, m;
            scale_min_k4(j, b->scales, &sc, &m);
            float d = bd * (float)sc;
            if (d != 0.0f) {
                float dm = bdmin * (float)m;
                for (int t = 0; t < 32; ++t) L[32 * j + t] = (uint8_t)clampi(nearest_int((xb[32 * j + t] + dm) / d), 0, 15);
            }
        }
        for (int g = 0; g < 4; ++g)
            for (int t = 0; t < 32; ++t) b->qs[32 * g + t] = (uint8_t)(L[64 * g + t] | (L[64 * g + 32 + t] << 4));
    }
}

static void quantize_row_q5k_imatrix(const float *x, blk_q5k *y, int64_t k, const float *imatrix) {
    for (int64_t i = 0; i < k / QK_K; ++i) {
        const float *xb = x + i * QK_K;
        blk_q5k *b = &y[i];
        memset(b, 0, sizeof(*b));
        kquant_imatrix_header(xb, imatrix + QK_K * i, 31, 1, &b->d, &b->dmin, b->scales);
        uint8_t L[QK_K];
        memset(L, 0, sizeof(L));
        float bd = lo_f16_to_f32(b->d), bdmin = lo_f16_to_f32(b->dmin);
        for (int j = 0; j < 8; ++j) {
            uint8_t sc, m;
            scale_min_k4(j, b->scales, &sc, &m);
            float d = bd * (float)sc;
            if (d != 0.0f) {
                float dm = bdmin * (float)m;
                for (int t = 0; t < 32; ++t) L[32 * j + t] = (uint8_t)clampi(nearest_int((xb[32 * j + t] + dm) / d), 0, 31);
            }
        }
        uint8_t m1 = 1, m2 = 2;
        for (int n = 0; n < QK_K; n += 64) {
            int off = (n / 64) * 32;
            for (int j = 0; j < 32; ++j) {
                uint8_t l1 = L[n + j], l2 = L[n + j + 32];
                if (l1 > 15) { l1 -= 16; b->qh[j] |= m1; }
                if (l2 > 15) { l2 -= 16; b->qh[j] |= m2; }
                b->qs[off + j] = (uint8_t)(l1 | (l2 << 4));
            }
            m1 <<= 2;
            m2 <<= 2;
        }
    }
}

/* ---- vec_dot, scalar generic order (vec_dot_unopt) ---- */

/* BlockQ8_0::vec_dot_unopt, k_quants.rs:800-818 */
static float vec_dot_q8_0_unopt(int64_t k, const blk_q8_0 *x, const blk_q8_0 *y) {
    float sumf = 0.0f;
    for (int64_t i = 0; i < k / QK8_0; ++i) {
        int32_t s = 0;
        for (int j = 0; j < QK8_0; ++j) s += (int32_t)x[i].qs[j] * (int32_t)y[i].qs[j];
        sumf += (float)s * lo_f16_to_f32(x[i].d) * lo_f16_to_f32(y[i].d);
    }
    return sumf;
}

/* the eight (scale, min) pairs of a Q4_K block, as the reference's utmp shuffle yields them */
static inline void q4k_scales_mins(const blk_q4k *b, uint8_t *sc, uint8_t *mn) {
    for (int j = 0; j < 8; ++j) scale_min_k4(j, b->scales, &sc[j], &mn[j]);
}

/* BlockQ4K::vec_dot_unopt, k_quants.rs:1540-1620 */
static float vec_dot_q4k_unopt(int64_t k, const blk_q4k *x, const blk_q8k *y) {
    float sums[8] = {0};
    float sumf = 0.0f;
    int8_t a[QK_K];
    for (int64_t i = 0; i < k / QK_K; ++i) {
        const blk_q4k *b = &x[i];
        for (int g = 0; g < 4; ++g)
            for (int t = 0; t < 32; ++t) {
                a[64 * g + t] = (int8_t)(b->qs[32 * g + t] & 0xF);
                a[64 * g + 32 + t] = (int8_t)(b->qs[32 * g + t] >> 4);
            }
        uint8_t sc[8], mn[8];
        q4k_scales_mins(b, sc, mn);
        int32_t sumi = 0;
        for (int j = 0; j < 16; ++j) sumi += (int32_t)y[i].bsums[j] * (int32_t)mn[j / 2];
        int32_t aux32[8] = {0};
        for (int j = 0; j < 8; ++j)
            for (int t = 0; t < 32; ++t)
                aux32[t & 7] += (int32_t)sc[j] * (int32_t)(int16_t)((int16_t)y[i].qs[32 * j + t] * (int16_t)a[32 * j + t]);
        float d = lo_f16_to_f32(b->d) * y[i].d;
        for (int l = 0; l < 8; ++l) sums[l] += d * (float)aux32[l];
        float dmin = lo_f16_to_f32(b->dmin) * y[i].d;
        sumf -= dmin * (float)sumi;
    }
    float s = 0.0f;
    for (int l = 0; l < 8; ++l) s += sums[l];
    return sumf + s;
}

/* BlockQ4_0::vec_dot_unopt, k_quants.rs:371-391 */
static float vec_dot_q4_0_unopt(int64_t k, const blk_q4_0 *x, const blk_q8_0 *y) {
    float sumf = 0.0f;
    int8_t c[32];
    for (int64_t i = 0; i < k / QK8_0; ++i) {
        q4_0_codes(&x[i], c);
        int32_t s = 0;
        for (int j = 0; j < 16; ++j) s += (int32_t)c[j] * y[i].qs[j] + (int32_t)c[j + 16] * y[i].qs[j + 16];
        sumf += (float)s * lo_f16_to_f32(x[i].d) * lo_f16_to_f32(y[i].d);
    }
    return sumf;
}

/* BlockQ5_0::vec_dot == vec_dot_unopt on every target, k_quants.rs:500-534 */
static float vec_dot_q5_0_unopt(int64_t k, const blk_q5_0 *x, const blk_q8_0 *y) {
    float sumf = 0.0f;
    int8_t c[32];
    for (int64_t i = 0; i < k / QK8_0; ++i) {
        q5_0_codes(&x[i], c);
        int32_t s = 0;
        for (int j = 0; j < 16; ++j) s += (int32_t)c[j] * y[i].qs[j] + (int32_t)c[j + 16] * y[i].qs[j + 16];
        sumf += (float)s * lo_f16_to_f32(x[i].d) * lo_f16_to_f32(y[i].d);
    }
    return sumf;
}

/* BlockQ5K::vec_dot_unopt, k_quants.rs:1795-1880 */
static float vec_dot_q5k_unopt(int64_t k, const blk_q5k *x, const blk_q8k *y) {
    float sums[8] = {0};
    float sumf = 0.0f;
    int8_t a[QK_K];
    for (int64_t i = 0; i < k / QK_K; ++i) {
        const blk_q5k *b = &x[i];
        q5k_codes(b, a);
        uint8_t sc[8], mn[8];
        q5k_scales_mins(b, sc, mn);
        int32_t sumi = 0;
        for (int j = 0; j < 16; ++j) sumi += (int32_t)y[i].bsums[j] * (int32_t)mn[j / 2];
        int32_t aux32[8] = {0};
        for (int j = 0; j < 8; ++j)
            for (int t = 0; t < 32; ++t)
                aux32[t & 7] += (int32_t)sc[j] * (int32_t)(int16_t)((int16_t)y[i].qs[32 * j + t] * (int16_t)a[32 * j + t]);
        float d = lo_f16_to_f32(b->d) * y[i].d;
        for (int l = 0; l < 8; ++l) sums[l] += d * (float)aux32[l];
        float dmin = lo_f16_to_f32(b->dmin) * y[i].d;
        sumf -= dmin * (float)sumi;
    }
    float s = 0.0f;
    for (int l = 0; l < 8; ++l) s += sums[l];
    return sumf + s;
}

/* BlockQ6K::vec_dot_unopt, k_quants.rs:2115-2172 (per-lane partial sums kept in f32 as there) */
static float vec_dot_q6k_unopt(int64_t k, const blk_q6k *x, const blk_q8k *y) {
    float sums[8] = {0};
    int8_t a[QK_K];
    for (int64_t i = 0; i < k / QK_K; ++i) {
        float aux32[8] = {0};
        q6k_codes(&x[i], a);
        for (int j = 0; j < 16; ++j) {
            float scale = (float)x[i].scales[j];
            for (int half = 0; half < 2; ++half)
                for (int l = 0; l < 8; ++l) {
                    int idx = 16 * j + 8 * half + l;
                    int16_t p = (int16_t)((int16_t)y[i].qs[idx] * (int16_t)a[idx]);
                    aux32[l] += scale * (float)p;
                }
        }
        float d = lo_f16_to_f32(x[i].d) * y[i].d;
        for (int l = 0; l < 8; ++l) sums[l] += aux32[l] * d;
    }
    float s = 0.0f;
    for (int l = 0; l < 8; ++l) s += sums[l];
    return s;
}

/* ---- vec_dot, AVX2 arm's order, emulated lane by lane in portable C ---- */

/* avx.rs:26-32 hsum_float_8: (hi128 + lo128), then (x + movehl), then (x + movehdup) */
static inline float hsum8_order(const float *v) {
    float r0 = v[4] + v[0], r1 = v[5] + v[1], r2 = v[6] + v[2], r3 = v[7] + v[3];
    float s0 = r0 + r2, s1 = r1 + r3;
    return s0 + s1;
}

/* avx.rs:71-87 vec_dot_q8_0_q8_0: lane i = bytes 4i..4i+3; acc = fma(dx*dy, lane, acc) */
static float vec_dot_q8_0_avx2_emu(int64_t k, const blk_q8_0 *x, const blk_q8_0 *y) {
    float acc[8] = {0};
    for (int64_t i = 0; i < k / QK8_0; ++i) {
        float d = lo_f16_to_f32(x[i].d) * lo_f16_to_f32(y[i].d);
        for (int l = 0; l < 8; ++l) {
            int32_t s = 0;
            for (int t = 0; t < 4; ++t) s += (int32_t)x[i].qs[4 * l + t] * (int32_t)y[i].qs[4 * l + t];
            acc[l] = fmaf(d, (float)s, acc[l]);
        }
    }
    return hsum8_order(acc);
}

/* avx.rs:443-525 vec_dot_q4k_q8k */
static float vec_dot_q4k_avx2_emu(int64_t k, const blk_q4k *x, const blk_q8k *y) {
    float acc[8] = {0}, acc_m[4] = {0};
    for (int64_t i = 0; i < k / QK_K; ++i) {
        const blk_q4k *b = &x[i];
        float d = y[i].d * lo_f16_to_f32(b->d);
        float dmin = -y[i].d * lo_f16_to_f32(b->dmin);
        uint8_t sc[8], mn[8];
        q4k_scales_mins(b, sc, mn);
        int16_t s[8];
        for (int j = 0; j < 8; ++j) s[j] = (int16_t)(y[i].bsums[2 * j] + y[i].bsums[2 * j + 1]);
        for (int p = 0; p < 4; ++p) {
            int32_t prod = (int32_t)mn[2 * p] * s[2 * p] + (int32_t)mn[2 * p + 1] * s[2 * p + 1];
            acc_m[p] = fmaf(dmin, (float)prod, acc_m[p]);
        }
        int32_t sumi[8] = {0};
        for (int g = 0; g < 4; ++g)
            for (int l = 0; l < 8; ++l) {
                int32_t lo = 0, hi = 0;
                for (int t = 0; t < 4; ++t) {
                    uint8_t q = b->qs[32 * g + 4 * l + t];
                    lo += (int32_t)(q & 0xF) * (int32_t)y[i].qs[64 * g + 4 * l + t];
                    hi += (int32_t)(q >> 4) * (int32_t)y[i].qs[64 * g + 32 + 4 * l + t];
                }
                sumi[l] += (int32_t)sc[2 * g] * lo + (int32_t)sc[2 * g + 1] * hi;
            }
        for (int l = 0; l < 8; ++l) acc[l] = fmaf(d, (float)sumi[l], acc[l]);
    }
    float m0 = acc_m[0] + acc_m[2], m1 = acc_m[1] + acc_m[3];
    return hsum8_order(acc) + (m0 + m1);
}

/* avx.rs:50-69 vec_dot_q4_0_q8_0: lane i = bytes 4i..4i+3 of (nibble - 8) * q8; acc = fma(dx*dy, lane, acc) */
static float vec_dot_q4_0_avx2_emu(int64_t k, const blk_q4_0 *x, const blk_q8_0 *y) {
    float acc[8] = {0};
    int8_t c[32];
    for (int64_t i = 0; i < k / QK8_0; ++i) {
        float d = lo_f16_to_f32(x[i].d) * lo_f16_to_f32(y[i].d);
        q4_0_codes(&x[i], c);
        for (int l = 0; l < 8; ++l) {
            int32_t s = 0;
            for (int t = 0; t < 4; ++t) s += (int32_t)c[4 * l + t] * (int32_t)y[i].qs[4 * l + t];
            acc[l] = fmaf(d, (float)s, acc[l]);
        }
    }
    return hsum8_order(acc);
}

/* avx.rs:528-640 vec_dot_q5k_q8k: eight int32 lanes of scale-weighted products, one fma per superblock; the min
 * term is one scalar product per superblock added to a scalar f32 */
static float vec_dot_q5k_avx2_emu(int64_t k, const blk_q5k *x, const blk_q8k *y) {
    float acc[8] = {0};
    float summs = 0.0f;
    int8_t a[QK_K];
    for (int64_t i = 0; i < k / QK_K; ++i) {
        const blk_q5k *b = &x[i];
        float d = y[i].d * lo_f16_to_f32(b->d);
        float dmin = -y[i].d * lo_f16_to_f32(b->dmin);
        uint8_t sc[8], mn[8];
        q5k_scales_mins(b, sc, mn);
        int32_t msum = 0;
        for (int j = 0; j < 8; ++j) msum += (int32_t)mn[j] * (int32_t)(int16_t)(y[i].bsums[2 * j] + y[i].bsums[2 * j + 1]);
        summs += dmin * (float)msum;
        q5k_codes(b, a);
        int32_t sumi[8] = {0};
        for (int j = 0; j < 8; ++j)
            for (int l = 0; l < 8; ++l) {
                int32_t p = 0;
                for (int t = 0; t < 4; ++t) p += (int32_t)a[32 * j + 4 * l + t] * (int32_t)y[i].qs[32 * j + 4 * l + t];
                sumi[l] += (int32_t)sc[j] * p;
            }
        for (int l = 0; l < 8; ++l) acc[l] = fmaf(d, (float)sumi[l], acc[l]);
    }
    return hsum8_order(acc) + summs;
}

/* avx.rs:131-216 vec_dot_q6k_q8k */
static float vec_dot_q6k_avx2_emu(int64_t k, const blk_q6k *x, const blk_q8k *y) {
    float acc[8] = {0};
    int8_t a[QK_K];
    for (int64_t i = 0; i < k / QK_K; ++i) {
        float d = y[i].d * lo_f16_to_f32(x[i].d);
        q6k_codes(&x[i], a);
        int32_t sumi[8] = {0};
        for (int g = 0; g < 8; ++g) /* eight groups of 32 elements; two 16-element scales each */
            for (int l = 0; l < 8; ++l) {
                int32_t p = 0;
                for (int t = 0; t < 4; ++t) p += (int32_t)a[32 * g + 4 * l + t] * (int32_t)y[i].qs[32 * g + 4 * l + t];
                sumi[l] += (int32_t)x[i].scales[2 * g + l / 4] * p;
            }
        for (int l = 0; l < 8; ++l) acc[l] = fmaf(d, (float)sumi[l], acc[l]);
    }
    return hsum8_order(acc);
}

/* ---- vec_dot, AVX2 arm with intrinsics (timed CPU baseline) ---- */
#ifdef LO_X86
#define LO_AVX2 __attribute__((target("avx2,fma")))

LO_AVX2 static inline float hsum_float_8(__m256 x) {
    __m128 r = _mm256_extractf128_ps(x, 1);
    r = _mm_add_ps(r, _mm256_castps256_ps128(x));
    r = _mm_add_ps(r, _mm_movehl_ps(r, r));
    r = _mm_add_ss(r, _mm_movehdup_ps(r));
    return _mm_cvtss_f32(r);
}

LO_AVX2 static float vec_dot_q8_0_avx2(int64_t k, const blk_q8_0 *x, const blk_q8_0 *y) {
    __m256 acc = _mm256_setzero_ps();
    const __m256i ones = _mm256_set1_epi16(1);
    for (int64_t i = 0; i < k / QK8_0; ++i) {
        __m256 d = _mm256_set1_ps(lo_f16_to_f32(x[i].d) * lo_f16_to_f32(y[i].d));
        __m256i bx = _mm256_loadu_si256((const __m256i *)x[i].qs);
        __m256i by = _mm256_loadu_si256((const __m256i *)y[i].qs);
        __m256i ax = _mm256_sign_epi8(bx, bx);
        __m256i sy = _mm256_sign_epi8(by, bx);
        __m256i dot = _mm256_maddubs_epi16(ax, sy);
        __m256 q = _mm256_cvtepi32_ps(_mm256_madd_epi16(ones, dot));
        acc = _mm256_fmadd_ps(d, q, acc);
    }
    return hsum_float_8(acc);
}

LO_AVX2 static float vec_dot_q4k_avx2(int64_t k, const blk_q4k *x, const blk_q8k *y) {
    const __m256i m4 = _mm256_set1_epi8(0xF);
    __m256 acc = _mm256_setzero_ps();
    __m128 acc_m = _mm_setzero_ps();
    for (int64_t i = 0; i < k / QK_K; ++i) {
        const blk_q4k *b = &x[i];
        float d = y[i].d * lo_f16_to_f32(b->d);
        float dmin = -y[i].d * lo_f16_to_f32(b->dmin);
        uint8_t sm[16]; /* scales 0..7 then mins 0..7 */
        q4k_scales_mins(b, sm, sm + 8);
        __m256i mins_and_scales = _mm256_cvtepu8_epi16(_mm_loadu_si128((const __m128i *)sm));
        __m256i q8sums = _mm256_loadu_si256((const __m256i *)y[i].bsums);
        __m128i q8s = _mm_hadd_epi16(_mm256_extracti128_si256(q8sums, 0), _mm256_extracti128_si256(q8sums, 1));
        __m128i prod = _mm_madd_epi16(_mm256_extracti128_si256(mins_and_scales, 1), q8s);
        acc_m = _mm_fmadd_ps(_mm_set1_ps(dmin), _mm_cvtepi32_ps(prod), acc_m);
        __m256i sumi = _mm256_setzero_si256();
        const uint8_t *q4 = b->qs;
        const int8_t *q8 = y[i].qs;
        for (int g = 0; g < 4; ++g) {
            __m256i scale_l = _mm256_set1_epi16((short)sm[2 * g]);
            __m256i scale_h = _mm256_set1_epi16((short)sm[2 * g + 1]);
            __m256i q4bits = _mm256_loadu_si256((const __m256i *)(q4 + 32 * g));
            __m256i q4l = _mm256_and_si256(q4bits, m4);
            __m256i q4h = _mm256_and_si256(_mm256_srli_epi16(q4bits, 4), m4);
            __m256i q8l = _mm256_loadu_si256((const __m256i *)(q8 + 64 * g));
            __m256i q8h = _mm256_loadu_si256((const __m256i *)(q8 + 64 * g + 32));
            sumi = _mm256_add_epi32(sumi, _mm256_madd_epi16(scale_l, _mm256_maddubs_epi16(q4l, q8l)));
            sumi = _mm256_add_epi32(sumi, _mm256_madd_epi16(scale_h, _mm256_maddubs_epi16(q4h, q8h)));
        }
        acc = _mm256_fmadd_ps(_mm256_set1_ps(d), _mm256_cvtepi32_ps(sumi), acc);
    }
    acc_m = _mm_add_ps(acc_m, _mm_movehl_ps(acc_m, acc_m));
    acc_m = _mm_add_ss(acc_m, _mm_movehdup_ps(acc_m));
    return hsum_float_8(acc) + _mm_cvtss_f32(acc_m);
}

LO_AVX2 static float vec_dot_q6k_avx2(int64_t k, const blk_q6k *x, const blk_q8k *y) {
    const __m256i m4 = _mm256_set1_epi8(0xF);
    const __m256i m2 = _mm256_set1_epi8(3);
    const __m256i m32s = _mm256_set1_epi8(32);
    __m256 acc = _mm256_setzero_ps();
    for (int64_t i = 0; i < k / QK_K; ++i) {
        float d = y[i].d * lo_f16_to_f32(x[i].d);
        const uint8_t *ql = x[i].ql;
        const uint8_t *qh = x[i].qh;
        const int8_t *q8 = y[i].qs;
        const int8_t *sc = x[i].scales;
        __m256i sumi = _mm256_setzero_si256();
        for (int h = 0; h < 2; ++h) {
            __m256i lo1 = _mm256_loadu_si256((const __m256i *)(ql + 64 * h));
            __m256i lo2 = _mm256_loadu_si256((const __m256i *)(ql + 64 * h + 32));
            __m256i hb = _mm256_loadu_si256((const __m256i *)(qh + 32 * h));
            __m256i q[4];
            q[0] = _mm256_or_si256(_mm256_and_si256(lo1, m4), _mm256_slli_epi16(_mm256_and_si256(hb, m2), 4));
            q[1] = _mm256_or_si256(_mm256_and_si256(lo2, m4),
                                   _mm256_slli_epi16(_mm256_and_si256(_mm256_srli_epi16(hb, 2), m2), 4));
            q[2] = _mm256_or_si256(_mm256_and_si256(_mm256_srli_epi16(lo1, 4), m4),
                                   _mm256_slli_epi16(_mm256_and_si256(_mm256_srli_epi16(hb, 4), m2), 4));
            q[3] = _mm256_or_si256(_mm256_and_si256(_mm256_srli_epi16(lo2, 4), m4),
                                   _mm256_slli_epi16(_mm256_and_si256(_mm256_srli_epi16(hb, 6), m2), 4));
            for (int g = 0; g < 4; ++g) {
                __m256i a8 = _mm256_loadu_si256((const __m256i *)(q8 + 128 * h + 32 * g));
                __m256i p16 = _mm256_sub_epi16(_mm256_maddubs_epi16(q[g], a8), _mm256_maddubs_epi16(m32s, a8));
                int8_t s0 = sc[8 * h + 2 * g], s1 = sc[8 * h + 2 * g + 1];
                __m256i scale = _mm256_set_m128i(_mm_set1_epi16(s1), _mm_set1_epi16(s0));
                sumi = _mm256_add_epi32(sumi, _mm256_madd_epi16(scale, p16));
            }
        }
        acc = _mm256_fmadd_ps(_mm256_set1_ps(d), _mm256_cvtepi32_ps(sumi), acc);
    }
    return hsum_float_8(acc);
}

int lo_has_avx2(void) { return __builtin_cpu_supports("avx2") && __builtin_cpu_supports("fma"); }
#else
int lo_has_avx2(void) { return 0; }
#endif

/* ---- per-element error scale ----
 * Sum of the magnitudes of the f32 summands the AVX2 arm actually adds for this element: per block,
 * the eight lane terms d * lane_sum (and, for Q4_K, the four min-lane terms).  Any re-ordering of that
 * f32 summation -- including the reference's own lane order -- is bounded relative to this scale. */
static float vec_dot_absum(int w_dtype, int64_t k, const void *w, const void *act) {
    float a = 0.0f;
    if (w_dtype == LO_Q8_0) {
        const blk_q8_0 *x = w, *y = act;
        for (int64_t i = 0; i < k / QK8_0; ++i) {
            float d = lo_f16_to_f32(x[i].d) * lo_f16_to_f32(y[i].d);
            for (int l = 0; l < 8; ++l) {
                int32_t s = 0;
                for (int t = 0; t < 4; ++t) s += (int32_t)x[i].qs[4 * l + t] * (int32_t)y[i].qs[4 * l + t];
                a += fabsf(d * (float)s);
            }
        }
    } else if (w_dtype == LO_Q4_K) {
        const blk_q4k *x = w;
        const blk_q8k *y = act;
        for (int64_t i = 0; i < k / QK_K; ++i) {
            const blk_q4k *b = &x[i];
            float d = y[i].d * lo_f16_to_f32(b->d);
            float dmin = y[i].d * lo_f16_to_f32(b->dmin);
            uint8_t sc[8], mn[8];
            q4k_scales_mins(b, sc, mn);
            for (int p = 0; p < 4; ++p) {
                int32_t prod = (int32_t)mn[2 * p] * ((int32_t)y[i].bsums[4 * p] + y[i].bsums[4 * p + 1]) +
                               (int32_t)mn[2 * p + 1] * ((int32_t)y[i].bsums[4 * p + 2] + y[i].bsums[4 * p + 3]);
                a += fabsf(dmin * (float)prod);
            }
            for (int l = 0; l < 8; ++l) {
                int32_t sumi = 0;
                for (int g = 0; g < 4; ++g) {
                    int32_t lo = 0, hi = 0;
                    for (int t = 0; t < 4; ++t) {
                        uint8_t q = b->qs[32 * g + 4 * l + t];
                        lo += (int32_t)(q & 0xF) * (int32_t)y[i].qs[64 * g + 4 * l + t];
                        hi += (int32_t)(q >> 4) * (int32_t)y[i].qs[64 * g + 32 + 4 * l + t];
                    }
                    sumi += (int32_t)sc[2 * g] * lo + (int32_t)sc[2 * g + 1] * hi;
                }
                a += fabsf(d * (float)sumi);
            }
        }
    } else if (w_dtype == LO_Q4_0) {
        const blk_q4_0 *x = w;
        const blk_q8_0 *y = act;
        int8_t c[32];
        for (int64_t i = 0; i < k / QK8_0; ++i) {
            float d = lo_f16_to_f32(x[i].d) * lo_f16_to_f32(y[i].d);
            q4_0_codes(&x[i], c);
            for (int l = 0; l < 8; ++l) {
                int32_t s = 0;
                for (int t = 0; t < 4; ++t) s += (int32_t)c[4 * l + t] * (int32_t)y[i].qs[4 * l + t];
                a += fabsf(d * (float)s);
            }
        }
    } else if (w_dtype == LO_Q5_0) { /* scalar arm: one f32 summand per block */
        const blk_q5_0 *x = w;
        const blk_q8_0 *y = act;
        int8_t c[32];
        for (int64_t i = 0; i < k / QK8_0; ++i) {
            q5_0_codes(&x[i], c);
            int32_t s = 0;
            for (int j = 0; j < 32; ++j) s += (int32_t)c[j] * (int32_t)y[i].qs[j];
            a += fabsf((float)s * lo_f16_to_f32(x[i].d) * lo_f16_to_f32(y[i].d));
        }
    } else if (w_dtype == LO_Q5_K) {
        const blk_q5k *x = w;
        const blk_q8k *y = act;
        int8_t c5[QK_K];
        for (int64_t i = 0; i < k / QK_K; ++i) {
            const blk_q5k *b = &x[i];
            float d = y[i].d * lo_f16_to_f32(b->d);
            float dmin = y[i].d * lo_f16_to_f32(b->dmin);
            uint8_t sc[8], mn[8];
            q5k_scales_mins(b, sc, mn);
            int32_t msum = 0;
            for (int j = 0; j < 8; ++j) msum += (int32_t)mn[j] * ((int32_t)y[i].bsums[2 * j] + y[i].bsums[2 * j + 1]);
            a += fabsf(dmin * (float)msum);
            q5k_codes(b, c5);
            for (int l = 0; l < 8; ++l) {
                int32_t sumi = 0;
                for (int j = 0; j < 8; ++j) {
                    int32_t p = 0;
                    for (int t = 0; t < 4; ++t) p += (int32_t)c5[32 * j + 4 * l + t] * (int32_t)y[i].qs[32 * j + 4 * l + t];
                    sumi += (int32_t)sc[j] * p;
                }
                a += fabsf(d * (float)sumi);
            }
        }
    } else if (w_dtype == LO_Q6_K) {
        const blk_q6k *x = w;
        const blk_q8k *y = act;
        int8_t c[QK_K];
        for (int64_t i = 0; i < k / QK_K; ++i) {
            float d = y[i].d * lo_f16_to_f32(x[i].d);
            q6k_codes(&x[i], c);
            for (int l = 0; l < 8; ++l) {
                int32_t sumi = 0;
                for (int g = 0; g < 8; ++g) {
                    int32_t p = 0;
                    for (int t = 0; t < 4; ++t) p += (int32_t)c[32 * g + 4 * l + t] * (int32_t)y[i].qs[32 * g + 4 * l + t];
                    sumi += (int32_t)x[i].scales[2 * g + l / 4] * p;
                }
                a += fabsf(d * (float)sumi);
            }
        }
    }
    return a;
}

/* ---- BarrierPool (lloom-tensor/src/utils.rs:10-307): persistent workers, one 64-byte slot each with a `go`
 * generation the parent release-stores and a `done` generation the worker release-stores; a two-level tree (main
 * signals one leader per cluster, leaders signal their followers; completion reduces the same way) that is flat
 * where the cluster size is unknown (utils.rs:94-103: every platform but macOS); workers spin 10,000 times on `go`,
 * then park; main runs the last share itself and spins on the roots' `done` (utils.rs:233-275). ---- */
typedef void (*lo_task_fn)(int tid, void *ctx);
#define LO_MAX_THREADS 256
#define LO_SPIN_LIMIT 10000
struct lo_slot {
    _Alignas(64) atomic_ulong go;
    atomic_ulong done;
    /* park / unpark with a token, like std::thread::park (an unpark before the park makes it return at once) */
    pthread_mutex_t mu;
    pthread_cond_t cv;
    int token;
    int n_children;
    int children[LO_MAX_THREADS / 2];
};
static struct {
    pthread_mutex_t call_lock; /* serializes callers; guards everything below but the slots' atomics */
    int n_workers;             /* workers of the current tree (threads started: n_started >= n_workers) */
    int n_started;
    size_t cluster_size;       /* 0 or 1: flat */
    unsigned long gen;
    lo_task_fn fn;
    void *ctx;
    int n_roots;
    int roots[LO_MAX_THREADS];
    pthread_t th[LO_MAX_THREADS];
    struct lo_slot slots[LO_MAX_THREADS];
} g_pool = {.call_lock = PTHREAD_MUTEX_INITIALIZER};

static inline void lo_spin(void) {
#ifdef LO_X86
    __builtin_ia32_pause();
#endif
}
static void lo_park(struct lo_slot *s) {
    pthread_mutex_lock(&s->mu);
    while (!s->token) pthread_cond_wait(&s->cv, &s->mu);
    s->token = 0;
    pthread_mutex_unlock(&s->mu);
}
static void lo_unpark(struct lo_slot *s) {
    pthread_mutex_lock(&s->mu);
    s->token = 1;
    pthread_cond_signal(&s->cv);
    pthread_mutex_unlock(&s->mu);
}

/* compute_tree (utils.rs:62-92): the first worker of each cluster leads it; the first cluster is main plus
 * cluster_size - 1 workers, whose first worker stands in as leader for main */
static void lo_build_tree(int n_workers, size_t cluster_size) {
    for (int i = 0; i < n_workers; ++i) g_pool.slots[i].n_children = 0;
    g_pool.n_roots = 0;
    if (n_workers == 0 || cluster_size <= 1 || cluster_size >= (size_t)LO_MAX_THREADS) {
        for (int i = 0; i < n_workers; ++i) g_pool.roots[g_pool.n_roots++] = i;
        return;
    }
    int c0 = (int)cluster_size - 1 < n_workers ? (int)cluster_size - 1 : n_workers;
    g_pool.roots[g_pool.n_roots++] = 0;
    for (int f = 1; f < c0; ++f) g_pool.slots[0].children[g_pool.slots[0].n_children++] = f;
    int next = c0;
    while (next < n_workers) {
        const int leader = next;
        g_pool.roots[g_pool.n_roots++] = leader;
        const int end = n_workers < next + (int)cluster_size ? n_workers : next + (int)cluster_size;
        for (int f = leader + 1; f < end; ++f) g_pool.slots[leader].children[g_pool.slots[leader].n_children++] = f;
        next = end;
    }
}

static void *pool_worker(void *arg) {
    const int tid = (int)(intptr_t)arg;
    struct lo_slot *slot = &g_pool.slots[tid];
    unsigned long gen = atomic_load_explicit(&slot->done, memory_order_acquire); /* the generation it was started in */
    for (;;) {
        unsigned spins = 0;
        for (;;) { /* spin briefly, then park, waiting for the next work item */
            const unsigned long g = atomic_load_explicit(&slot->go, memory_order_acquire);
            if (g != gen) { gen = g; break; }
            if (++spins < LO_SPIN_LIMIT) lo_spin();
            else { lo_park(slot); spins = 0; }
        }
        /* fan the work out to the children */
        for (int c = 0; c < slot->n_children; ++c) {
            struct lo_slot *ch = &g_pool.slots[slot->children[c]];
            atomic_store_explicit(&ch->go, gen, memory_order_release);
            lo_unpark(ch);
        }
        g_pool.fn(tid, g_pool.ctx);
        /* reduce: all children before the parent hears of it */
        for (int c = 0; c < slot->n_children; ++c)
            while (atomic_load_explicit(&g_pool.slots[slot->children[c]].done, memory_order_acquire) != gen) lo_spin();
        atomic_store_explicit(&slot->done, gen, memory_order_release);
    }
    return 0;
}

/* cluster size of the tree (utils.rs:94-103 hard-codes 6 on macOS and "flat" elsewhere); 0 = flat.  Takes effect with
 * the next lo_parallel call. */
void lo_set_cluster_size(int cluster_size) {
    pthread_mutex_lock(&g_pool.call_lock);
    g_pool.cluster_size = cluster_size > 0 ? (size_t)cluster_size : 0;
    g_pool.n_workers = -1; /* rebuild the tree */
    pthread_mutex_unlock(&g_pool.call_lock);
}

/* BarrierPool::execute (utils.rs:233-275): runs fn(tid, ctx) for tid in 0..nthreads; workers are 0..nthreads-2, the
 * caller takes part as the last tid */
static void lo_parallel(int nthreads, lo_task_fn fn, void *ctx) {
    if (nthreads > LO_MAX_THREADS) nthreads = LO_MAX_THREADS;
    if (nthreads <= 1) { fn(0, ctx); return; }
    pthread_mutex_lock(&g_pool.call_lock);
    int want = nthreads - 1;
    while (g_pool.n_started < want) {
        const int tid = g_pool.n_started;
        struct lo_slot *s = &g_pool.slots[tid];
        atomic_store(&s->go, g_pool.gen);
        atomic_store(&s->done, g_pool.gen);
        pthread_mutex_init(&s->mu, 0);
        pthread_cond_init(&s->cv, 0);
        s->token = 0;
        s->n_children = 0;
        if (pthread_create(&g_pool.th[tid], 0, pool_worker, (void *)(intptr_t)tid) != 0) break;
        pthread_detach(g_pool.th[tid]);
        ++g_pool.n_started;
    }
    if (want > g_pool.n_started) want = g_pool.n_started;
    if (want != g_pool.n_workers) { /* all workers are idle here: nobody reads the tree */
        lo_build_tree(want, g_pool.cluster_size);
        g_pool.n_workers = want;
    }
    const unsigned long gen = ++g_pool.gen;
    g_pool.fn = fn;
    g_pool.ctx = ctx;
    for (int r = 0; r < g_pool.n_roots; ++r) {
        struct lo_slot *s = &g_pool.slots[g_pool.roots[r]];
        atomic_store_explicit(&s->go, gen, memory_order_release);
        lo_unpark(s);
    }
    for (int t = want; t < nthreads; ++t) fn(t, ctx); /* main's share (and that of any thread that could not start) */
    for (int r = 0; r < g_pool.n_roots; ++r)
        while (atomic_load_explicit(&g_pool.slots[g_pool.roots[r]].done, memory_order_acquire) != gen) lo_spin();
    pthread_mutex_unlock(&g_pool.call_lock);
}

/* ---- public entry points ---- */

int lo_quantize_row(int dtype, const float *x, void *blocks, int64_t k) {
    int64_t be = lo_block_elems(dtype);
    if (be == 0 || k % be != 0) return -2;
    switch (dtype) {
    case LO_Q8_0: quantize_row_q8_0(x, blocks, k); return 0;
    case LO_Q4_K: quantize_row_q4k(x, blocks, k); return 0;
    case LO_Q6_K: quantize_row_q6k(x, blocks, k); return 0;
    case LO_Q8_K: quantize_row_q8k(x, blocks, k); return 0;
    case LO_Q4_0: quantize_row_q4_0(x, blocks, k); return 0;
    case LO_Q5_0: quantize_row_q5_0(x, blocks, k); return 0;
    case LO_Q5_K: quantize_row_q5k(x, blocks, k); return 0;
    }
    return -2;
}

/* T::from_float_imatrix over one row of k = n_per_row elements: the importance weights are one per column
 * (QTensor::quantize_imatrix, mod.rs:940-975); only Q4K, Q5K and Q6K of this oracle's formats implement it. */
int lo_quantize_row_imatrix(int dtype, const float *x, void *blocks, int64_t k, const float *imatrix) {
    if (k % QK_K != 0) return -2;
    switch (dtype) {
    case LO_Q4_K: quantize_row_q4k_imatrix(x, blocks, k, imatrix); return 0;
    case LO_Q5_K: quantize_row_q5k_imatrix(x, blocks, k, imatrix); return 0;
    case LO_Q6_K: quantize_row_q6k_w(x, blocks, k, imatrix); return 0;
    }
    return -2;
}

struct qrows_ctx { int dtype; const float *x; void *blocks; int64_t rows, k, row_bytes; int nthreads; };
static void qrows_task(int tid, void *p) {
    struct qrows_ctx *c = p;
    int64_t per = (c->rows + c->nthreads - 1) / c->nthreads;
    int64_t r0 = tid * per, r1 = r0 + per < c->rows ? r0 + per : c->rows;
    for (int64_t r = r0; r < r1; ++r)
        lo_quantize_row(c->dtype, c->x + r * c->k, (char *)c->blocks + r * c->row_bytes, c->k);
}

int lo_quantize_rows(int dtype, const float *x, void *blocks, int64_t rows, int64_t k, int nthreads) {
    int64_t be = lo_block_elems(dtype), bb = lo_block_bytes(dtype);
    if (be == 0 || k % be != 0) return -2;
    if (nthreads < 1) nthreads = 1;
    struct qrows_ctx c = {dtype, x, blocks, rows, k, k / be * bb, nthreads};
    lo_parallel(nthreads, qrows_task, &c);
    return 0;
}

int lo_dequantize_row(int dtype, const void *blocks, float *y, int64_t k) {
    int64_t be = lo_block_elems(dtype);
    if (be == 0 || k % be != 0) return -2;
    switch (dtype) {
    case LO_Q8_0: dequantize_row_q8_0(blocks, y, k); return 0;
    case LO_Q4_K: dequantize_row_q4k(blocks, y, k); return 0;
    case LO_Q6_K: dequantize_row_q6k(blocks, y, k); return 0;
    case LO_Q8_K: dequantize_row_q8k(blocks, y, k); return 0;
    case LO_Q4_0: dequantize_row_q4_0(blocks, y, k); return 0;
    case LO_Q5_0: dequantize_row_q5_0(blocks, y, k); return 0;
    case LO_Q5_K: dequantize_row_q5k(blocks, y, k); return 0;
    }
    return -2;
}

typedef float (*dot_fn)(int64_t, const void *, const void *);

static dot_fn pick_dot(int w_dtype, int order) {
    /* Q5_0 has no vectorised arm: vec_dot is vec_dot_unopt on every target (k_quants.rs:500-513).  Q4_0 and Q5_K
     * have AVX2 arms (avx.rs:50-69, 528-640); the oracle holds their lane order in portable C only. */
    if (w_dtype == LO_Q5_0) return (dot_fn)vec_dot_q5_0_unopt;
    if (order == LO_ORDER_AVX2 && (w_dtype == LO_Q4_0 || w_dtype == LO_Q5_K)) order = LO_ORDER_AVX2_EMU;
#ifdef LO_X86
    if (order == LO_ORDER_AVX2) {
        if (!lo_has_avx2()) return 0;
        switch (w_dtype) {
        case LO_Q8_0: return (dot_fn)vec_dot_q8_0_avx2;
        case LO_Q4_K: return (dot_fn)vec_dot_q4k_avx2;
        case LO_Q6_K: return (dot_fn)vec_dot_q6k_avx2;
        }
        return 0;
    }
#endif
    if (order == LO_ORDER_AVX2_EMU) {
        switch (w_dtype) {
        case LO_Q8_0: return (dot_fn)vec_dot_q8_0_avx2_emu;
        case LO_Q4_K: return (dot_fn)vec_dot_q4k_avx2_emu;
        case LO_Q6_K: return (dot_fn)vec_dot_q6k_avx2_emu;
        case LO_Q4_0: return (dot_fn)vec_dot_q4_0_avx2_emu;
        case LO_Q5_K: return (dot_fn)vec_dot_q5k_avx2_emu;
        }
        return 0;
    }
    if (order == LO_ORDER_UNOPT) {
        switch (w_dtype) {
        case LO_Q4_0: return (dot_fn)vec_dot_q4_0_unopt;
        case LO_Q5_K: return (dot_fn)vec_dot_q5k_unopt;
        case LO_Q8_0: return (dot_fn)vec_dot_q8_0_unopt;
        case LO_Q4_K: return (dot_fn)vec_dot_q4k_unopt;
        case LO_Q6_K: return (dot_fn)vec_dot_q6k_unopt;
        }
    }
    return 0;
}

float lo_vec_dot(int w_dtype, int64_t k, const void *w, const void *act, int order) {
    dot_fn f = pick_dot(w_dtype, order);
    if (!f) return NAN;
    return f(k, w, act);
}

float lo_vec_dot_absum(int w_dtype, int64_t k, const void *w, const void *act) {
    return vec_dot_absum(w_dtype, k, w, act);
}

/* VecDotType of each weight type: k_quants.rs:717 (Q8_0 -> Q8_0), 1507 (Q4K -> Q8K), 2082 (Q6K -> Q8K) */
static int act_dtype_of(int w_dtype) {
    switch (w_dtype) {
    case LO_Q8_0: case LO_Q4_0: case LO_Q5_0: return LO_Q8_0;   /* k_quants.rs:296, 498 */
    case LO_Q4_K: case LO_Q5_K: case LO_Q6_K: return LO_Q8_K;   /* k_quants.rs:1781 */
    }
    return 0;
}

int lo_quantize_act(int w_dtype, const float *lhs, void *act_blocks, int64_t m, int64_t k) {
    int adt = act_dtype_of(w_dtype);
    if (!adt) return -2;
    int64_t be = lo_block_elems(adt), bb = lo_block_bytes(adt);
    if (k % be != 0) return -2;
    for (int64_t r = 0; r < m; ++r) lo_quantize_row(adt, lhs + r * k, (char *)act_blocks + r * (k / be) * bb, k);
    return 0;
}

/* k_quants::matmul, k_quants.rs:2455-2641.  mode 0: vec_dot in `order`; mode 1: absum. */
struct mm_ctx {
    int w_dtype, mode, nthreads;
    int64_t m, k, n, w_row, a_row, quads_total, qpt, row; /* row: the single LHS row of the m == 1 dispatch */
    const char *wb, *act;
    float *dst;
    dot_fn dot;
};
static inline float mm_dot(const struct mm_ctx *c, int64_t col, int64_t r) {
    const char *wp = c->wb + col * c->w_row, *ap = c->act + r * c->a_row;
    return c->mode == 0 ? c->dot(c->k, wp, ap) : vec_dot_absum(c->w_dtype, c->k, wp, ap);
}
/* m > 1: per thread, column tiles of 4 quads x row tiles of 16 (k_quants.rs:2518-2585) */
static void mm_task_tiled(int tid, void *p) {
    const struct mm_ctx *c = p;
    int64_t start = tid * c->qpt;
    int64_t end = start + c->qpt < c->quads_total ? start + c->qpt : c->quads_total;
    for (int64_t ct = start; ct < end; ct += 4) {
        int64_t ce = ct + 4 < end ? ct + 4 : end;
        for (int64_t rt = 0; rt < c->m; rt += 16)
            for (int64_t q = ct; q < ce; ++q)
                for (int64_t r = rt; r < (rt + 16 < c->m ? rt + 16 : c->m); ++r)
                    for (int j = 0; j < 4; ++j) c->dst[r * c->n + q * 4 + j] = mm_dot(c, q * 4 + j, r);
    }
}
/* m == 1: column quads split evenly (k_quants.rs:2587-2618) */
static void mm_task_row(int tid, void *p) {
    const struct mm_ctx *c = p;
    int64_t start = tid * c->qpt;
    int64_t end = (tid + 1) * c->qpt < c->quads_total ? (tid + 1) * c->qpt : c->quads_total;
    for (int64_t q = start; q < end; ++q)
        for (int j = 0; j < 4; ++j) c->dst[c->row * c->n + q * 4 + j] = mm_dot(c, q * 4 + j, c->row);
}

static int matmul_impl(int w_dtype, int64_t m, int64_t k, int64_t n, const float *lhs, const void *w, float *dst,
                       int64_t dst_len, int nthreads, int order, int mode) {
    int adt = act_dtype_of(w_dtype);
    if (!adt) return -2;
    int64_t be = lo_block_elems(w_dtype);
    if (k % be != 0) return -2;
    dot_fn dot = mode == 0 ? pick_dot(w_dtype, order) : 0;
    if (mode == 0 && !dot) return -2;
    if (m > 1 && dst_len < m * n) return -1; /* "destination is too short", k_quants.rs:2522-2524 */
    if (nthreads < 1) nthreads = 1;
    if (nthreads > LO_MAX_THREADS) nthreads = LO_MAX_THREADS;
    struct mm_ctx c;
    c.w_dtype = w_dtype; c.mode = mode; c.nthreads = nthreads;
    c.m = m; c.k = k; c.n = n;
    c.w_row = k / be * lo_block_bytes(w_dtype);
    c.a_row = k / lo_block_elems(adt) * lo_block_bytes(adt);
    char *act = malloc((size_t)(m * c.a_row) + 8);
    if (!act) return -3;
    lo_quantize_act(w_dtype, lhs, act, m, k);
    c.wb = w; c.act = act; c.dst = dst; c.dot = dot;
    int64_t n_quad = n & ~(int64_t)3;
    c.quads_total = n_quad / 4;
    c.qpt = (c.quads_total + nthreads - 1) / nthreads;
    c.row = 0;
    if (m > 1) {
        lo_parallel(nthreads, mm_task_tiled, &c);
        for (int64_t r = 0; r < m; ++r)
            for (int64_t col = n_quad; col < n; ++col) dst[r * n + col] = mm_dot(&c, col, r);
    } else {
        for (int64_t r = 0; r < m; ++r) {
            c.row = r;
            lo_parallel(nthreads, mm_task_row, &c);
            for (int64_t col = n_quad; col < n; ++col) dst[r * n + col] = mm_dot(&c, col, r);
        }
    }
    free(act);
    return 0;
}

int lo_matmul(int w_dtype, int64_t m, int64_t k, int64_t n, const float *lhs, const void *w, float *dst,
              int64_t dst_len, int nthreads, int order) {
    return matmul_impl(w_dtype, m, k, n, lhs, w, dst, dst_len, nthreads, order, 0);
}

int lo_matmul_absum(int w_dtype, int64_t m, int64_t k, int64_t n, const float *lhs, const void *w, float *dst,
                    int nthreads) {
    return matmul_impl(w_dtype, m, k, n, lhs, w, dst, m * n, nthreads, 0, 1);
}
