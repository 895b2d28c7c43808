// C++ host layer over the C ABI (see qcuda_storage.hpp) and its C view (include/lloom_b200_host.h).
#include "qcuda_storage.hpp"

#include <cuda_runtime.h>

#include <algorithm>
#include <cmath>
#include <cstring>
#include <limits>
#include <mutex>
#include <thread>

#include "../../../include/lloom_b200.h"
#include "../../../include/lloom_b200_host.h"

namespace lloom {
namespace host {

namespace {

constexpr int64_t kMatrixRowPadding = 512;  // cuda.rs MATRIX_ROW_PADDING: tail padding in elements

void cuda_check(cudaError_t e, const char *what) {
    if (e != cudaSuccess) throw Error(LLOOM_ERR_LAUNCH, std::string(what) + ": " + cudaGetErrorString(e));
}
void status_check(int status, const char *what) {
    if (status != LLOOM_OK) throw Error(status, std::string(what) + ": " + lloom_b200_error_string(status));
}

struct DeviceGuard {
    int prev = 0;
    explicit DeviceGuard(int ordinal) {
        cuda_check(cudaGetDevice(&prev), "cudaGetDevice");
        if (prev != ordinal) cuda_check(cudaSetDevice(ordinal), "cudaSetDevice");
    }
    ~DeviceGuard() { cudaSetDevice(prev); }
};

// Grow-only scratch per device, held under a lock across the launches that use it -- the role of
// WORKSPACES in fast_mmvq.rs:44-81 / fast_mmq.rs:135-174.
struct Workspace {
    std::mutex mu;
    void *ptr = nullptr;
    int64_t bytes = 0;
};
Workspace &workspace_for(int ordinal) {
    static Workspace ws[64];
    return ws[(ordinal >= 0 && ordinal < 64) ? ordinal : 0];
}

// ---- scalar conventions of the reference's quantizers ----
// f32 -> f16 bits, round to nearest even, subnormals kept (crate `half`).
uint16_t f32_to_f16(float f) {
    uint32_t x;
    std::memcpy(&x, &f, 4);
    const uint16_t sign = (uint16_t)((x >> 16) & 0x8000u);
    const uint32_t exp = (x >> 23) & 0xff;
    uint32_t man = x & 0x7fffffu;
    if (exp == 0xff) return (uint16_t)(sign | 0x7c00u | (man ? (0x200u | (man >> 13)) : 0));
    const int e = (int)exp - 112;
    if (e >= 31) return (uint16_t)(sign | 0x7c00u);
    if (e <= 0) {
        if (e < -10) return sign;
        man |= 0x800000u;
        const int shift = 14 - e;
        uint32_t h = man >> shift;
        const uint32_t rem = man & ((1u << shift) - 1), half = 1u << (shift - 1);
        if (rem > half || (rem == half && (h & 1))) ++h;
        return (uint16_t)(sign | h);
    }
    uint32_t h = ((uint32_t)e << 10) | (man >> 13);
    const uint32_t rem = man & 0x1fffu;
    if (rem > 0x1000u || (rem == 0x1000u && (h & 1))) ++h;
    return (uint16_t)(sign | h);
}
float f16_to_f32(uint16_t h) {
    const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1f, man = h & 0x3ffu, bits;
    if (exp == 0) {
        if (man == 0) bits = sign;
        else {
            int shift = 0;
            while (!(man & 0x400u)) { man <<= 1; ++shift; }
            bits = sign | ((uint32_t)(113 - shift) << 23) | ((man & 0x3ffu) << 13);
        }
    } else if (exp == 31) bits = sign | 0x7f800000u | (man << 13);
    else bits = sign | ((exp + 112) << 23) | (man << 13);
    float f;
    std::memcpy(&f, &bits, 4);
    return f;
}
// Rust `as i32` / `as i8` from f32 saturate and send NaN to 0; f32::round is half-away = roundf.
int32_t to_i32(float v) {
    if (std::isnan(v)) return 0;
    if (v >= 2147483648.0f) return std::numeric_limits<int32_t>::max();
    if (v <= -2147483648.0f) return std::numeric_limits<int32_t>::min();
    return (int32_t)v;
}
int32_t nearest_int(float v) { return to_i32(std::round(v)); }
int32_t clampi(int32_t v, int32_t lo, int32_t hi) { return std::min(std::max(v, lo), hi); }

// ---- Q8_0: k_quants.rs:738-767 ----
void quantize_q8_0(const float *x, uint8_t *out, int64_t k) {
    for (int64_t b = 0; b < k / 32; ++b, x += 32, out += 34) {
        float amax = 0.0f;
        for (int i = 0; i < 32; ++i) {
            const float a = std::fabs(x[i]);
            if (a > amax) amax = a;  // f32::max skips NaN
        }
        const float d = amax / 127.0f;
        const float id = d != 0.0f ? 1.0f / d : 0.0f;
        const uint16_t hd = f32_to_f16(d);
        std::memcpy(out, &hd, 2);
        for (int i = 0; i < 32; ++i) {
            const float r = std::round(x[i] * id);
            out[2 + i] = (uint8_t)(int8_t)(std::isnan(r) ? 0 : (int)std::min(std::max(r, -128.0f), 127.0f));
        }
    }
}

// ---- Q4_K: k_quants.rs:1622-1680 + utils.rs:227-284 (make_qkx1_quants(15, 5, .)) ----
void qkx1(const float *x, float &scale_out, float &min_out, int nmax = 15) {
    constexpr int n = 32, ntry = 5;
    uint8_t L[n] = {0};
    float mn = x[0], mx = x[0];
    for (int i = 1; i < n; ++i) { mn = std::min(mn, x[i]); mx = std::max(mx, x[i]); }
    if (mx == mn) { scale_out = 0.0f; min_out = 0.0f; return; }
    if (mn > 0.0f) mn = 0.0f;
    float iscale = (float)nmax / (mx - mn);
    float scale = 1.0f / iscale;
    for (int it = 0; it < ntry; ++it) {
        float sumlx = 0.0f;
        int32_t suml2 = 0;
        bool changed = false;
        for (int i = 0; i < n; ++i) {
            const int32_t li = clampi(nearest_int(iscale * (x[i] - mn)), 0, nmax);
            if ((uint8_t)li != L[i]) { L[i] = (uint8_t)li; changed = true; }
            sumlx += (x[i] - mn) * (float)li;
            suml2 += li * li;
        }
        scale = sumlx / (float)suml2;
        float sum = 0.0f;
        for (int i = 0; i < n; ++i) sum += x[i] - scale * (float)L[i];
        mn = sum / (float)n;
        if (mn > 0.0f) mn = 0.0f;
        iscale = 1.0f / scale;
        if (!changed) break;
    }
    scale_out = scale;
    min_out = -mn;
}
void scale_min_k4(int j, const uint8_t *q, uint8_t &sc, uint8_t &m) {  // utils.rs:50-60
    if (j < 4) { sc = q[j] & 63; m = q[j + 4] & 63; }
    else { sc = (uint8_t)((q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4)); m = (uint8_t)((q[j + 4] >> 4) | ((q[j] >> 6) << 4)); }
}
void quantize_q4k(const float *x, uint8_t *out, int64_t k) {
    for (int64_t b = 0; b < k / 256; ++b, x += 256, out += 144) {
        std::memset(out, 0, 144);
        uint8_t *scales = out + 4, *qs = out + 16;
        float mins[8], sc[8];
        for (int j = 0; j < 8; ++j) qkx1(x + 32 * j, sc[j], mins[j]);
        float max_scale = 0.0f, max_min = 0.0f;
        for (int j = 0; j < 8; ++j) { max_scale = std::max(sc[j], max_scale); max_min = std::max(mins[j], max_min); }
        const float inv_scale = max_scale > 0.0f ? 63.0f / max_scale : 0.0f;
        const float inv_min = max_min > 0.0f ? 63.0f / max_min : 0.0f;
        for (int j = 0; j < 8; ++j) {
            const uint8_t ls = (uint8_t)std::min(nearest_int(inv_scale * sc[j]), 63);
            const uint8_t lm = (uint8_t)std::min(nearest_int(inv_min * mins[j]), 63);
            if (j < 4) { scales[j] = ls; scales[j + 4] = lm; }
            else {
                scales[j + 4] = (uint8_t)((ls & 0xF) | ((lm & 0xF) << 4));
                scales[j - 4] |= (uint8_t)((ls >> 4) << 6);
                scales[j] |= (uint8_t)((lm >> 4) << 6);
            }
        }
        const uint16_t hd = f32_to_f16(max_scale / 63.0f), hm = f32_to_f16(max_min / 63.0f);
        std::memcpy(out, &hd, 2);
        std::memcpy(out + 2, &hm, 2);
        const float d = f16_to_f32(hd), dmin = f16_to_f32(hm);
        uint8_t L[256] = {0};
        for (int j = 0; j < 8; ++j) {
            uint8_t s, m;
            scale_min_k4(j, scales, s, m);
            const float dj = d * (float)s;
            if (dj == 0.0f) continue;
            const float dm = dmin * (float)m;
            for (int t = 0; t < 32; ++t) L[32 * j + t] = (uint8_t)clampi(nearest_int((x[32 * j + t] + dm) / dj), 0, 15);
        }
        for (int g = 0; g < 4; ++g)
            for (int t = 0; t < 32; ++t) qs[32 * g + t] = (uint8_t)(L[64 * g + t] | (L[64 * g + 32 + t] << 4));
    }
}

// ---- Q5_K: k_quants.rs:1883-1968 (make_qkx1_quants(31, 5, .), the Q4_K scale scheme, a fifth bit in qh) ----
void quantize_q5k(const float *x, uint8_t *out, int64_t k) {
    for (int64_t b = 0; b < k / 256; ++b, x += 256, out += 176) {
        std::memset(out, 0, 176);
        uint8_t *scales = out + 4, *qh = out + 16, *qs = out + 48;
        float mins[8], sc[8];
        for (int j = 0; j < 8; ++j) qkx1(x + 32 * j, sc[j], mins[j], 31);
        float max_scale = 0.0f, max_min = 0.0f;
        for (int j = 0; j < 8; ++j) { max_scale = std::max(sc[j], max_scale); max_min = std::max(mins[j], max_min); }
        const float inv_scale = max_scale > 0.0f ? 63.0f / max_scale : 0.0f;
        const float inv_min = max_min > 0.0f ? 63.0f / max_min : 0.0f;
        for (int j = 0; j < 8; ++j) {
            const uint8_t ls = (uint8_t)std::min(nearest_int(inv_scale * sc[j]), 63);
            const uint8_t lm = (uint8_t)std::min(nearest_int(inv_min * mins[j]), 63);
            if (j < 4) { scales[j] = ls; scales[j + 4] = lm; }
            else {
                scales[j + 4] = (uint8_t)((ls & 0xF) | ((lm & 0xF) << 4));
                scales[j - 4] |= (uint8_t)((ls >> 4) << 6);
                scales[j] |= (uint8_t)((lm >> 4) << 6);
            }
        }
        const uint16_t hd = f32_to_f16(max_scale / 63.0f), hm = f32_to_f16(max_min / 63.0f);
        std::memcpy(out, &hd, 2);
        std::memcpy(out + 2, &hm, 2);
        const float d = f16_to_f32(hd), dmin = f16_to_f32(hm);
        uint8_t L[256] = {0};
        for (int j = 0; j < 8; ++j) {
            uint8_t s, m;
            scale_min_k4(j, scales, s, m);
            const float dj = d * (float)s;
            if (dj == 0.0f) continue;
            const float dm = dmin * (float)m;
            for (int t = 0; t < 32; ++t) L[32 * j + t] = (uint8_t)clampi(nearest_int((x[32 * j + t] + dm) / dj), 0, 31);
        }
        uint8_t m1 = 1, m2 = 2;
        for (int g = 0; g < 4; ++g) {
            for (int t = 0; t < 32; ++t) {
                uint8_t l1 = L[64 * g + t], l2 = L[64 * g + 32 + t];
                if (l1 > 15) { l1 -= 16; qh[t] |= m1; }
                if (l2 > 15) { l2 -= 16; qh[t] |= m2; }
                qs[32 * g + t] = (uint8_t)(l1 | (l2 << 4));
            }
            m1 <<= 2;
            m2 <<= 2;
        }
    }
}

// Rust `f32 as u8` / `as i8`: truncation toward zero, saturating, NaN -> 0.
uint8_t trunc_u8(float v) {
    if (std::isnan(v) || v <= 0.0f) return 0;
    return v >= 255.0f ? 255 : (uint8_t)v;
}
int8_t trunc_i8(float v) {
    if (std::isnan(v)) return 0;
    if (v <= -128.0f) return -128;
    return v >= 127.0f ? 127 : (int8_t)v;
}
// The element of largest magnitude, first one on ties (`if amax < x.abs()`).
float first_max_by_abs(const float *x, int n) {
    float amax = 0.0f, mx = 0.0f;
    for (int i = 0; i < n; ++i)
        if (amax < std::fabs(x[i])) { amax = std::fabs(x[i]); mx = x[i]; }
    return mx;
}
// ---- Q4_0: k_quants.rs:320-352 ----
void quantize_q4_0(const float *x, uint8_t *out, int64_t k) {
    for (int64_t b = 0; b < k / 32; ++b, x += 32, out += 18) {
        const float d = first_max_by_abs(x, 32) / -8.0f;
        const float id = d != 0.0f ? 1.0f / d : 0.0f;
        const uint16_t hd = f32_to_f16(d);
        std::memcpy(out, &hd, 2);
        for (int j = 0; j < 16; ++j) {
            const uint8_t xi0 = std::min<uint8_t>(15, trunc_u8(x[j] * id + 8.5f));
            const uint8_t xi1 = std::min<uint8_t>(15, trunc_u8(x[16 + j] * id + 8.5f));
            out[2 + j] = (uint8_t)(xi0 | (xi1 << 4));
        }
    }
}
// ---- Q5_0: k_quants.rs:536-575 ----
void quantize_q5_0(const float *x, uint8_t *out, int64_t k) {
    for (int64_t b = 0; b < k / 32; ++b, x += 32, out += 22) {
        const float d = first_max_by_abs(x, 32) / -16.0f;
        const float id = d != 0.0f ? 1.0f / d : 0.0f;
        const uint16_t hd = f32_to_f16(d);
        std::memcpy(out, &hd, 2);
        uint32_t qh = 0;
        for (int j = 0; j < 16; ++j) {
            const uint8_t xi0 = (uint8_t)std::min<int8_t>(trunc_i8(x[j] * id + 16.5f), 31);
            const uint8_t xi1 = (uint8_t)std::min<int8_t>(trunc_i8(x[j + 16] * id + 16.5f), 31);
            out[6 + j] = (uint8_t)((xi0 & 0x0F) | ((xi1 & 0x0F) << 4));
            qh |= (((uint32_t)xi0 & 0x10u) >> 4) << j;
            qh |= (((uint32_t)xi1 & 0x10u) >> 4) << (j + 16);
        }
        std::memcpy(out + 2, &qh, 4);  // little-endian host, as LittleEndian::write_u32
    }
}

// ---- Q6_K: k_quants.rs:2174-2244 + utils.rs:62-224 (make_qx_quants(16, 32, ., ., 1, null)) ----
float qx_w2(const float *x, int8_t *ls, const float *qw = nullptr) {
    constexpr int n = 16, nmax = 32;
    float mx = 0.0f, amax = 0.0f;
    for (int i = 0; i < n; ++i) {
        const float a = std::fabs(x[i]);
        if (a > amax) { amax = a; mx = x[i]; }
    }
    if (amax == 0.0f) { std::memset(ls, 0, n); return 0.0f; }
    const float iscale0 = -(float)nmax / mx;
    float sumlx = 0.0f, suml2 = 0.0f;
    for (int i = 0; i < n; ++i) {
        const int32_t l = clampi(nearest_int(iscale0 * x[i]), -nmax, nmax - 1);
        ls[i] = (int8_t)(l + nmax);
        const float w = qw ? qw[i] : x[i] * x[i], lf = (float)l;
        sumlx += w * x[i] * lf;
        suml2 += w * lf * lf;
    }
    float scale = sumlx / suml2;
    float best = scale * sumlx;
    for (int itry = 0; itry < 3; ++itry) {
        const float is = 1.0f / scale;
        float slx = 0.0f, sl2 = 0.0f;
        bool changed = false;
        for (int i = 0; i < n; ++i) {
            const int32_t l = clampi(nearest_int(is * x[i]), -nmax, nmax - 1);
            if (l + nmax != (int32_t)ls[i]) changed = true;
            const float w = qw ? qw[i] : x[i] * x[i], lf = (float)l;
            slx += w * x[i] * lf;
            sl2 += w * lf * lf;
        }
        if (!changed || sl2 == 0.0f || slx * slx <= best * sl2) break;
        for (int i = 0; i < n; ++i) ls[i] = (int8_t)(nmax + clampi(nearest_int(is * x[i]), -nmax, nmax - 1));
        sumlx = slx;
        suml2 = sl2;
        scale = sumlx / suml2;
        best = scale * sumlx;
    }
    for (int itry = 0; itry < 5; ++itry) {
        int n_changed = 0;
        for (int i = 0; i < n; ++i) {
            const float w = qw ? qw[i] : x[i] * x[i];
            const int32_t l = (int32_t)ls[i] - nmax;
            float slx = sumlx - w * x[i] * (float)l;
            if (slx > 0.0f) {
                float sl2 = suml2 - w * (float)l * (float)l;
                const int32_t nl = clampi(nearest_int(x[i] * sl2 / slx), -nmax, nmax - 1);
                if (nl != l) {
                    slx += w * x[i] * (float)nl;
                    sl2 += w * (float)nl * (float)nl;
                    if (sl2 > 0.0f && slx * slx * suml2 > sumlx * sumlx * sl2) {
                        ls[i] = (int8_t)(nmax + nl);
                        sumlx = slx;
                        suml2 = sl2;
                        scale = sumlx / suml2;
                        ++n_changed;
                    }
                }
            }
        }
        if (n_changed == 0) break;
    }
    return scale;
}
// imatrix == nullptr: from_float; else from_float_imatrix (k_quants.rs:2246-2325), one importance weight per column
void quantize_q6k(const float *x, uint8_t *out, int64_t k, const float *imatrix = nullptr) {
    int8_t L[256] = {0};
    float scales[16];
    for (int64_t b = 0; b < k / 256; ++b, x += 256, out += 210) {
        uint8_t *ql = out, *qh = out + 128;
        int8_t *sc = reinterpret_cast<int8_t *>(out + 192);
        float max_scale = 0.0f, max_abs = 0.0f;
        for (int ib = 0; ib < 16; ++ib) {
            const float s = qx_w2(x + 16 * ib, L + 16 * ib, imatrix ? imatrix + 256 * b + 16 * ib : nullptr);
            scales[ib] = s;
            if (std::fabs(s) > max_abs) { max_abs = std::fabs(s); max_scale = s; }
        }
        const float iscale = -128.0f / max_scale;  // -inf for an all-zero block, as in the reference
        const uint16_t hd = f32_to_f16(1.0f / iscale);
        std::memcpy(out + 208, &hd, 2);
        for (int ib = 0; ib < 16; ++ib) sc[ib] = (int8_t)std::min(nearest_int(iscale * scales[ib]), 127);
        const float d = f16_to_f32(hd);
        for (int j = 0; j < 16; ++j) {
            const float dj = d * (float)sc[j];
            if (dj == 0.0f) continue;
            for (int t = 0; t < 16; ++t) L[16 * j + t] = (int8_t)(clampi(nearest_int(x[16 * j + t] / dj), -32, 31) + 32);
        }
        for (int h = 0; h < 2; ++h) {
            const int8_t *Lh = L + 128 * h;
            for (int t = 0; t < 32; ++t) {
                ql[64 * h + t] = (uint8_t)((Lh[t] & 0xF) | ((Lh[t + 64] & 0xF) << 4));
                ql[64 * h + 32 + t] = (uint8_t)((Lh[t + 32] & 0xF) | ((Lh[t + 96] & 0xF) << 4));
                qh[32 * h + t] = (uint8_t)((Lh[t] >> 4) | ((Lh[t + 32] >> 4) << 2) | ((Lh[t + 64] >> 4) << 4) |
                                           ((Lh[t + 96] >> 4) << 6));
            }
        }
    }
}

// ---- importance-matrix quantizers of the k-quants with 6-bit (scale, min) pairs: from_float_imatrix of Q4K
// (k_quants.rs:1682-1745) and Q5K (:1959-2041); make_qkx3_quants utils.rs:372-466, make_qp_quants utils.rs:469-560 ----
void qkx3(int nmax, const float *x, const float *weights, float &scale_out, float &min_out) {
    constexpr int n = 32, nstep = 36;
    constexpr float rmin = -0.9f, rdelta = 0.05f;
    uint8_t L[n] = {0}, Laux[n];
    float min_val = x[0], max_val = x[0];
    float sum_w = weights[0];
    float sum_x = sum_w * x[0];
    for (int i = 1; i < n; ++i) {
        if (x[i] < min_val) min_val = x[i];
        if (x[i] > max_val) max_val = x[i];
        sum_w += weights[i];
        sum_x += weights[i] * x[i];
    }
    if (min_val > 0.0f) min_val = 0.0f;
    if (max_val <= min_val) { scale_out = 0.0f; min_out = -min_val; return; }
    float iscale = (float)nmax / (max_val - min_val);
    float scale = 1.0f / iscale;
    float best_mad = 0.0f;
    for (int i = 0; i < n; ++i) {
        const uint8_t l = (uint8_t)clampi(nearest_int(iscale * (x[i] - min_val)), 0, nmax);
        L[i] = l;
        const float diff = scale * (float)l + min_val - x[i];
        best_mad += weights[i] * (diff * diff);
    }
    for (int is = 0; is <= nstep; ++is) {
        iscale = (rmin + rdelta * (float)is + (float)nmax) / (max_val - min_val);
        float sum_l = 0.0f, sum_l2 = 0.0f, sum_xl = 0.0f;
        for (int i = 0; i < n; ++i) {
            const uint8_t l = (uint8_t)clampi(nearest_int(iscale * (x[i] - min_val)), 0, nmax);
            Laux[i] = l;
            const float w = weights[i], lf = (float)l;
            sum_l += w * lf;
            sum_l2 += w * (lf * lf);
            sum_xl += w * lf * x[i];
        }
        const float d = sum_w * sum_l2 - sum_l * sum_l;
        if (d > 0.0f) {
            float this_scale = (sum_w * sum_xl - sum_x * sum_l) / d;
            float this_min = (sum_l2 * sum_x - sum_l * sum_xl) / d;
            if (this_min > 0.0f) { this_min = 0.0f; this_scale = sum_xl / sum_l2; }
            float mad = 0.0f;
            for (int i = 0; i < n; ++i) {
                const float diff = this_scale * (float)Laux[i] + this_min - x[i];
                mad += weights[i] * (diff * diff);
            }
            if (mad < best_mad) {
                std::memcpy(L, Laux, n);
                best_mad = mad;
                scale = this_scale;
                min_val = this_min;
            }
        }
    }
    scale_out = scale;
    min_out = -min_val;
}
float qp_quants(const float *x, uint8_t *L, const float *qw) {
    constexpr int n = 8;
    constexpr uint8_t nmax = 63;
    float mx = 0.0f;
    for (int i = 0; i < n; ++i) mx = std::isnan(x[i]) ? mx : std::max(mx, x[i]);  // f32::max skips NaN
    if (mx == 0.0f) { std::memset(L, 0, n); return 0.0f; }
    float iscale = (float)nmax / mx;
    for (int i = 0; i < n; ++i) L[i] = (uint8_t)nearest_int(iscale * x[i]);  // i32 -> u8 wraps, as Rust `as`
    const float scale = 1.0f / iscale;
    float best_mse = 0.0f;
    for (int i = 0; i < n; ++i) { const float diff = x[i] - scale * (float)L[i]; best_mse += qw[i] * diff * diff; }
    for (int is = -4; is <= 4; ++is) {
        if (is == 0) continue;
        const float iscale_is = (0.1f * (float)is + (float)nmax) / mx;
        const float scale_is = 1.0f / iscale_is;
        float mse = 0.0f;
        for (int i = 0; i < n; ++i) {
            const uint8_t li = std::min((uint8_t)nearest_int(iscale_is * x[i]), nmax);
            const float diff = x[i] - scale_is * (float)li;
            mse += qw[i] * diff * diff;
        }
        if (mse < best_mse) { best_mse = mse; iscale = iscale_is; }
    }
    float sumlx = 0.0f, suml2 = 0.0f;
    for (int i = 0; i < n; ++i) {
        const uint8_t li = std::min(trunc_u8(std::round(iscale * x[i])), nmax);  // f32 -> u8 saturates
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
                const uint8_t nl = std::min((uint8_t)nearest_int(x[i] * sl2 / slx), nmax);
                if (nl != L[i]) {
                    slx += qw[i] * x[i] * (float)nl;
                    sl2 += qw[i] * ((float)nl * (float)nl);
                    if ((slx * slx) * suml2 > (sumlx * sumlx) * sl2) {
                        L[i] = nl;
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
// d, dmin and the twelve scale bytes of one superblock (out + 0 .. 15), imatrix form; the block is zeroed by the caller
void kquant_imatrix_header(const float *x, const float *iw, int nmax, bool clamp63, uint8_t *out) {
    float mins[8], scales[8], weights[32], sw[8];
    uint8_t ls[8] = {0}, lm[8] = {0};
    float sum_x2 = 0.0f;
    for (int t = 0; t < 256; ++t) sum_x2 += x[t] * x[t];
    const float sigma2 = 2.0f * sum_x2 / 256.0f;
    for (int j = 0; j < 8; ++j) {
        for (int l = 0; l < 32; ++l) weights[l] = iw[32 * j + l] * std::sqrt(sigma2 + x[32 * j + l] * x[32 * j + l]);
        float sumw = 0.0f;
        for (int l = 0; l < 32; ++l) sumw += weights[l];
        sw[j] = sumw;
        qkx3(nmax, x + 32 * j, weights, scales[j], mins[j]);
    }
    const float d_block = qp_quants(scales, ls, sw);
    const float m_block = qp_quants(mins, lm, sw);
    uint8_t *sc = out + 4;
    for (int j = 0; j < 8; ++j) {
        const uint8_t lsv = clamp63 ? std::min<uint8_t>(ls[j], 63) : ls[j], lmv = clamp63 ? std::min<uint8_t>(lm[j], 63) : lm[j];
        if (j < 4) { sc[j] = lsv; sc[j + 4] = lmv; }
        else {
            sc[j + 4] = (uint8_t)((lsv & 0xF) | ((lmv & 0xF) << 4));
            sc[j - 4] |= (uint8_t)((lsv >> 4) << 6);
            sc[j] |= (uint8_t)((lmv >> 4) << 6);
        }
    }
    const uint16_t hd = f32_to_f16(d_block), hm = f32_to_f16(m_block);
    std::memcpy(out, &hd, 2);
    std::memcpy(out + 2, &hm, 2);
}
void quantize_q4k_imatrix(const float *x, uint8_t *out, int64_t k, const float *imatrix) {
    for (int64_t b = 0; b < k / 256; ++b, x += 256, out += 144) {
        std::memset(out, 0, 144);
        kquant_imatrix_header(x, imatrix + 256 * b, 15, false, out);
        uint16_t hd, hm;
        std::memcpy(&hd, out, 2);
        std::memcpy(&hm, out + 2, 2);
        const float d = f16_to_f32(hd), dmin = f16_to_f32(hm);
        uint8_t L[256] = {0};
        for (int j = 0; j < 8; ++j) {
            uint8_t s, m;
            scale_min_k4(j, out + 4, s, m);
            const float dj = d * (float)s;
            if (dj == 0.0f) continue;
            const float dm = dmin * (float)m;
            for (int t = 0; t < 32; ++t) L[32 * j + t] = (uint8_t)clampi(nearest_int((x[32 * j + t] + dm) / dj), 0, 15);
        }
        for (int g = 0; g < 4; ++g)
            for (int t = 0; t < 32; ++t) out[16 + 32 * g + t] = (uint8_t)(L[64 * g + t] | (L[64 * g + 32 + t] << 4));
    }
}
void quantize_q5k_imatrix(const float *x, uint8_t *out, int64_t k, const float *imatrix) {
    for (int64_t b = 0; b < k / 256; ++b, x += 256, out += 176) {
        std::memset(out, 0, 176);
        kquant_imatrix_header(x, imatrix + 256 * b, 31, true, out);
        uint16_t hd, hm;
        std::memcpy(&hd, out, 2);
        std::memcpy(&hm, out + 2, 2);
        const float d = f16_to_f32(hd), dmin = f16_to_f32(hm);
        uint8_t *qh = out + 16, *qs = out + 48;
        uint8_t L[256] = {0};
        for (int j = 0; j < 8; ++j) {
            uint8_t s, m;
            scale_min_k4(j, out + 4, s, m);
            const float dj = d * (float)s;
            if (dj == 0.0f) continue;
            const float dm = dmin * (float)m;
            for (int t = 0; t < 32; ++t) L[32 * j + t] = (uint8_t)clampi(nearest_int((x[32 * j + t] + dm) / dj), 0, 31);
        }
        uint8_t m1 = 1, m2 = 2;
        for (int g = 0; g < 4; ++g) {
            for (int t = 0; t < 32; ++t) {
                uint8_t l1 = L[64 * g + t], l2 = L[64 * g + 32 + t];
                if (l1 > 15) { l1 -= 16; qh[t] |= m1; }
                if (l2 > 15) { l2 -= 16; qh[t] |= m2; }
                qs[32 * g + t] = (uint8_t)(l1 | (l2 << 4));
            }
            m1 <<= 2;
            m2 <<= 2;
        }
    }
}

void quantize_row_imatrix(GgmlDType t, const float *x, uint8_t *out, int64_t k, const float *imatrix) {
    switch (t) {
    case GgmlDType::Q4K: quantize_q4k_imatrix(x, out, k, imatrix); return;
    case GgmlDType::Q5K: quantize_q5k_imatrix(x, out, k, imatrix); return;
    case GgmlDType::Q6K: quantize_q6k(x, out, k, imatrix); return;
    default: throw Error(LLOOM_ERR_DTYPE, "`from_float_imatrix` is unimplemented for this type");
    }
}

void quantize_row(GgmlDType t, const float *x, uint8_t *out, int64_t k) {
    switch (t) {
    case GgmlDType::Q8_0: quantize_q8_0(x, out, k); return;
    case GgmlDType::Q4K: quantize_q4k(x, out, k); return;
    case GgmlDType::Q6K: quantize_q6k(x, out, k); return;
    case GgmlDType::Q5K: quantize_q5k(x, out, k); return;
    case GgmlDType::Q4_0: quantize_q4_0(x, out, k); return;
    case GgmlDType::Q5_0: quantize_q5_0(x, out, k); return;
    default: throw Error(LLOOM_ERR_DTYPE, "quantize: not a weight type of this backend");
    }
}

}  // namespace

int64_t block_size(GgmlDType t) { return lloom_b200_block_elems((int)t); }
int64_t type_size(GgmlDType t) { return lloom_b200_block_bytes((int)t); }

void quantize_rows(GgmlDType t, const float *x, void *blocks, int64_t rows, int64_t k, int nthreads,
                   const float *imatrix) {
    if (t != GgmlDType::Q8_0 && t != GgmlDType::Q4K && t != GgmlDType::Q6K && t != GgmlDType::Q5K &&
        t != GgmlDType::Q4_0 && t != GgmlDType::Q5_0)
        throw Error(LLOOM_ERR_DTYPE, "quantize: not a weight type of this backend");
    if (imatrix && t != GgmlDType::Q4K && t != GgmlDType::Q5K && t != GgmlDType::Q6K)
        throw Error(LLOOM_ERR_DTYPE, "`from_float_imatrix` is unimplemented for this type");
    if (k <= 0 || k % block_size(t) != 0) throw Error(LLOOM_ERR_SHAPE, "quantize: k is not a whole number of blocks");
    const int64_t row_bytes = k / block_size(t) * type_size(t);
    nthreads = (int)std::max<int64_t>(1, std::min<int64_t>(nthreads, rows));
    auto work = [&](int tid) {
        const int64_t per = (rows + nthreads - 1) / nthreads;
        const int64_t r1 = std::min(rows, (tid + 1) * per);
        for (int64_t r = tid * per; r < r1; ++r) {
            if (imatrix) quantize_row_imatrix(t, x + r * k, (uint8_t *)blocks + r * row_bytes, k, imatrix);
            else quantize_row(t, x + r * k, (uint8_t *)blocks + r * row_bytes, k);
        }
    };
    std::vector<std::thread> pool;
    for (int tid = 1; tid < nthreads; ++tid) pool.emplace_back(work, tid);
    work(0);
    for (auto &th : pool) th.join();
}

// ---- QCudaStorage ----

QCudaStorage::~QCudaStorage() {
    if (data_) cudaFree(data_);
}

std::unique_ptr<QCudaStorage> QCudaStorage::zeros(const CudaDevice &dev, int64_t el_count, GgmlDType dtype) {
    const int64_t bs = block_size(dtype), ts = type_size(dtype);
    if (bs == 0) throw Error(LLOOM_ERR_DTYPE, "zeros: unsupported dtype");
    std::unique_ptr<QCudaStorage> s(new QCudaStorage(dev, dtype));
    s->len_ = (el_count + bs - 1) / bs * ts;
    s->padded_ = (el_count + kMatrixRowPadding + bs - 1) / bs * ts;
    DeviceGuard g(dev.ordinal);
    cuda_check(cudaMalloc((void **)&s->data_, (size_t)s->padded_), "cudaMalloc");
    cuda_check(cudaMemsetAsync(s->data_, 0, (size_t)s->padded_, (cudaStream_t)dev.stream), "cudaMemsetAsync");
    return s;
}

std::unique_ptr<QCudaStorage> QCudaStorage::load_quantized(const CudaDevice &dev, const void *data, int64_t nbytes,
                                                           GgmlDType dtype) {
    const int64_t bs = block_size(dtype), ts = type_size(dtype);
    if (dtype == GgmlDType::Q8K || bs == 0) throw Error(LLOOM_ERR_DTYPE, "load_quantized: unsupported dtype");
    if (nbytes < 0 || nbytes % ts != 0) throw Error(LLOOM_ERR_SHAPE, "load_quantized: payload length");
    auto s = zeros(dev, nbytes / ts * bs, dtype);
    DeviceGuard g(dev.ordinal);
    if (nbytes > 0) {
        cuda_check(cudaMemcpyAsync(s->data_, data, (size_t)nbytes, cudaMemcpyHostToDevice, (cudaStream_t)dev.stream),
                   "cudaMemcpyAsync");
        cuda_check(cudaStreamSynchronize((cudaStream_t)dev.stream), "cudaStreamSynchronize");  // `data` may be pageable
    }
    return s;
}

void QCudaStorage::quantize_onto(const float *host_src, int64_t el_count, int64_t k, int nthreads) {
    quantize_imatrix_onto(host_src, el_count, nullptr, k, nthreads);
}

void QCudaStorage::quantize_imatrix_onto(const float *host_src, int64_t el_count, const float *imatrix_weights,
                                         int64_t n_per_row, int nthreads) {
    const int64_t k = n_per_row;
    if (k <= 0 || el_count % k != 0) throw Error(LLOOM_ERR_SHAPE, "quantize_onto: shape");
    const int64_t need = el_count / block_size(dtype_) * type_size(dtype_);
    if (need != len_) throw Error(LLOOM_ERR_SHAPE, "quantize_onto: storage size does not match the source");
    std::vector<uint8_t> blocks((size_t)need);
    quantize_rows(dtype_, host_src, blocks.data(), el_count / k, k, nthreads, imatrix_weights);
    DeviceGuard g(dev_.ordinal);
    cuda_check(cudaMemcpyAsync(data_, blocks.data(), (size_t)need, cudaMemcpyHostToDevice, (cudaStream_t)dev_.stream),
               "cudaMemcpyAsync");
    cuda_check(cudaStreamSynchronize((cudaStream_t)dev_.stream), "cudaStreamSynchronize");
}

std::vector<uint8_t> QCudaStorage::data() const {
    std::vector<uint8_t> out((size_t)len_);
    DeviceGuard g(dev_.ordinal);
    if (len_ > 0) {
        cuda_check(cudaMemcpyAsync(out.data(), data_, (size_t)len_, cudaMemcpyDeviceToHost, (cudaStream_t)dev_.stream),
                   "cudaMemcpyAsync");
        cuda_check(cudaStreamSynchronize((cudaStream_t)dev_.stream), "cudaStreamSynchronize");
    }
    return out;
}

void QCudaStorage::dequantize(int64_t elem_count, void *out, bool f16) const {
    DeviceGuard g(dev_.ordinal);
    status_check(lloom_b200_dequantize((int)dtype_, data_, elem_count, out, f16 ? 1 : 0, dev_.stream), "dequantize");
}

void QCudaStorage::embedding(int64_t rows, int64_t hidden, const uint32_t *ids, int64_t n_ids, float *out) const {
    if (hidden % block_size(dtype_) != 0)
        throw Error(LLOOM_ERR_SHAPE, "quantized embedding hidden size is not divisible by block size");
    if (rows * hidden / block_size(dtype_) * type_size(dtype_) != len_)
        throw Error(LLOOM_ERR_SHAPE, "quantized tensor has a different byte size than rows x hidden");
    DeviceGuard g(dev_.ordinal);
    status_check(lloom_b200_get_rows((int)dtype_, data_, rows, hidden, ids, n_ids, out, dev_.stream), "get_rows");
}

void QCudaStorage::fwd(int64_t n, int64_t k, const float *x, int64_t m, float *y, int64_t ldy, int store) const {
    if (n * k / block_size(dtype_) * type_size(dtype_) != len_)
        throw Error(LLOOM_ERR_SHAPE, "fwd: weight shape does not match the storage");
    const int64_t need = lloom_b200_workspace_bytes((int)dtype_, m, n, k);
    if (need <= 0) throw Error(LLOOM_ERR_SHAPE, "fwd: unsupported shape");
    DeviceGuard g(dev_.ordinal);
    Workspace &ws = workspace_for(dev_.ordinal);
    std::lock_guard<std::mutex> lock(ws.mu);  // held across the launches, like the reference's guard
    if (ws.bytes < need) {
        if (ws.ptr) cuda_check(cudaFree(ws.ptr), "cudaFree");  // implicit device sync: earlier launches are done
        ws.ptr = nullptr;
        ws.bytes = 0;
        const int64_t grow = std::max<int64_t>(need, 1 << 20);
        cuda_check(cudaMalloc(&ws.ptr, (size_t)grow), "cudaMalloc");
        ws.bytes = grow;
    }
    if (store != LLOOM_STORE_PLAIN)
        status_check(lloom_b200_qmatmul_fwd_store((int)dtype_, data_, x, y, m, n, k, ldy, store, ws.ptr, ws.bytes, dev_.stream),
                     "qmatmul_fwd_store");
    else
        status_check(lloom_b200_qmatmul_fwd((int)dtype_, data_, x, y, m, n, k, ldy, ws.ptr, ws.bytes, dev_.stream),
                     "qmatmul_fwd");
}

// ---- QTensor / QMatMul ----

QTensor::QTensor(std::unique_ptr<QCudaStorage> storage, std::vector<int64_t> shape)
    : storage_(std::move(storage)), shape_(std::move(shape)) {
    const int64_t bs = block_size(storage_->dtype());
    if (shape_.empty()) throw Error(-1, "scalar tensor cannot be quantized");
    if (shape_.back() % bs != 0) throw Error(-1, "quantized tensor must have their last dim divisible by block size");
    if (elem_count() / bs * type_size(storage_->dtype()) != storage_->storage_size_in_bytes())
        throw Error(-1, "storage size does not match the shape");
}

int64_t QTensor::elem_count() const {
    int64_t e = 1;
    for (int64_t d : shape_) e *= d;
    return e;
}

std::shared_ptr<QTensor> QTensor::quantize(const CudaDevice &dev, const float *src, std::vector<int64_t> shape,
                                           GgmlDType dtype, int nthreads) {
    if (shape.empty()) throw Error(-1, "scalar tensor cannot be quantized");
    int64_t elems = 1;
    for (int64_t d : shape) elems *= d;
    if (shape.back() % block_size(dtype) != 0)
        throw Error(-1, "quantized tensor must have their last dim divisible by block size");
    auto st = QCudaStorage::zeros(dev, elems, dtype);
    st->quantize_onto(src, elems, shape.back(), nthreads);
    return std::make_shared<QTensor>(std::move(st), std::move(shape));
}

std::shared_ptr<QTensor> QTensor::quantize_imatrix(const CudaDevice &dev, const float *src, const float *imatrix_weights,
                                                   int64_t imatrix_len, std::vector<int64_t> shape, GgmlDType dtype,
                                                   int nthreads) {
    if (shape.empty()) throw Error(-1, "scalar tensor cannot be quantized");
    if (imatrix_len != shape.back()) throw Error(-1, "imatrix weights must have the same length as the last dim of src");
    int64_t elems = 1;
    for (int64_t d : shape) elems *= d;
    if (shape.back() % block_size(dtype) != 0)
        throw Error(-1, "quantized tensor must have their last dim divisible by block size");
    auto st = QCudaStorage::zeros(dev, elems, dtype);
    st->quantize_imatrix_onto(src, elems, imatrix_weights, shape.back(), nthreads);
    return std::make_shared<QTensor>(std::move(st), std::move(shape));
}

std::shared_ptr<QTensor> QTensor::from_data(const CudaDevice &dev, const void *bytes, int64_t nbytes, GgmlDType dtype,
                                            std::vector<int64_t> shape) {
    int64_t elems = 1;
    for (int64_t d : shape) elems *= d;
    const int64_t need = elems / std::max<int64_t>(block_size(dtype), 1) * type_size(dtype);
    if (nbytes < need) throw Error(-1, "payload length is shorter than the shape");
    return std::make_shared<QTensor>(QCudaStorage::load_quantized(dev, bytes, need, dtype), std::move(shape));
}

void QMatMul::forward(const float *xs, const std::vector<int64_t> &xs_dims, float *y) const {
    const auto &ws = w_->shape();
    if (ws.size() != 2) throw Error(-1, "qmatmul weight is not rank 2");
    if (xs_dims.size() < 2) throw Error(-1, "input tensor has only one dimension");
    const int64_t n = ws[0], k = ws[1];
    if (xs_dims.back() != k) throw Error(-1, "input tensor incompatible with the weight shape");
    int64_t m = 1;
    for (size_t i = 0; i + 1 < xs_dims.size(); ++i) m *= xs_dims[i];
    w_->storage().fwd(n, k, xs, m, y, n);
}

bool QMatMul::forward_store(const float *xs, const std::vector<int64_t> &xs_dims, float *y, int store) const {
    const auto &ws = w_->shape();
    if (ws.size() != 2 || xs_dims.size() < 2 || xs_dims.back() != ws[1]) return false;
    int64_t m = 1;
    for (size_t i = 0; i + 1 < xs_dims.size(); ++i) m *= xs_dims[i];
    if (m > 8) return false;  // the store blocks serve the matvec path only
    w_->storage().fwd(ws[0], ws[1], xs, m, y, ws[0], store);
    return true;
}

bool QMatMul::forward_silu(const float *xs, const std::vector<int64_t> &xs_dims, float *y) const {
    return forward_store(xs, xs_dims, y, LLOOM_STORE_SILU);
}

bool QMatMul::forward_mul_into(const float *xs, const std::vector<int64_t> &xs_dims, float *gate) const {
    return forward_store(xs, xs_dims, gate, LLOOM_STORE_MUL_INTO);
}

}  // namespace host
}  // namespace lloom

// ---- C view for drivers that cannot call C++ (the Python tests and bench) ----
using namespace lloom::host;

namespace {
thread_local std::string t_host_error;
template <class F>
int guarded(F &&f) {
    try {
        f();
        return 0;
    } catch (const Error &e) {
        t_host_error = e.what();
        return e.status != 0 ? e.status : -1;
    } catch (const std::exception &e) {
        t_host_error = e.what();
        return -1;
    }
}
struct Handle {
    std::shared_ptr<QTensor> t;
};
}  // namespace

extern "C" {

const char *lloom_b200_host_last_error(void) { return t_host_error.c_str(); }

int lloom_b200_host_quantize_rows(int dtype, const float *x, void *blocks, int64_t rows, int64_t k, int nthreads) {
    return guarded([&] { quantize_rows((GgmlDType)dtype, x, blocks, rows, k, nthreads); });
}

int lloom_b200_host_quantize_rows_imatrix(int dtype, const float *x, const float *imatrix, void *blocks, int64_t rows,
                                          int64_t k, int nthreads) {
    return guarded([&] {
        if (!imatrix) throw Error(LLOOM_ERR_NULL, "quantize_imatrix: no importance weights");
        quantize_rows((GgmlDType)dtype, x, blocks, rows, k, nthreads, imatrix);
    });
}

int lloom_b200_host_qtensor_quantize_imatrix(int device, void *stream, const float *src, const float *imatrix, int64_t n,
                                             int64_t k, int dtype, int nthreads, void **out) {
    return guarded([&] {
        CudaDevice dev{device, stream};
        *out = new Handle{QTensor::quantize_imatrix(dev, src, imatrix, k, {n, k}, (GgmlDType)dtype, nthreads)};
    });
}

int lloom_b200_host_qtensor_quantize(int device, void *stream, const float *src, int64_t n, int64_t k, int dtype,
                                     int nthreads, void **out) {
    return guarded([&] {
        CudaDevice dev{device, stream};
        *out = new Handle{QTensor::quantize(dev, src, {n, k}, (GgmlDType)dtype, nthreads)};
    });
}

int lloom_b200_host_qtensor_from_data(int device, void *stream, const void *bytes, int64_t nbytes, int dtype,
                                      int64_t n, int64_t k, void **out) {
    return guarded([&] {
        CudaDevice dev{device, stream};
        *out = new Handle{QTensor::from_data(dev, bytes, nbytes, (GgmlDType)dtype, {n, k})};
    });
}

void lloom_b200_host_qtensor_free(void *h) { delete static_cast<Handle *>(h); }

int64_t lloom_b200_host_qtensor_nbytes(void *h) { return static_cast<Handle *>(h)->t->storage().storage_size_in_bytes(); }

const void *lloom_b200_host_qtensor_device_ptr(void *h) { return static_cast<Handle *>(h)->t->storage().device_ptr(); }

int lloom_b200_host_qtensor_data(void *h, void *out, int64_t capacity) {
    return guarded([&] {
        auto bytes = static_cast<Handle *>(h)->t->storage().data();
        if ((int64_t)bytes.size() > capacity) throw Error(LLOOM_ERR_SHAPE, "data: output buffer too small");
        std::memcpy(out, bytes.data(), bytes.size());
    });
}

int lloom_b200_host_qmatmul_forward(void *h, const float *x_dev, int64_t m, float *y_dev) {
    return guarded([&] {
        auto &t = static_cast<Handle *>(h)->t;
        QMatMul::from_arc(t).forward(x_dev, {m, t->shape()[1]}, y_dev);
    });
}

int lloom_b200_host_qtensor_dequantize(void *h, void *out_dev, int f16) {
    return guarded([&] {
        auto &t = static_cast<Handle *>(h)->t;
        t->storage().dequantize(t->elem_count(), out_dev, f16 != 0);
    });
}

int lloom_b200_host_qtensor_embedding(void *h, const uint32_t *ids_dev, int64_t n_ids, float *out_dev) {
    return guarded([&] {
        auto &t = static_cast<Handle *>(h)->t;
        t->storage().embedding(t->shape()[0], t->shape()[1], ids_dev, n_ids, out_dev);
    });
}

}  // extern "C"
