// Dequantize and row gather (embedding) for the six weight formats, exact T::to_float arithmetic.
// Bandwidth kernels: one thread produces four consecutive elements (one 16-byte store).
#pragma once

#include "common.cuh"

namespace lloom {

// Four consecutive elements e..e+3 (e % 4 == 0) of a row of canonical blocks.
// Every product is an explicit round-to-nearest multiply: no contraction into FMA, so the values
// equal the reference's sequential f32 expressions bit for bit.
__device__ __forceinline__ float4 dequant4(int dtype, const uint8_t *__restrict__ row, int64_t e) {
    float r[4];
    if (dtype == LLOOM_Q8_0) {
        // k_quants.rs:720-736   y = q as f32 * d
        const uint8_t *blk = row + (e >> 5) * Q8_0_BYTES;
        const float d = f16_bits_to_f32(*reinterpret_cast<const unsigned short *>(blk));
        const int8_t *q = reinterpret_cast<const int8_t *>(blk + 2 + (e & 31));
#pragma unroll
        for (int i = 0; i < 4; ++i) r[i] = __fmul_rn((float)q[i], d);
    } else if (dtype == LLOOM_Q4_K) {
        // k_quants.rs:1747-1774   y = (d*sc)*q - (dmin*m)
        const uint8_t *blk = row + (e >> 8) * Q4K_BYTES;
        const int w = (int)(e & 255);
        const int g = w >> 6, hi = (w >> 5) & 1, t = w & 31;
        const uint32_t dd = *reinterpret_cast<const uint32_t *>(blk);
        const float d = f16_bits_to_f32(dd & 0xffffu), dmin = f16_bits_to_f32(dd >> 16);
        const uint32_t s[3] = {*reinterpret_cast<const uint32_t *>(blk + 4), *reinterpret_cast<const uint32_t *>(blk + 8),
                               *reinterpret_cast<const uint32_t *>(blk + 12)};
        int sc, mn;
        q4k_scale_min(s, 2 * g + hi, sc, mn);
        const float d1 = __fmul_rn(d, (float)sc), m1 = __fmul_rn(dmin, (float)mn);
        const uint32_t qw = *reinterpret_cast<const uint32_t *>(blk + 16 + 32 * g + t);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int q = (qw >> (8 * i + 4 * hi)) & 0xF;
            r[i] = __fsub_rn(__fmul_rn(d1, (float)q), m1);
        }
    } else if (dtype == LLOOM_Q4_0) {
        // k_quants.rs:299-318   y = (nibble - 8) as f32 * d; low nibbles are elements 0..15, high 16..31
        const uint8_t *blk = row + (e >> 5) * Q4_0_BYTES;
        const float d = f16_bits_to_f32(*reinterpret_cast<const unsigned short *>(blk));
        const int w = (int)(e & 31);
        const uint8_t *q = blk + 2 + (w & 15);
#pragma unroll
        for (int i = 0; i < 4; ++i) r[i] = __fmul_rn((float)(((w & 16) ? (q[i] >> 4) : (q[i] & 0xF)) - 8), d);
    } else if (dtype == LLOOM_Q5_0) {
        // k_quants.rs:578-600   y = ((nibble | fifth bit << 4) - 16) as f32 * d
        const uint8_t *blk = row + (e >> 5) * Q5_0_BYTES;
        const float d = f16_bits_to_f32(*reinterpret_cast<const unsigned short *>(blk));
        const uint32_t qh = (uint32_t)blk[2] | ((uint32_t)blk[3] << 8) | ((uint32_t)blk[4] << 16) | ((uint32_t)blk[5] << 24);
        const int w = (int)(e & 31);
        const uint8_t *q = blk + 6 + (w & 15);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int nib = (w & 16) ? (q[i] >> 4) : (q[i] & 0xF);
            r[i] = __fmul_rn((float)((nib | (int)(((qh >> (w + i)) & 1u) << 4)) - 16), d);
        }
    } else if (dtype == LLOOM_Q5_K) {
        // k_quants.rs:2043-2076   y = (d*sc) * (nibble + 16 * fifth bit) - (dmin*m), the code summed in f32
        const uint8_t *blk = row + (e >> 8) * Q5K_BYTES;
        const int w = (int)(e & 255);
        const int g = w >> 6, hi = (w >> 5) & 1, t = w & 31;
        const uint32_t dd = *reinterpret_cast<const uint32_t *>(blk);
        const float d = f16_bits_to_f32(dd & 0xffffu), dmin = f16_bits_to_f32(dd >> 16);
        const uint32_t s[3] = {*reinterpret_cast<const uint32_t *>(blk + 4), *reinterpret_cast<const uint32_t *>(blk + 8),
                               *reinterpret_cast<const uint32_t *>(blk + 12)};
        int sc, mn;
        q4k_scale_min(s, 2 * g + hi, sc, mn);
        const float d1 = __fmul_rn(d, (float)sc), m1 = __fmul_rn(dmin, (float)mn);
        const uint32_t qw = *reinterpret_cast<const uint32_t *>(blk + 48 + 32 * g + t);
        const uint32_t hw = *reinterpret_cast<const uint32_t *>(blk + 16 + t);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int q = (qw >> (8 * i + 4 * hi)) & 0xF;
            const float add = ((hw >> (8 * i + 2 * g + hi)) & 1u) ? 16.0f : 0.0f;
            r[i] = __fsub_rn(__fmul_rn(d1, __fadd_rn((float)q, add)), m1);
        }
    } else {
        // k_quants.rs:2327-2358   y = d * sc * q   (left to right)
        const uint8_t *blk = row + (e >> 8) * Q6K_BYTES;
        const int w = (int)(e & 255);
        const int h = w >> 7, gq = (w >> 5) & 3, l = w & 31;
        const float d = f16_bits_to_f32(*reinterpret_cast<const unsigned short *>(blk + 208));
        const int sc = reinterpret_cast<const int8_t *>(blk + 192)[8 * h + (l >> 4) + 2 * gq];
        const float dsc = __fmul_rn(d, (float)sc);
        const uint8_t *ql = blk + 64 * h + 32 * (gq & 1) + l;
        const uint8_t *qh = blk + 128 + 32 * h + l;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int lo = (gq & 2) ? (ql[i] >> 4) : (ql[i] & 0xF);
            const int q = (lo | (((qh[i] >> (2 * gq)) & 3) << 4)) - 32;
            r[i] = __fmul_rn(dsc, (float)q);
        }
    }
    return make_float4(r[0], r[1], r[2], r[3]);
}

template <bool F16>
__global__ void __launch_bounds__(256) dequantize_kernel(int dtype, const uint8_t *__restrict__ blocks, int64_t elems,
                                                         void *__restrict__ out) {
    const int64_t e = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (e >= elems) return;
    const float4 v = dequant4(dtype, blocks, e);
    if (F16) {
        __half2 *o = reinterpret_cast<__half2 *>(reinterpret_cast<__half *>(out) + e);
        o[0] = __halves2half2(__float2half_rn(v.x), __float2half_rn(v.y));
        o[1] = __halves2half2(__float2half_rn(v.z), __float2half_rn(v.w));
    } else {
        *reinterpret_cast<float4 *>(reinterpret_cast<float *>(out) + e) = v;
    }
}

// out[i, :] = to_float(table row ids[i]); ids outside [0, rows) give a zero row.
__global__ void __launch_bounds__(256) get_rows_kernel(int dtype, const uint8_t *__restrict__ blocks, int64_t rows,
                                                       int64_t hidden, int64_t row_bytes,
                                                       const uint32_t *__restrict__ ids, int64_t n_ids,
                                                       float *__restrict__ out) {
    const int64_t per_row = hidden >> 2;
    const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= n_ids * per_row) return;
    const int64_t i = t / per_row, e = (t - i * per_row) * 4;
    const uint32_t id = __ldg(ids + i);
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if ((int64_t)id < rows) v = dequant4(dtype, blocks + (int64_t)id * row_bytes, e);
    *reinterpret_cast<float4 *>(out + i * hidden + e) = v;
}

}  // namespace lloom
