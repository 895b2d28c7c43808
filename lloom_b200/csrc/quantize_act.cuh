// Activation quantizers: f32 rows -> canonical Q8_0 / Q8_K blocks, bit-exact with the reference's
// CPU quantizers.  Every float operation is an explicit round-to-nearest intrinsic so that no
// compiler flag can fuse or reorder it.
#pragma once

#include "common.cuh"

namespace lloom {

// Rust `f32 as i8` after `round()`: saturating, NaN -> 0.
__device__ __forceinline__ int sat_i8_from_rounded(float v) {
    if (v != v) return 0;
    v = fminf(fmaxf(v, -128.0f), 127.0f);
    return (int)v;
}

// BlockQ8_0::from_float (lloom-tensor/src/quantized/k_quants.rs:738-767):
//   amax = max|x|; d = amax/127; id = d != 0 ? 1/d : 0; block.d = f16(d); q = (i8)round(x*id).
// Four lanes share a 32-element block (8 consecutive elements each); a warp covers 8 blocks.
__global__ void __launch_bounds__(256) quantize_q8_0_kernel(const float *__restrict__ x, uint8_t *__restrict__ out,
                                                            int64_t total_blocks) {
    const int64_t gthread = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t blk = gthread >> 2;
    const int part = (int)(gthread & 3);
    const bool live = blk < total_blocks;
    float v[8];
    if (live) {
        const float4 *src = reinterpret_cast<const float4 *>(x + blk * QK8_0 + part * 8);
        float4 a = __ldg(src), b = __ldg(src + 1);
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
        v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = 0.0f;
    }
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));  // fmaxf ignores NaN like f32::max
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    const float d = __fdiv_rn(amax, 127.0f);
    const float id = (d != 0.0f) ? __fdiv_rn(1.0f, d) : 0.0f;
    if (!live) return;
    uint8_t *dst = out + blk * Q8_0_BYTES;
    if (part == 0) *reinterpret_cast<unsigned short *>(dst) = __half_as_ushort(__float2half_rn(d));
    unsigned short *q16 = reinterpret_cast<unsigned short *>(dst + 2 + part * 8);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        int q0 = sat_i8_from_rounded(roundf(__fmul_rn(v[2 * i], id)));
        int q1 = sat_i8_from_rounded(roundf(__fmul_rn(v[2 * i + 1], id)));
        q16[i] = (unsigned short)((q0 & 0xff) | ((q1 & 0xff) << 8));
    }
}

// BlockQ8K::from_float, x86 arm (k_quants.rs:2400-2438):
//   max = the element of largest |x|, FIRST one on ties; all-zero block -> d = 0, qs = 0;
//   else iscale = -127/max; q = clamp(round(iscale*x), -128, 127); bsums[j] = sum of 16 q; d = 1/iscale.
// One warp per 256-element block; lane l owns elements [8l, 8l+8).  For an all-zero block bsums are
// written as 0 (the reference leaves them untouched; they only ever multiply d == 0).
__global__ void __launch_bounds__(256) quantize_q8k_kernel(const float *__restrict__ x, uint8_t *__restrict__ out,
                                                           int64_t total_blocks) {
    const int lane = threadIdx.x & 31;
    const int64_t blk = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    if (blk >= total_blocks) return;  // whole warp leaves together
    const float4 *src = reinterpret_cast<const float4 *>(x + blk * QK_K + lane * 8);
    float4 a = __ldg(src), b = __ldg(src + 1);
    float v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
    float amax = 0.0f, vmax = 0.0f;
    int idx = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        float ax = fabsf(v[i]);
        if (amax < ax) { amax = ax; vmax = v[i]; idx = lane * 8 + i; }
    }
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
        float oa = __shfl_xor_sync(0xffffffffu, amax, off);
        float ov = __shfl_xor_sync(0xffffffffu, vmax, off);
        int oi = __shfl_xor_sync(0xffffffffu, idx, off);
        // larger magnitude wins; equal magnitudes -> lower index (the sequential scan's first hit)
        if (oa > amax || (oa == amax && oi < idx)) { amax = oa; vmax = ov; idx = oi; }
    }
    uint8_t *dst = out + blk * Q8K_BYTES;
    uint32_t *q32 = reinterpret_cast<uint32_t *>(dst + 4 + lane * 8);
    short *bs = reinterpret_cast<short *>(dst + 4 + QK_K);
    if (amax == 0.0f) {
        if (lane == 0) *reinterpret_cast<float *>(dst) = 0.0f;
        q32[0] = 0;
        q32[1] = 0;
        if ((lane & 1) == 0) bs[lane >> 1] = 0;
        return;
    }
    const float iscale = __fdiv_rn(-127.0f, vmax);
    int q[8], s = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        q[i] = sat_i8_from_rounded(roundf(__fmul_rn(iscale, v[i])));
        s += q[i];
    }
    q32[0] = (q[0] & 0xff) | ((q[1] & 0xff) << 8) | ((q[2] & 0xff) << 16) | ((uint32_t)(q[3] & 0xff) << 24);
    q32[1] = (q[4] & 0xff) | ((q[5] & 0xff) << 8) | ((q[6] & 0xff) << 16) | ((uint32_t)(q[7] & 0xff) << 24);
    s += __shfl_xor_sync(0xffffffffu, s, 1);
    if ((lane & 1) == 0) bs[lane >> 1] = (short)s;
    if (lane == 0) *reinterpret_cast<float *>(dst) = __fdiv_rn(1.0f, iscale);
}

inline cudaError_t launch_quantize_act(int w_dtype, const float *x, int64_t m, int64_t k, void *out,
                                       cudaStream_t stream) {
    if (w_dtype == LLOOM_Q8_0) {
        int64_t blocks = m * (k / QK8_0);
        int64_t threads = blocks * 4;
        quantize_q8_0_kernel<<<(unsigned)ceil_div64(threads, 256), 256, 0, stream>>>(x, (uint8_t *)out, blocks);
    } else {
        int64_t blocks = m * (k / QK_K);
        int64_t threads = blocks * 32;
        quantize_q8k_kernel<<<(unsigned)ceil_div64(threads, 256), 256, 0, stream>>>(x, (uint8_t *)out, blocks);
    }
    return cudaGetLastError();
}

}  // namespace lloom
