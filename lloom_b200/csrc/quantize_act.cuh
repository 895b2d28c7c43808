// Activation quantizers: f32 rows -> Q8_0 / Q8_K blocks, bit-exact with the reference's CPU
// quantizers.  Every float operation is an explicit round-to-nearest intrinsic so that no compiler
// flag can fuse or reorder it.  The block arithmetic lives in two warp-level device functions that
// both the stand-alone kernels (canonical blocks in global memory) and the GEMV's fused prologue
// (planes in shared memory) call, so the two cannot drift apart.
#pragma once

#include "common.cuh"

namespace lloom {

// Rust `f32 as i8` after `round()`: saturating, NaN -> 0.  The float -> s32 conversion saturates and maps NaN
// to 0 in hardware; the s32 -> s8 step saturates again.  v is integer-valued (or NaN / infinite), so the
// rounding mode of the first conversion does not matter.
__device__ __forceinline__ int sat_i8_from_rounded(float v) {
    int r;
    asm("{\n"
        ".reg .s32 t;\n"
        "cvt.rzi.s32.f32 t, %1;\n"
        "cvt.sat.s8.s32 %0, t;\n"
        "}\n"
        : "=r"(r)
        : "f"(v));
    return r;
}

__device__ __forceinline__ uint32_t pack4(int a, int b, int c, int d) {
    return (uint32_t)(a & 0xff) | ((uint32_t)(b & 0xff) << 8) | ((uint32_t)(c & 0xff) << 16) | ((uint32_t)(d & 0xff) << 24);
}

// BlockQ8K::from_float, x86 arm (lloom-tensor/src/quantized/k_quants.rs:2400-2438):
//   max = the element of largest |x|, FIRST one on ties; all-zero block -> d = 0, qs = 0;
//   else iscale = -127/max; q = clamp(round(iscale*x), -128, 127); bsums[j] = sum of 16 q; d = 1/iscale.
// One warp per 256-element block; lane l owns elements [8l, 8l+8) in v.  Returns the lane's 8 codes
// packed in two words, d (same on every lane) and sum16 = the bsum of the lane's 16-element group
// (same on lanes 2j and 2j+1).  For an all-zero block the sums are 0 (the reference leaves bsums
// untouched; they only ever multiply d == 0).
__device__ __forceinline__ void q8k_quantize_warp(const float (&v)[8], int lane, uint32_t &q_lo, uint32_t &q_hi,
                                                  float &d, int &sum16) {
    // The sequential scan keeps the FIRST element of largest magnitude (`if amax < ax`; NaN never wins).  In-lane:
    // the same scan over the lane's 8 elements.  Across lanes: the largest magnitude by a max-reduction, then the
    // lowest lane holding it (ballot + find-first) hands over its candidate -- lanes are in element order.
    float amax = 0.0f, vmax = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const float ax = fabsf(v[i]);
        if (amax < ax) { amax = ax; vmax = v[i]; }
    }
    float wmax = amax;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) wmax = fmaxf(wmax, __shfl_xor_sync(0xffffffffu, wmax, off));
    const unsigned holders = __ballot_sync(0xffffffffu, amax == wmax);
    vmax = __shfl_sync(0xffffffffu, vmax, __ffs(holders) - 1);
    amax = wmax;
    if (amax == 0.0f) {
        q_lo = q_hi = 0;
        d = 0.0f;
        sum16 = 0;
        return;
    }
    const float iscale = __fdiv_rn(-127.0f, vmax);
    int q[8], s = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        q[i] = sat_i8_from_rounded(roundf(__fmul_rn(iscale, v[i])));
        s += q[i];
    }
    q_lo = pack4(q[0], q[1], q[2], q[3]);
    q_hi = pack4(q[4], q[5], q[6], q[7]);
    sum16 = s + __shfl_xor_sync(0xffffffffu, s, 1);
    d = __fdiv_rn(1.0f, iscale);
}

// BlockQ8_0::from_float (k_quants.rs:738-767):
//   amax = max|x|; d = amax/127; id = d != 0 ? 1/d : 0; block.d = f16(d); q = (i8)round(x*id).
// Four consecutive lanes share a 32-element block (8 consecutive elements each).  All 32 lanes must
// call it.  Returns the lane's 8 codes and the f16 bits of d.
__device__ __forceinline__ void q8_0_quantize_quad(const float (&v)[8], uint32_t &q_lo, uint32_t &q_hi,
                                                   unsigned short &d_f16) {
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));  // fmaxf ignores NaN like f32::max
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    const float d = __fdiv_rn(amax, 127.0f);
    const float id = (d != 0.0f) ? __fdiv_rn(1.0f, d) : 0.0f;
    int q[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) q[i] = sat_i8_from_rounded(roundf(__fmul_rn(v[i], id)));
    q_lo = pack4(q[0], q[1], q[2], q[3]);
    q_hi = pack4(q[4], q[5], q[6], q[7]);
    d_f16 = __half_as_ushort(__float2half_rn(d));
}

__device__ __forceinline__ void load8(const float *p, float (&v)[8]) {
    const float4 a = __ldg(reinterpret_cast<const float4 *>(p)), b = __ldg(reinterpret_cast<const float4 *>(p) + 1);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
    v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}

// Stand-alone Q8_0 quantizer: canonical 34-byte blocks {f16 d; i8 qs[32]}.  A warp covers 8 blocks.
static __global__ void __launch_bounds__(256) quantize_q8_0_kernel(const float *__restrict__ x, uint8_t *__restrict__ out,
                                                            int64_t total_blocks) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");  // the GEMV behind may start streaming weights
    const int64_t gthread = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t blk = gthread >> 2;
    const int part = (int)(gthread & 3);
    const bool live = blk < total_blocks;
    float v[8];
    if (live) load8(x + blk * QK8_0 + part * 8, v);
    else {
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = 0.0f;
    }
    uint32_t q_lo, q_hi;
    unsigned short d16;
    q8_0_quantize_quad(v, q_lo, q_hi, d16);
    if (!live) return;
    uint8_t *dst = out + blk * Q8_0_BYTES;  // 2-byte aligned
    if (part == 0) *reinterpret_cast<unsigned short *>(dst) = d16;
    unsigned short *q16 = reinterpret_cast<unsigned short *>(dst + 2 + part * 8);
    q16[0] = (unsigned short)(q_lo & 0xffffu);
    q16[1] = (unsigned short)(q_lo >> 16);
    q16[2] = (unsigned short)(q_hi & 0xffffu);
    q16[3] = (unsigned short)(q_hi >> 16);
}

// Stand-alone Q8_K quantizer: canonical 292-byte blocks {f32 d; i8 qs[256]; i16 bsums[16]}.
static __global__ void __launch_bounds__(256) quantize_q8k_kernel(const float *__restrict__ x, uint8_t *__restrict__ out,
                                                           int64_t total_blocks) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");  // the GEMV behind may start streaming weights
    const int lane = threadIdx.x & 31;
    const int64_t blk = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    if (blk >= total_blocks) return;  // whole warp leaves together
    float v[8];
    load8(x + blk * QK_K + lane * 8, v);
    uint32_t q_lo, q_hi;
    float d;
    int sum16;
    q8k_quantize_warp(v, lane, q_lo, q_hi, d, sum16);
    uint8_t *dst = out + blk * Q8K_BYTES;
    uint32_t *q32 = reinterpret_cast<uint32_t *>(dst + 4 + lane * 8);
    q32[0] = q_lo;
    q32[1] = q_hi;
    if ((lane & 1) == 0) reinterpret_cast<short *>(dst + 4 + QK_K)[lane >> 1] = (short)sum16;
    if (lane == 0) *reinterpret_cast<float *>(dst) = d;
}

static inline cudaError_t launch_quantize_act(int w_dtype, const float *x, int64_t m, int64_t k, void *out,
                                       cudaStream_t stream) {
    if (w_dtype == LLOOM_Q8_0 || w_dtype == LLOOM_Q4_0 || w_dtype == LLOOM_Q5_0) {  // VecDotType = BlockQ8_0
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
