// Decode GEMV (1 <= M <= 8) over canonical GGUF block rows, HBM-bound by design.
//
// One persistent CTA per SM, each owning an equal contiguous range of weight rows.  A producer warp
// streams tiles of consecutive rows (one contiguous byte range of the canonical [n][k/block] stream)
// into a ring of shared-memory stages with the bulk-async copy engine; consumer warps unpack nibbles
// / 6-bit codes in registers, take exact integer dot products with dp4a against the quantized
// activations (held once per CTA in shared memory as aligned planes), apply the block scales in f32
// in the reference's algebraic form -- one FMA per 256-element superblock (per 32-element block for
// Q8_0), exactly the reference's granularity -- and reduce across lanes with warp shuffles.
// Per-row arithmetic never depends on the row's position in a tile or on n, so any row shard of a
// matrix gives bit-identical rows.
#pragma once

#include <mutex>

#include "common.cuh"
#include "gemv_params.h"
#include "quantize_act.cuh"

namespace lloom {

// Activation planes in shared memory, built once per CTA from the canonical blocks:
//   qs   int8  per unit, padded by 16 bytes so that the lanes of a quarter-warp, one unit apart, hit
//              distinct banks: Q8_K acts [M][K/256][256+16], Q8_0 acts [M][K/64][64+16]
//   d    f32   [M][K/32]  (Q8_0 acts: f16 scale widened)   or [M][K/256] (Q8_K acts)
//   sums int16 [M][K/32]  for Q4_K weights: bsums[2j] + bsums[2j+1] (one per 32-element sub-block)
//        int16 [M][2][K/256][8] for Q6_K weights: the 16-element bsums, split by superblock half
struct ActPlanes {
    const int8_t *qs;
    const float *d;
    const short *sums;
    int k;
};

// Read NWORDS 32-bit words starting at a 2-byte aligned shared-memory address.
template <int NWORDS>
__device__ __forceinline__ void lds_words_unaligned(const uint8_t *p, uint32_t (&out)[NWORDS]) {
    const uint32_t addr = smem_u32(p);
    const uint32_t sh = (addr & 3u) * 8u;
    const uint32_t *wp = reinterpret_cast<const uint32_t *>(p - (addr & 3u));
    uint32_t prev = wp[0];
#pragma unroll
    for (int i = 0; i < NWORDS; ++i) {
        const uint32_t next = wp[i + 1];
        out[i] = __funnelshift_r(prev, next, sh);
        prev = next;
    }
}

__device__ __forceinline__ int dot16(const uint4 &a, const uint4 &b, int c) {
    c = __dp4a((int)a.x, (int)b.x, c);
    c = __dp4a((int)a.y, (int)b.y, c);
    c = __dp4a((int)a.z, (int)b.z, c);
    return __dp4a((int)a.w, (int)b.w, c);
}

// unsigned bytes of a times signed bytes of b (dp4a.u32.s32)
__device__ __forceinline__ int dp4a_us(uint32_t a, uint32_t b, int c) {
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ int dot16_us(const uint4 &a, const uint4 &b, int c) {
    c = dp4a_us(a.x, b.x, c);
    c = dp4a_us(a.y, b.y, c);
    c = dp4a_us(a.z, b.z, c);
    return dp4a_us(a.w, b.w, c);
}

// ---------------------------------------------------------------------------------------------
// Per-format units.  A unit is the span of one weight row that a single lane owns: one 256-element
// superblock for the k-quants, two 32-element blocks for Q8_0.  The lane loads the matching
// activation bytes once and reuses them for the RW rows it handles.  MC = activation rows handled
// per pass (<= 4 keeps the activation registers bounded; M > 4 takes two passes over the unit).
// ---------------------------------------------------------------------------------------------

// Q4_K x Q8_K (k_quants.rs:1540-1620, avx.rs:443-525), per superblock:
//   out += (d_a*d_w) * sum_j sc_j * dot32(q4_j, q8_j)  +  (-d_a*dmin_w) * sum_j m_j * (bsums[2j]+bsums[2j+1])
struct FmtQ4K {
    static constexpr int kUnitElems = 256;
    template <int MC, int RW>
    __device__ static __forceinline__ void unit(const ActPlanes &p, int m0, int b, const uint8_t *const (&rowp)[RW],
                                                const bool (&valid)[RW], float (&acc)[RW][MC]) {
        // headers of the RW rows: d, dmin and the 6-bit (scale, min) pairs (utils.rs:50-60) unpacked to bytes
        float dw[RW], dminw[RW];
        uint32_t scw[RW][2], mnw[RW][2];
#pragma unroll
        for (int r = 0; r < RW; ++r) {
            if (valid[r]) {
                const uint4 h = *reinterpret_cast<const uint4 *>(rowp[r] + (size_t)b * Q4K_BYTES);
                dw[r] = f16_bits_to_f32(h.x & 0xffffu);
                dminw[r] = f16_bits_to_f32(h.x >> 16);
                scw[r][0] = h.y & 0x3f3f3f3fu;
                scw[r][1] = (h.w & 0x0f0f0f0fu) | (((h.y >> 6) & 0x03030303u) << 4);
                mnw[r][0] = h.z & 0x3f3f3f3fu;
                mnw[r][1] = ((h.w >> 4) & 0x0f0f0f0fu) | (((h.z >> 6) & 0x03030303u) << 4);
            } else {
                dw[r] = dminw[r] = 0.0f;
                scw[r][0] = scw[r][1] = mnw[r][0] = mnw[r][1] = 0;
            }
        }
        int S[RW][MC];
#pragma unroll
        for (int r = 0; r < RW; ++r)
#pragma unroll
            for (int m = 0; m < MC; ++m) S[r][m] = 0;
#pragma unroll
        for (int g = 0; g < 4; ++g) {
            uint4 alo[MC][2], ahi[MC][2];
#pragma unroll
            for (int m = 0; m < MC; ++m) {
                const uint4 *q = reinterpret_cast<const uint4 *>(
                    p.qs + ((size_t)(m0 + m) * (p.k >> 8) + b) * kQ8KUnitStride + g * 64);
                alo[m][0] = q[0]; alo[m][1] = q[1];
                ahi[m][0] = q[2]; ahi[m][1] = q[3];
            }
#pragma unroll
            for (int r = 0; r < RW; ++r) {
                if (!valid[r]) continue;
                const uint4 *qp = reinterpret_cast<const uint4 *>(rowp[r] + (size_t)b * Q4K_BYTES + 16 + g * 32);
                const uint4 q0 = qp[0], q1 = qp[1];
                uint4 l0, l1, h0, h1;
                l0.x = q0.x & 0x0f0f0f0fu; l0.y = q0.y & 0x0f0f0f0fu; l0.z = q0.z & 0x0f0f0f0fu; l0.w = q0.w & 0x0f0f0f0fu;
                l1.x = q1.x & 0x0f0f0f0fu; l1.y = q1.y & 0x0f0f0f0fu; l1.z = q1.z & 0x0f0f0f0fu; l1.w = q1.w & 0x0f0f0f0fu;
                // high nibbles stay in place (16*q as unsigned bytes); the exact factor 16 comes out of the sum below
                h0.x = q0.x & 0xf0f0f0f0u; h0.y = q0.y & 0xf0f0f0f0u; h0.z = q0.z & 0xf0f0f0f0u; h0.w = q0.w & 0xf0f0f0f0u;
                h1.x = q1.x & 0xf0f0f0f0u; h1.y = q1.y & 0xf0f0f0f0u; h1.z = q1.z & 0xf0f0f0f0u; h1.w = q1.w & 0xf0f0f0f0u;
                const int sc_lo = (scw[r][g >> 1] >> (16 * (g & 1))) & 0xff;
                const int sc_hi = (scw[r][g >> 1] >> (16 * (g & 1) + 8)) & 0xff;
#pragma unroll
                for (int m = 0; m < MC; ++m) {
                    const int pl = dot16(l1, alo[m][1], dot16(l0, alo[m][0], 0));
                    const int ph = dot16_us(h1, ahi[m][1], dot16_us(h0, ahi[m][0], 0)) >> 4;  // a multiple of 16: exact
                    S[r][m] += sc_lo * pl + sc_hi * ph;
                }
            }
        }
#pragma unroll
        for (int m = 0; m < MC; ++m) {
            // eight sub-block sums of this superblock, packed 2 x int16 per word
            const uint4 sp = *reinterpret_cast<const uint4 *>(p.sums + (size_t)(m0 + m) * (p.k >> 5) + b * 8);
            const float da = p.d[(m0 + m) * (p.k >> 8) + b];
#pragma unroll
            for (int r = 0; r < RW; ++r) {
                int mv = __dp2a_lo((int)sp.x, (int)mnw[r][0], 0);
                mv = __dp2a_hi((int)sp.y, (int)mnw[r][0], mv);
                mv = __dp2a_lo((int)sp.z, (int)mnw[r][1], mv);
                mv = __dp2a_hi((int)sp.w, (int)mnw[r][1], mv);
                acc[r][m] = fmaf(__fmul_rn(da, dw[r]), (float)S[r][m], acc[r][m]);
                acc[r][m] = fmaf(__fmul_rn(-da, dminw[r]), (float)mv, acc[r][m]);
            }
        }
    }
};

// Q6_K x Q8_K (k_quants.rs:2115-2172, avx.rs:131-216), per superblock:
//   out += (d_a*d_w) * sum_{j<16} sc_j * dot16(q6_j - 32, q8_j),   (q6-32).q8 taken as q6u.q8 - 32*bsum
struct FmtQ6K {
    static constexpr int kUnitElems = 256;
    template <int MC, int RW>
    __device__ static __forceinline__ void unit(const ActPlanes &p, int m0, int b, const uint8_t *const (&rowp)[RW],
                                                const bool (&valid)[RW], float (&acc)[RW][MC]) {
        int S[RW][MC];
#pragma unroll
        for (int r = 0; r < RW; ++r)
#pragma unroll
            for (int m = 0; m < MC; ++m) S[r][m] = 0;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            // the half's eight 16-element sums and its scales
            uint4 bsw[MC];
#pragma unroll
            for (int m = 0; m < MC; ++m)
                bsw[m] = *reinterpret_cast<const uint4 *>(p.sums + (((size_t)(m0 + m) * 2 + h) * (p.k >> 8) + b) * 8);
            uint32_t scw[RW][2];
#pragma unroll
            for (int r = 0; r < RW; ++r) {
                scw[r][0] = scw[r][1] = 0;
                if (valid[r]) lds_words_unaligned<2>(rowp[r] + (size_t)b * Q6K_BYTES + 192 + 8 * h, scw[r]);
            }
#pragma unroll
            for (int lq = 0; lq < 2; ++lq) {  // l0 = 16*lq
                uint4 aq[MC][4];
#pragma unroll
                for (int m = 0; m < MC; ++m) {
                    const int8_t *base =
                        p.qs + ((size_t)(m0 + m) * (p.k >> 8) + b) * kQ8KUnitStride + h * 128 + lq * 16;
#pragma unroll
                    for (int gq = 0; gq < 4; ++gq) aq[m][gq] = *reinterpret_cast<const uint4 *>(base + 32 * gq);
                }
#pragma unroll
                for (int r = 0; r < RW; ++r) {
                    if (!valid[r]) continue;
                    const uint8_t *blk = rowp[r] + (size_t)b * Q6K_BYTES;  // 2-byte aligned
                    uint32_t la[4], lb[4], hh[4];
                    lds_words_unaligned<4>(blk + 64 * h + 16 * lq, la);
                    lds_words_unaligned<4>(blk + 64 * h + 32 + 16 * lq, lb);
                    lds_words_unaligned<4>(blk + 128 + 32 * h + 16 * lq, hh);
                    uint32_t cw[4][4];
#pragma unroll
                    for (int w = 0; w < 4; ++w) {
                        cw[0][w] = (la[w] & 0x0f0f0f0fu) | ((hh[w] << 4) & 0x30303030u);
                        cw[1][w] = (lb[w] & 0x0f0f0f0fu) | ((hh[w] << 2) & 0x30303030u);
                        cw[2][w] = ((la[w] >> 4) & 0x0f0f0f0fu) | (hh[w] & 0x30303030u);
                        cw[3][w] = ((lb[w] >> 4) & 0x0f0f0f0fu) | ((hh[w] >> 2) & 0x30303030u);
                    }
#pragma unroll
                    for (int gq = 0; gq < 4; ++gq) {
                        // scale index within the half: lq + 2*gq  (byte of scw), sum index the same
                        const int idx = lq + 2 * gq;
                        const int sc = (int)(int8_t)((scw[r][idx >> 2] >> (8 * (idx & 3))) & 0xff);
                        const uint4 cv = make_uint4(cw[gq][0], cw[gq][1], cw[gq][2], cw[gq][3]);
#pragma unroll
                        for (int m = 0; m < MC; ++m) {
                            const uint32_t bsv[4] = {bsw[m].x, bsw[m].y, bsw[m].z, bsw[m].w};
                            const uint32_t bw = bsv[idx >> 1];
                            const int bs = (int)(short)((idx & 1) ? (bw >> 16) : (bw & 0xffffu));
                            S[r][m] += sc * (dot16(cv, aq[m][gq], 0) - 32 * bs);
                        }
                    }
                }
            }
        }
#pragma unroll
        for (int r = 0; r < RW; ++r) {
            float dw = 0.0f;
            if (valid[r]) dw = f16_bits_to_f32(*reinterpret_cast<const unsigned short *>(rowp[r] + (size_t)b * Q6K_BYTES + 208));
#pragma unroll
            for (int m = 0; m < MC; ++m) {
                const float da = p.d[(m0 + m) * (p.k >> 8) + b];
                acc[r][m] = fmaf(__fmul_rn(da, dw), (float)S[r][m], acc[r][m]);
            }
        }
    }
};

// Q8_0 x Q8_0 (k_quants.rs:800-818, avx.rs:71-87):  out += (d_w*d_a) * dot32(q_w, q_a) per 32-element block.
// unit = two consecutive 34-byte blocks (k must be a multiple of 64).
struct FmtQ8_0 {
    static constexpr int kUnitElems = 64;
    template <int MC, int RW>
    __device__ static __forceinline__ void unit(const ActPlanes &p, int m0, int u, const uint8_t *const (&rowp)[RW],
                                                const bool (&valid)[RW], float (&acc)[RW][MC]) {
        uint4 aq[MC][4];
        float da[MC][2];
#pragma unroll
        for (int m = 0; m < MC; ++m) {
            const uint4 *q = reinterpret_cast<const uint4 *>(
                p.qs + ((size_t)(m0 + m) * (p.k >> 6) + u) * kQ8_0UnitStride);
#pragma unroll
            for (int i = 0; i < 4; ++i) aq[m][i] = q[i];
            const float2 dd = *reinterpret_cast<const float2 *>(p.d + (size_t)(m0 + m) * (p.k >> 5) + u * 2);
            da[m][0] = dd.x;
            da[m][1] = dd.y;
        }
#pragma unroll
        for (int r = 0; r < RW; ++r) {
            if (!valid[r]) continue;
            const uint8_t *blk = rowp[r] + (size_t)u * (2 * Q8_0_BYTES);  // 2-byte aligned
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const uint8_t *bp = blk + half * Q8_0_BYTES;
                const float dw = f16_bits_to_f32(*reinterpret_cast<const unsigned short *>(bp));
                uint32_t q[8];
                lds_words_unaligned<8>(bp + 2, q);
                const uint4 q0 = make_uint4(q[0], q[1], q[2], q[3]), q1 = make_uint4(q[4], q[5], q[6], q[7]);
#pragma unroll
                for (int m = 0; m < MC; ++m) {
                    const int pi = dot16(q1, aq[m][2 * half + 1], dot16(q0, aq[m][2 * half], 0));
                    acc[r][m] = fmaf(__fmul_rn(dw, da[m][half]), (float)pi, acc[r][m]);
                }
            }
        }
    }
};

// Q5_K x Q8_K (k_quants.rs:1795-1880, avx.rs:528-640): Q4_K's scale scheme with a fifth code bit per element in
// qh (bit 2g of qh[t]: element 64g + t, bit 2g + 1: element 64g + 32 + t), per superblock:
//   out += (d_a*d_w) * sum_j sc_j * dot32(q5_j, q8_j)  +  (-d_a*dmin_w) * sum_j m_j * (bsums[2j]+bsums[2j+1])
// Block: f16 d @0, f16 dmin @2, scales[12] @4, qh[32] @16, qs[128] @48 (176 bytes, rows stay 16-byte multiples).
struct FmtQ5K {
    static constexpr int kUnitElems = 256;
    template <int MC, int RW>
    __device__ static __forceinline__ void unit(const ActPlanes &p, int m0, int b, const uint8_t *const (&rowp)[RW],
                                                const bool (&valid)[RW], float (&acc)[RW][MC]) {
        float dw[RW], dminw[RW];
        uint32_t scw[RW][2], mnw[RW][2];
        uint4 qh[RW][2];
#pragma unroll
        for (int r = 0; r < RW; ++r) {
            if (valid[r]) {
                const uint4 *bp = reinterpret_cast<const uint4 *>(rowp[r] + (size_t)b * Q5K_BYTES);
                const uint4 h = bp[0];
                qh[r][0] = bp[1];
                qh[r][1] = bp[2];
                dw[r] = f16_bits_to_f32(h.x & 0xffffu);
                dminw[r] = f16_bits_to_f32(h.x >> 16);
                scw[r][0] = h.y & 0x3f3f3f3fu;
                scw[r][1] = (h.w & 0x0f0f0f0fu) | (((h.y >> 6) & 0x03030303u) << 4);
                mnw[r][0] = h.z & 0x3f3f3f3fu;
                mnw[r][1] = ((h.w >> 4) & 0x0f0f0f0fu) | (((h.z >> 6) & 0x03030303u) << 4);
            } else {
                dw[r] = dminw[r] = 0.0f;
                scw[r][0] = scw[r][1] = mnw[r][0] = mnw[r][1] = 0;
                qh[r][0] = qh[r][1] = make_uint4(0, 0, 0, 0);
            }
        }
        int S[RW][MC];
#pragma unroll
        for (int r = 0; r < RW; ++r)
#pragma unroll
            for (int m = 0; m < MC; ++m) S[r][m] = 0;
#pragma unroll
        for (int g = 0; g < 4; ++g) {
            uint4 alo[MC][2], ahi[MC][2];
#pragma unroll
            for (int m = 0; m < MC; ++m) {
                const uint4 *q = reinterpret_cast<const uint4 *>(
                    p.qs + ((size_t)(m0 + m) * (p.k >> 8) + b) * kQ8KUnitStride + g * 64);
                alo[m][0] = q[0]; alo[m][1] = q[1];
                ahi[m][0] = q[2]; ahi[m][1] = q[3];
            }
#pragma unroll
            for (int r = 0; r < RW; ++r) {
                if (!valid[r]) continue;
                const uint4 *qp = reinterpret_cast<const uint4 *>(rowp[r] + (size_t)b * Q5K_BYTES + 48 + g * 32);
                const uint4 q0 = qp[0], q1 = qp[1];
                const uint32_t qw[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
                const uint32_t hw[8] = {qh[r][0].x, qh[r][0].y, qh[r][0].z, qh[r][0].w,
                                        qh[r][1].x, qh[r][1].y, qh[r][1].z, qh[r][1].w};
                uint32_t lo[8], hi[8];
#pragma unroll
                for (int w = 0; w < 8; ++w) {
                    lo[w] = (qw[w] & 0x0f0f0f0fu) | (((hw[w] >> (2 * g)) & 0x01010101u) << 4);
                    hi[w] = ((qw[w] >> 4) & 0x0f0f0f0fu) | (((hw[w] >> (2 * g + 1)) & 0x01010101u) << 4);
                }
                const uint4 l0 = make_uint4(lo[0], lo[1], lo[2], lo[3]), l1 = make_uint4(lo[4], lo[5], lo[6], lo[7]);
                const uint4 h0 = make_uint4(hi[0], hi[1], hi[2], hi[3]), h1 = make_uint4(hi[4], hi[5], hi[6], hi[7]);
                const int sc_lo = (scw[r][g >> 1] >> (16 * (g & 1))) & 0xff;
                const int sc_hi = (scw[r][g >> 1] >> (16 * (g & 1) + 8)) & 0xff;
#pragma unroll
                for (int m = 0; m < MC; ++m) {
                    const int pl = dot16(l1, alo[m][1], dot16(l0, alo[m][0], 0));
                    const int ph = dot16(h1, ahi[m][1], dot16(h0, ahi[m][0], 0));
                    S[r][m] += sc_lo * pl + sc_hi * ph;
                }
            }
        }
#pragma unroll
        for (int m = 0; m < MC; ++m) {
            const uint4 sp = *reinterpret_cast<const uint4 *>(p.sums + (size_t)(m0 + m) * (p.k >> 5) + b * 8);
            const float da = p.d[(m0 + m) * (p.k >> 8) + b];
#pragma unroll
            for (int r = 0; r < RW; ++r) {
                int mv = __dp2a_lo((int)sp.x, (int)mnw[r][0], 0);
                mv = __dp2a_hi((int)sp.y, (int)mnw[r][0], mv);
                mv = __dp2a_lo((int)sp.z, (int)mnw[r][1], mv);
                mv = __dp2a_hi((int)sp.w, (int)mnw[r][1], mv);
                acc[r][m] = fmaf(__fmul_rn(da, dw[r]), (float)S[r][m], acc[r][m]);
                acc[r][m] = fmaf(__fmul_rn(-da, dminw[r]), (float)mv, acc[r][m]);
            }
        }
    }
};

// Q4_0 x Q8_0 (k_quants.rs:371-391, avx.rs:50-69) and Q5_0 x Q8_0 (k_quants.rs:500-534), per 32-element block:
//   Q4_0: out += (d_w*d_a) * dot32(nibble - 8, q_a)            (the AVX2 arm's one product d = d_w*d_a, then fma)
//   Q5_0: out += ((dot32(code5 - 16, q_a) * d_w) * d_a)        (the scalar arm, the only one this format has)
// Low nibble j = element j, high nibble j = element j + 16; Q5_0's fifth bits: qh bit j / bit j + 16.
// The offset comes out of the sum: dot(code - o, q_a) = dot(code, q_a) - o * sum(q_a), with the block sums of the
// activations precomputed in the planes.  unit = two consecutive blocks (k must be a multiple of 64).
template <bool FIVE_BIT>
struct FmtQ4or5_0 {
    static constexpr int kUnitElems = 64;
    static constexpr int kBlockBytes = FIVE_BIT ? Q5_0_BYTES : Q4_0_BYTES;
    template <int MC, int RW>
    __device__ static __forceinline__ void unit(const ActPlanes &p, int m0, int u, const uint8_t *const (&rowp)[RW],
                                                const bool (&valid)[RW], float (&acc)[RW][MC]) {
        uint4 aq[MC][4];
        float da[MC][2];
        int asum[MC][2];
        const int *sums32 = reinterpret_cast<const int *>(p.sums);
#pragma unroll
        for (int m = 0; m < MC; ++m) {
            const uint4 *q = reinterpret_cast<const uint4 *>(
                p.qs + ((size_t)(m0 + m) * (p.k >> 6) + u) * kQ8_0UnitStride);
#pragma unroll
            for (int i = 0; i < 4; ++i) aq[m][i] = q[i];
            const float2 dd = *reinterpret_cast<const float2 *>(p.d + (size_t)(m0 + m) * (p.k >> 5) + u * 2);
            da[m][0] = dd.x;
            da[m][1] = dd.y;
            const int2 ss = *reinterpret_cast<const int2 *>(sums32 + (size_t)(m0 + m) * (p.k >> 5) + u * 2);
            asum[m][0] = ss.x;
            asum[m][1] = ss.y;
        }
#pragma unroll
        for (int r = 0; r < RW; ++r) {
            if (!valid[r]) continue;
            const uint8_t *blk = rowp[r] + (size_t)u * (2 * kBlockBytes);  // 2-byte aligned
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const uint8_t *bp = blk + half * kBlockBytes;
                const float dw = f16_bits_to_f32(*reinterpret_cast<const unsigned short *>(bp));
                uint32_t lo[4], hi[4];
                if (FIVE_BIT) {
                    uint32_t w[5];  // qh, then the 16 nibble bytes
                    lds_words_unaligned<5>(bp + 2, w);
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const uint32_t hb_lo = (((w[0] >> (4 * i)) & 0xFu) * 0x00204081u) & 0x01010101u;
                        const uint32_t hb_hi = (((w[0] >> (16 + 4 * i)) & 0xFu) * 0x00204081u) & 0x01010101u;
                        lo[i] = (w[1 + i] & 0x0f0f0f0fu) | (hb_lo << 4);
                        hi[i] = ((w[1 + i] >> 4) & 0x0f0f0f0fu) | (hb_hi << 4);
                    }
                } else {
                    uint32_t w[4];
                    lds_words_unaligned<4>(bp + 2, w);
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        lo[i] = w[i] & 0x0f0f0f0fu;
                        hi[i] = (w[i] >> 4) & 0x0f0f0f0fu;
                    }
                }
                const uint4 l4 = make_uint4(lo[0], lo[1], lo[2], lo[3]), h4 = make_uint4(hi[0], hi[1], hi[2], hi[3]);
#pragma unroll
                for (int m = 0; m < MC; ++m) {
                    const int pi = dot16(h4, aq[m][2 * half + 1], dot16(l4, aq[m][2 * half], 0)) -
                                   (FIVE_BIT ? 16 : 8) * asum[m][half];
                    if (FIVE_BIT) acc[r][m] = __fadd_rn(acc[r][m], __fmul_rn(__fmul_rn((float)pi, dw), da[m][half]));
                    else acc[r][m] = fmaf(__fmul_rn(dw, da[m][half]), (float)pi, acc[r][m]);
                }
            }
        }
    }
};
using FmtQ4_0 = FmtQ4or5_0<false>;
using FmtQ5_0 = FmtQ4or5_0<true>;

// The matrix (or row range of one) a CTA is working on: a launch has one, a grouped launch up to kMaxGroup.
struct GemvSeg {
    const uint8_t *w;  // first block of the matrix
    int64_t w_bytes;   // its size (the bulk engine may touch whole 16-byte lines below this)
    float *y;
    int64_t ldy;
    int store;         // block on the store
    int r_begin, r_end;  // rows of this matrix the CTA owns
    int64_t row_base;  // rows between `w` and the matrix's first row (routed experts: `w` is the whole stack, so that
                       // an expert whose byte offset is not a multiple of 16 still streams from an aligned base)
};

// One output value to its destination(s).  SiLU in the reference's f32 form v / (1 + exp(-v)) (op.rs:755-757,
// kernels/metal_src/quantized_store.metal:17-25); MulInto reads the destination and multiplies it by the product.
// Only the EPI = 1 kernel instances contain this code: inlined into the sixteen unrolled stores of an 8-row
// instance it cost the plain forward 25-60 % of that instance's time, and as an out-of-line call it still cost
// every instance 5-20 % (registers held across the call sites).
__device__ __forceinline__ void store_out(const GemvParams &p, const GemvSeg &sg, int64_t idx, float v) {
    if (sg.store == LLOOM_STORE_SILU) v = __fdiv_rn(v, __fadd_rn(1.0f, expf(-v)));
    if (p.n_peers == 0) {
        sg.y[idx] = (sg.store == LLOOM_STORE_MUL_INTO) ? __fmul_rn(sg.y[idx], v) : v;
    } else {
        for (int g = 0; g < p.n_peers; ++g) p.y_peer[g][idx] = v;
    }
}

// Output of row `row` (of this CTA's range starting at r_begin), activation row m: staged in shared memory when the
// launch has a staging area, else straight to its destination(s).
__device__ __forceinline__ void emit_out(const GemvParams &p, const GemvSeg &sg, float *out_s, int m, int row, float v) {
    if (p.out_bytes) {
        if (sg.store == LLOOM_STORE_SILU) v = __fdiv_rn(v, __fadd_rn(1.0f, expf(-v)));
        out_s[m * p.out_pitch + (row - sg.r_begin)] = v;
    } else {
        store_out(p, sg, (int64_t)m * sg.ldy + row, v);
    }
}

// The staged rows of this CTA to every peer buffer: consecutive threads write consecutive floats, so a peer
// receives whole 128-byte lines instead of one small packet per value.  Called by `nthreads` consumer threads
// after a barrier among them.
__device__ __forceinline__ void flush_out(const GemvParams &p, const float *out_s, int r_begin, int r_end, int tid,
                                          int nthreads) {
    const int rows = r_end - r_begin;
    for (int g = 0; g < p.n_peers; ++g)
        for (int m = 0; m < p.m; ++m) {
            float *dst = p.y_peer[g] + (int64_t)m * p.ldy + r_begin;
            const float *src = out_s + m * p.out_pitch;
            for (int i = tid; i < rows; i += nthreads) dst[i] = src[i];
        }
}

// Bounded wait for a fused gather to complete on this GPU: every slot of this GPU's flag array has reached the
// count this GPU's own GEMV published (word kMaxPeers of the array).  Every thread may call it; each polls by
// itself (the flags sit in L2 after the first read).  On a time-out the status word is set and false returned.
__device__ __forceinline__ bool wait_exchange(const GemvParams &p) {
    const unsigned int *flags = p.wait_flags;
    unsigned int want;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(want) : "l"(flags + kMaxPeers) : "memory");
    unsigned long long t0 = 0;
    int g = 0;
    for (uint32_t i = 0; i < kMaxSpins; ++i) {
        unsigned int seen;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(flags + g) : "memory");
        if ((int)(seen - want) >= 0) {
            if (++g == p.wait_peers) return true;
            continue;
        }
        if ((i & 63) == 63) {
            const unsigned long long now = global_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > wait_limit_ns()) break;
        }
        __nanosleep(100);
    }
    atomicExch(&g_device_status, LLOOM_ERR_TIMEOUT);
    return false;
}

// Fused gather with the cross-GPU barrier folded in (p.publish != 0): every CTA, once its peer stores
// are issued, makes them visible system-wide and bumps this GPU's arrival counter; the CTA that arrives last
// advances the GPU's call counter and publishes it in slot [peer_rank] of every GPU's flag array with a
// system-scope release store.  A consumer that has seen the same count in all slots of its own flag array
// (lloom_b200_peer_wait) may read the gathered rows.  Called by one thread per CTA after a CTA-wide barrier.
__device__ __forceinline__ void publish_arrival(const GemvParams &p) {
    // words of this GPU's flag array: [kMaxPeers] = its call counter, [kMaxPeers + 1] = CTAs arrived so far
    unsigned int *mine = p.peer_flags[p.peer_rank];
    // This CTA's peer stores (ordered before this thread by the CTA barrier) become visible device-wide, then the
    // arrival is counted.  Only the CTA that arrives last pays for a system-scope fence: it has observed every other
    // CTA's arrival (acquire on the counter), so its release at system scope covers their stores as well.
    __threadfence();
    unsigned int prev;
    asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], 1;" : "=r"(prev) : "l"(mine + kMaxPeers + 1) : "memory");
    if (prev + 1 == gridDim.x) {
        mine[kMaxPeers + 1] = 0;  // ready for the next launch on this stream
        const unsigned int epoch = mine[kMaxPeers] + 1;
        mine[kMaxPeers] = epoch;
        __threadfence_system();
        for (int g = 0; g < p.n_peers; ++g)
            asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p.peer_flags[g] + p.peer_rank), "r"(epoch) : "memory");
    }
}

// Canonical activation blocks (global) -> planes (shared); all `nthreads` consumer threads take part.
__device__ __forceinline__ void stage_acts(const GemvParams &p, uint8_t *act_smem, int tid, int nthreads,
                                           ActPlanes &planes) {
    const size_t qs_bytes = round16(act_qs_bytes(p.w_dtype, p.m, p.k));
    float *dpl = reinterpret_cast<float *>(act_smem + qs_bytes);
    planes.qs = reinterpret_cast<const int8_t *>(act_smem);
    planes.d = dpl;
    planes.k = p.k;
    constexpr int kUnroll = 4;
    if (act_is_q8_0(p.w_dtype)) {
        // 17 half-words per block: [0] = f16 d, [1..16] = 32 int8
        const unsigned short *src = reinterpret_cast<const unsigned short *>(p.act);
        unsigned short *q16 = reinterpret_cast<unsigned short *>(act_smem);
        const int total = p.m * (p.k / 32) * 17;
        if (p.w_dtype != LLOOM_Q8_0) {
            // Q4_0 / Q5_0 weights: the sum of each block's 32 codes (the code offset comes out of the dot product)
            int *sums32 = reinterpret_cast<int *>(act_smem + qs_bytes + round16((int64_t)p.m * (p.k / 32) * 4));
            for (int blk = tid; blk < p.m * (p.k / 32); blk += nthreads) {
                int s = 0;
                for (int i = 1; i <= 16; ++i) {
                    const unsigned short v = __ldg(src + blk * 17 + i);
                    s += (int)(int8_t)(v & 0xff) + (int)(int8_t)(v >> 8);
                }
                sums32[blk] = s;
            }
            planes.sums = reinterpret_cast<const short *>(sums32);
        } else {
            planes.sums = nullptr;
        }
        for (int base = tid; base < total; base += nthreads * kUnroll) {
            unsigned short v[kUnroll];
#pragma unroll
            for (int j = 0; j < kUnroll; ++j) {
                const int i = base + j * nthreads;
                v[j] = i < total ? __ldg(src + i) : (unsigned short)0;
            }
#pragma unroll
            for (int j = 0; j < kUnroll; ++j) {
                const int i = base + j * nthreads;
                if (i < total) {
                    const int blk = i / 17, hw = i - blk * 17;
                    if (hw == 0) dpl[blk] = __half2float(__ushort_as_half(v[j]));
                    else q16[(blk >> 1) * (kQ8_0UnitStride / 2) + (blk & 1) * 16 + hw - 1] = v[j];
                }
            }
        }
    } else {
        // 73 words per block: [0] = f32 d, [1..64] = 256 int8, [65..72] = 16 int16 bsums
        const int nb = p.k / 256;
        short *sums = reinterpret_cast<short *>(act_smem + qs_bytes + round16((int64_t)p.m * nb * 4));
        const uint32_t *src = reinterpret_cast<const uint32_t *>(p.act);
        uint32_t *q32 = reinterpret_cast<uint32_t *>(act_smem);
        const bool pair = p.w_dtype != LLOOM_Q6_K;  // Q4_K / Q5_K: one sum per 32-element sub-block
        const int total = p.m * nb * 73;
        for (int base = tid; base < total; base += nthreads * kUnroll) {
            uint32_t v[kUnroll];
#pragma unroll
            for (int j = 0; j < kUnroll; ++j) {
                const int i = base + j * nthreads;
                v[j] = i < total ? __ldg(src + i) : 0u;
            }
#pragma unroll
            for (int j = 0; j < kUnroll; ++j) {
                const int i = base + j * nthreads;
                if (i < total) {
                    const int blk = i / 73, w = i - blk * 73;
                    if (w == 0) dpl[blk] = __uint_as_float(v[j]);
                    else if (w <= 64) q32[blk * (kQ8KUnitStride / 4) + w - 1] = v[j];
                    else if (pair) sums[blk * 8 + w - 65] = (short)((int)(short)(v[j] & 0xffffu) + (int)(short)(v[j] >> 16));
                    else {
                        const int mrow = blk / nb, b = blk - mrow * nb, jj = w - 65;  // word jj: bsums 2jj, 2jj+1
                        reinterpret_cast<uint32_t *>(sums)[((mrow * 2 + (jj >> 2)) * nb + b) * 4 + (jj & 3)] = v[j];
                    }
                }
            }
        }
        planes.sums = sums;
    }
}

// f32 activations (global) -> planes (shared), quantized on the way with the same warp-level block
// arithmetic as the stand-alone quantizer kernels (bit-identical codes, scales and sums).
__device__ __forceinline__ void quantize_acts_to_planes(const GemvParams &p, uint8_t *act_smem, int warp, int lane,
                                                        ActPlanes &planes) {
    const size_t qs_bytes = round16(act_qs_bytes(p.w_dtype, p.m, p.k));
    float *dpl = reinterpret_cast<float *>(act_smem + qs_bytes);
    uint32_t *q32 = reinterpret_cast<uint32_t *>(act_smem);
    planes.qs = reinterpret_cast<const int8_t *>(act_smem);
    planes.d = dpl;
    planes.k = p.k;
    if (act_is_q8_0(p.w_dtype)) {
        const int total = p.m * (p.k / 32);
        int *sums32 = reinterpret_cast<int *>(act_smem + qs_bytes + round16((int64_t)total * 4));
        for (int base = warp * 8; base < total; base += p.n_cwarps * 8) {
            const int blk = base + (lane >> 2), part = lane & 3;
            const bool live = blk < total;
            float v[8];
            if (live) load8(p.x + (size_t)blk * 32 + part * 8, v);
            else {
#pragma unroll
                for (int i = 0; i < 8; ++i) v[i] = 0.0f;
            }
            uint32_t q_lo, q_hi;
            unsigned short d16;
            q8_0_quantize_quad(v, q_lo, q_hi, d16);
            if (live) {
                uint32_t *dst = q32 + ((blk >> 1) * kQ8_0UnitStride + (blk & 1) * 32 + part * 8) / 4;
                dst[0] = q_lo;
                dst[1] = q_hi;
                if (part == 0) dpl[blk] = __half2float(__ushort_as_half(d16));
            }
            if (p.w_dtype != LLOOM_Q8_0) {  // block sums of the codes, for the formats with an offset code
                int s = __dp4a((int)q_lo, 0x01010101, __dp4a((int)q_hi, 0x01010101, 0));
                s += __shfl_xor_sync(0xffffffffu, s, 1);
                s += __shfl_xor_sync(0xffffffffu, s, 2);
                if (live && part == 0) sums32[blk] = s;
            }
        }
        planes.sums = p.w_dtype != LLOOM_Q8_0 ? reinterpret_cast<const short *>(sums32) : nullptr;
    } else {
        const int nb = p.k / 256;
        short *sums = reinterpret_cast<short *>(act_smem + qs_bytes + round16((int64_t)p.m * nb * 4));
        const int total = p.m * nb;
        // two blocks per warp in flight: both loads are issued before either is quantized (one L2 round trip)
        for (int blk0 = warp; blk0 < total; blk0 += 2 * p.n_cwarps) {
            const int blk1 = blk0 + p.n_cwarps;
            float va[8], vb[8];
            load8(p.x + (size_t)blk0 * 256 + lane * 8, va);
            if (blk1 < total) load8(p.x + (size_t)blk1 * 256 + lane * 8, vb);
#pragma unroll
            for (int rep = 0; rep < 2; ++rep) {
                const int blk = rep == 0 ? blk0 : blk1;
                if (blk >= total) break;  // warp-uniform
                uint32_t q_lo, q_hi;
                float d;
                int sum16;
                q8k_quantize_warp(rep == 0 ? va : vb, lane, q_lo, q_hi, d, sum16);
                q32[blk * (kQ8KUnitStride / 4) + lane * 2] = q_lo;
                q32[blk * (kQ8KUnitStride / 4) + lane * 2 + 1] = q_hi;
                if (lane == 0) dpl[blk] = d;
                if (p.w_dtype != LLOOM_Q6_K) {
                    const int sum32 = sum16 + __shfl_xor_sync(0xffffffffu, sum16, 2);
                    if ((lane & 3) == 0) sums[blk * 8 + (lane >> 2)] = (short)sum32;
                } else if ((lane & 1) == 0) {
                    const int mrow = blk / nb, b = blk - mrow * nb, j = lane >> 1;
                    sums[((mrow * 2 + (j >> 3)) * nb + b) * 8 + (j & 7)] = (short)sum16;
                }
            }
        }
        planes.sums = sums;
    }
}

// The producer warp's loop over one matrix: streams tiles of `tile_rows` consecutive rows of the segment's row range
// into the stage ring.  `it` counts the work items of the launch (it carries on across the matrices of a group).
__device__ __forceinline__ bool gemv_producer(const GemvParams &p, const GemvSeg &sg, uint64_t *full, uint64_t *empty,
                                              uint8_t *stage0, int tile_rows, int lane, int &it) {
    for (int row0 = sg.r_begin; row0 < sg.r_end; row0 += tile_rows, ++it) {
        const int s = it % p.stages;
        if (it >= p.stages) {
            if (!mbar_wait(&empty[s], ((it / p.stages) - 1) & 1)) return false;
        }
        const int rows = min(tile_rows, sg.r_end - row0);
        const int64_t start = (sg.row_base + row0) * p.row_bytes;
        const int64_t end = start + (int64_t)rows * p.row_bytes;
        const int64_t a_start = start & ~(int64_t)15;
        int64_t a_end = (end + 15) & ~(int64_t)15;
        const int64_t bulk_limit = sg.w_bytes & ~(int64_t)15;  // bytes the bulk engine may touch
        if (a_end > bulk_limit) a_end = bulk_limit;
        uint8_t *dst = stage0 + (size_t)s * p.stage_bytes;
        // ragged end of the weight stream (< 16 bytes): plain loads
        if (end > a_end) {
            const int64_t from = a_end > a_start ? a_end : a_start;
            for (int64_t i = from + lane; i < end; i += 32) dst[i - a_start] = __ldg(sg.w + i);
        }
        __syncwarp();
        if (lane == 0) {
            if (a_end > a_start) {
                const uint32_t bytes = (uint32_t)(a_end - a_start);
                mbar_arrive_expect_tx(&full[s], bytes);
                bulk_g2s(dst, sg.w + a_start, bytes, &full[s]);
            } else {
                mbar_arrive(&full[s]);
            }
        }
    }
    return true;
}

// The producer loop for rows cut into pieces (long rows: a whole-row tile would not leave room for two stages in
// the side-by-side shape).  Work items in order -- tile 0: pieces 0.., tile 1: ... -- each `chunk_units` units
// (fewer in a row's last piece) of up to `tile_rows` rows, one bulk copy per row, the pieces of a tile's rows packed
// `chunk_units * unit_bytes` apart.  Needs row sizes and piece sizes that are multiples of 16 bytes.
__device__ __forceinline__ bool gemv_producer_pieces(const GemvParams &p, const GemvSeg &sg, uint64_t *full, uint64_t *empty,
                                                     uint8_t *stage0, int tile_rows, int units, int lane, int &it) {
    const int pitch = p.chunk_units * p.unit_bytes;
    for (int row0 = sg.r_begin; row0 < sg.r_end; row0 += tile_rows) {
        const int rows = min(tile_rows, sg.r_end - row0);
        for (int c = 0; c < p.nchunks; ++c, ++it) {
            const int s = it % p.stages;
            if (it >= p.stages) {
                if (!mbar_wait(&empty[s], ((it / p.stages) - 1) & 1)) return false;
            }
            const int u0 = c * p.chunk_units;
            const uint32_t bytes = (uint32_t)(min(p.chunk_units, units - u0) * p.unit_bytes);
            uint8_t *dst = stage0 + (size_t)s * p.stage_bytes;
            if (lane == 0) mbar_arrive_expect_tx(&full[s], (uint32_t)rows * bytes);
            __syncwarp();
            for (int r = lane; r < rows; r += 32)
                bulk_g2s(dst + (size_t)r * pitch, sg.w + (sg.row_base + row0 + r) * p.row_bytes + (int64_t)u0 * p.unit_bytes,
                         bytes, &full[s]);
        }
    }
    return true;
}

// Segment g of the launch as seen by this CTA, which owns rows [r_begin, r_end) of the concatenation.
template <bool GROUP>
__device__ __forceinline__ GemvSeg gemv_segment(const GemvParams &p, int g, int r_begin, int r_end) {
    GemvSeg sg;
    if (GROUP) {
        const int off = p.goff[g], rows = p.goff[g + 1] - off;
        sg.w = p.gw[g];
        sg.w_bytes = (int64_t)rows * p.row_bytes;
        sg.row_base = 0;
        if (p.moe_ids) {
            uint32_t e = __ldg(p.moe_ids + g);
            if (e >= (uint32_t)p.moe_experts) {  // reported through the status word; the last expert stands in
                e = (uint32_t)p.moe_experts - 1;
                atomicExch(&g_device_status, LLOOM_ERR_SHAPE);
            }
            sg.w = p.w;
            sg.row_base = (int64_t)e * rows;
            sg.w_bytes = (int64_t)p.moe_experts * rows * p.row_bytes;
        }
        sg.y = p.gy[g];
        sg.ldy = p.gldy[g];
        sg.store = p.gstore[g];
        sg.r_begin = max(r_begin - off, 0);
        sg.r_end = min(r_end - off, rows);
    } else {
        sg.w = p.w;
        sg.w_bytes = p.w_bytes;
        sg.y = p.y;
        sg.ldy = p.ldy;
        sg.store = p.store_mode;
        sg.r_begin = r_begin;
        sg.r_end = r_end;
        sg.row_base = 0;
    }
    return sg;
}

// Dynamic shared memory: [barriers 128 B][act planes][staged output rows, fused gather only][stage 0][stage 1]...
// Launch overlap: the kernel lets its stream successor start as soon as it is set up
// (griddepcontrol.launch_dependents) and itself waits for its predecessor (griddepcontrol.wait) only
// before it reads activations or writes outputs.  The producer warp starts streaming weights right
// away -- weights are read-only for the life of a QTensor.  Without the programmatic-serialization
// launch attribute both instructions do nothing.  RW == 1 instances are built to fit two per SM, so
// a successor's CTA can sit beside its predecessor's and keep the HBM stream going across launches.
// CW = most consumer warps the instance may be launched with (8, or 12 for the side-by-side m <= 2 shapes).
// PIECES = the instance for rows cut into pieces (p.nchunks > 1); the whole-row instances keep the loop over pieces
// out of their code.  EPI = 1: the instance with the store blocks and the fused gather (store_out / emit_out);
// EPI = 0 stores every value to its matrix's y and nothing else.  GROUP = the instance that walks several matrices
// (p.n_group of them, sharing the activations) as one concatenated row range.
template <class Fmt, int M, int RW, int CW = 8, bool PIECES = false, int EPI = 0, bool GROUP = false>
__global__ void __launch_bounds__(32 * (CW + 1), RW == 1 ? 2 : 1) gemv_kernel(const GemvParams p) {
    constexpr int MC = M > 4 ? (M + 1) / 2 : M;  // activation rows per pass
    constexpr int NPASS = (M + MC - 1) / MC;
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t *full = reinterpret_cast<uint64_t *>(smem);
    uint64_t *empty = full + kMaxStages;
    uint8_t *act_smem = smem + 128;
    uint8_t *stage0 = act_smem + p.act_bytes + p.out_bytes;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int lpr = 1 << p.lpr_log2;
    const int groups = 32 >> p.lpr_log2;
    const int tile_rows = p.n_cwarps * groups * RW;
    // equal contiguous row ranges per CTA: HBM bytes per SM differ by at most one row
    const int r_begin = (int)(((int64_t)blockIdx.x * p.n) / gridDim.x);
    const int r_end = (int)(((int64_t)(blockIdx.x + 1) * p.n) / gridDim.x);
    const int nseg = GROUP ? p.n_group : 1;

    if (threadIdx.x == 0) {
        for (int s = 0; s < p.stages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], p.n_cwarps);
        }
        fence_mbar_init();
    }
    __syncthreads();
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    if (warp == p.n_cwarps) {
        // ---------------- producer warp ----------------
        // routed experts: which matrices to stream is device data that the stream predecessor may have written
        if (GROUP && p.moe_ids) asm volatile("griddepcontrol.wait;" ::: "memory");
        int it = 0;
        for (int g = 0; g < nseg; ++g) {
            const GemvSeg sg = gemv_segment<GROUP>(p, g, r_begin, r_end);
            if (sg.r_begin >= sg.r_end) continue;
            const bool ok = PIECES ? gemv_producer_pieces(p, sg, full, empty, stage0, tile_rows, p.k / Fmt::kUnitElems, lane, it)
                                   : gemv_producer(p, sg, full, empty, stage0, tile_rows, lane, it);
            if (!ok) break;
        }
        return;
    }

    // ---------------- consumer warps ----------------
    ActPlanes planes;
    bool ok_wait = true;
    {
        const int nthreads = p.n_cwarps * 32;
        asm volatile("griddepcontrol.wait;" ::: "memory");  // predecessor's writes (x, act blocks) are visible
        if (EPI != 0 && p.wait_flags) ok_wait = wait_exchange(p);  // x came out of a fused gather: all peers' rows are in
        if (p.x) quantize_acts_to_planes(p, act_smem, warp, lane, planes);
        else stage_acts(p, act_smem, threadIdx.x, nthreads, planes);
        asm volatile("bar.sync 1, %0;" ::"r"(nthreads) : "memory");
    }

    const int units = p.k / Fmt::kUnitElems;
    const int group = lane >> p.lpr_log2, lig = lane & (lpr - 1);
    float *out_s = reinterpret_cast<float *>(act_smem + p.act_bytes);
    int it = 0;  // work items so far: a tile, or one piece of a tile's rows when the rows are cut into pieces
    bool ok = ok_wait;  // a timed-out wait ends the loop; the warp still meets the others at the flush barrier
    const int nchunks = PIECES ? p.nchunks : 1;
    const int unit_chunk = PIECES ? p.chunk_units : units;
    const int piece_pitch = unit_chunk * p.unit_bytes;
    for (int g = 0; g < nseg && ok; ++g) {
        const GemvSeg sg = gemv_segment<GROUP>(p, g, r_begin, r_end);
        for (int trow = sg.r_begin; trow < sg.r_end && ok; trow += tile_rows) {
            const int local0 = (warp * groups + group) * RW;
            const int row0 = trow + local0;
            bool valid[RW];
#pragma unroll
            for (int r = 0; r < RW; ++r) valid[r] = row0 + r < sg.r_end;
            float accs[NPASS][RW][MC];
#pragma unroll
            for (int pass = 0; pass < NPASS; ++pass)
#pragma unroll
                for (int r = 0; r < RW; ++r)
#pragma unroll
                    for (int m = 0; m < MC; ++m) accs[pass][r][m] = 0.0f;
            for (int c = 0; c < nchunks; ++c, ++it) {
                const int s = it % p.stages;
                if (!mbar_wait(&full[s], (it / p.stages) & 1)) {
                    ok = false;
                    break;
                }
                const uint8_t *rowp[RW];
                const int u0 = c * unit_chunk, u1 = min(units, u0 + unit_chunk);
                if (PIECES) {
                    // pieces packed back to back; the pointer is the row's virtual start, so that unit u sits at
                    // u * unit_bytes as in a whole row
                    const uint8_t *tile_base = stage0 + (size_t)s * p.stage_bytes;
#pragma unroll
                    for (int r = 0; r < RW; ++r)
                        rowp[r] = tile_base + (size_t)(local0 + r) * piece_pitch - (size_t)u0 * p.unit_bytes;
                } else {
                    const int64_t start = (sg.row_base + trow) * p.row_bytes;
                    const uint8_t *tile_base = stage0 + (size_t)s * p.stage_bytes + (start & 15);
#pragma unroll
                    for (int r = 0; r < RW; ++r) rowp[r] = tile_base + (size_t)(local0 + r) * p.row_bytes;
                }
                if (valid[0]) {
#pragma unroll
                    for (int pass = 0; pass < NPASS; ++pass) {
                        const int m0 = pass * MC;
                        // the last pass of an odd M starts at M - MC: it overlaps the previous pass instead of running past M
                        for (int u = u0 + lig; u < u1; u += lpr) {
                            if (m0 + MC <= M) Fmt::template unit<MC, RW>(planes, m0, u, rowp, valid, accs[pass]);
                            else Fmt::template unit<MC, RW>(planes, M - MC, u, rowp, valid, accs[pass]);
                        }
                    }
                }
                // this warp is done reading the stage once every sum its loads feed has been computed
#pragma unroll
                for (int pass = 0; pass < NPASS; ++pass)
#pragma unroll
                    for (int r = 0; r < RW; ++r)
#pragma unroll
                        for (int m = 0; m < MC; ++m) pin_value(accs[pass][r][m]);
                __syncwarp();
                if (lane == 0) mbar_arrive(&empty[s]);
            }
            if (!ok) break;
            float out[RW][M];
#pragma unroll
            for (int pass = 0; pass < NPASS; ++pass)
#pragma unroll
                for (int r = 0; r < RW; ++r)
#pragma unroll
                    for (int m = 0; m < MC; ++m) {
                        const int m0 = pass * MC;
                        const int mi = (m0 + MC <= M) ? m0 + m : M - MC + m;
                        out[r][mi] = accs[pass][r][m];
                    }

#pragma unroll
            for (int r = 0; r < RW; ++r)
#pragma unroll
                for (int m = 0; m < M; ++m) {
                    float v = out[r][m];
                    for (int off = lpr >> 1; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
                    out[r][m] = v;
                }
            if (lig == 0) {
#pragma unroll
                for (int r = 0; r < RW; ++r)
                    if (valid[r]) {
#pragma unroll
                        for (int m = 0; m < M; ++m) {
                            if (EPI == 0) sg.y[(int64_t)m * sg.ldy + row0 + r] = out[r][m];
                            else emit_out(p, sg, out_s, m, row0 + r, out[r][m]);
                        }
                    }
            }
        }
    }
    if (EPI != 0 && p.out_bytes) {
        const int nthreads = p.n_cwarps * 32;
        asm volatile("bar.sync 1, %0;" ::"r"(nthreads) : "memory");
        if (ok) flush_out(p, out_s, r_begin, r_end, threadIdx.x, nthreads);
    }
    if (EPI != 0 && p.publish) {
        // every consumer thread's peer stores are issued; one thread reports the CTA (also after a timed-out wait,
        // so that the peers' waits end with the right count and the status word tells the story)
        const int nthreads = p.n_cwarps * 32;
        asm volatile("bar.sync 1, %0;" ::"r"(nthreads) : "memory");
        if (threadIdx.x == 0) publish_arrival(p);
    }
}

// ---- launch of one format's instances (each format is a translation unit of its own) ----

struct FuncSmemConfig {  // per kernel instance: the dynamic shared memory each device has opted into
    std::mutex mu;
    int smem[64] = {0};
};

template <class Kern>
static cudaError_t ensure_smem(Kern kern, FuncSmemConfig &cfg, int smem, bool carveout) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    std::lock_guard<std::mutex> lock(cfg.mu);
    if (cfg.smem[dev] >= smem) return cudaSuccess;
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    if (carveout) {
        // ask for the largest shared-memory carve-out, so that two half-size CTAs really fit side by side
        e = cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        if (e != cudaSuccess) return e;
    }
    cfg.smem[dev] = smem;
    return cudaSuccess;
}

template <class Kern, class Params>
static cudaError_t launch_with_overlap(Kern kern, const Params &p, int grid, int threads, int smem, bool overlap,
                                       cudaStream_t stream) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3((unsigned)threads);
    cfg.dynamicSmemBytes = (size_t)smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = overlap ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, p);
}

// EPI = 1 instances carry the store blocks and the fused gather; the plain forward uses the EPI = 0 instances.
inline bool gemv_needs_epi(const GemvParams &p) {
    if (p.n_peers != 0 || p.store_mode != LLOOM_STORE_PLAIN || p.wait_flags != nullptr) return true;
    for (int g = 0; g < p.n_group; ++g)
        if (p.gstore[g] != LLOOM_STORE_PLAIN) return true;
    return false;
}

template <class Fmt, int M, int RW, int CW, bool PIECES, int EPI, bool GROUP>
static cudaError_t launch_gemv_inst2(const GemvParams &p, int grid, int smem, bool overlap, cudaStream_t stream) {
    auto kern = gemv_kernel<Fmt, M, RW, CW, PIECES, EPI, GROUP>;
    static FuncSmemConfig cfg;
    cudaError_t e = ensure_smem(kern, cfg, smem, true);
    if (e != cudaSuccess) return e;
    return launch_with_overlap(kern, p, grid, 32 * (p.n_cwarps + 1), smem, overlap, stream);
}

template <class Fmt, int M, int RW, int CW = 8, bool PIECES = false, bool GROUP = false>
static cudaError_t launch_gemv_inst(const GemvParams &p, int grid, int smem, bool overlap, cudaStream_t stream) {
    if (gemv_needs_epi(p)) return launch_gemv_inst2<Fmt, M, RW, CW, PIECES, 1, GROUP>(p, grid, smem, overlap, stream);
    return launch_gemv_inst2<Fmt, M, RW, CW, PIECES, 0, GROUP>(p, grid, smem, overlap, stream);
}

template <class Fmt, int RW>
static cudaError_t launch_gemv_m(const GemvParams &p, int grid, int smem, bool overlap, cudaStream_t stream) {
    if (p.n_group >= 1) {  // grouped launch: eight consumer warps, one row per lane, m <= 2 (rows in pieces: m == 1)
        if (RW != 1 || p.n_cwarps > 8) return cudaErrorInvalidValue;
        if (p.nchunks > 1) {
            if (p.m == 1) return launch_gemv_inst<Fmt, 1, 1, 8, true, true>(p, grid, smem, overlap, stream);
            return cudaErrorInvalidValue;
        }
        if (p.m == 1) return launch_gemv_inst<Fmt, 1, 1, 8, false, true>(p, grid, smem, overlap, stream);
        if (p.m == 2) return launch_gemv_inst<Fmt, 2, 1, 8, false, true>(p, grid, smem, overlap, stream);
        return cudaErrorInvalidValue;
    }
    if (RW == 1 && p.nchunks > 1) {  // rows cut into pieces: side-by-side shapes with eight consumer warps, m <= 2 only
        if (p.n_cwarps > 8) return cudaErrorInvalidValue;
        if (p.m == 1) return launch_gemv_inst<Fmt, 1, 1, 8, true>(p, grid, smem, overlap, stream);
        if (p.m == 2) return launch_gemv_inst<Fmt, 2, 1, 8, true>(p, grid, smem, overlap, stream);
        return cudaErrorInvalidValue;
    }
    if (RW == 1 && p.n_cwarps > 8) {  // twelve-consumer-warp instances exist for m <= 2 only
        if (p.m == 1) return launch_gemv_inst<Fmt, 1, 1, 12>(p, grid, smem, overlap, stream);
        if (p.m == 2) return launch_gemv_inst<Fmt, 2, 1, 12>(p, grid, smem, overlap, stream);
        return cudaErrorInvalidValue;
    }
    switch (p.m) {
    case 1: return launch_gemv_inst<Fmt, 1, RW>(p, grid, smem, overlap, stream);
    case 2: return launch_gemv_inst<Fmt, 2, RW>(p, grid, smem, overlap, stream);
    case 3: return launch_gemv_inst<Fmt, 3, RW>(p, grid, smem, overlap, stream);
    case 4: return launch_gemv_inst<Fmt, 4, RW>(p, grid, smem, overlap, stream);
    case 5: return launch_gemv_inst<Fmt, 5, RW>(p, grid, smem, overlap, stream);
    case 6: return launch_gemv_inst<Fmt, 6, RW>(p, grid, smem, overlap, stream);
    case 7: return launch_gemv_inst<Fmt, 7, RW>(p, grid, smem, overlap, stream);
    case 8: return launch_gemv_inst<Fmt, 8, RW>(p, grid, smem, overlap, stream);
    }
    return cudaErrorInvalidValue;
}

template <class Fmt>
static cudaError_t launch_gemv_format(const GemvParams &p, int grid, int smem, bool overlap, int rw, cudaStream_t stream) {
    return rw == 2 ? launch_gemv_m<Fmt, 2>(p, grid, smem, overlap, stream) : launch_gemv_m<Fmt, 1>(p, grid, smem, overlap, stream);
}

}  // namespace lloom
