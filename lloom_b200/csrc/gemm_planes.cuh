// Prefill GEMM for Q8_0, Q4_0, Q5_0 and Q6_K weights on tcgen05 tensor cores (sm_100a), exact-integer formulation.
//
//   Q8_0 x Q8_0 (k_quants.rs:800-818, avx.rs:71-87):     y[m,n] = sum over 32-element blocks b of (d_w[n,b]*d_a[m,b]) * dot32(q_w, q_a)
//   Q6_K x Q8_K (k_quants.rs:2115-2172, avx.rs:131-216):  y[m,n] = sum over superblocks b of (d_a[m,b]*d_w[n,b]) * S,
//                                                         S = sum_{j<16} sc_j * dot16(q6_j - 32, q8_j)
// through the m > 1 arm of k_quants::matmul (k_quants.rs:2518-2585).
//
// The block sums are integer contractions, so they run on the tensor cores (kind::f16, f32 accumulators in tensor
// memory) with every operand an integer that f16 represents exactly:
//   Q8_0: A = q_w, B = q_a (|.| <= 127); one accumulator drain per 32 of K, where the two f16 block scales meet.
//   Q4_0 / Q5_0 (k_quants.rs:320-392, 602-700; dotted with Q8_0 activations like Q8_0): the same with A = nibble - 8
//         / (nibble | fifth bit << 4) - 16; only the weight image and the place of the block scale differ.
//   Q6_K: v = sc_j * (q6 - 32) has up to 13 significant bits, so it is split v = hi + lo with lo = v mod 64 in
//         [0, 63] and hi a multiple of 64 in [-4096, 4032]: both exact in f16.  The two planes multiply the same
//         B = q8 codes and add into the same accumulator, which then holds S itself; one drain per 256 of K.
// The kernel is the Q4_K GEMM's frame (gemm_q4k.cuh) with the drain group, the plane count and the activation rows
// per tile (BM, the UMMA N) as parameters: 128 x BM output tile per CTA; operands arrive as ready-made
// 128-byte-swizzled K-major images by bulk copies; 512 / BM accumulators in tensor memory, so the drain of group g
// overlaps the MMAs of the following groups.  An MMA reads both operands from shared memory (8 KB per M = 128,
// N = 128, K = 16 instruction, 12 KB for twice the work at N = 256) and the bulk copies write as much again, so with
// the instruction stream kept short the shared-memory port sets the pace of the MMA side: Q6_K (one drain per 256 of
// K) runs at BM = 256; Q8_0 / Q4_0 / Q5_0 (one drain per 32 of K) are bound by their epilogue and stay at 128.
// Warp roles: 0-7 epilogue, 8 operand copies, 9 MMA issuer (one elected lane), 10 scale tiles (bulk copy of the
// activation scales; for the 32-of-K formats also the gather of the weight rows' f16 scales from the canonical blocks).
// The scale tiles travel in their own ring (a slot = 8 drain groups for the 32-of-K formats), released by the epilogue
// warps separately from the accumulators.  Epilogue of the 32-of-K formats: accumulators are read in the MMA fragment
// layout (tcgen05.ld.16x256b: 4 rows x 16 columns per thread), so a thread needs 16 + 4 scale words per group instead
// of 64 + 1; per output one exact product d_w * d_a and one fused multiply-add, the AVX2 arm's two operations.
// All waits are bounded and abortable; tensor memory is released on every path.
#pragma once

#include "gemm_q4k.cuh"

namespace lloom {

template <int GROUP_K, int PLANES, int BM>
struct PlanesCfg {
    static constexpr int kEpiWarps = 8;                // BM / 2 accumulator columns per warp (sixteen warps of BM / 4
                                                       // columns measured 1.6x slower on the 32-of-K formats)
    static constexpr int kGroupK = GROUP_K;            // K elements per accumulator drain
    static constexpr int kPlanes = PLANES;             // f16 images per weight element
    static constexpr int kBM = BM;                     // activation rows per tile (UMMA N): 128 or 256
    static constexpr int kStageK = PLANES == 1 ? 128 : 64;  // K elements per pipeline stage
    static constexpr int kStages = (PLANES == 1 || BM == 256) ? 3 : 4;
    static constexpr int kAtomsPerStage = kStageK / 64;
    static constexpr int kBAtomBytes = BM * 64 * 2;    // B atom: BM rows x 64 of K
    static constexpr int kStageABytes = kAtomsPerStage * PLANES * kGemmAtomBytes;
    static constexpr int kStageBBytes = kAtomsPerStage * kBAtomBytes;
    static constexpr int kAccBufs = 512 / BM;
    static constexpr int kDaBytes = BM * 4;             // activation scales of one drain group
    // The scale tiles travel in a ring of their own: a slot holds the scales of kDaGroups consecutive drain groups.
    // With a drain every 32 of K a slot covers eight groups, so a copy's trip to L2 is paid once per 256 of K and is
    // not on the path from one drain of an accumulator to its next use.
    static constexpr int kDaGroups = GROUP_K >= 256 ? 1 : 8;
    static constexpr int kDaSlots = GROUP_K >= 256 ? kAccBufs : 3;
    static constexpr int kDaSlotBytes = kDaGroups * kDaBytes;
    // Where a group is 32 of K the weight rows' scales ride in the same ring (gathered from the canonical blocks by the
    // scale warp, 128 f32 per group); where a group is 256 of K each epilogue thread fetches its row's scale itself.
    static constexpr bool kSmemW = GROUP_K < 256;
    static constexpr int kDwSlotBytes = kSmemW ? kDaGroups * kGemmBN * 4 : 0;
    // BM = 256: 128 running sums per epilogue thread; three whole warpgroups, so that the two epilogue warpgroups can
    // take registers from the third (setmaxnreg)
    static constexpr int kThreads = BM == 256 ? 384 : 32 * (kEpiWarps + 3);  // epilogue warps + operand copies + MMA issuer + scale copies
    // shared memory map (offsets from a 1024-byte aligned base)
    static constexpr int kOffA = 0;
    static constexpr int kOffB = kOffA + kStages * kStageABytes;
    static constexpr int kOffDa = kOffB + kStages * kStageBBytes;
    static constexpr int kOffDw = kOffDa + kDaSlots * kDaSlotBytes;
    static constexpr int kOffBars = kOffDw + kDaSlots * kDwSlotBytes;
    static constexpr int kNumBars = 2 * kStages + 2 * kAccBufs + 2 * kDaSlots;
    static constexpr int kOffMisc = kOffBars + kNumBars * 8;
    static constexpr int kSmemBytes = kOffMisc + 16 + 1024;  // + alignment slack
};

// Operand images: activation side [m-tile][k/64 atoms][BM x 128 B] + scales [m-tile][k/GROUP_K][BM] f32;
// weight side [n-tile][k/64 atoms][PLANES][16 KB].
struct PlanesActLayout {
    int64_t bimg, dat, total;
};
__host__ __device__ inline PlanesActLayout planes_act_layout(int64_t m, int64_t k, int group_k, int bm) {
    PlanesActLayout s;
    const int64_t mt = (m + bm - 1) / bm;
    s.bimg = 0;
    s.dat = mt * (k / 64) * bm * 128;
    s.total = (s.dat + mt * (k / group_k) * bm * 4 + 1023) / 1024 * 1024;
    return s;
}
__host__ __device__ inline int64_t planes_weight_bytes(int64_t n, int64_t k, int planes) {
    return (n + kGemmBN - 1) / kGemmBN * (k / 64) * planes * kGemmAtomBytes;
}

__device__ __forceinline__ uint32_t f16x2_from_ints(int a, int b) {
    const __half2 h = __halves2half2(__int2half_rn(a), __int2half_rn(b));
    return *reinterpret_cast<const uint32_t *>(&h);
}

// Canonical activation blocks -> B image + scale plane.  One CTA per (m-tile, 64-element atom of K), one thread
// per activation row of the tile (BM threads).  ACT_Q8_0: 34-byte Q8_0 blocks (f16 d, 32 codes); else 292-byte Q8_K
// blocks (f32 d, 256 codes).
template <bool ACT_Q8_0, int BM>
__global__ void __launch_bounds__(BM) planes_prep_kernel(const uint8_t *__restrict__ act, int m, int k,
                                                         uint8_t *__restrict__ scratch) {
    const int atoms = k / 64;
    const int mt = blockIdx.x / atoms, atom = blockIdx.x % atoms;
    const int t = threadIdx.x, row = mt * BM + t;
    const int group_k = ACT_Q8_0 ? 32 : 256;
    const PlanesActLayout lay = planes_act_layout(m, k, group_k, BM);
    uint8_t *img = scratch + lay.bimg + ((int64_t)mt * atoms + atom) * (BM * 128);
    float *dat = reinterpret_cast<float *>(scratch + lay.dat) + (int64_t)mt * (k / group_k) * BM;
    int q[64];
#pragma unroll
    for (int i = 0; i < 64; ++i) q[i] = 0;
    if (row < m) {
        if (ACT_Q8_0) {
            const uint8_t *blk = act + ((int64_t)row * (k / 32) + atom * 2) * Q8_0_BYTES;  // 2-byte aligned
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const unsigned short *p16 = reinterpret_cast<const unsigned short *>(blk + h * Q8_0_BYTES);
                dat[(atom * 2 + h) * BM + t] = f16_bits_to_f32(p16[0]);
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const unsigned short w = p16[1 + i];
                    q[h * 32 + 2 * i] = (int)(int8_t)(w & 0xff);
                    q[h * 32 + 2 * i + 1] = (int)(int8_t)(w >> 8);
                }
            }
        } else {
            const uint8_t *blk = act + ((int64_t)row * (k / 256) + (atom >> 2)) * Q8K_BYTES;  // 4-byte aligned
            if ((atom & 3) == 0) dat[(atom >> 2) * BM + t] = *reinterpret_cast<const float *>(blk);
            const uint32_t *p32 = reinterpret_cast<const uint32_t *>(blk + 4 + (atom & 3) * 64);
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const uint32_t w = p32[i];
#pragma unroll
                for (int j = 0; j < 4; ++j) q[4 * i + j] = (int)(int8_t)(w >> (8 * j));
            }
        }
    } else {
        if (ACT_Q8_0) {
            dat[(atom * 2) * BM + t] = 0.0f;
            dat[(atom * 2 + 1) * BM + t] = 0.0f;
        } else if ((atom & 3) == 0) {
            dat[(atom >> 2) * BM + t] = 0.0f;
        }
    }
#pragma unroll
    for (int c = 0; c < 8; ++c) {
        const uint4 out = make_uint4(f16x2_from_ints(q[8 * c], q[8 * c + 1]), f16x2_from_ints(q[8 * c + 2], q[8 * c + 3]),
                                     f16x2_from_ints(q[8 * c + 4], q[8 * c + 5]), f16x2_from_ints(q[8 * c + 6], q[8 * c + 7]));
        *reinterpret_cast<uint4 *>(img + sw128_offset(t, 8 * c)) = out;
    }
}

// f32 activations -> the same B image + scale plane in one pass (the forward entries: no canonical blocks in between).
// One warp per (padded activation row, 256-element span of K), lane l holding elements 8l .. 8l + 7 of the span, i.e.
// one 16-byte chunk of the image; the quantizers are the warp functions of the stand-alone quantizer kernels, so the
// codes and scales are those of the canonical blocks bit for bit.  ACT_Q8_0: eight 32-element blocks per span (four
// lanes each; k may end in the middle of a span); else one Q8_K block.
template <bool ACT_Q8_0, int BM>
__global__ void __launch_bounds__(256) planes_prep_f32_kernel(const float *__restrict__ x, int m, int k, uint8_t *__restrict__ scratch) {
    const int spans = (k + 255) / 256, atoms = k / 64;
    const int lane = threadIdx.x & 31;
    const int64_t item = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);  // (padded row, span)
    const int64_t prow = item / spans;
    const int sp = (int)(item % spans);
    const int64_t mt = prow / BM;
    const int t = (int)(prow % BM);
    if (mt >= (m + BM - 1) / BM) return;  // whole warp
    const int group_k = ACT_Q8_0 ? 32 : 256;
    const PlanesActLayout lay = planes_act_layout(m, k, group_k, BM);
    const int e0 = sp * 256 + lane * 8;      // first of the lane's elements
    const bool in_k = e0 < k;
    float v[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = 0.0f;
    if (prow < m && in_k) load8(x + prow * k + e0, v);  // rows of the last tile past m stay zero
    uint32_t q_lo = 0, q_hi = 0;
    float *dat = reinterpret_cast<float *>(scratch + lay.dat) + mt * (k / group_k) * BM;
    if (ACT_Q8_0) {
        unsigned short d16;
        q8_0_quantize_quad(v, q_lo, q_hi, d16);
        if (in_k && (lane & 3) == 0) dat[(int64_t)(sp * 8 + (lane >> 2)) * BM + t] = f16_bits_to_f32(d16);
    } else {
        float d;
        int sum16;
        q8k_quantize_warp(v, lane, q_lo, q_hi, d, sum16);
        if (lane == 0) dat[(int64_t)sp * BM + t] = d;
    }
    if (!in_k) return;
    auto cvt2 = [](uint32_t w, int sh) -> uint32_t {
        const __half2 h = __floats2half2_rn((float)(int)(int8_t)(w >> sh), (float)(int)(int8_t)(w >> (sh + 8)));
        return *reinterpret_cast<const uint32_t *>(&h);
    };
    const int atom = sp * 4 + (lane >> 3), e = (lane & 7) * 8;
    uint8_t *img = scratch + lay.bimg + (mt * atoms + atom) * (int64_t)(BM * 128);
    *reinterpret_cast<uint4 *>(img + sw128_offset(t, e)) = make_uint4(cvt2(q_lo, 0), cvt2(q_lo, 16), cvt2(q_hi, 0), cvt2(q_hi, 16));
}

// Q8_0 weight blocks -> A image (one plane: the codes as f16).  One CTA per (n-tile, 64-element atom), one thread
// per weight row; rows past n are zero.  `row0` is the first row of the image's slab within the matrix.
__global__ void __launch_bounds__(128) planes_expand_q8_0_kernel(const uint8_t *__restrict__ w, int64_t row0, int n_end,
                                                                 int k, uint8_t *__restrict__ image) {
    const int atoms = k / 64;
    const int nt = blockIdx.x / atoms, atom = blockIdx.x % atoms;
    const int r = threadIdx.x;
    const int64_t row = row0 + (int64_t)nt * kGemmBN + r;
    uint8_t *img = image + ((int64_t)nt * atoms + atom) * kGemmAtomBytes;
    int q[64];
#pragma unroll
    for (int i = 0; i < 64; ++i) q[i] = 0;
    if (row < n_end) {
        const uint8_t *blk = w + (row * (k / 32) + atom * 2) * Q8_0_BYTES;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const unsigned short *p16 = reinterpret_cast<const unsigned short *>(blk + h * Q8_0_BYTES);
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const unsigned short v = __ldg(p16 + 1 + i);
                q[h * 32 + 2 * i] = (int)(int8_t)(v & 0xff);
                q[h * 32 + 2 * i + 1] = (int)(int8_t)(v >> 8);
            }
        }
    }
#pragma unroll
    for (int c = 0; c < 8; ++c) {
        const uint4 out = make_uint4(f16x2_from_ints(q[8 * c], q[8 * c + 1]), f16x2_from_ints(q[8 * c + 2], q[8 * c + 3]),
                                     f16x2_from_ints(q[8 * c + 4], q[8 * c + 5]), f16x2_from_ints(q[8 * c + 6], q[8 * c + 7]));
        *reinterpret_cast<uint4 *>(img + sw128_offset(r, 8 * c)) = out;
    }
}

// Q4_0 / Q5_0 weight blocks -> A image (one plane: nibble - 8, or (nibble | fifth bit << 4) - 16, as f16;
// k_quants.rs:299-318, 578-600: low nibbles are elements 0..15 of a block, high nibbles 16..31).  Same grid as Q8_0.
template <bool FIVE_BIT>
__global__ void __launch_bounds__(128) planes_expand_q4or5_0_kernel(const uint8_t *__restrict__ w, int64_t row0, int n_end,
                                                                    int k, uint8_t *__restrict__ image) {
    constexpr int kBlk = FIVE_BIT ? Q5_0_BYTES : Q4_0_BYTES;
    const int atoms = k / 64;
    const int nt = blockIdx.x / atoms, atom = blockIdx.x % atoms;
    const int r = threadIdx.x;
    const int64_t row = row0 + (int64_t)nt * kGemmBN + r;
    uint8_t *img = image + ((int64_t)nt * atoms + atom) * kGemmAtomBytes;
    int q[64];
#pragma unroll
    for (int i = 0; i < 64; ++i) q[i] = 0;
    if (row < n_end) {
        const uint8_t *blk = w + (row * (k / 32) + atom * 2) * kBlk;  // 2-byte aligned
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const unsigned short *p16 = reinterpret_cast<const unsigned short *>(blk + h * kBlk);
            uint32_t bits = 0;
            if (FIVE_BIT) bits = (uint32_t)__ldg(p16 + 1) | ((uint32_t)__ldg(p16 + 2) << 16);
            const unsigned short *qs = p16 + (FIVE_BIT ? 3 : 1);
#pragma unroll
            for (int i = 0; i < 8; ++i) {  // bytes 2i, 2i+1: elements 2i, 2i+1 (low nibbles) and 16 + 2i, 17 + 2i (high)
                const unsigned short v = __ldg(qs + i);
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    const int byte = (v >> (8 * j)) & 0xff, l = 2 * i + j;
                    if (FIVE_BIT) {
                        q[h * 32 + l] = ((byte & 0xF) | (int)(((bits >> l) & 1u) << 4)) - 16;
                        q[h * 32 + 16 + l] = ((byte >> 4) | (int)(((bits >> (16 + l)) & 1u) << 4)) - 16;
                    } else {
                        q[h * 32 + l] = (byte & 0xF) - 8;
                        q[h * 32 + 16 + l] = (byte >> 4) - 8;
                    }
                }
            }
        }
    }
#pragma unroll
    for (int c = 0; c < 8; ++c) {
        const uint4 out = make_uint4(f16x2_from_ints(q[8 * c], q[8 * c + 1]), f16x2_from_ints(q[8 * c + 2], q[8 * c + 3]),
                                     f16x2_from_ints(q[8 * c + 4], q[8 * c + 5]), f16x2_from_ints(q[8 * c + 6], q[8 * c + 7]));
        *reinterpret_cast<uint4 *>(img + sw128_offset(r, 8 * c)) = out;
    }
}

// Q6_K weight blocks -> A image, two planes per atom: hi = v - (v mod 64), lo = v mod 64 with v = sc_j * (q6 - 32)
// (k_quants.rs:2327-2358 for the code layout).  One CTA per (n-tile, 64-element atom), one thread per weight row.
__global__ void __launch_bounds__(128) planes_expand_q6k_kernel(const uint8_t *__restrict__ w, int64_t row0, int n_end,
                                                                int k, uint8_t *__restrict__ image) {
    const int atoms = k / 64;
    const int nt = blockIdx.x / atoms, atom = blockIdx.x % atoms;
    const int r = threadIdx.x;
    const int64_t row = row0 + (int64_t)nt * kGemmBN + r;
    uint8_t *img_hi = image + (((int64_t)nt * atoms + atom) * 2) * kGemmAtomBytes;
    uint8_t *img_lo = img_hi + kGemmAtomBytes;
    const int a = atom & 3;         // atom of the superblock: elements 64a .. 64a+63
    const int h = a >> 1;           // half of the superblock
    const int gq0 = (a & 1) * 2;    // element e = 128h + 32gq + l: this atom holds gq0 (l = 0..31) and gq0 + 1
    int v[64];
#pragma unroll
    for (int i = 0; i < 64; ++i) v[i] = 0;
    if (row < n_end) {
        const uint8_t *blk = w + (row * (k / 256) + (atom >> 2)) * Q6K_BYTES;  // 2-byte aligned
        const unsigned short *ql16 = reinterpret_cast<const unsigned short *>(blk + 64 * h);
        const unsigned short *qh16 = reinterpret_cast<const unsigned short *>(blk + 128 + 32 * h);
        const unsigned short *sc16 = reinterpret_cast<const unsigned short *>(blk + 192 + 8 * h);
        int sc[8];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const unsigned short s2 = __ldg(sc16 + i);
            sc[2 * i] = (int)(int8_t)(s2 & 0xff);
            sc[2 * i + 1] = (int)(int8_t)(s2 >> 8);
        }
#pragma unroll
        for (int gi = 0; gi < 2; ++gi) {
            const int gq = gq0 + gi;  // gq 0: ql[l] low nibble, 1: ql[l+32] low, 2: ql[l] high, 3: ql[l+32] high
#pragma unroll
            for (int i = 0; i < 16; ++i) {  // two elements l = 2i, 2i+1 per 16-bit load
                const unsigned short lw = __ldg(ql16 + ((gq & 1) * 32 + 2 * i) / 2);
                const unsigned short hw = __ldg(qh16 + i);
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    const int l = 2 * i + j;
                    const int lb = (lw >> (8 * j)) & 0xff, hb = (hw >> (8 * j)) & 0xff;
                    const int lo4 = (gq & 2) ? (lb >> 4) : (lb & 0xF);
                    const int code = (lo4 | (((hb >> (2 * gq)) & 3) << 4)) - 32;
                    v[gi * 32 + l] = sc[(l >> 4) + 2 * gq] * code;
                }
            }
        }
    }
#pragma unroll
    for (int c = 0; c < 8; ++c) {
        int lo[8], hi[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            lo[i] = v[8 * c + i] & 63;
            hi[i] = v[8 * c + i] - lo[i];
        }
        const int off = sw128_offset(r, 8 * c);
        *reinterpret_cast<uint4 *>(img_hi + off) = make_uint4(f16x2_from_ints(hi[0], hi[1]), f16x2_from_ints(hi[2], hi[3]),
                                                              f16x2_from_ints(hi[4], hi[5]), f16x2_from_ints(hi[6], hi[7]));
        *reinterpret_cast<uint4 *>(img_lo + off) = make_uint4(f16x2_from_ints(lo[0], lo[1]), f16x2_from_ints(lo[2], lo[3]),
                                                              f16x2_from_ints(lo[4], lo[5]), f16x2_from_ints(lo[6], lo[7]));
    }
}

// 16 lanes x 64 columns of tensor memory as the MMA accumulator fragment: thread T = 4*g + c holds, for each block i of
// eight columns, v[4i], v[4i+1] = lane g, columns 8i + 2c, 8i + 2c + 1 and v[4i+2], v[4i+3] = lane g + 8, same columns.
__device__ __forceinline__ void tmem_ld_frag64(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.16x256b.x8.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
          "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
          "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr));
}

struct PlanesParams {
    const uint8_t *w;        // canonical weight blocks of the whole matrix (for the per-group f16 scales)
    const uint8_t *act_img;  // planes_prep_kernel output
    const uint8_t *w_img;    // expand kernel output for rows [row0, row0 + n_tiles * 128)
    float *y;
    int64_t ldy;
    int64_t row_bytes;
    int64_t row0;   // first weight row of this launch (a slab of the matrix)
    int m, n_end, k;  // n_end: rows of the whole matrix (rows >= n_end are masked)
    int n_tiles, m_tiles;
    int scale_stride, scale_off;  // weight scale of group g of a row: f16 at row + g * scale_stride + scale_off
};

template <class Cfg>
__global__ void __launch_bounds__(Cfg::kThreads, 1) gemm_planes_kernel(const PlanesParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + Cfg::kOffBars);
    uint64_t *full = bars, *empty = bars + Cfg::kStages;
    uint64_t *acc_full = bars + 2 * Cfg::kStages, *acc_empty = acc_full + Cfg::kAccBufs;
    uint64_t *da_full = acc_empty + Cfg::kAccBufs, *da_empty = da_full + Cfg::kDaSlots;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem + Cfg::kOffMisc);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + Cfg::kOffMisc + 4);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // m-tiles of one n-tile are neighbours in launch order, so the n-tile's A images are shared through L2
    const int mt = blockIdx.x % p.m_tiles, nt = blockIdx.x / p.m_tiles;
    const int m0 = mt * Cfg::kBM;
    const int64_t n0 = p.row0 + (int64_t)nt * kGemmBN;
    const int atoms = p.k / 64;
    const int ngroups = p.k / Cfg::kGroupK;
    const int nstages = p.k / Cfg::kStageK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < Cfg::kStages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int i = 0; i < Cfg::kAccBufs; ++i) {
            mbar_init(&acc_full[i], 1);
            mbar_init(&acc_empty[i], Cfg::kEpiWarps);
        }
        for (int i = 0; i < Cfg::kDaSlots; ++i) {
            mbar_init(&da_full[i], Cfg::kSmemW ? 2 : 1);  // the copy's bytes (+ the gathered weight scales)
            mbar_init(&da_empty[i], Cfg::kEpiWarps);
        }
        *abort_flag = 0;
        fence_mbar_init();
    }
    if (warp == Cfg::kEpiWarps + 1) {  // tensor memory: all 512 columns, 512 / BM accumulators
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512u)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    // BM = 256, per scheduler: two epilogue warps of 216 registers and one other warp of 72.  One setmaxnreg per
    // warpgroup, executed by all of its warps at the top of the branch that holds all of the warpgroup's code.
    if (warp < Cfg::kEpiWarps) {
        // ------------------------------ epilogue ------------------------------
        // warp w: TMEM lanes 32*(w%4).. (hardware rule), accumulator columns (BM/2)*(w/4)..
        if (Cfg::kBM == 256) asm volatile("setmaxnreg.inc.sync.aligned.u32 216;" ::: "memory");
        constexpr int kCW = Cfg::kBM / (Cfg::kEpiWarps / 4);  // columns per warp
        const int q = warp & 3, half = warp >> 2;
        if (Cfg::kSmemW) {
            // A drain every 32 of K: the scales, not the sums, set the cost.  With a tensor-memory lane per thread every
            // thread would fetch all 64 activation scales of its columns for every group (the same words in all 32
            // lanes, 64 shared-memory wavefronts per warp and group); in the accumulator-fragment layout a thread
            // holds 4 rows x 16 columns, so it needs 16 activation scales and 4 weight scales (20 wavefronts).
            const int fg = lane >> 2, fc = lane & 3;
            float acc[4][16];  // [row j: 32q + fg + 8j][2i + e: column 64*half + 8i + 2fc + e]
#pragma unroll
            for (int j = 0; j < 4; ++j)
#pragma unroll
                for (int i = 0; i < 16; ++i) acc[j][i] = 0.0f;
            bool ok = true;
            for (int g = 0; g < ngroups && ok; ++g) {
                const int buf = g % Cfg::kAccBufs;
                const uint32_t par = (g / Cfg::kAccBufs) & 1;
                const int slot_i = g / Cfg::kDaGroups, in_slot = g % Cfg::kDaGroups, slot = slot_i % Cfg::kDaSlots;
                if (in_slot == 0) ok = mbar_wait_abortable<64>(&da_full[slot], (slot_i / Cfg::kDaSlots) & 1, abort_flag);
                if (!ok) break;
                const float *dws = reinterpret_cast<const float *>(smem + Cfg::kOffDw + slot * Cfg::kDwSlotBytes) +
                                   in_slot * kGemmBN + q * 32 + fg;
                const float2 *das = reinterpret_cast<const float2 *>(smem + Cfg::kOffDa + slot * Cfg::kDaSlotBytes +
                                                                     in_slot * Cfg::kDaBytes + half * kCW * 4) + fc;
                float dw[4];
                float2 da2[8];
#pragma unroll
                for (int j = 0; j < 4; ++j) dw[j] = dws[8 * j];
#pragma unroll
                for (int i = 0; i < 8; ++i) da2[i] = das[4 * i];
                ok = mbar_wait_abortable<64>(&acc_full[buf], par, abort_flag);
                if (!ok) break;
                tc_fence_after();
                const uint32_t t_main = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * Cfg::kBM + half * kCW);
                uint32_t va[32], vb[32];
                tmem_ld_frag64(t_main, va);                     // lanes 32q .. 32q + 15
                tmem_ld_frag64(t_main + (16u << 16), vb);       // lanes 32q + 16 .. 32q + 31
                tmem_ld_wait();
                // everything this warp needs from tensor memory and from the scale tiles is in registers now
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&acc_empty[buf]);
                if (in_slot == Cfg::kDaGroups - 1 || g == ngroups - 1) {
                    // the slot is rewritten by a bulk copy (async proxy) right after the arrivals, so this warp's reads
                    // of it (generic proxy) are fenced first
                    fence_proxy_async();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&da_empty[slot]);
                }
                // scalar multiplies and fused multiply-adds: they issue on both FMA pipes, the packed f32x2 forms on one
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const uint32_t *v = (j < 2) ? va : vb;
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const int ix = 4 * i + 2 * (j & 1);
                        acc[j][2 * i] = __fmaf_rn(__fmul_rn(da2[i].x, dw[j]), __uint_as_float(v[ix]), acc[j][2 * i]);
                        acc[j][2 * i + 1] = __fmaf_rn(__fmul_rn(da2[i].y, dw[j]), __uint_as_float(v[ix + 1]), acc[j][2 * i + 1]);
                    }
                }
            }
            if (ok) {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int64_t n = n0 + q * 32 + fg + 8 * j;
                    if (n >= p.n_end) continue;
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const int mrow = m0 + half * kCW + 8 * i + 2 * fc;
                        if (mrow < p.m) p.y[(int64_t)mrow * p.ldy + n] = acc[j][2 * i];
                        if (mrow + 1 < p.m) p.y[(int64_t)(mrow + 1) * p.ldy + n] = acc[j][2 * i + 1];
                    }
                }
            }
        } else {
        const int r = q * 32 + lane;  // row of the tile == TMEM lane
        const int64_t n = n0 + r;
        const bool row_ok = n < p.n_end;
        const uint8_t *wrow = p.w + (row_ok ? n : 0) * p.row_bytes + p.scale_off;
        uint64_t out2[kCW / 2];
#pragma unroll
        for (int j = 0; j < kCW / 2; ++j) out2[j] = 0ull;
        // group >= 256 of K: the row's weight scale of the next group is fetched while this group is drained
        unsigned short hdr_nxt = 0;
        if (row_ok) hdr_nxt = __ldg(reinterpret_cast<const unsigned short *>(wrow));
        bool ok = true;
        for (int g = 0; g < ngroups && ok; ++g) {
            const int buf = g % Cfg::kAccBufs;
            const uint32_t par = (g / Cfg::kAccBufs) & 1;
            const int slot_i = g / Cfg::kDaGroups, in_slot = g % Cfg::kDaGroups, slot = slot_i % Cfg::kDaSlots;
            if (in_slot == 0) ok = mbar_wait_abortable<64>(&da_full[slot], (slot_i / Cfg::kDaSlots) & 1, abort_flag);
            if (!ok) break;
            const float dw = f16_bits_to_f32(hdr_nxt);
            if (row_ok && g + 1 < ngroups)
                hdr_nxt = __ldg(reinterpret_cast<const unsigned short *>(wrow + (int64_t)(g + 1) * p.scale_stride));
            const uint64_t dw2 = pack2f(dw, dw);
            ok = mbar_wait_abortable<64>(&acc_full[buf], par, abort_flag);
            if (!ok) break;
            tc_fence_after();
            const uint32_t t_main = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * Cfg::kBM + half * kCW);
            // the activation scales of this warp's columns, as f32 pairs, times the weight scale: (d_a * d_w)
            const ulonglong2 *dap = reinterpret_cast<const ulonglong2 *>(smem + Cfg::kOffDa + slot * Cfg::kDaSlotBytes +
                                                                         in_slot * Cfg::kDaBytes + half * kCW * 4);
#pragma unroll
            for (int c = 0; c < kCW / 64; ++c) {  // 64 columns at a time: two loads in flight
                uint32_t va[32], vb[32];
                tmem_ld32(t_main + 64 * c, va);
                tmem_ld32(t_main + 64 * c + 32, vb);
                uint64_t d2[16];
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const ulonglong2 t = dap[16 * c + j];
                    d2[2 * j] = mul_f32x2(t.x, dw2);
                    d2[2 * j + 1] = mul_f32x2(t.y, dw2);
                }
                tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 16; ++j)
                    out2[32 * c + j] = fma_f32x2(d2[j], (uint64_t)va[2 * j] | ((uint64_t)va[2 * j + 1] << 32), out2[32 * c + j]);
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const ulonglong2 t = dap[16 * c + 8 + j];
                    d2[2 * j] = mul_f32x2(t.x, dw2);
                    d2[2 * j + 1] = mul_f32x2(t.y, dw2);
                }
                if (c == kCW / 64 - 1) {
                    // everything this warp needs from tensor memory and from the scale tiles is in registers now
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&acc_empty[buf]);
                    if (in_slot == Cfg::kDaGroups - 1 || g == ngroups - 1) {
                        // the slot is rewritten by a bulk copy (async proxy) right after the arrivals, so this warp's
                        // reads of it (generic proxy) are fenced first
                        fence_proxy_async();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&da_empty[slot]);
                    }
                }
#pragma unroll
                for (int j = 0; j < 16; ++j)
                    out2[32 * c + 16 + j] = fma_f32x2(d2[j], (uint64_t)vb[2 * j] | ((uint64_t)vb[2 * j + 1] << 32), out2[32 * c + 16 + j]);
            }
        }
        if (ok && row_ok) {
#pragma unroll
            for (int j = 0; j < kCW / 2; ++j) {
                const int mrow = m0 + half * kCW + 2 * j;
                if (mrow < p.m) p.y[(int64_t)mrow * p.ldy + n] = __uint_as_float((uint32_t)(out2[j] & 0xffffffffu));
                if (mrow + 1 < p.m) p.y[(int64_t)(mrow + 1) * p.ldy + n] = __uint_as_float((uint32_t)(out2[j] >> 32));
            }
        }
        }
    } else {
    if (Cfg::kBM == 256) asm volatile("setmaxnreg.dec.sync.aligned.u32 72;" ::: "memory");
    if (warp == Cfg::kEpiWarps) {
        // ------------------------------ operand tiles: bulk copies ------------------------------
        // The whole warp walks the loop (lanes stay converged); lane 0 issues the copies.
        const uint8_t *aimg = p.w_img + (int64_t)nt * atoms * Cfg::kPlanes * kGemmAtomBytes;
        const uint8_t *bimg = p.act_img + (int64_t)mt * atoms * Cfg::kBAtomBytes;
        bool ok = true;
        for (int it = 0; it < nstages && ok; ++it) {
            const int s = it % Cfg::kStages;
            if (it >= Cfg::kStages) ok = mbar_wait_abortable<32>(&empty[s], ((it / Cfg::kStages) - 1) & 1, abort_flag);
            if (!ok) break;
            if (lane == 0) {
                mbar_arrive_expect_tx(&full[s], Cfg::kStageABytes + Cfg::kStageBBytes);
                bulk_g2s(smem + Cfg::kOffA + s * Cfg::kStageABytes, aimg + (int64_t)it * Cfg::kStageABytes, Cfg::kStageABytes, &full[s]);
                bulk_g2s(smem + Cfg::kOffB + s * Cfg::kStageBBytes, bimg + (int64_t)it * Cfg::kStageBBytes, Cfg::kStageBBytes, &full[s]);
            }
            __syncwarp();
        }
    } else if (warp == Cfg::kEpiWarps + 2) {
        // ------------------------------ activation scales, a slot of drain groups at a time ------------------------------
        const PlanesActLayout lay = planes_act_layout(p.m, p.k, Cfg::kGroupK, Cfg::kBM);
        const uint8_t *dat = p.act_img + lay.dat + (int64_t)mt * ngroups * Cfg::kDaBytes;
        const int nslots = (ngroups + Cfg::kDaGroups - 1) / Cfg::kDaGroups;
        bool ok = true;
        for (int si = 0; si < nslots && ok; ++si) {
            const int slot = si % Cfg::kDaSlots;
            if (si >= Cfg::kDaSlots) ok = mbar_wait_abortable<32>(&da_empty[slot], ((si / Cfg::kDaSlots) - 1) & 1, abort_flag);
            if (!ok) break;
            if (lane == 0) {
                const int groups = min(Cfg::kDaGroups, ngroups - si * Cfg::kDaGroups);
                const uint32_t bytes = (uint32_t)(groups * Cfg::kDaBytes);
                mbar_arrive_expect_tx(&da_full[slot], bytes);
                bulk_g2s(smem + Cfg::kOffDa + slot * Cfg::kDaSlotBytes, dat + (int64_t)si * Cfg::kDaSlotBytes, bytes, &da_full[slot]);
            }
            if (Cfg::kSmemW) {
                // the f16 scales of the tile's 128 weight rows for the slot's groups: lane l gathers rows l, l + 32, ...
                const int groups = min(Cfg::kDaGroups, ngroups - si * Cfg::kDaGroups);
                float *dws = reinterpret_cast<float *>(smem + Cfg::kOffDw + slot * Cfg::kDwSlotBytes);
#pragma unroll
                for (int j = 0; j < kGemmBN / 32; ++j) {
                    const int rr = lane + 32 * j;
                    const bool rok = n0 + rr < p.n_end;
                    const uint8_t *wp = p.w + (rok ? n0 + rr : 0) * p.row_bytes + p.scale_off +
                                        (int64_t)si * Cfg::kDaGroups * p.scale_stride;
                    unsigned short h[Cfg::kDaGroups];
#pragma unroll
                    for (int gi = 0; gi < Cfg::kDaGroups; ++gi)
                        h[gi] = (rok && gi < groups) ? __ldg(reinterpret_cast<const unsigned short *>(wp + (int64_t)gi * p.scale_stride))
                                                     : (unsigned short)0;
#pragma unroll
                    for (int gi = 0; gi < Cfg::kDaGroups; ++gi) dws[gi * kGemmBN + rr] = f16_bits_to_f32(h[gi]);
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&da_full[slot]);
            }
            __syncwarp();
        }
    } else if (warp == Cfg::kEpiWarps + 1) {
        // ------------------------------ MMA issuer ------------------------------
        // The whole warp walks the loop; lane 0 issues the MMAs and commits.
        // instruction descriptor: D = f32, A = B = f16, both K-major, N = BM, M = 128
        const uint32_t idesc = (1u << 4) | ((uint32_t)(Cfg::kBM >> 3) << 17) | ((uint32_t)(kGemmBN >> 4) << 24);
        const uint32_t a_lo0 = umma_desc_lo(smem_u32(smem + Cfg::kOffA), 16), b_lo0 = umma_desc_lo(smem_u32(smem + Cfg::kOffB), 16);
        constexpr int kStepsPerStage = Cfg::kStageK / 16;
        constexpr int kStepsPerGroup = Cfg::kGroupK / 16;
        bool ok = true;
        for (int it = 0; it < nstages && ok; ++it) {
            const int s = it % Cfg::kStages;
            ok = mbar_wait_abortable<0>(&full[s], (it / Cfg::kStages) & 1, abort_flag);
            if (!ok) break;
            tc_fence_after();
            const uint32_t a_lo = a_lo0 + (uint32_t)(s * (Cfg::kStageABytes >> 4));
            const uint32_t b_lo = b_lo0 + (uint32_t)(s * (Cfg::kStageBBytes >> 4));
#pragma unroll
            for (int kk = 0; kk < kStepsPerStage; ++kk) {  // K = 16 per instruction: atom kk/4, 32 bytes along its swizzled row
                const int step = it * kStepsPerStage + kk;
                const int g = step / kStepsPerGroup, in_group = step % kStepsPerGroup;
                const int buf = g % Cfg::kAccBufs;
                if (in_group == 0 && g >= Cfg::kAccBufs) {
                    ok = mbar_wait_abortable<0>(&acc_empty[buf], ((g / Cfg::kAccBufs) - 1) & 1, abort_flag);
                    if (!ok) break;
                    tc_fence_after();
                }
                if (lane == 0) {
                    const uint32_t d_acc = tmem_base + (uint32_t)(buf * Cfg::kBM);
                    const uint32_t boff = (uint32_t)((kk >> 2) * (Cfg::kBAtomBytes >> 4) + (kk & 3) * 2);
#pragma unroll
                    for (int pl = 0; pl < Cfg::kPlanes; ++pl) {
                        const uint32_t aoff = (uint32_t)(((kk >> 2) * Cfg::kPlanes + pl) * (kGemmAtomBytes >> 4) + (kk & 3) * 2);
                        if (pl != 0 || (kk % kStepsPerGroup) != 0) umma_f16_lo<true>(d_acc, a_lo + aoff, b_lo + boff, idesc);
                        else umma_f16_lo_rt(d_acc, a_lo + aoff, b_lo + boff, idesc, in_group != 0 ? 1u : 0u);
                    }
                    if (in_group == kStepsPerGroup - 1) umma_commit(&acc_full[buf]);
                }
                __syncwarp();
            }
            if (!ok) break;
            if (lane == 0) umma_commit(&empty[s]);
            __syncwarp();
        }
    }
    }
    // ------------------------------ teardown ------------------------------
    tc_fence_before();
    __syncthreads();
    if (warp == Cfg::kEpiWarps + 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
    }
}

}  // namespace lloom
