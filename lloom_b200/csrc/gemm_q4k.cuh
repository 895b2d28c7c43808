// Prefill GEMM for Q4_K weights on tcgen05 tensor cores (sm_100a), exact-integer formulation.
//
//   y[m, n] = sum over superblocks b of  (d_a[m,b]*d_w[n,b]) * S[n,m,b]  +  (-d_a[m,b]*dmin_w[n,b]) * Mn[n,m,b]
//   S  = sum_j sc_j * dot32(q4_j, q8_j)      Mn = sum_j m_j * (bsums[2j] + bsums[2j+1])
// (BlockQ4K::vec_dot, lloom-tensor/src/quantized/k_quants.rs:1540-1620 / avx.rs:443-525, through the
// m > 1 arm of k_quants::matmul, :2518-2585).
//
// S and Mn are integer contractions, so they run on the tensor cores with every operand an integer
// that f16 represents exactly:  A = sc_j*q4 (<= 945),  B = q8 codes (|.| <= 127),  A_min = m_j (<= 63,
// each duplicated against the two 16-element bsums it multiplies),  B_min = bsums (|.| <= 2032); the
// f32 accumulators in tensor memory then hold the integers.  One 128x128 accumulator pair (S, Mn)
// is produced per 256-element superblock and drained by the epilogue warps, which apply the two f32
// scales in the reference's algebraic form and keep the running sum in registers -- the per-block
// scale granularity of the format is what forces a drain per superblock.  Tensor memory holds two
// accumulator pairs (2 x (128 + 128) = 512 columns), so the drain of superblock b overlaps the MMAs
// of superblock b+1.
//
// Three launches per call:
//   gemm_prep_f32_kernel f32 activations -> f16 operand images (B, B_min) + scale planes, quantizing on the way (the
//                        forward entries); gemm_prep_kernel: the same from canonical Q8_K blocks (lloom_b200_gemm)
//   gemm_expand_kernel   Q4_K weight blocks -> f16 operand images (A = sc*q, A_min = m_j); a bandwidth pass
//                        (33 MB in, 125 MB out for [14336, 4096]) that spares every output tile from
//                        re-unpacking its 128 weight rows on CUDA cores beside the MMAs
//   gemm_q4k_kernel      one CTA per 128 x 128 output tile; all operands arrive as ready-made shared-memory
//                        images (128-byte-swizzled K-major UMMA layout) by bulk copies.  Warp roles:
//                          warps 0-15 epilogue: tcgen05.ld in the MMA fragment layout -> f32x2 FMAs; warp w reads
//                                     TMEM lanes 32*(w%4).., columns 32*(w/4)..
//                          warp 16    bulk-copy (TMA engine) producer
//                          warp 17    MMA issuer (one elected lane): 8 x tcgen05.mma.kind::f16 (K = 16) per stage
//                          warp 18    the tile's 128 row headers (d, dmin) per superblock -> shared memory
// An MMA reads its 8 KB of operands from shared memory in 65 cycles and the bulk copies write the same bytes first:
// the shared-memory port, not the tensor pipe, bounds this tile shape, so everything else is kept off that port
// (row headers gathered once per tile, activation scales loaded once per fragment column pair).
// All mbarrier waits are bounded and abortable; on a time-out the status word is set, every role
// leaves its loop, and tensor memory is still released.
#pragma once

#include <cuda_fp16.h>

#include "common.cuh"
#include "quantize_act.cuh"

namespace lloom {

constexpr int kGemmBN = 128;          // weight rows per tile (UMMA M)
constexpr int kGemmBM = 128;          // activation rows per tile (UMMA N)
constexpr int kGemmAtomBytes = 128 * 64 * 2;   // one swizzle atom: 128 rows x 64 of K, f16
constexpr int kGemmStageAtoms = 2;                   // swizzle atoms per operand and pipeline stage (64 of K each); one atom per stage and six stages measured 13% slower
constexpr int kGemmStageBytes = kGemmStageAtoms * kGemmAtomBytes;
constexpr int kGemmStagesPerSb = 4 / kGemmStageAtoms;  // stages per 256-element superblock
constexpr int kGemmMinBytes = 128 * 16 * 2;    // min-term operand tile (K = 16), f16
constexpr int kGemmDaBytes = 128 * 4;
constexpr int kGemmStages = 6 / kGemmStageAtoms;     // 192 KB of operand stages
constexpr int kGemmThreads = 320;  // 8 epilogue warps + bulk-copy warp + MMA warp (plane GEMMs)
constexpr int kGemmEpiWarps = 8;
// Q4_K kernel: sixteen epilogue warps (four per tensor-memory lane quarter, 32 accumulator columns each): with S and Mn
// to drain per superblock, eight warps at two per scheduler left part of the drain exposed
constexpr int kQ4kEpiWarps = 16;
constexpr int kQ4kThreads = 32 * (kQ4kEpiWarps + 3);  // + copy warp, MMA warp, row-scale warp

// ---- shared memory map (offsets from a 1024-byte aligned base) ----
constexpr int kOffA = 0;
constexpr int kOffB = kOffA + kGemmStages * kGemmStageBytes;
constexpr int kOffMinA = kOffB + kGemmStages * kGemmStageBytes;
constexpr int kOffMinB = kOffMinA + 2 * kGemmMinBytes;
constexpr int kOffDa = kOffMinB + 2 * kGemmMinBytes;
constexpr int kOffHdr = kOffDa + 2 * kGemmDaBytes;   // (d_w, -dmin_w) of the tile's 128 weight rows, per superblock
constexpr int kGemmHdrBytes = 128 * 8;
constexpr int kOffBars = kOffHdr + 2 * kGemmHdrBytes;
constexpr int kGemmNumBars = 2 * kGemmStages + 6;
constexpr int kOffMisc = kOffBars + kGemmNumBars * 8;
constexpr int kGemmSmemBytes = kOffMisc + 16 + 1024;  // + alignment slack

__host__ __device__ inline int64_t gemm_m_tiles(int64_t m) { return (m + kGemmBM - 1) / kGemmBM; }

// Operand images the GEMM reads.  Activation side (per call, in the caller's workspace): B images, min-B images,
// scales.  Weight side: A images and min-A images -- built per call in the workspace, or once per weight matrix
// into a caller-owned buffer (lloom_b200_weight_image_build) that later calls pass instead.
struct GemmActLayout {
    int64_t bimg, minb, dat, total;
};
struct GemmWeightLayout {
    int64_t aimg, mina, total;
};
__host__ __device__ inline GemmActLayout gemm_act_layout(int64_t m, int64_t k) {
    GemmActLayout s;
    const int64_t mt = gemm_m_tiles(m), nb = k / 256;
    s.bimg = 0;
    s.minb = s.bimg + mt * (k / 64) * kGemmAtomBytes;
    s.dat = s.minb + mt * nb * kGemmMinBytes;
    s.total = (s.dat + mt * nb * kGemmDaBytes + 1023) / 1024 * 1024;
    return s;
}
__host__ __device__ inline GemmWeightLayout gemm_weight_layout(int64_t n, int64_t k) {
    GemmWeightLayout s;
    const int64_t nt = (n + kGemmBN - 1) / kGemmBN, nb = k / 256;
    s.aimg = 0;
    s.mina = s.aimg + nt * (k / 64) * kGemmAtomBytes;
    s.total = (s.mina + nt * nb * kGemmMinBytes + 1023) / 1024 * 1024;
    return s;
}

// Byte offset of element (row r, k-element e in [0,64)) inside a 128-row k-stage image:
// K-major, 128-byte rows, 8-row groups of 1024 bytes, 16-byte chunks XOR-swizzled by the row (SWIZZLE_128B).
__host__ __device__ inline int sw128_offset(int r, int e) {
    return (r >> 3) * 1024 + (r & 7) * 128 + ((((e >> 3) ^ (r & 7)) & 7) << 4) + (e & 7) * 2;
}
// Byte offset inside a min-term tile (128 rows x 16 f16), K-major without swizzle:
// core matrices of 8 rows x 16 bytes; K-chunk stride 128 bytes, 8-row-group stride 256 bytes.
__host__ __device__ inline int min_tile_offset(int r, int e) {
    return ((r >> 3) * 2 + (e >> 3)) * 128 + (r & 7) * 16 + (e & 7) * 2;
}

// Canonical Q8_K activation blocks -> the GEMM's operand images.  One CTA per (m-tile, superblock):
// thread (t, c) converts 8 consecutive codes of token t to f16 and stores one 16-byte chunk.
__global__ void __launch_bounds__(256) gemm_prep_kernel(const uint8_t *__restrict__ act, int m, int k,
                                                        uint8_t *__restrict__ scratch) {
    const int nb = k / 256;
    const int quarter = blockIdx.x & 3;  // 32 tokens of the tile per CTA
    const int mt = (blockIdx.x >> 2) / nb, b = (blockIdx.x >> 2) % nb;
    const GemmActLayout lay = gemm_act_layout(m, k);
    uint8_t *bimg = scratch + lay.bimg + ((int64_t)mt * (k / 64) + (int64_t)b * 4) * kGemmAtomBytes;
    uint8_t *minb = scratch + lay.minb + ((int64_t)mt * nb + b) * kGemmMinBytes;
    float *dat = reinterpret_cast<float *>(scratch + lay.dat) + ((int64_t)mt * nb + b) * 128;
    for (int i = threadIdx.x; i < 32 * 32; i += blockDim.x) {
        const int t = quarter * 32 + (i >> 5), c = i & 31;  // token in tile, 8-element chunk of the superblock
        const int row = mt * kGemmBM + t;
        uint4 out = make_uint4(0, 0, 0, 0);
        if (row < m) {
            const uint8_t *blk = act + ((int64_t)row * nb + b) * Q8K_BYTES;
            const uint32_t *qp = reinterpret_cast<const uint32_t *>(blk + 4 + c * 8);  // 4-byte aligned only
            const uint2 q = make_uint2(qp[0], qp[1]);
            auto cvt2 = [](uint32_t w, int sh) -> uint32_t {
                const __half2 h = __floats2half2_rn((float)(int)(int8_t)(w >> sh), (float)(int)(int8_t)(w >> (sh + 8)));
                return *reinterpret_cast<const uint32_t *>(&h);
            };
            out = make_uint4(cvt2(q.x, 0), cvt2(q.x, 16), cvt2(q.y, 0), cvt2(q.y, 16));
        }
        const int ks = c >> 3, e = (c & 7) * 8;
        *reinterpret_cast<uint4 *>(bimg + (int64_t)ks * kGemmAtomBytes + sw128_offset(t, e)) = out;
    }
    for (int i = threadIdx.x; i < 32 * 2; i += blockDim.x) {
        const int t = quarter * 32 + (i >> 1), c = i & 1;
        const int row = mt * kGemmBM + t;
        uint4 out = make_uint4(0, 0, 0, 0);
        if (row < m) {
            const uint8_t *blk = act + ((int64_t)row * nb + b) * Q8K_BYTES;
            const short *bs = reinterpret_cast<const short *>(blk + 4 + 256) + c * 8;
            uint32_t w[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const __half2 h = __floats2half2_rn((float)bs[2 * j], (float)bs[2 * j + 1]);
                w[j] = *reinterpret_cast<const uint32_t *>(&h);
            }
            out = make_uint4(w[0], w[1], w[2], w[3]);
        }
        *reinterpret_cast<uint4 *>(minb + min_tile_offset(t, c * 8)) = out;
    }
    for (int t = quarter * 32 + threadIdx.x; t < quarter * 32 + 32; t += blockDim.x) {
        const int row = mt * kGemmBM + t;
        dat[t] = row < m ? *reinterpret_cast<const float *>(act + ((int64_t)row * nb + b) * Q8K_BYTES) : 0.0f;
    }
}

// f32 activations -> the same operand images in one pass (the forward entries: no canonical blocks in between).  One
// warp per (activation row, superblock): BlockQ8K::from_float by the warp function every other kernel uses (so the
// codes, sums and scale are those of the canonical block), lane l holding elements 8l..8l+7, i.e. exactly one 16-byte
// chunk of the B image.
__global__ void __launch_bounds__(256) gemm_prep_f32_kernel(const float *__restrict__ x, int m, int k, uint8_t *__restrict__ scratch) {
    const int nb = k / 256;
    const int lane = threadIdx.x & 31;
    const int64_t item = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);  // (padded row, superblock)
    const int64_t prow = item / nb;
    const int b = (int)(item % nb);
    const int64_t mt = prow / kGemmBM;
    const int t = (int)(prow % kGemmBM);
    if (mt >= gemm_m_tiles(m)) return;  // whole warp
    const GemmActLayout lay = gemm_act_layout(m, k);
    uint8_t *bimg = scratch + lay.bimg + (mt * (k / 64) + (int64_t)b * 4) * kGemmAtomBytes;
    uint8_t *minb = scratch + lay.minb + (mt * nb + b) * kGemmMinBytes;
    float *dat = reinterpret_cast<float *>(scratch + lay.dat) + (mt * nb + b) * 128;
    uint32_t q_lo = 0, q_hi = 0;
    float d = 0.0f;
    int sum16 = 0;
    if (prow < m) {  // rows of the last tile past m stay zero
        float v[8];
        load8(x + prow * k + (int64_t)b * 256 + lane * 8, v);
        q8k_quantize_warp(v, lane, q_lo, q_hi, d, sum16);
    }
    auto cvt2 = [](uint32_t w, int sh) -> uint32_t {
        const __half2 h = __floats2half2_rn((float)(int)(int8_t)(w >> sh), (float)(int)(int8_t)(w >> (sh + 8)));
        return *reinterpret_cast<const uint32_t *>(&h);
    };
    const int ks = lane >> 3, e = (lane & 7) * 8;
    *reinterpret_cast<uint4 *>(bimg + (int64_t)ks * kGemmAtomBytes + sw128_offset(t, e)) =
        make_uint4(cvt2(q_lo, 0), cvt2(q_lo, 16), cvt2(q_hi, 0), cvt2(q_hi, 16));
    // the 16 bsums sit on lane pairs (group j on lanes 2j, 2j+1); lanes 0 and 1 collect eight each
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int j0 = 8 * (lane & 1) + 2 * i;
        const int s0 = __shfl_sync(0xffffffffu, sum16, 2 * j0), s1 = __shfl_sync(0xffffffffu, sum16, 2 * (j0 + 1));
        const __half2 h = __floats2half2_rn((float)s0, (float)s1);
        w[i] = *reinterpret_cast<const uint32_t *>(&h);
    }
    if (lane < 2) *reinterpret_cast<uint4 *>(minb + min_tile_offset(t, lane * 8)) = make_uint4(w[0], w[1], w[2], w[3]);
    if (lane == 0) dat[t] = d;
}

// Q4_K / Q5_K weight blocks -> the GEMM's A images.  One CTA per (n-tile, superblock), one thread per weight row:
// the 144-byte block becomes four 128-byte rows of f16 (sc_j * q, exact) in the four swizzle atoms of the
// superblock, plus the 32-byte min row (m_j duplicated against the two 16-element bsums of sub-block j).
// FIVE_BIT: Q5_K blocks (176 bytes: the same header, 32 bytes of fifth bits, then the nibbles; k_quants.rs:1778-2077):
// the code is nibble + 16 * bit, sc_j * q <= 63 * 31 = 1953 is still exact in f16, everything else is Q4_K's.
template <bool FIVE_BIT>
__global__ void __launch_bounds__(128) gemm_expand_kernel(const uint8_t *__restrict__ w, int n, int k,
                                                          uint8_t *__restrict__ scratch) {
    // [4 atoms x 16 KB][min tile 4 KB]: assembled in shared memory, written out by two bulk stores
    extern __shared__ __align__(1024) uint8_t ex_smem[];
    const int nb = k / 256;
    const int nt = blockIdx.x / nb, b = blockIdx.x % nb;
    const GemmWeightLayout lay = gemm_weight_layout(n, k);
    const int r = threadIdx.x, row = nt * kGemmBN + r;
    // blk[0]: header; blk[1..8]: the 128 nibble bytes; qh[0..1]: the 32 bytes of fifth bits (Q5_K)
    uint4 blk[9], qh[2];
#pragma unroll
    for (int i = 0; i < 9; ++i) blk[i] = make_uint4(0, 0, 0, 0);
    qh[0] = qh[1] = make_uint4(0, 0, 0, 0);
    if (row < n) {
        const uint4 *src = reinterpret_cast<const uint4 *>(w + ((int64_t)row * nb + b) * (FIVE_BIT ? Q5K_BYTES : Q4K_BYTES));
        blk[0] = __ldg(src);
        if (FIVE_BIT) {
            qh[0] = __ldg(src + 1);
            qh[1] = __ldg(src + 2);
        }
#pragma unroll
        for (int i = 1; i < 9; ++i) blk[i] = __ldg(src + i + (FIVE_BIT ? 2 : 0));
    }
    const uint4 hq = blk[0];
    // 6-bit scales / mins (utils.rs:50-60), four per word
    const uint32_t scw[2] = {hq.y & 0x3f3f3f3fu, (hq.w & 0x0f0f0f0fu) | (((hq.y >> 6) & 0x03030303u) << 4)};
    const uint32_t mnw[2] = {hq.z & 0x3f3f3f3fu, ((hq.w >> 4) & 0x0f0f0f0fu) | (((hq.z >> 6) & 0x03030303u) << 4)};
    uint8_t *img = ex_smem + (r >> 3) * 1024 + (r & 7) * 128;
    const int sw = r & 7;
#pragma unroll
    for (int g = 0; g < 4; ++g) {
        const uint4 q0 = blk[1 + 2 * g], q1 = blk[2 + 2 * g];
        const uint32_t sc_lo = (scw[g >> 1] >> (16 * (g & 1))) & 0xff, sc_hi = (scw[g >> 1] >> (16 * (g & 1) + 8)) & 0xff;
        // f16 value of sc*q without an int->float convert: (1024 + q) * sc - 1024 * sc, one exact FMA
        const __half2 s_lo = __half2half2(__ushort2half_rn((unsigned short)sc_lo));
        const __half2 s_hi = __half2half2(__ushort2half_rn((unsigned short)sc_hi));
        const __half2 c_lo = __hmul2(s_lo, __float2half2_rn(-1024.0f)), c_hi = __hmul2(s_hi, __float2half2_rn(-1024.0f));
        const uint32_t qw[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
        uint8_t *dst = img + g * kGemmAtomBytes;
#pragma unroll
        for (int c = 0; c < 8; ++c) {  // 16-byte chunk c of the row: k-elements 8c..8c+7 of the atom
            // chunks 0-3: low nibbles of bytes 8c..8c+7; chunks 4-7: high nibbles of bytes 8(c-4)..
            const uint32_t w0 = qw[2 * (c & 3)], w1 = qw[2 * (c & 3) + 1];
            uint32_t n0w = (c < 4) ? (w0 & 0x0f0f0f0fu) : ((w0 >> 4) & 0x0f0f0f0fu);
            uint32_t n1w = (c < 4) ? (w1 & 0x0f0f0f0fu) : ((w1 >> 4) & 0x0f0f0f0fu);
            if (FIVE_BIT) {  // element l of sub-block 2g + (c >= 4) takes bit 2g + (c >= 4) of fifth-bit byte l
                const uint32_t hw[8] = {qh[0].x, qh[0].y, qh[0].z, qh[0].w, qh[1].x, qh[1].y, qh[1].z, qh[1].w};
                const int bit = 2 * g + (c >> 2);
                n0w |= ((hw[2 * (c & 3)] >> bit) & 0x01010101u) << 4;
                n1w |= ((hw[2 * (c & 3) + 1] >> bit) & 0x01010101u) << 4;
            }
            const __half2 sc2 = (c < 4) ? s_lo : s_hi, cc2 = (c < 4) ? c_lo : c_hi;
            uint32_t h[4];
            h[0] = __byte_perm(n0w, 0x64646464u, 0x4140);
            h[1] = __byte_perm(n0w, 0x64646464u, 0x4342);
            h[2] = __byte_perm(n1w, 0x64646464u, 0x4140);
            h[3] = __byte_perm(n1w, 0x64646464u, 0x4342);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const __half2 v = __hfma2(*reinterpret_cast<const __half2 *>(&h[j]), sc2, cc2);
                h[j] = *reinterpret_cast<const uint32_t *>(&v);
            }
            *reinterpret_cast<uint4 *>(dst + ((c ^ sw) << 4)) = make_uint4(h[0], h[1], h[2], h[3]);
        }
    }
    uint8_t *md = ex_smem + 4 * kGemmAtomBytes;
#pragma unroll
    for (int c = 0; c < 2; ++c) {
        uint32_t h[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const unsigned short mv = (unsigned short)((mnw[c] >> (8 * j)) & 0xff);
            const __half2 v = __half2half2(__ushort2half_rn(mv));
            h[j] = *reinterpret_cast<const uint32_t *>(&v);
        }
        *reinterpret_cast<uint4 *>(md + min_tile_offset(r, c * 8)) = make_uint4(h[0], h[1], h[2], h[3]);
    }
    fence_proxy_async();  // generic-proxy stores -> visible to the bulk-copy engine
    __syncthreads();
    if (threadIdx.x == 0) {
        uint8_t *ga = scratch + lay.aimg + ((int64_t)nt * (k / 64) + (int64_t)b * 4) * kGemmAtomBytes;
        uint8_t *gm = scratch + lay.mina + ((int64_t)nt * nb + b) * kGemmMinBytes;
        asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(ga), "r"(smem_u32(ex_smem)),
                     "r"(4 * kGemmAtomBytes)
                     : "memory");
        asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gm), "r"(smem_u32(md)),
                     "r"(kGemmMinBytes)
                     : "memory");
        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");  // shared memory must outlive the copies
    }
}

// ---- tcgen05 wrappers ----
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes, uint32_t layout) {
    return (uint64_t)((smem_addr >> 4) & 0x3FFFu) | ((uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16) |
           ((uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32) | (1ull << 46) | ((uint64_t)layout << 61);
}
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t"
        "}\n" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u), "r"(0u), "r"(0u), "r"(0u)
        : "memory");
}
// The issue loop's form of the same: for a K-major, 128-byte-swizzled operand only the low word of the descriptor
// (address and leading offset) changes from step to step, by a compile-time amount; the high word (stride 1024 bytes,
// version, swizzle mode) is a constant.  Built this way an MMA costs its issuing thread a handful of instructions; with
// the descriptors rebuilt from addresses for every instruction the issuing thread, not the tensor pipe, set the pace
// (about 200 cycles per M = 128, N = 128, K = 16 instruction against 65 when issued back to back).
constexpr uint32_t kUmmaDescHiSw128 = (1024u >> 4) | (1u << 14) | (2u << 29);
__device__ __forceinline__ uint32_t umma_desc_lo(uint32_t smem_addr, uint32_t lbo_bytes) {
    return ((smem_addr >> 4) & 0x3FFFu) | (((lbo_bytes >> 4) & 0x3FFFu) << 16);
}
template <bool ACC>
__device__ __forceinline__ void umma_f16_lo(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t idesc) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        ".reg .b64 da, db;\n\t"
        "setp.ne.b32 p, %5, 0;\n\t"
        "mov.b64 da, {%1, %3};\n\t"
        "mov.b64 db, {%2, %3};\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, p;\n\t"
        "}\n" ::"r"(d_tmem),
        "r"(a_lo), "r"(b_lo), "r"(kUmmaDescHiSw128), "r"(idesc), "n"(ACC ? 1 : 0)
        : "memory");
}
__device__ __forceinline__ void umma_f16_lo_rt(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        ".reg .b64 da, db;\n\t"
        "setp.ne.b32 p, %5, 0;\n\t"
        "mov.b64 da, {%1, %3};\n\t"
        "mov.b64 db, {%2, %3};\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, p;\n\t"
        "}\n" ::"r"(d_tmem),
        "r"(a_lo), "r"(b_lo), "r"(kUmmaDescHiSw128), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
          "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
          "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];\n"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(taddr));
}
// 16 lanes x 32 columns of tensor memory as the MMA accumulator fragment: thread T = 4*g + c holds, for each block i of
// eight columns, v[4i], v[4i+1] = lane g, columns 8i + 2c, 8i + 2c + 1 and v[4i+2], v[4i+3] = lane g + 8, same columns.
__device__ __forceinline__ void tmem_ld_frag32(uint32_t taddr, uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.16x256b.x4.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];\n"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ uint64_t pack2f(float lo, float hi) {
    return (uint64_t)__float_as_uint(lo) | ((uint64_t)__float_as_uint(hi) << 32);
}
__device__ __forceinline__ uint64_t mul_f32x2(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ uint64_t fma_f32x2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}

// Abortable bounded wait: gives up when the CTA-wide abort flag is raised or the time budget runs out.
// kSleepNs > 0 makes the waiter back off between polls: every role except the MMA issuer waits this
// way, so that their polling does not crowd the shared-memory pipe the issuer's own barrier
// operations and commits go through.
template <int kSleepNs>
__device__ __forceinline__ bool mbar_wait_abortable(uint64_t *bar, uint32_t parity, volatile int *abort_flag) {
    if (mbar_try_wait(bar, parity)) return true;
    unsigned long long t0 = 0;
    for (uint32_t i = 0; i < kMaxSpins; ++i) {
        if (kSleepNs > 0) __nanosleep(kSleepNs);
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 63) == 63) {
            if (*abort_flag) return false;
            const unsigned long long now = global_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > wait_limit_ns()) break;
        }
    }
    *abort_flag = 1;
    atomicExch(&g_device_status, LLOOM_ERR_TIMEOUT);
    return false;
}

struct GemmParams {
    const uint8_t *w;        // Q4_K blocks [n][k/256], 16-byte aligned
    const uint8_t *act_img;  // planes written by gemm_prep_kernel
    const uint8_t *w_img;    // images written by gemm_expand_kernel
    float *y;
    int64_t ldy;
    int64_t row_bytes;
    int m, n, k;
    int n_tiles;  // tiles along the weight rows
    int m_tiles;  // tiles along the activation rows
    int blk_bytes;  // bytes of a weight block (144 for Q4_K, 176 for Q5_K): where the next superblock's d / dmin sit
};

// Pipeline barriers.  A stage (128 of K of both operands, 64 KB) has one "full" barrier, completed by the
// bulk copies' transaction bytes, and one "empty" barrier, completed by a single tcgen05.commit -- one
// commit and one wait per stage keep the issuing thread's serial overhead below the tensor time of the
// stage.  Per superblock parity (two of each): min_full (min tiles + activation scales landed), acc_full
// (commit after the superblock's last MMA: accumulators ready, min tiles free), acc_empty (the eight
// epilogue warps have read the accumulators out of tensor memory and hold the scales in registers).
__global__ void __launch_bounds__(kQ4kThreads, 1) gemm_q4k_kernel(const GemmParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + kOffBars);
    uint64_t *full = bars, *empty = bars + kGemmStages;
    uint64_t *min_full = bars + 2 * kGemmStages, *acc_full = min_full + 2, *acc_empty = min_full + 4;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem + kOffMisc);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + kOffMisc + 4);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // m-tiles of one n-tile are neighbours in launch order, so the n-tile's A images are shared through L2
    const int mt = blockIdx.x % p.m_tiles, nt = blockIdx.x / p.m_tiles;
    const int n0 = nt * kGemmBN, m0 = mt * kGemmBM;
    const int nb = p.k / 256;
    const GemmActLayout alay = gemm_act_layout(p.m, p.k);
    const GemmWeightLayout wlay = gemm_weight_layout(p.n, p.k);

    if (threadIdx.x == 0) {
        for (int s = 0; s < kGemmStages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&min_full[i], 2);  // the copies' bytes + the gathered row scales
            mbar_init(&acc_full[i], 1);
            mbar_init(&acc_empty[i], kQ4kEpiWarps);
        }
        *abort_flag = 0;
        fence_mbar_init();
    }
    if (warp == kQ4kEpiWarps + 1) {  // tensor memory: all 512 columns, two (S, Mn) accumulator pairs
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512u)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp < kQ4kEpiWarps) {
        // ------------------------------ epilogue ------------------------------
        // warp w: TMEM lanes 32*(w%4).. (hardware rule), accumulator columns 32*(w/4)..  The accumulators are read in
        // the MMA fragment layout: thread 4*fg + fc holds rows 32q + fg + 8j (j < 4) and columns 32*part + 8i + 2fc, + 1
        // (i < 4), so it needs 8 activation scales per superblock instead of the 32 a thread owning one tensor-memory
        // lane would fetch (the same words in all 32 lanes: a quarter of the shared-memory port, which the MMA operand
        // reads and the bulk copies already fill).
        const int q = warp & 3, part = warp >> 2;
        const int fg = lane >> 2, fc = lane & 3;
        bool row_ok[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) row_ok[j] = n0 + q * 32 + fg + 8 * j < p.n;
        uint64_t out2[4][4];  // [row j][column pair i]
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int i = 0; i < 4; ++i) out2[j][i] = 0ull;
        bool ok = true;
        for (int b = 0; b < nb && ok; ++b) {
            const int buf = b & 1;
            const uint32_t par = (b >> 1) & 1;
            ok = mbar_wait_abortable<64>(&min_full[buf], par, abort_flag);
            if (!ok) break;
            // the rows' (d_w, -dmin_w), gathered once per tile and superblock by the copy warp
            uint64_t dw2[4], ndmin2[4];
            {
                const float2 *hp = reinterpret_cast<const float2 *>(smem + kOffHdr + buf * kGemmHdrBytes) + q * 32 + fg;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float2 h = hp[8 * j];
                    dw2[j] = pack2f(h.x, h.x);
                    ndmin2[j] = pack2f(h.y, h.y);
                }
            }
            const uint64_t *dap = reinterpret_cast<const uint64_t *>(smem + kOffDa + buf * kGemmDaBytes + part * 128) + fc;
            uint64_t da2[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) da2[i] = dap[4 * i];
            ok = mbar_wait_abortable<64>(&acc_full[buf], par, abort_flag);
            if (!ok) break;
            tc_fence_after();
            const uint32_t t_main = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * 256 + part * 32);
            // two halves of 16 lanes: S and Mn of a half are loaded together, the next half's loads run under this half's FMAs
            uint32_t va[2][16], vb[2][16];
            tmem_ld_frag32(t_main, va[0]);
            tmem_ld_frag32(t_main + 128, vb[0]);
            tmem_ld_wait();
            tmem_ld_frag32(t_main + (16u << 16), va[1]);
            tmem_ld_frag32(t_main + (16u << 16) + 128, vb[1]);
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                if (h == 1) {
                    tmem_ld_wait();
                    // everything this warp needs from tensor memory is in registers now
                    tc_fence_before();
                }
#pragma unroll
                for (int i = 0; i < 4; ++i) {
#pragma unroll
                    for (int jj = 0; jj < 2; ++jj) {
                        const int j = 2 * h + jj;
                        const uint32_t *a = va[h] + 4 * i + 2 * jj, *m = vb[h] + 4 * i + 2 * jj;
                        uint64_t o = out2[j][i];
                        o = fma_f32x2(mul_f32x2(da2[i], dw2[j]), (uint64_t)a[0] | ((uint64_t)a[1] << 32), o);
                        out2[j][i] = fma_f32x2(mul_f32x2(da2[i], ndmin2[j]), (uint64_t)m[0] | ((uint64_t)m[1] << 32), o);
                    }
                }
            }
            // the scale tile is rewritten by a bulk copy (async proxy) after the arrivals, so this warp's reads of it
            // (generic proxy) are fenced first
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[buf]);
        }
        if (ok) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                if (!row_ok[j]) continue;
                const int n = n0 + q * 32 + fg + 8 * j;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int mrow = m0 + part * 32 + 8 * i + 2 * fc;
                    if (mrow < p.m) p.y[(int64_t)mrow * p.ldy + n] = __uint_as_float((uint32_t)(out2[j][i] & 0xffffffffu));
                    if (mrow + 1 < p.m) p.y[(int64_t)(mrow + 1) * p.ldy + n] = __uint_as_float((uint32_t)(out2[j][i] >> 32));
                }
            }
        }
    } else if (warp == kQ4kEpiWarps) {
        // ------------------------------ operand tiles: bulk copies ------------------------------
        // The whole warp walks the loop (lanes stay converged); lane 0 issues the copies.
        const uint8_t *aimg = p.w_img + wlay.aimg + (int64_t)nt * (p.k / 64) * kGemmAtomBytes;
        const uint8_t *mina = p.w_img + wlay.mina + (int64_t)nt * nb * kGemmMinBytes;
        const uint8_t *bimg = p.act_img + alay.bimg + (int64_t)mt * (p.k / 64) * kGemmAtomBytes;
        const uint8_t *minb = p.act_img + alay.minb + (int64_t)mt * nb * kGemmMinBytes;
        const uint8_t *dat = p.act_img + alay.dat + (int64_t)mt * nb * kGemmDaBytes;
        bool ok = true;
        for (int b = 0; b < nb && ok; ++b) {
            for (int h = 0; h < kGemmStagesPerSb && ok; ++h) {
                const int it = b * kGemmStagesPerSb + h, s = it % kGemmStages;
                if (it >= kGemmStages) ok = mbar_wait_abortable<32>(&empty[s], ((it / kGemmStages) - 1) & 1, abort_flag);
                if (!ok) break;
                if (lane == 0) {
                    mbar_arrive_expect_tx(&full[s], 2 * kGemmStageBytes);
                    bulk_g2s(smem + kOffA + s * kGemmStageBytes, aimg + (int64_t)it * kGemmStageBytes, kGemmStageBytes, &full[s]);
                    bulk_g2s(smem + kOffB + s * kGemmStageBytes, bimg + (int64_t)it * kGemmStageBytes, kGemmStageBytes, &full[s]);
                }
                __syncwarp();
            }
            if (!ok) break;
            const int buf = b & 1;
            if (b >= 2) {  // min tiles are free after the MMAs of b-2, the scales after the epilogue of b-2
                const uint32_t pp = ((b >> 1) - 1) & 1;
                ok = mbar_wait_abortable<32>(&acc_full[buf], pp, abort_flag) && mbar_wait_abortable<32>(&acc_empty[buf], pp, abort_flag);
            }
            if (!ok) break;
            if (lane == 0) {
                mbar_arrive_expect_tx(&min_full[buf], 2 * kGemmMinBytes + kGemmDaBytes);
                bulk_g2s(smem + kOffMinA + buf * kGemmMinBytes, mina + (int64_t)b * kGemmMinBytes, kGemmMinBytes, &min_full[buf]);
                bulk_g2s(smem + kOffMinB + buf * kGemmMinBytes, minb + (int64_t)b * kGemmMinBytes, kGemmMinBytes, &min_full[buf]);
                bulk_g2s(smem + kOffDa + buf * kGemmDaBytes, dat + (int64_t)b * kGemmDaBytes, kGemmDaBytes, &min_full[buf]);
            }
            __syncwarp();
        }
    } else if (warp == kQ4kEpiWarps + 2) {
        // ------------------------------ row scales ------------------------------
        // The block headers (f16 d | f16 dmin) of the tile's 128 weight rows, once per tile and superblock instead of once
        // per epilogue warp: lane l gathers rows l, l + 32, l + 64, l + 96; the next superblock's loads are in flight
        // while this one's values go to shared memory as (d_w, -dmin_w).
        const uint8_t *hrow[4];
        uint32_t hdr_next[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + lane + 32 * j;
            hrow[j] = n < p.n ? p.w + (int64_t)n * p.row_bytes : nullptr;
            hdr_next[j] = hrow[j] ? __ldg(reinterpret_cast<const uint32_t *>(hrow[j])) : 0u;
        }
        bool ok = true;
        for (int b = 0; b < nb && ok; ++b) {
            const int buf = b & 1;
            if (b >= 2) ok = mbar_wait_abortable<32>(&acc_empty[buf], ((b >> 1) - 1) & 1, abort_flag);  // the epilogue of b-2 has read its scales
            if (!ok) break;
            float2 *hp = reinterpret_cast<float2 *>(smem + kOffHdr + buf * kGemmHdrBytes);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint32_t hdr = hdr_next[j];
                if (b + 1 < nb && hrow[j]) hdr_next[j] = __ldg(reinterpret_cast<const uint32_t *>(hrow[j] + (int64_t)(b + 1) * p.blk_bytes));
                hp[lane + 32 * j] = make_float2(f16_bits_to_f32(hdr & 0xffffu), -f16_bits_to_f32(hdr >> 16));
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&min_full[buf]);
            __syncwarp();
        }
    } else if (warp == kQ4kEpiWarps + 1) {
        // ------------------------------ MMA issuer ------------------------------
        // The whole warp walks the loop; lane 0 issues the MMAs and commits.
        // instruction descriptor: D = f32, A = B = f16, both K-major, N = 128, M = 128
        const uint32_t idesc = (1u << 4) | ((uint32_t)(kGemmBM >> 3) << 17) | ((uint32_t)(kGemmBN >> 4) << 24);
        const uint32_t a_lo0 = umma_desc_lo(smem_u32(smem + kOffA), 16), b_lo0 = umma_desc_lo(smem_u32(smem + kOffB), 16);
        bool ok = true;
        for (int b = 0; b < nb && ok; ++b) {
            const int buf = b & 1;
            const uint32_t par = (b >> 1) & 1;
            if (b >= 2) ok = mbar_wait_abortable<0>(&acc_empty[buf], ((b >> 1) - 1) & 1, abort_flag);
            if (!ok) break;
            tc_fence_after();
            const uint32_t d_main = tmem_base + (uint32_t)(buf * 256), d_min = d_main + 128;
#pragma unroll
            for (int h = 0; h < kGemmStagesPerSb; ++h) {
                if (!ok) break;
                const int it = b * kGemmStagesPerSb + h, s = it % kGemmStages;
                ok = mbar_wait_abortable<0>(&full[s], (it / kGemmStages) & 1, abort_flag);
                if (!ok) break;
                tc_fence_after();
                if (lane == 0) {
                    const uint32_t a_lo = a_lo0 + (uint32_t)(s * (kGemmStageBytes >> 4));
                    const uint32_t b_lo = b_lo0 + (uint32_t)(s * (kGemmStageBytes >> 4));
#pragma unroll
                    for (int kk = 0; kk < 4 * kGemmStageAtoms; ++kk) {  // K = 16 per instruction: atom kk/4, 32 bytes along its swizzled row
                        constexpr int kAtom16 = kGemmAtomBytes >> 4;
                        const uint32_t off = (uint32_t)((kk >> 2) * kAtom16 + (kk & 3) * 2);
                        if (h == 0 && kk == 0) umma_f16_lo<false>(d_main, a_lo + off, b_lo + off, idesc);
                        else umma_f16_lo<true>(d_main, a_lo + off, b_lo + off, idesc);
                    }
                    umma_commit(&empty[s]);
                }
                __syncwarp();
            }
            if (!ok) break;
            ok = mbar_wait_abortable<0>(&min_full[buf], par, abort_flag);
            if (!ok) break;
            tc_fence_after();
            if (lane == 0) {
                const uint64_t mad = umma_desc(smem_u32(smem + kOffMinA + buf * kGemmMinBytes), 128, 256, 0);
                const uint64_t mbd = umma_desc(smem_u32(smem + kOffMinB + buf * kGemmMinBytes), 128, 256, 0);
                umma_f16(d_min, mad, mbd, idesc, 0u);
                umma_commit(&acc_full[buf]);
            }
            __syncwarp();
        }
    }
    // ------------------------------ teardown ------------------------------
    tc_fence_before();
    __syncthreads();
    if (warp == kQ4kEpiWarps + 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
    }
}

}  // namespace lloom
