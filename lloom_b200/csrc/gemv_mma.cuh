// Decode GEMV for 2 <= M <= 8 activation rows over Q4_K weights, on the integer tensor cores.
//
// With several activation rows the dp4a kernel (gemv.cuh) spends its time issuing dot-product
// instructions, not waiting for HBM.  Here one warp-level `mma.sync.m16n8k32.s8` multiplies a
// 16-row x 32-element weight sub-block (nibbles unpacked to int8 in registers) by the 32 x 8 block of
// activation codes (8 = the activation rows; columns past M compute on row 0's codes and are never
// stored), giving exact int32 sums for 16 weight rows x 8 activation rows at once.  The 6-bit
// sub-block scale is applied to the four accumulators of each MMA as an integer multiply, so the
// superblock sum S stays an exact integer; the min term sum_j m_j * bsum_j is two more MMAs over the
// sub-block sums split as 64*h + l (both halves fit int8); the f32 scales are applied once per
// superblock in the reference's form (k_quants.rs:1540-1620, avx.rs:443-525).
//
// Frame: persistent CTA per SM over a contiguous row range; a producer warp streams 16-row tiles
// through a bulk-copy ring, one copy per row so that rows sit `row_pitch` bytes apart (8 banks mod 32:
// the 64-bit fragment loads of four rows are conflict-free).  The
// sixteen consumer warps work as four teams of four; tile i goes to team i mod 4, warp j of the team walks
// superblocks j, j+4, ... in order, and the team's first warp adds the four partial sums in warp order, so a
// row's f32 sum has one fixed order whatever the batch, the shard or the launch.  (Measured on [14336, 4096],
// 8 rows: teams of 2 / 4 / 8 / 16 warps give 11.9 / 11.1 / 11.2 / 12.5 us per forward.)  Every CTA quantizing
// all activation rows itself was measured too: from three rows on the blocks x ~200 instructions per CTA cost more
// than the separate quantizer kernel's launch gap, so those batches keep that kernel.  (Two rows, prologue
// quantizer: 10.2 us here against 12.2 us on the dp4a kernel; one row stays there, 8.6 us against 11.0 us.)
#pragma once

#include "gemv.cuh"

namespace lloom {

// Activation planes of the tensor-core kernel, per activation row t and superblock b:
//   codes  [t][b][64 words]  the 256 int8 codes, words permuted so that lane (gid, tig) finds the four words of
//                            group g it feeds to the MMAs -- low sub-block words 2tig, 2tig+1, high sub-block
//                            words 2tig, 2tig+1 -- in one 16-byte load at word 16g + 4tig; rows act_pitch apart
//   lh     [t][b][16 bytes]  l_j = bsum_j & 63 (j = 0..7, the 32-element sub-blocks), then h_j = bsum_j >> 6
//   d      [t][b] f32

__device__ __forceinline__ void mma_s8_16x8x32(int (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};\n"
        : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

// Where word c (0..63) of a block's codes goes inside the block's 64-word slot of the codes plane.
__host__ __device__ inline int mma_code_pos(int c) {
    const int g = c >> 4, r = c & 15;
    return 16 * g + 4 * ((r & 7) >> 1) + 2 * (r >> 3) + (r & 1);
}

// Canonical Q8_K blocks (292 B: f32 d, 256 codes, 16 i16 sums of 16) -> the three planes above.
__device__ __forceinline__ void stage_acts_mma(const GemvParams &p, uint8_t *act_smem, int tid, int nthreads) {
    const int nb = p.k >> 8;
    uint8_t *lh = act_smem + (size_t)p.m * p.act_pitch;
    float *dpl = reinterpret_cast<float *>(lh + (size_t)p.m * nb * 16);
    const uint32_t *src = reinterpret_cast<const uint32_t *>(p.act);
    const int total = p.m * nb * (Q8K_BYTES / 4);
    constexpr int kUnroll = 8;  // loads of a batch in flight together: the latency is paid once per batch
    for (int i0 = tid; i0 < total; i0 += nthreads * kUnroll) {
        uint32_t v[kUnroll];
#pragma unroll
        for (int j = 0; j < kUnroll; ++j) {
            const int i = i0 + j * nthreads;
            v[j] = i < total ? __ldg(src + i) : 0u;
        }
#pragma unroll
        for (int j = 0; j < kUnroll; ++j) {
            const int i = i0 + j * nthreads;
            if (i >= total) break;
            const int blk = i / (Q8K_BYTES / 4), w = i - blk * (Q8K_BYTES / 4);
            const int t = blk / nb, b = blk - t * nb;
            if (w == 0) {
                dpl[blk] = __uint_as_float(v[j]);
            } else if (w <= 64) {
                reinterpret_cast<uint32_t *>(act_smem + (size_t)t * p.act_pitch + (size_t)b * 256)[mma_code_pos(w - 1)] = v[j];
            } else {
                const int sb = w - 65;  // sub-block sb = i16 sums 2sb, 2sb+1
                const int s = (int)(short)(v[j] & 0xffffu) + (int)(short)(v[j] >> 16);
                lh[(size_t)blk * 16 + sb] = (uint8_t)(s & 63);
                lh[(size_t)blk * 16 + 8 + sb] = (uint8_t)((s >> 6) & 0xff);
            }
        }
    }
}

// One warp quantizes 256-element block (t, b) of the f32 activations into the three planes at `out` (global
// or shared memory).  Block arithmetic: q8k_quantize_warp, shared with the canonical quantizer.
__device__ __forceinline__ void q8k_values_to_planes(const float (&v)[8], uint8_t *out, int t, int b, int m, int nb,
                                                     int act_pitch, int lane) {
    const int blk = t * nb + b;
    uint32_t q_lo, q_hi;
    float d;
    int sum16;
    q8k_quantize_warp(v, lane, q_lo, q_hi, d, sum16);
    const int sum32 = sum16 + __shfl_xor_sync(0xffffffffu, sum16, 2);
    uint32_t *codes = reinterpret_cast<uint32_t *>(out + (size_t)t * act_pitch + (size_t)b * 256);
    *reinterpret_cast<uint2 *>(codes + mma_code_pos(2 * lane)) = make_uint2(q_lo, q_hi);  // words 2l, 2l+1 stay adjacent
    uint8_t *lh = out + (size_t)m * act_pitch + (size_t)blk * 16;
    if ((lane & 3) == 0) {
        lh[lane >> 2] = (uint8_t)(sum32 & 63);
        lh[8 + (lane >> 2)] = (uint8_t)((sum32 >> 6) & 0xff);
    }
    if (lane == 0) reinterpret_cast<float *>(out + (size_t)m * act_pitch + (size_t)m * nb * 16)[blk] = d;
}
__device__ __forceinline__ void q8k_block_to_planes(const float *__restrict__ x, uint8_t *out, int t, int b, int m, int nb,
                                                    int act_pitch, int lane) {
    float v[8];
    load8(x + (int64_t)(t * nb + b) * QK_K + lane * 8, v);
    q8k_values_to_planes(v, out, t, b, m, nb, act_pitch, lane);
}

// f32 activations -> the plane image in global memory (the same bytes stage_acts_mma leaves in shared
// memory), one warp per 256-element block; the GEMV then fetches the image with one bulk copy.
__global__ void __launch_bounds__(256) quantize_q8k_planes_kernel(const float *__restrict__ x, uint8_t *__restrict__ out,
                                                                  int m, int nb, int act_pitch) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");  // the GEMV may start streaming weights
    const int lane = threadIdx.x & 31;
    const int blk = (int)(((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5);
    if (blk >= m * nb) return;  // whole warp leaves together
    q8k_block_to_planes(x, out, blk / nb, blk % nb, m, nb, act_pitch, lane);
}

// Producer loop: work items in order (tile 0: chunks 0.., tile 1: ...).  An item is `chunk_sb` superblocks (fewer in a
// row's last chunk) of up to 16 consecutive rows: one bulk copy per row, rows `row_pitch` bytes apart in the stage.
// Every item completes a barrier of its own (item_full[it], used once): the consumers of a stage are different
// warps from one use to the next, and a phase parity cannot tell a late warp which use it is looking at.
__device__ __forceinline__ void gemv_mma_producer(const GemvParams &p, uint64_t *item_full, uint64_t *empty, uint8_t *stage0,
                                                  int r_begin, int r_end, int lane) {
    const int nb = p.k >> 8;
    const int ntiles = (r_end - r_begin + kMmaTileRows - 1) / kMmaTileRows;
    int it = 0;
    for (int tile = 0; tile < ntiles; ++tile) {
        const int row0 = r_begin + tile * kMmaTileRows;
        const int rows = min(kMmaTileRows, r_end - row0);
        for (int c = 0; c < p.nchunks; ++c, ++it) {
            const int s = it % p.stages;
            if (it >= p.stages) {
                if (!mbar_wait(&empty[s], ((it / p.stages) - 1) & 1)) return;
            }
            const int sb0 = c * p.chunk_sb;
            const uint32_t bytes = (uint32_t)(min(p.chunk_sb, nb - sb0) * Q4K_BYTES);
            uint8_t *dst = stage0 + (size_t)s * p.stage_bytes;
            if (lane == 0) mbar_arrive_expect_tx(&item_full[it], (uint32_t)rows * bytes);
            __syncwarp();
            for (int r = lane; r < rows; r += 32)
                bulk_g2s(dst + (size_t)r * p.row_pitch, p.w + (int64_t)(row0 + r) * p.row_bytes + (int64_t)sb0 * Q4K_BYTES, bytes,
                         &item_full[it]);
        }
    }
}


// Dynamic shared memory: [barriers 128 B][per-tile barriers][partial sums][act planes][staged output rows, fused
// gather only][stage 0][stage 1]...
template <int SPLIT, int EPI = 0>
__global__ void __launch_bounds__(32 * (kMmaWarps + 1), 1) gemv_mma_q4k_kernel(const GemvParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t *empty = reinterpret_cast<uint64_t *>(smem);
    uint64_t *act_bar = empty + kMaxStages;
    uint64_t *tile_full = reinterpret_cast<uint64_t *>(smem + kMmaBarBytes);
    float4 *red = reinterpret_cast<float4 *>(smem + kMmaBarBytes + p.tile_bar_bytes);
    uint8_t *act_smem = smem + kMmaBarBytes + p.tile_bar_bytes + kMmaRedBytes;
    float *out_s = reinterpret_cast<float *>(act_smem + p.act_bytes);  // staged output rows (fused gather only)
    uint8_t *stage0 = act_smem + p.act_bytes + p.out_bytes;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // whole 16-row tiles per CTA (a ragged split would leave most CTAs a last tile of a row or two that costs a
    // full tile's latency)
    const int total_tiles = (p.n + kMmaTileRows - 1) / kMmaTileRows;
    const int r_begin = (int)(((int64_t)blockIdx.x * total_tiles) / gridDim.x) * kMmaTileRows;
    const int r_end = min(p.n, (int)(((int64_t)(blockIdx.x + 1) * total_tiles) / gridDim.x) * kMmaTileRows);
    const GemvSeg sg = gemv_segment<false>(p, 0, r_begin, r_end);
    int *cta_ok = reinterpret_cast<int *>(smem + kMmaBarBytes - 8);  // cleared by a warp whose bounded wait ran out

    const int ntiles = (r_end - r_begin + kMmaTileRows - 1) / kMmaTileRows;
    for (int i = threadIdx.x; i < ntiles * p.nchunks; i += blockDim.x) mbar_init(&tile_full[i], 1);
    if (threadIdx.x < p.stages) mbar_init(&empty[threadIdx.x], SPLIT);
    if (threadIdx.x == 32) mbar_init(act_bar, 1);
    if (threadIdx.x == 0) *cta_ok = 1;
    fence_mbar_init();
    __syncthreads();
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    if (warp == kMmaWarps) {
        gemv_mma_producer(p, tile_full, empty, stage0, r_begin, r_end, lane);
        return;
    }

    constexpr int nthreads = kMmaWarps * 32;
    bool alive = true;  // after a timed-out wait the warp keeps meeting its partner at the pair barrier but computes nothing
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (EPI != 0 && p.wait_flags) alive = wait_exchange(p);  // x came out of a fused gather: all peers' rows are in
    if (p.x) {  // quantizer as prologue: this CTA quantizes the activation rows into its own planes
        // a warp's blocks are loaded four at a time before any is quantized: one L2 round trip per batch
        const int nbq = p.k >> 8, nblk = p.m * nbq;
        for (int base = warp; base < nblk; base += 4 * kMmaWarps) {
            float v[4][8];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int blk = base + j * kMmaWarps;
                if (blk < nblk) load8(p.x + (int64_t)blk * QK_K + lane * 8, v[j]);
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int blk = base + j * kMmaWarps;
                if (blk < nblk) q8k_values_to_planes(v[j], act_smem, blk / nbq, blk % nbq, p.m, nbq, p.act_pitch, lane);
            }
        }
        asm volatile("bar.sync 9, %0;" ::"r"(nthreads) : "memory");
    } else if (p.act_planes) {
        if (threadIdx.x == 0) {
            mbar_arrive_expect_tx(act_bar, (uint32_t)p.act_bytes);
            bulk_g2s(act_smem, p.act, (uint32_t)p.act_bytes, act_bar);
        }
        alive = mbar_wait(act_bar, 0) && alive;
    } else {
        stage_acts_mma(p, act_smem, threadIdx.x, nthreads);
        asm volatile("bar.sync 9, %0;" ::"r"(nthreads) : "memory");
    }

    const int nb = p.k >> 8;
    const int gid = lane >> 2, tig = lane & 3;  // MMA fragment coordinates
    // B fragments come from activation row gid (rows past m read row 0; their columns are never stored)
    const int tb = gid < p.m ? gid : 0;
    const uint8_t *codes = act_smem + (size_t)tb * p.act_pitch + 16 * tig;
    const uint8_t *lh_base = act_smem + (size_t)p.m * p.act_pitch;
    const uint32_t *lh_b = reinterpret_cast<const uint32_t *>(lh_base + (size_t)tb * nb * 16) + (tig & 1);
    const float *dpl = reinterpret_cast<const float *>(lh_base + (size_t)p.m * nb * 16);
    // the accumulators of this lane belong to activation rows 2*tig and 2*tig + 1
    const int t0 = 2 * tig, t1 = 2 * tig + 1;
    const float *d0 = dpl + (t0 < p.m ? t0 : 0) * nb, *d1 = dpl + (t1 < p.m ? t1 : 0) * nb;
    const bool min_lane = tig < 2;  // lanes that carry the eight mins / sub-block sums in the min-term MMAs

    constexpr int kTeams = kMmaWarps / SPLIT;
    const int team = warp / SPLIT, member = warp % SPLIT;
    int round = 0;
    for (int it = team; it < ntiles; it += kTeams, ++round) {
        const int trow = r_begin + it * kMmaTileRows;
        const int rows = min(kMmaTileRows, r_end - trow);
        // rows of the A fragment held by this lane; rows past the end of the range read row 0 and are dropped later
        const int ra = gid < rows ? gid : 0, rb = gid + 8 < rows ? gid + 8 : 0;
        float out[4] = {0.f, 0.f, 0.f, 0.f};  // (row gid, t0), (gid, t1), (gid+8, t0), (gid+8, t1)
        // the tile's chunks of superblocks, in order: a warp's partial sums run over all of them
        for (int c = 0; c < p.nchunks; ++c) {
        const int item = it * p.nchunks + c, s = item % p.stages;
        alive = alive && mbar_wait(&tile_full[item], 0);
        const uint8_t *tile_base = stage0 + (size_t)s * p.stage_bytes;
        const uint8_t *rowa = tile_base + (size_t)ra * p.row_pitch, *rowb = tile_base + (size_t)rb * p.row_pitch;
        const int sb0 = c * p.chunk_sb, nsb = min(p.chunk_sb, nb - sb0);
#pragma unroll 2
        for (int bl = member; alive && bl < nsb; bl += SPLIT) {
            const int b = sb0 + bl;  // superblock of the row; bl: its place in the stage
            const uint4 ha = *reinterpret_cast<const uint4 *>(rowa + (size_t)bl * Q4K_BYTES);
            const uint4 hb = *reinterpret_cast<const uint4 *>(rowb + (size_t)bl * Q4K_BYTES);
            // 6-bit scales / mins (utils.rs:50-60), four per word, for the two rows
            const uint32_t sca[2] = {ha.y & 0x3f3f3f3fu, (ha.w & 0x0f0f0f0fu) | (((ha.y >> 6) & 0x03030303u) << 4)};
            const uint32_t scb[2] = {hb.y & 0x3f3f3f3fu, (hb.w & 0x0f0f0f0fu) | (((hb.y >> 6) & 0x03030303u) << 4)};
            const uint32_t mna[2] = {ha.z & 0x3f3f3f3fu, ((ha.w >> 4) & 0x0f0f0f0fu) | (((ha.z >> 6) & 0x03030303u) << 4)};
            const uint32_t mnb[2] = {hb.z & 0x3f3f3f3fu, ((hb.w >> 4) & 0x0f0f0f0fu) | (((hb.z >> 6) & 0x03030303u) << 4)};
            const uint2 *qa = reinterpret_cast<const uint2 *>(rowa + (size_t)bl * Q4K_BYTES + 16) + tig;
            const uint2 *qb = reinterpret_cast<const uint2 *>(rowb + (size_t)bl * Q4K_BYTES + 16) + tig;
            const uint4 *act = reinterpret_cast<const uint4 *>(codes + (size_t)b * 256);
            int S[4] = {0, 0, 0, 0};
#pragma unroll
            for (int g = 0; g < 4; ++g) {
                // bytes 8*tig .. 8*tig+7 of the group's 32 nibble bytes, rows gid / gid+8; the same element
                // positions of the low (2g) and high (2g+1) sub-blocks of the activations
                const uint2 wa = qa[4 * g], wb = qb[4 * g];
                const uint4 av = act[4 * g];
                const uint32_t bl[2] = {av.x, av.y}, bh[2] = {av.z, av.w};
                const uint32_t alo[4] = {wa.x & 0x0f0f0f0fu, wb.x & 0x0f0f0f0fu, wa.y & 0x0f0f0f0fu, wb.y & 0x0f0f0f0fu};
                const uint32_t ahi[4] = {(wa.x >> 4) & 0x0f0f0f0fu, (wb.x >> 4) & 0x0f0f0f0fu, (wa.y >> 4) & 0x0f0f0f0fu,
                                         (wb.y >> 4) & 0x0f0f0f0fu};
                int cl[4] = {0, 0, 0, 0}, ch[4] = {0, 0, 0, 0};
                mma_s8_16x8x32(cl, alo, bl);
                mma_s8_16x8x32(ch, ahi, bh);
                const int sh = 16 * (g & 1);
                const int sa_lo = (sca[g >> 1] >> sh) & 0xff, sa_hi = (sca[g >> 1] >> (sh + 8)) & 0xff;
                const int sb_lo = (scb[g >> 1] >> sh) & 0xff, sb_hi = (scb[g >> 1] >> (sh + 8)) & 0xff;
                S[0] += sa_lo * cl[0] + sa_hi * ch[0];
                S[1] += sa_lo * cl[1] + sa_hi * ch[1];
                S[2] += sb_lo * cl[2] + sb_hi * ch[2];
                S[3] += sb_lo * cl[3] + sb_hi * ch[3];
            }
            // min term: k = 0..7 of one MMA carry the eight mins against the eight l (then h) halves of the sums
            const uint32_t am[4] = {min_lane ? (tig ? mna[1] : mna[0]) : 0u, min_lane ? (tig ? mnb[1] : mnb[0]) : 0u, 0u, 0u};
            const uint32_t lv = lh_b[b * 4], hv = lh_b[b * 4 + 2];
            const uint32_t bml[2] = {min_lane ? lv : 0u, 0u}, bmh[2] = {min_lane ? hv : 0u, 0u};
            int ml[4] = {0, 0, 0, 0}, mh[4] = {0, 0, 0, 0};
            mma_s8_16x8x32(ml, am, bml);
            mma_s8_16x8x32(mh, am, bmh);

            const float dwa = f16_bits_to_f32(ha.x & 0xffffu), dma = f16_bits_to_f32(ha.x >> 16);
            const float dwb = f16_bits_to_f32(hb.x & 0xffffu), dmb = f16_bits_to_f32(hb.x >> 16);
            const float da0 = d0[b], da1 = d1[b];
            out[0] = fmaf(__fmul_rn(da0, dwa), (float)S[0], out[0]);
            out[0] = fmaf(__fmul_rn(-da0, dma), (float)(ml[0] + 64 * mh[0]), out[0]);
            out[1] = fmaf(__fmul_rn(da1, dwa), (float)S[1], out[1]);
            out[1] = fmaf(__fmul_rn(-da1, dma), (float)(ml[1] + 64 * mh[1]), out[1]);
            out[2] = fmaf(__fmul_rn(da0, dwb), (float)S[2], out[2]);
            out[2] = fmaf(__fmul_rn(-da0, dmb), (float)(ml[2] + 64 * mh[2]), out[2]);
            out[3] = fmaf(__fmul_rn(da1, dwb), (float)S[3], out[3]);
            out[3] = fmaf(__fmul_rn(-da1, dmb), (float)(ml[3] + 64 * mh[3]), out[3]);
        }
        // this warp is done reading the stage once the sums its loads feed have been computed
#pragma unroll
        for (int i = 0; i < 4; ++i) pin_value(out[i]);
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[s]);
        }  // chunks

        // partial sums of the team meet in shared memory; its first warp adds them in member order
        float4 *slot = red + ((round & 1) * kMmaWarps + team * SPLIT) * 32 + lane;
        if (member != 0) slot[member * 32] = make_float4(out[0], out[1], out[2], out[3]);
        asm volatile("bar.sync %0, %1;" ::"r"(1 + team), "n"(SPLIT * 32) : "memory");
        if (member != 0 || !alive) continue;
#pragma unroll
        for (int j = 1; j < SPLIT; ++j) {
            const float4 o = slot[j * 32];
            out[0] += o.x;
            out[1] += o.y;
            out[2] += o.z;
            out[3] += o.w;
        }
        if (EPI == 0) {
            if (t0 < p.m) {
                if (gid < rows) p.y[(int64_t)t0 * p.ldy + trow + gid] = out[0];
                if (gid + 8 < rows) p.y[(int64_t)t0 * p.ldy + trow + gid + 8] = out[2];
            }
            if (t1 < p.m) {
                if (gid < rows) p.y[(int64_t)t1 * p.ldy + trow + gid] = out[1];
                if (gid + 8 < rows) p.y[(int64_t)t1 * p.ldy + trow + gid + 8] = out[3];
            }
        } else {
            if (t0 < p.m) {
                if (gid < rows) emit_out(p, sg, out_s, t0, trow + gid, out[0]);
                if (gid + 8 < rows) emit_out(p, sg, out_s, t0, trow + gid + 8, out[2]);
            }
            if (t1 < p.m) {
                if (gid < rows) emit_out(p, sg, out_s, t1, trow + gid, out[1]);
                if (gid + 8 < rows) emit_out(p, sg, out_s, t1, trow + gid + 8, out[3]);
            }
        }
    }
    if (EPI != 0 && (p.out_bytes || p.publish)) {  // every consumer warp gets here, timed-out ones included
        if (!alive) *cta_ok = 0;
        asm volatile("bar.sync 9, %0;" ::"r"(nthreads) : "memory");
        // staged rows leave for the peers only if every warp finished its tiles (a timed-out warp left gaps)
        if (p.out_bytes && *cta_ok) flush_out(p, out_s, r_begin, r_end, threadIdx.x, nthreads);
        if (p.publish) {
            asm volatile("bar.sync 9, %0;" ::"r"(nthreads) : "memory");
            if (threadIdx.x == 0) publish_arrival(p);
        }
    }
}

}  // namespace lloom
