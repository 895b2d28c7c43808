// Decode GEMV for 3 <= M <= 8 activation rows over Q4_K weights, on the integer tensor cores.
//
// With several activation rows the dp4a kernel (gemv.cuh) spends its time issuing dot-product
// instructions, not waiting for HBM.  Here one warp-level `mma.sync.m16n8k32.s8` multiplies a
// 16-row x 32-element weight sub-block (nibbles unpacked to int8 in registers) by the 32 x 8 block of
// activation codes (8 = the activation rows, zero-padded), giving exact int32 sums for 16 rows x 8
// rows of activations at once; the 6-bit sub-block scale is applied to the four accumulators of each
// MMA as an integer multiply, so the superblock sum S stays an exact integer, and the f32 scales are
// applied once per superblock in the reference's form (k_quants.rs:1540-1620, avx.rs:443-525).
//
// Same frame as the dp4a kernel: persistent CTA per SM over a contiguous row range, producer warp
// streaming 16-row tiles through the bulk-copy ring, activation planes in shared memory.  The eight
// consumer warps split the superblocks of a tile (warp w takes b = w, w+8, ...); their partial f32
// tiles meet in shared memory and are summed in a fixed order, so results are run-to-run identical.
#pragma once

#include "gemv.cuh"

namespace lloom {

constexpr int kMmaTileRows = 16;
constexpr int kMmaWarps = 8;
constexpr int kMmaRedBytes = 2 * kMmaWarps * 16 * 8 * 4;  // double-buffered partial tiles

__device__ __forceinline__ void mma_s8_16x8x32(int (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};\n"
        : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

// Dynamic shared memory: [barriers 128 B][partial tiles 8 KB][act planes][stage 0][stage 1]...
template <int M>
__global__ void __launch_bounds__(32 * (kMmaWarps + 1), 1) gemv_mma_q4k_kernel(const GemvParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t *full = reinterpret_cast<uint64_t *>(smem);
    uint64_t *empty = full + kMaxStages;
    float *red = reinterpret_cast<float *>(smem + 128);
    uint8_t *act_smem = smem + 128 + kMmaRedBytes;
    uint8_t *stage0 = act_smem + p.act_bytes;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r_begin = (int)(((int64_t)blockIdx.x * p.n) / gridDim.x);
    const int r_end = (int)(((int64_t)(blockIdx.x + 1) * p.n) / gridDim.x);

    if (threadIdx.x == 0) {
        for (int s = 0; s < p.stages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], kMmaWarps);
        }
        fence_mbar_init();
    }
    __syncthreads();
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    const int row_pitch = (int)p.row_bytes + 16;  // consecutive rows four banks apart: conflict-free fragment loads
    if (warp == kMmaWarps) {
        gemv_producer_rows(p, full, empty, stage0, kMmaTileRows, row_pitch, r_begin, r_end, lane);
        return;
    }

    ActPlanes planes;
    constexpr int nthreads = kMmaWarps * 32;
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (p.x) quantize_acts_to_planes(p, act_smem, warp, lane, planes);
    else stage_acts(p, act_smem, threadIdx.x, nthreads, planes);
    asm volatile("bar.sync 1, %0;" ::"r"(nthreads) : "memory");

    const int nb = p.k >> 8;
    const int gid = lane >> 2, tig = lane & 3;  // MMA fragment coordinates
    const bool tok_ok = gid < M;                // this lane's activation row (B-fragment column) exists
    // activation rows this lane's accumulators belong to (C-fragment columns 2*tig, 2*tig + 1)
    const int t0 = 2 * tig, t1 = 2 * tig + 1;
    int it = 0;
    bool alive = true;  // after a timed-out wait the warp keeps walking the tiles (the CTA barrier below needs it) but idles
    for (int trow = r_begin; trow < r_end; trow += kMmaTileRows, ++it) {
        const int s = it % p.stages;
        alive = alive && mbar_wait(&full[s], (it / p.stages) & 1);
        const uint8_t *tile_base = stage0 + (size_t)s * p.stage_bytes;
        const int rows = min(kMmaTileRows, r_end - trow);
        // rows of the A fragment held by this lane; rows past the end of the range read row 0 and are dropped later
        const int ra = gid < rows ? gid : 0, rb = gid + 8 < rows ? gid + 8 : 0;
        const uint8_t *rowa = tile_base + (size_t)ra * row_pitch, *rowb = tile_base + (size_t)rb * row_pitch;

        float out[4] = {0.f, 0.f, 0.f, 0.f};  // (row gid, t0), (gid, t1), (gid+8, t0), (gid+8, t1)
        for (int b = warp; alive && b < nb; b += kMmaWarps) {
            const uint4 ha = *reinterpret_cast<const uint4 *>(rowa + (size_t)b * Q4K_BYTES);
            const uint4 hb = *reinterpret_cast<const uint4 *>(rowb + (size_t)b * Q4K_BYTES);
            // 6-bit scales / mins (utils.rs:50-60), four per word, for the two rows
            const uint32_t sca[2] = {ha.y & 0x3f3f3f3fu, (ha.w & 0x0f0f0f0fu) | (((ha.y >> 6) & 0x03030303u) << 4)};
            const uint32_t scb[2] = {hb.y & 0x3f3f3f3fu, (hb.w & 0x0f0f0f0fu) | (((hb.y >> 6) & 0x03030303u) << 4)};
            const uint32_t mna[2] = {ha.z & 0x3f3f3f3fu, ((ha.w >> 4) & 0x0f0f0f0fu) | (((ha.z >> 6) & 0x03030303u) << 4)};
            const uint32_t mnb[2] = {hb.z & 0x3f3f3f3fu, ((hb.w >> 4) & 0x0f0f0f0fu) | (((hb.z >> 6) & 0x03030303u) << 4)};
            const uint32_t *qa = reinterpret_cast<const uint32_t *>(rowa + (size_t)b * Q4K_BYTES + 16);
            const uint32_t *qb = reinterpret_cast<const uint32_t *>(rowb + (size_t)b * Q4K_BYTES + 16);
            const uint32_t *act = reinterpret_cast<const uint32_t *>(
                planes.qs + (size_t)(tok_ok ? gid : 0) * ((size_t)nb * kQ8KUnitStride + p.act_row_pad) + (size_t)b * kQ8KUnitStride);
            int S[4] = {0, 0, 0, 0};
#pragma unroll
            for (int g = 0; g < 4; ++g) {
                // weight words of this lane: bytes 4*tig.. and 16+4*tig.. of the group's 32 bytes, rows gid / gid+8
                const uint32_t wa0 = qa[8 * g + tig], wa1 = qa[8 * g + tig + 4];
                const uint32_t wb0 = qb[8 * g + tig], wb1 = qb[8 * g + tig + 4];
                // activation words: sub-block 2g at element 64g, sub-block 2g+1 at 64g + 32
                uint32_t bl[2], bh[2];
                bl[0] = tok_ok ? act[16 * g + tig] : 0u;
                bl[1] = tok_ok ? act[16 * g + 4 + tig] : 0u;
                bh[0] = tok_ok ? act[16 * g + 8 + tig] : 0u;
                bh[1] = tok_ok ? act[16 * g + 12 + tig] : 0u;
                const uint32_t alo[4] = {wa0 & 0x0f0f0f0fu, wb0 & 0x0f0f0f0fu, wa1 & 0x0f0f0f0fu, wb1 & 0x0f0f0f0fu};
                const uint32_t ahi[4] = {(wa0 >> 4) & 0x0f0f0f0fu, (wb0 >> 4) & 0x0f0f0f0fu, (wa1 >> 4) & 0x0f0f0f0fu,
                                         (wb1 >> 4) & 0x0f0f0f0fu};
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
            const float dwa = f16_bits_to_f32(ha.x & 0xffffu), dma = f16_bits_to_f32(ha.x >> 16);
            const float dwb = f16_bits_to_f32(hb.x & 0xffffu), dmb = f16_bits_to_f32(hb.x >> 16);
#pragma unroll
            for (int tt = 0; tt < 2; ++tt) {
                const int t = tt == 0 ? t0 : t1;
                if (t < M) {
                    const uint4 sp = *reinterpret_cast<const uint4 *>(planes.sums + ((size_t)t * nb + b) * 8);
                    const float da = planes.d[t * nb + b];
                    int ma = __dp2a_lo((int)sp.x, (int)mna[0], 0);
                    ma = __dp2a_hi((int)sp.y, (int)mna[0], ma);
                    ma = __dp2a_lo((int)sp.z, (int)mna[1], ma);
                    ma = __dp2a_hi((int)sp.w, (int)mna[1], ma);
                    int mb = __dp2a_lo((int)sp.x, (int)mnb[0], 0);
                    mb = __dp2a_hi((int)sp.y, (int)mnb[0], mb);
                    mb = __dp2a_lo((int)sp.z, (int)mnb[1], mb);
                    mb = __dp2a_hi((int)sp.w, (int)mnb[1], mb);
                    out[tt] = fmaf(__fmul_rn(da, dwa), (float)S[tt], out[tt]);
                    out[tt] = fmaf(__fmul_rn(-da, dma), (float)ma, out[tt]);
                    out[2 + tt] = fmaf(__fmul_rn(da, dwb), (float)S[2 + tt], out[2 + tt]);
                    out[2 + tt] = fmaf(__fmul_rn(-da, dmb), (float)mb, out[2 + tt]);
                }
            }
        }
        // this warp is done reading the stage
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[s]);

        // partial tiles of the eight warps meet in shared memory and are summed in warp order
        float *mine = red + ((it & 1) * kMmaWarps + warp) * 128;
        mine[gid * 8 + t0] = out[0];
        mine[gid * 8 + t1] = out[1];
        mine[(gid + 8) * 8 + t0] = out[2];
        mine[(gid + 8) * 8 + t1] = out[3];
        asm volatile("bar.sync 1, %0;" ::"r"(nthreads) : "memory");
        if (threadIdx.x < 128) {
            const int r = threadIdx.x >> 3, t = threadIdx.x & 7;
            if (alive && r < rows && t < M) {
                const float *src = red + (it & 1) * kMmaWarps * 128 + r * 8 + t;
                float v = 0.0f;
#pragma unroll
                for (int w = 0; w < kMmaWarps; ++w) v += src[w * 128];
                p.y[(int64_t)t * p.ldy + trow + r] = v;
            }
        }
    }
}

}  // namespace lloom
