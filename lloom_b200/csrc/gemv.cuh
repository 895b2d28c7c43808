// Decode GEMV (1 <= M <= 8) over canonical GGUF block rows, HBM-bound by design.
//
// One persistent CTA per SM.  A producer warp streams tiles of consecutive weight rows (one
// contiguous byte range of the canonical [n][k/block] stream) into a ring of shared-memory stages
// with the bulk-async copy engine; consumer warps unpack nibbles / 6-bit codes in registers, take
// exact integer dot products with dp4a against the quantized activations (held once per CTA in
// shared memory as aligned planes), apply the block scales in f32 in the reference's algebraic form
// and reduce with warp shuffles.  Per-row arithmetic never depends on the row's position in a tile
// or on n, so any row shard of a matrix gives bit-identical rows.
#pragma once

#include "common.cuh"

namespace lloom {

// Activation planes in shared memory (built by stage_acts from the canonical blocks):
//   qs    int8  [M][K]            16-byte aligned rows
//   d     f32   [M][K/32] (Q8_0 acts, f16 scale widened) or [M][K/256] (Q8_K acts)
//   bsums int16 [M][K/16]         (Q8_K acts only)
struct ActPlanes {
    const int8_t *qs;
    const float *d;
    const short *bsums;
    int k;
};

__host__ __device__ inline int64_t act_plane_bytes(int w_dtype, int64_t m, int64_t k) {
    int64_t qs = m * k;
    int64_t d = (w_dtype == LLOOM_Q8_0) ? m * (k / 32) * 4 : m * (k / 256) * 4;
    int64_t bs = (w_dtype == LLOOM_Q8_0) ? 0 : m * (k / 16) * 2;
    return ((qs + 15) / 16) * 16 + ((d + 15) / 16) * 16 + ((bs + 15) / 16) * 16;
}

// Read NWORDS 32-bit words starting at a 2-byte aligned shared-memory address.
template <int NWORDS>
__device__ __forceinline__ void lds_words_unaligned(const uint8_t *p, uint32_t (&out)[NWORDS]) {
    const uint32_t addr = smem_u32(p);
    const uint32_t sh = (addr & 3u) * 8u;
    const uint32_t *wp = reinterpret_cast<const uint32_t *>(p - (addr & 3u));
    uint32_t prev = wp[0];
#pragma unroll
    for (int i = 0; i < NWORDS; ++i) {
        uint32_t next = wp[i + 1];
        out[i] = __funnelshift_r(prev, next, sh);
        prev = next;
    }
}

// ---------------------------------------------------------------------------------------------
// Per-format work items.  An item is 64 consecutive-in-layout elements of one weight row; a lane
// loads the matching activation bytes once and reuses them for every row it handles.
// ---------------------------------------------------------------------------------------------

// Q4_K x Q8_K (k_quants.rs:1540-1620, avx.rs:443-525):
//   out += (d_a*d_w) * sum_j sc_j * dot32(q4_j, q8_j)  +  (-d_a*dmin_w) * sum_j m_j * (bsums[2j]+bsums[2j+1])
// item = (superblock b, 64-group g): sub-blocks 2g (low nibbles) and 2g+1 (high nibbles).
template <int M>
struct ItemQ4K {
    static constexpr int kItemsPerBlock = 4;
    static constexpr int kBlockBytes = Q4K_BYTES;
    struct Act {
        uint4 lo[M][2], hi[M][2];
        int s0[M], s1[M];
        float d[M];
    };
    __device__ static __forceinline__ void load_act(Act &a, const ActPlanes &p, int item) {
        const int b = item >> 2, g = item & 3;
#pragma unroll
        for (int m = 0; m < M; ++m) {
            const uint4 *q = reinterpret_cast<const uint4 *>(p.qs + (size_t)m * p.k + b * 256 + g * 64);
            a.lo[m][0] = q[0]; a.lo[m][1] = q[1];
            a.hi[m][0] = q[2]; a.hi[m][1] = q[3];
            const short *bs = p.bsums + (size_t)m * (p.k >> 4) + b * 16 + g * 4;
            a.s0[m] = (int)bs[0] + (int)bs[1];
            a.s1[m] = (int)bs[2] + (int)bs[3];
            a.d[m] = p.d[m * (p.k >> 8) + b];
        }
    }
    __device__ static __forceinline__ void row(const uint8_t *rowp, int item, const Act &a, float (&acc)[M]) {
        const int b = item >> 2, g = item & 3;
        const uint8_t *blk = rowp + b * Q4K_BYTES;
        const uint32_t dd = *reinterpret_cast<const uint32_t *>(blk);
        const float dw = f16_bits_to_f32(dd & 0xffffu), dminw = f16_bits_to_f32(dd >> 16);
        // 6-bit (scale, min) pairs of sub-blocks 2g and 2g+1 (utils.rs:50-60), as byte pairs
        const unsigned short *s16 = reinterpret_cast<const unsigned short *>(blk + 4);
        const uint32_t X = s16[g + 2];      // scale bytes 2g+4, 2g+5
        const uint32_t Y = s16[g & 1];      // scale bytes 2g (g<2) or 2g-4 (g>=2)
        const uint32_t Z = s16[g];          // scale bytes 2g, 2g+1
        uint32_t scp, mnp;
        if (g < 2) {
            scp = Y & 0x3f3fu;
            mnp = X & 0x3f3fu;
        } else {
            scp = (X & 0x0f0fu) | (((Y >> 6) & 0x0303u) << 4);
            mnp = ((X >> 4) & 0x0f0fu) | (((Z >> 6) & 0x0303u) << 4);
        }
        const int sc0 = scp & 0xff, sc1 = scp >> 8, mn0 = mnp & 0xff, mn1 = mnp >> 8;
        const uint4 *qp = reinterpret_cast<const uint4 *>(blk + 16 + g * 32);
        const uint4 q0 = qp[0], q1 = qp[1];
        const uint32_t qw[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
        uint32_t ql[8], qh[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            ql[i] = qw[i] & 0x0f0f0f0fu;
            qh[i] = (qw[i] >> 4) & 0x0f0f0f0fu;
        }
#pragma unroll
        for (int m = 0; m < M; ++m) {
            const uint32_t al[8] = {a.lo[m][0].x, a.lo[m][0].y, a.lo[m][0].z, a.lo[m][0].w,
                                    a.lo[m][1].x, a.lo[m][1].y, a.lo[m][1].z, a.lo[m][1].w};
            const uint32_t ah[8] = {a.hi[m][0].x, a.hi[m][0].y, a.hi[m][0].z, a.hi[m][0].w,
                                    a.hi[m][1].x, a.hi[m][1].y, a.hi[m][1].z, a.hi[m][1].w};
            int pl = 0, ph = 0;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                pl = __dp4a((int)ql[i], (int)al[i], pl);
                ph = __dp4a((int)qh[i], (int)ah[i], ph);
            }
            const int v = sc0 * pl + sc1 * ph;
            const int mv = mn0 * a.s0[m] + mn1 * a.s1[m];
            acc[m] = fmaf(__fmul_rn(a.d[m], dw), (float)v, acc[m]);
            acc[m] = fmaf(__fmul_rn(-a.d[m], dminw), (float)mv, acc[m]);
        }
    }
};

// Q6_K x Q8_K (k_quants.rs:2115-2172, avx.rs:131-216):
//   out += (d_a*d_w) * sum_{j<16} sc_j * dot16(q6_j - 32, q8_j)
// item = (superblock b, half h, 16 l-values at l0): the four 16-element groups l0 + {0,32,64,96}
// of the half, each with one scale.  (q6-32).q8 is taken as q6u.q8 - 32*bsum like the AVX2 arm.
template <int M>
struct ItemQ6K {
    static constexpr int kItemsPerBlock = 4;
    static constexpr int kBlockBytes = Q6K_BYTES;
    struct Act {
        uint4 q[M][4];
        int bs[M][4];
        float d[M];
    };
    __device__ static __forceinline__ void load_act(Act &a, const ActPlanes &p, int item) {
        const int b = item >> 2, h = (item >> 1) & 1, l0 = (item & 1) * 16;
#pragma unroll
        for (int m = 0; m < M; ++m) {
            const int8_t *base = p.qs + (size_t)m * p.k + b * 256 + h * 128 + l0;
            const short *bs = p.bsums + (size_t)m * (p.k >> 4) + b * 16 + h * 8 + (l0 >> 4);
#pragma unroll
            for (int gq = 0; gq < 4; ++gq) {
                a.q[m][gq] = *reinterpret_cast<const uint4 *>(base + 32 * gq);
                a.bs[m][gq] = (int)bs[2 * gq];
            }
            a.d[m] = p.d[m * (p.k >> 8) + b];
        }
    }
    __device__ static __forceinline__ void row(const uint8_t *rowp, int item, const Act &a, float (&acc)[M]) {
        const int b = item >> 2, h = (item >> 1) & 1, l0 = (item & 1) * 16;
        const uint8_t *blk = rowp + (size_t)b * Q6K_BYTES;  // 2-byte aligned
        uint32_t la[4], lb[4], hh[4];
        lds_words_unaligned<4>(blk + 64 * h + l0, la);
        lds_words_unaligned<4>(blk + 64 * h + 32 + l0, lb);
        lds_words_unaligned<4>(blk + 128 + 32 * h + l0, hh);
        const int8_t *scp = reinterpret_cast<const int8_t *>(blk + 192 + 8 * h + (l0 >> 4));
        const int sc[4] = {scp[0], scp[2], scp[4], scp[6]};
        const float dw = f16_bits_to_f32(*reinterpret_cast<const unsigned short *>(blk + 208));
        uint32_t c[4][4];
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            c[0][w] = (la[w] & 0x0f0f0f0fu) | ((hh[w] << 4) & 0x30303030u);
            c[1][w] = (lb[w] & 0x0f0f0f0fu) | ((hh[w] << 2) & 0x30303030u);
            c[2][w] = ((la[w] >> 4) & 0x0f0f0f0fu) | (hh[w] & 0x30303030u);
            c[3][w] = ((lb[w] >> 4) & 0x0f0f0f0fu) | ((hh[w] >> 2) & 0x30303030u);
        }
#pragma unroll
        for (int m = 0; m < M; ++m) {
            int v = 0;
#pragma unroll
            for (int gq = 0; gq < 4; ++gq) {
                const uint4 aq = a.q[m][gq];
                int p = __dp4a((int)c[gq][0], (int)aq.x, 0);
                p = __dp4a((int)c[gq][1], (int)aq.y, p);
                p = __dp4a((int)c[gq][2], (int)aq.z, p);
                p = __dp4a((int)c[gq][3], (int)aq.w, p);
                v += sc[gq] * (p - 32 * a.bs[m][gq]);
            }
            acc[m] = fmaf(__fmul_rn(a.d[m], dw), (float)v, acc[m]);
        }
    }
};

// Q8_0 x Q8_0 (k_quants.rs:800-818, avx.rs:71-87):  out += (d_w*d_a) * dot32(q_w, q_a) per block.
// item = two consecutive 34-byte blocks.
template <int M>
struct ItemQ8_0 {
    static constexpr int kItemsPerBlock = 0;  // items are pairs of blocks: items per row = k / 64
    static constexpr int kBlockBytes = Q8_0_BYTES;
    struct Act {
        uint4 q[M][4];
        float d[M][2];
    };
    __device__ static __forceinline__ void load_act(Act &a, const ActPlanes &p, int item) {
#pragma unroll
        for (int m = 0; m < M; ++m) {
            const uint4 *q = reinterpret_cast<const uint4 *>(p.qs + (size_t)m * p.k + item * 64);
#pragma unroll
            for (int i = 0; i < 4; ++i) a.q[m][i] = q[i];
            a.d[m][0] = p.d[m * (p.k >> 5) + item * 2];
            a.d[m][1] = p.d[m * (p.k >> 5) + item * 2 + 1];
        }
    }
    __device__ static __forceinline__ void row(const uint8_t *rowp, int item, const Act &a, float (&acc)[M]) {
        const uint8_t *blk = rowp + (size_t)item * (2 * Q8_0_BYTES);  // 2-byte aligned
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const uint8_t *bp = blk + half * Q8_0_BYTES;
            const float dw = f16_bits_to_f32(*reinterpret_cast<const unsigned short *>(bp));
            uint32_t q[8];
            lds_words_unaligned<8>(bp + 2, q);
#pragma unroll
            for (int m = 0; m < M; ++m) {
                const uint4 a0 = a.q[m][2 * half], a1 = a.q[m][2 * half + 1];
                int p = __dp4a((int)q[0], (int)a0.x, 0);
                p = __dp4a((int)q[1], (int)a0.y, p);
                p = __dp4a((int)q[2], (int)a0.z, p);
                p = __dp4a((int)q[3], (int)a0.w, p);
                p = __dp4a((int)q[4], (int)a1.x, p);
                p = __dp4a((int)q[5], (int)a1.y, p);
                p = __dp4a((int)q[6], (int)a1.z, p);
                p = __dp4a((int)q[7], (int)a1.w, p);
                acc[m] = fmaf(__fmul_rn(dw, a.d[m][half]), (float)p, acc[m]);
            }
        }
    }
};

struct GemvParams {
    const uint8_t *w;    // canonical blocks, 16-byte aligned
    const uint8_t *act;  // canonical activation blocks [m][k/block]
    float *y;
    int64_t ldy;
    int64_t row_bytes;
    int64_t w_bytes;  // n * row_bytes
    int n, k, m;
    int w_dtype;
    int n_cwarps;      // consumer warps; blockDim.x = 32 * (n_cwarps + 1)
    int stages;
    int stage_bytes;   // multiple of 128
    int act_bytes;     // multiple of 16
};

constexpr int kMaxStages = 8;

// Dynamic shared memory: [barriers 128 B][act planes][stage 0][stage 1]...
template <class Item, int M, int RW>
__global__ void __launch_bounds__(288, 1) gemv_kernel(const GemvParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t *full = reinterpret_cast<uint64_t *>(smem);
    uint64_t *empty = full + kMaxStages;
    uint8_t *act_smem = smem + 128;
    uint8_t *stage0 = act_smem + p.act_bytes;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile_rows = p.n_cwarps * RW;
    // equal contiguous row ranges per CTA: HBM bytes per SM differ by at most one row
    const int r_begin = (int)(((int64_t)blockIdx.x * p.n) / gridDim.x);
    const int r_end = (int)(((int64_t)(blockIdx.x + 1) * p.n) / gridDim.x);

    if (threadIdx.x == 0) {
        for (int s = 0; s < p.stages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], p.n_cwarps);
        }
        fence_mbar_init();
    }
    __syncthreads();

    if (warp == p.n_cwarps) {
        // ---------------- producer warp ----------------
        int it = 0;
        for (int row0 = r_begin; row0 < r_end; row0 += tile_rows, ++it) {
            const int s = it % p.stages;
            if (it >= p.stages) {
                if (!mbar_wait(&empty[s], ((it / p.stages) - 1) & 1)) return;
            }
            const int rows = min(tile_rows, r_end - row0);
            const int64_t start = (int64_t)row0 * p.row_bytes;
            const int64_t end = start + (int64_t)rows * p.row_bytes;
            const int64_t a_start = start & ~(int64_t)15;
            int64_t a_end = (end + 15) & ~(int64_t)15;
            const int64_t bulk_limit = p.w_bytes & ~(int64_t)15;  // bytes the bulk engine may touch
            if (a_end > bulk_limit) a_end = bulk_limit;
            uint8_t *dst = stage0 + (size_t)s * p.stage_bytes;
            // ragged end of the weight stream (< 16 bytes): plain loads
            if (end > a_end) {
                const int64_t from = a_end > a_start ? a_end : a_start;
                for (int64_t i = from + lane; i < end; i += 32) dst[i - a_start] = __ldg(p.w + i);
            }
            __syncwarp();
            if (lane == 0) {
                if (a_end > a_start) {
                    const uint32_t bytes = (uint32_t)(a_end - a_start);
                    mbar_arrive_expect_tx(&full[s], bytes);
                    bulk_g2s(dst, p.w + a_start, bytes, &full[s]);
                } else {
                    mbar_arrive(&full[s]);
                }
            }
        }
        return;
    }

    // ---------------- consumer warps ----------------
    ActPlanes planes;
    // all consumer warps stage the activations together (named barrier over consumers only)
    {
        const int nthreads = p.n_cwarps * 32;
        // canonical activation blocks (global) -> aligned planes (shared), once per CTA
        const size_t qs_bytes = (((size_t)p.m * p.k + 15) / 16) * 16;
        float *dpl = reinterpret_cast<float *>(act_smem + qs_bytes);
        if (p.w_dtype == LLOOM_Q8_0) {
            const int nb = p.k / 32;
            const unsigned short *src = reinterpret_cast<const unsigned short *>(p.act);
            unsigned short *q16 = reinterpret_cast<unsigned short *>(act_smem);
            const int total = p.m * nb * 17;
            for (int i = threadIdx.x; i < total; i += nthreads) {
                const int blk = i / 17, hw = i - blk * 17;
                const unsigned short v = __ldg(src + i);
                if (hw == 0) dpl[blk] = __half2float(__ushort_as_half(v));
                else q16[blk * 16 + hw - 1] = v;
            }
            planes.bsums = nullptr;
        } else {
            const int nb = p.k / 256;
            const size_t d_bytes = (((size_t)p.m * nb * 4 + 15) / 16) * 16;
            uint32_t *bs32 = reinterpret_cast<uint32_t *>(act_smem + qs_bytes + d_bytes);
            const uint32_t *src = reinterpret_cast<const uint32_t *>(p.act);
            uint32_t *q32 = reinterpret_cast<uint32_t *>(act_smem);
            const int total = p.m * nb * 73;
            for (int i = threadIdx.x; i < total; i += nthreads) {
                const int blk = i / 73, w = i - blk * 73;
                const uint32_t v = __ldg(src + i);
                if (w == 0) dpl[blk] = __uint_as_float(v);
                else if (w <= 64) q32[blk * 64 + w - 1] = v;
                else bs32[blk * 8 + w - 65] = v;
            }
            planes.bsums = reinterpret_cast<const short *>(bs32);
        }
        planes.qs = reinterpret_cast<const int8_t *>(act_smem);
        planes.d = dpl;
        planes.k = p.k;
        asm volatile("bar.sync 1, %0;" ::"r"(nthreads) : "memory");
    }

    const int items_per_row = p.k >> 6;
    int it = 0;
    for (int trow = r_begin; trow < r_end; trow += tile_rows, ++it) {
        const int s = it % p.stages;
        if (!mbar_wait(&full[s], (it / p.stages) & 1)) return;
        const int64_t start = (int64_t)trow * p.row_bytes;
        const uint8_t *tile_base = stage0 + (size_t)s * p.stage_bytes + (start & 15);
        const int row0 = trow + warp * RW;

        float acc[RW][M];
#pragma unroll
        for (int r = 0; r < RW; ++r)
#pragma unroll
            for (int m = 0; m < M; ++m) acc[r][m] = 0.0f;

        if (row0 < r_end) {
            for (int item = lane; item < items_per_row; item += 32) {
                typename Item::Act a;
                Item::load_act(a, planes, item);
#pragma unroll
                for (int r = 0; r < RW; ++r) {
                    if (row0 + r < r_end) {
                        const uint8_t *rowp = tile_base + (size_t)(warp * RW + r) * p.row_bytes;
                        Item::row(rowp, item, a, acc[r]);
                    }
                }
            }
        }
        // this warp is done reading the stage
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[s]);

        if (row0 < r_end) {
#pragma unroll
            for (int r = 0; r < RW; ++r)
#pragma unroll
                for (int m = 0; m < M; ++m) {
                    float v = acc[r][m];
#pragma unroll
                    for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
                    acc[r][m] = v;
                }
            // lane (r*M + m) writes its value
#pragma unroll
            for (int r = 0; r < RW; ++r)
#pragma unroll
                for (int m = 0; m < M; ++m)
                    if (lane == r * M + m && row0 + r < r_end) p.y[(int64_t)m * p.ldy + row0 + r] = acc[r][m];
        }
    }
}

}  // namespace lloom
