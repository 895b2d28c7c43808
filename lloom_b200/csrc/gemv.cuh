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

#include "common.cuh"
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

constexpr int kQ8KUnitStride = 256 + 16;
constexpr int kQ8_0UnitStride = 64 + 16;

__host__ __device__ inline int64_t round16(int64_t v) { return (v + 15) / 16 * 16; }

__host__ __device__ inline int64_t act_qs_bytes(int w_dtype, int64_t m, int64_t k) {
    return (w_dtype == LLOOM_Q8_0) ? m * (k / 64) * kQ8_0UnitStride : m * (k / 256) * kQ8KUnitStride;
}

__host__ __device__ inline int64_t act_plane_bytes(int w_dtype, int64_t m, int64_t k) {
    const int64_t qs = act_qs_bytes(w_dtype, m, k);
    const int64_t d = (w_dtype == LLOOM_Q8_0) ? m * (k / 32) * 4 : m * (k / 256) * 4;
    const int64_t sums = (w_dtype == LLOOM_Q8_0) ? 0 : (w_dtype == LLOOM_Q4_K ? m * (k / 32) * 2 : m * (k / 16) * 2);
    return round16(qs) + round16(d) + round16(sums);
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

constexpr int kMaxPeers = 8;  // GPUs of one node

struct GemvParams {
    const uint8_t *w;    // canonical blocks, 16-byte aligned
    const uint8_t *act;  // canonical activation blocks [m][k/block] (used when x == nullptr)
    const float *x;      // f32 activations [m][k], 16-byte aligned: quantized in the prologue (fused forward)
    float *y;
    int64_t ldy;
    int64_t row_bytes;
    int64_t w_bytes;  // n * row_bytes
    int n, k, m;
    int w_dtype;
    int n_cwarps;      // consumer warps; blockDim.x = 32 * (n_cwarps + 1)
    int lpr_log2;      // lanes per row = 1 << lpr_log2 (a warp handles 32 / lanes-per-row row groups)
    int stages;
    int stage_bytes;   // multiple of 128
    int act_bytes;     // multiple of 16
    int row_pitch;     // tensor-core kernel only: bytes between weight rows inside a stage
    int act_pitch;     // tensor-core kernel only: bytes between activation rows of the code plane
    int act_planes;    // tensor-core kernel only: `act` already holds the plane image (else canonical blocks)
    int tile_bar_bytes;  // tensor-core kernel only: bytes of the per-item barrier array (multiple of 16)
    int chunk_sb;        // tensor-core kernel only: superblocks of a row per stage (all of them unless K is large)
    int nchunks;         // both kernels: pieces a row is cut into, each a stage's worth (1: whole rows)
    int chunk_units;     // dp4a kernel, nchunks > 1: units (superblocks / pairs of Q8_0 blocks) of a row per piece
    int unit_bytes;      // dp4a kernel: bytes of a unit (144 / 210 / 68)
    // Fused gather: when n_peers > 0 every output value goes to the same place in each of these buffers (this GPU's
    // own and its peers', mapped into this process) instead of `y`, so the row-sharded forward needs no separate
    // all-gather: the stores cross NVLink while the rest of the rows are still being computed.
    int n_peers;
    // Fused gather with staging: bytes of the shared-memory area (after the activation planes) that collects the
    // CTA's output rows, [m][out_pitch] floats; the CTA writes them to the peers in whole lines when it is done.
    // 0: every value goes out on its own.
    int out_bytes;
    int out_pitch;
    // Block on the store (the reference's MvStore, lloom-tensor/src/quantized/mod.rs:1668-1696):
    // 0 plain, 1 silu(W.x), 2 dst <- dst * (W.x).
    int store_mode;
    float *y_peer[kMaxPeers];
};

// One output value to its destination(s).  SiLU in the reference's f32 form v / (1 + exp(-v)) (op.rs:755-757,
// kernels/metal_src/quantized_store.metal:17-25); MulInto reads the destination and multiplies it by the product.
// Only the EPI = 1 kernel instances contain this code: inlined into the sixteen unrolled stores of an 8-row
// instance it cost the plain forward 25-60 % of that instance's time, and as an out-of-line call it still cost
// every instance 5-20 % (registers held across the call sites).
__device__ __forceinline__ void store_out(const GemvParams &p, int64_t idx, float v) {
    if (p.store_mode == LLOOM_STORE_SILU) v = __fdiv_rn(v, __fadd_rn(1.0f, expf(-v)));
    if (p.n_peers == 0) {
        p.y[idx] = (p.store_mode == LLOOM_STORE_MUL_INTO) ? __fmul_rn(p.y[idx], v) : v;
    } else {
        for (int g = 0; g < p.n_peers; ++g) p.y_peer[g][idx] = v;
    }
}

constexpr int kMaxStages = 8;

#ifdef LLOOM_TRACE
// Development build only: per-CTA timestamps (ns) of the GEMV's phases.
__device__ unsigned long long g_trace[16][160][16];  // [launch ring][CTA][event]
__device__ unsigned int g_trace_cnt[160];
__shared__ unsigned int s_trace_slot;
__device__ __forceinline__ unsigned long long trace_now() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
#define LLOOM_TRACE_MARK(slot) do { if ((threadIdx.x & 31) == 0 && blockIdx.x < 160) g_trace[s_trace_slot & 15][blockIdx.x][slot] = trace_now(); } while (0)
#else
#define LLOOM_TRACE_MARK(slot) do { } while (0)
#endif

// Output of row `row` (of this CTA's range starting at r_begin), activation row m: staged in shared memory when the
// launch has a staging area, else straight to its destination(s).
__device__ __forceinline__ void emit_out(const GemvParams &p, float *out_s, int r_begin, int m, int row, float v) {
    if (p.out_bytes) {
        if (p.store_mode == LLOOM_STORE_SILU) v = __fdiv_rn(v, __fadd_rn(1.0f, expf(-v)));
        out_s[m * p.out_pitch + (row - r_begin)] = v;
    } else {
        store_out(p, (int64_t)m * p.ldy + row, v);
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

// Canonical activation blocks (global) -> planes (shared); all `nthreads` consumer threads take part.
__device__ __forceinline__ void stage_acts(const GemvParams &p, uint8_t *act_smem, int tid, int nthreads,
                                           ActPlanes &planes) {
    const size_t qs_bytes = round16(act_qs_bytes(p.w_dtype, p.m, p.k));
    float *dpl = reinterpret_cast<float *>(act_smem + qs_bytes);
    planes.qs = reinterpret_cast<const int8_t *>(act_smem);
    planes.d = dpl;
    planes.k = p.k;
    constexpr int kUnroll = 4;
    if (p.w_dtype == LLOOM_Q8_0) {
        // 17 half-words per block: [0] = f16 d, [1..16] = 32 int8
        const unsigned short *src = reinterpret_cast<const unsigned short *>(p.act);
        unsigned short *q16 = reinterpret_cast<unsigned short *>(act_smem);
        const int total = p.m * (p.k / 32) * 17;
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
        planes.sums = nullptr;
    } else {
        // 73 words per block: [0] = f32 d, [1..64] = 256 int8, [65..72] = 16 int16 bsums
        const int nb = p.k / 256;
        short *sums = reinterpret_cast<short *>(act_smem + qs_bytes + round16((int64_t)p.m * nb * 4));
        const uint32_t *src = reinterpret_cast<const uint32_t *>(p.act);
        uint32_t *q32 = reinterpret_cast<uint32_t *>(act_smem);
        const bool pair = p.w_dtype == LLOOM_Q4_K;
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
    if (p.w_dtype == LLOOM_Q8_0) {
        const int total = p.m * (p.k / 32);
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
        }
        planes.sums = nullptr;
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
                if (p.w_dtype == LLOOM_Q4_K) {
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

// The producer warp's loop: streams tiles of `tile_rows` consecutive rows of [r_begin, r_end) into the stage ring.
__device__ __forceinline__ void gemv_producer(const GemvParams &p, uint64_t *full, uint64_t *empty, uint8_t *stage0,
                                              int tile_rows, int r_begin, int r_end, int lane) {
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
}

// The producer loop for rows cut into pieces (long rows: a whole-row tile would not leave room for two stages in
// the side-by-side shape).  Work items in order -- tile 0: pieces 0.., tile 1: ... -- each `chunk_units` units
// (fewer in a row's last piece) of up to `tile_rows` rows, one bulk copy per row, the pieces of a tile's rows packed
// `chunk_units * unit_bytes` apart.  Needs row sizes and piece sizes that are multiples of 16 bytes.
__device__ __forceinline__ void gemv_producer_pieces(const GemvParams &p, uint64_t *full, uint64_t *empty, uint8_t *stage0,
                                                     int tile_rows, int units, int r_begin, int r_end, int lane) {
    const int pitch = p.chunk_units * p.unit_bytes;
    int it = 0;
    for (int row0 = r_begin; row0 < r_end; row0 += tile_rows) {
        const int rows = min(tile_rows, r_end - row0);
        for (int c = 0; c < p.nchunks; ++c, ++it) {
            const int s = it % p.stages;
            if (it >= p.stages) {
                if (!mbar_wait(&empty[s], ((it / p.stages) - 1) & 1)) return;
            }
            const int u0 = c * p.chunk_units;
            const uint32_t bytes = (uint32_t)(min(p.chunk_units, units - u0) * p.unit_bytes);
            uint8_t *dst = stage0 + (size_t)s * p.stage_bytes;
            if (lane == 0) mbar_arrive_expect_tx(&full[s], (uint32_t)rows * bytes);
            __syncwarp();
            for (int r = lane; r < rows; r += 32)
                bulk_g2s(dst + (size_t)r * pitch, p.w + (int64_t)(row0 + r) * p.row_bytes + (int64_t)u0 * p.unit_bytes, bytes,
                         &full[s]);
        }
    }
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
// EPI = 0 stores every value to p.y and nothing else.
template <class Fmt, int M, int RW, int CW = 8, bool PIECES = false, int EPI = 0>
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

#ifdef LLOOM_TRACE
    if (threadIdx.x == 0) s_trace_slot = blockIdx.x < 160 ? g_trace_cnt[blockIdx.x]++ : 0;
    __syncthreads();
#endif
    if (threadIdx.x == 0) LLOOM_TRACE_MARK(0);
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
        if (PIECES) gemv_producer_pieces(p, full, empty, stage0, tile_rows, p.k / Fmt::kUnitElems, r_begin, r_end, lane);
        else gemv_producer(p, full, empty, stage0, tile_rows, r_begin, r_end, lane);
        return;
    }

    // ---------------- consumer warps ----------------
    ActPlanes planes;
    {
        const int nthreads = p.n_cwarps * 32;
        asm volatile("griddepcontrol.wait;" ::: "memory");  // predecessor's writes (x, act blocks) are visible
        if (threadIdx.x == 0) LLOOM_TRACE_MARK(14);
        if (p.x) quantize_acts_to_planes(p, act_smem, warp, lane, planes);
        else stage_acts(p, act_smem, threadIdx.x, nthreads, planes);
        asm volatile("bar.sync 1, %0;" ::"r"(nthreads) : "memory");
        if (threadIdx.x == 0) LLOOM_TRACE_MARK(1);
    }

    const int units = p.k / Fmt::kUnitElems;
    const int group = lane >> p.lpr_log2, lig = lane & (lpr - 1);
    float *out_s = reinterpret_cast<float *>(act_smem + p.act_bytes);
    int it = 0;  // work items so far: a tile, or one piece of a tile's rows when the rows are cut into pieces
    bool ok = true;  // a timed-out wait ends the loop; the warp still meets the others at the flush barrier
    const int nchunks = PIECES ? p.nchunks : 1;
    const int unit_chunk = PIECES ? p.chunk_units : units;
    const int piece_pitch = unit_chunk * p.unit_bytes;
    for (int trow = r_begin; trow < r_end && ok; trow += tile_rows) {
        const int local0 = (warp * groups + group) * RW;
        const int row0 = trow + local0;
        bool valid[RW];
#pragma unroll
        for (int r = 0; r < RW; ++r) valid[r] = row0 + r < r_end;
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
            if (threadIdx.x == 0 && it < 6) LLOOM_TRACE_MARK(2 + 2 * it);
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
                const int64_t start = (int64_t)trow * p.row_bytes;
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
            // this warp is done reading the stage
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[s]);
            if (threadIdx.x == 0 && it < 6) LLOOM_TRACE_MARK(3 + 2 * it);
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
                        if (EPI == 0) p.y[(int64_t)m * p.ldy + row0 + r] = out[r][m];
                        else emit_out(p, out_s, r_begin, m, row0 + r, out[r][m]);
                    }
                }
        }
    }
    if (EPI != 0 && p.out_bytes) {
        const int nthreads = p.n_cwarps * 32;
        asm volatile("bar.sync 1, %0;" ::"r"(nthreads) : "memory");
        if (ok) flush_out(p, out_s, r_begin, r_end, threadIdx.x, nthreads);
    }
    if (threadIdx.x == 0) LLOOM_TRACE_MARK(15);
}

}  // namespace lloom
