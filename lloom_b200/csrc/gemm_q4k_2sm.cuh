// Prefill GEMM for Q4_K weights, CTA-pair variant: `tcgen05.mma.cta_group::2`, 256 weight rows x 128
// activation rows per pair of SMs.
//
// Same arithmetic, operand images, accumulator scheme and epilogue as the one-SM kernel (gemm_q4k.cuh).
// What changes is who reads what from shared memory.  A one-SM 128x128x16 MMA reads 8 KB of operands in
// its 64 cycles -- the whole shared-memory port -- and the bulk copies write as much again, which caps
// the tensor pipe near one half.  In a CTA pair each SM keeps its own 128 weight rows (A) but only half of
// the activation tile (64 rows of B); the pair's tensor cores exchange the halves themselves.  Per 128 of
// K an SM then takes in 48 KB and reads 48 KB in 512 cycles instead of 64 KB + 64 KB.
//
// Pair protocol (rank 0 = leader, issues every MMA and commit):
//   * both CTAs copy their own operands and complete their own `full` / `min_full` barriers (a plain bulk
//     copy can only signal a barrier of the CTA it writes to); in the peer a relay warp waits on those and
//     arrives on the leader's `peer_full` / `peer_min_full` barriers across the cluster;
//   * the leader's commits are multicast to both CTAs' `empty` / `acc_full` barriers;
//   * epilogue warps of both CTAs arrive on the leader's `pair_empty` (accumulators drained) and on their
//     own `min_free` (scale tile read; the commit after the Mn MMA is its ninth arrival);
//   * tensor memory is allocated and freed by the same warp of both CTAs (cta_group::2 rule), with a
//     cluster barrier after the allocation and before the release.
// Every mbarrier wait is time-bounded and abortable, as in the one-SM kernel; the two cluster barriers are
// reached by every thread on every path.
#pragma once

#include "gemm_q4k.cuh"

namespace lloom {

constexpr int k2StageA = 2 * kGemmAtomBytes;      // 128 weight rows x 128 of K, f16
constexpr int k2StageB = kGemmAtomBytes;          // 64 activation rows x 128 of K: two half atoms
constexpr int k2Stages = 4;
constexpr int k2MinB = kGemmMinBytes / 2;         // 64 activation rows x 16
constexpr int k2Threads = 352;                    // 8 epilogue warps, producer, MMA issuer, relay
constexpr int k2OffA = 0;
constexpr int k2OffB = k2OffA + k2Stages * k2StageA;
constexpr int k2OffMinA = k2OffB + k2Stages * k2StageB;
constexpr int k2MinBufs = 4;  // min tiles + activation scales: small, so buffered deeper than the accumulators --
                              // with two, the producer stalls on the epilogue two superblocks back and the
                              // operand prefetch never gets more than one superblock ahead
constexpr int k2OffMinB = k2OffMinA + k2MinBufs * kGemmMinBytes;
constexpr int k2OffDa = k2OffMinB + k2MinBufs * k2MinB;
constexpr int k2OffBars = k2OffDa + k2MinBufs * kGemmDaBytes;
// full[4] empty[4] peer_full[4] | min_full[4] peer_min_full[4] min_free[4] | acc_full[2] pair_empty[2]
constexpr int k2NumBars = 3 * k2Stages + 3 * k2MinBufs + 4;
constexpr int k2OffMisc = k2OffBars + k2NumBars * 8;
constexpr int k2SmemBytes = k2OffMisc + 16 + 1024;

#ifdef LLOOM_TRACE
// Development build only: clock64 stamps of CTA 0's roles, [role][superblock][event].
__device__ long long g_gemm2_trace[4][64][8];
#define G2_MARK(role, b, ev) do { if (blockIdx.x == 0 && lane == 0 && (b) < 64) g_gemm2_trace[role][b][ev] = clock64(); } while (0)
#else
#define G2_MARK(role, b, ev) do { } while (0)
#endif

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Arrive on the barrier at the same shared-memory offset in CTA `rank` of the cluster.
__device__ __forceinline__ void mbar_arrive_cluster(uint64_t *local_bar, uint32_t rank) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(local_bar)), "r"(rank));
    // default semantics (release at CTA scope): a cluster-scope release is a full fence per arrival, and the
    // data these arrivals order -- tensor memory and bulk-copied shared memory -- is ordered by the tcgen05
    // fences and the copy's own completion, not by this thread's earlier stores
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(remote) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait_cluster(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// mbar_wait_abortable with cluster-scope acquire: for barriers another CTA arrives on.
template <int kSleepNs>
__device__ __forceinline__ bool mbar_wait_abortable_cluster(uint64_t *bar, uint32_t parity, volatile int *abort_flag) {
    if (mbar_try_wait_cluster(bar, parity)) return true;
    unsigned long long t0 = 0;
    for (uint32_t i = 0; i < kMaxSpins; ++i) {
        if (kSleepNs > 0) __nanosleep(kSleepNs);
        if (mbar_try_wait_cluster(bar, parity)) return true;
        if ((i & 63) == 63) {
            if (*abort_flag) return false;
            const unsigned long long now = global_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > kMaxWaitNs) break;
        }
    }
    *abort_flag = 1;
    atomicExch(&g_device_status, LLOOM_ERR_TIMEOUT);
    return false;
}

__device__ __forceinline__ void umma_f16_2sm(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n\t"
        "}\n" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u)
        : "memory");
}
// Commit of the pair's outstanding MMAs, arriving on the barrier at this offset in both CTAs.
__device__ __forceinline__ void umma_commit_pair(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
                     smem_u32(bar)),
                 "h"((unsigned short)3)
                 : "memory");
}

// Grid: 2 * (pairs of n-tiles) * m_tiles CTAs in clusters of two; the m-tiles of one pair of n-tiles are
// neighbours in launch order.  The weight images cover an even number of n-tiles (rows past n are zero).
__global__ void __launch_bounds__(k2Threads, 1) gemm_q4k_2sm_kernel(const GemmParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + k2OffBars);
    uint64_t *full = bars, *empty = bars + k2Stages, *peer_full = bars + 2 * k2Stages;
    uint64_t *min_full = bars + 3 * k2Stages, *peer_min_full = min_full + k2MinBufs, *min_free = min_full + 2 * k2MinBufs;
    uint64_t *acc_full = min_full + 3 * k2MinBufs, *pair_empty = acc_full + 2;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem + k2OffMisc);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + k2OffMisc + 4);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const int pair = blockIdx.x >> 1;
    const int mt = pair % p.m_tiles, nt = 2 * (pair / p.m_tiles) + (int)rank;
    const int n0 = nt * kGemmBN, m0 = mt * kGemmBM;
    const int nb = p.k / 256;
    const GemmScratch lay = gemm_scratch_layout(p.m, p.n, p.k);

    if (threadIdx.x == 0) {
        for (int s = 0; s < k2Stages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
            mbar_init(&peer_full[s], 1);
        }
        for (int i = 0; i < k2MinBufs; ++i) {
            mbar_init(&min_full[i], 1);
            mbar_init(&peer_min_full[i], 1);
            mbar_init(&min_free[i], kGemmEpiWarps + 1);  // local epilogue warps (scales read) + the commit after the Mn MMA
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&acc_full[i], 1);
            mbar_init(&pair_empty[i], 2 * kGemmEpiWarps);
        }
        *abort_flag = 0;
        fence_mbar_init();
    }
    if (warp == kGemmEpiWarps + 1) {  // tensor memory: all 512 columns in both CTAs, two (S, Mn) accumulator pairs
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512u)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();  // the peer's barriers are initialised and its tensor memory allocated
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp < kGemmEpiWarps) {
        // ------------------------------ epilogue (this CTA's 128 weight rows x 128 activation rows) ------------------------------
        const int q = warp & 3, half = warp >> 2;
        const int r = q * 32 + lane;
        const int n = n0 + r;
        const bool row_ok = n < p.n;
        const uint8_t *wrow = p.w + (int64_t)(row_ok ? n : 0) * p.row_bytes;
        uint64_t out2[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) out2[j] = 0ull;
        uint32_t hdr_next = row_ok ? __ldg(reinterpret_cast<const uint32_t *>(wrow)) : 0u;
        bool ok = true;
        for (int b = 0; b < nb && ok; ++b) {
            const int buf = b & 1;
            const uint32_t par = (b >> 1) & 1;
            const uint32_t hdr = hdr_next;
            if (b + 1 < nb && row_ok) hdr_next = __ldg(reinterpret_cast<const uint32_t *>(wrow + (int64_t)(b + 1) * Q4K_BYTES));
            const float dw = f16_bits_to_f32(hdr & 0xffffu), ndmin = -f16_bits_to_f32(hdr >> 16);
            const uint64_t dw2 = pack2f(dw, dw), ndmin2 = pack2f(ndmin, ndmin);
            const int mb = b % k2MinBufs;
            ok = mbar_wait_abortable<64>(&min_full[mb], (b / k2MinBufs) & 1, abort_flag);
            if (!ok) break;
            uint64_t da2[32];
            {
                const ulonglong2 *dap = reinterpret_cast<const ulonglong2 *>(smem + k2OffDa + mb * kGemmDaBytes + half * 256);
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const ulonglong2 t = dap[j];
                    da2[2 * j] = t.x;
                    da2[2 * j + 1] = t.y;
                }
            }
            if (warp == 0) G2_MARK(1, b, 0);
            ok = mbar_wait_abortable_cluster<64>(&acc_full[buf], par, abort_flag);
            if (!ok) break;
            tc_fence_after();
            if (warp == 0) G2_MARK(1, b, 1);
            const uint32_t t_main = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * 256 + half * 64);
            uint32_t va[32], vb[32];
            tmem_ld32(t_main, va);
            tmem_ld_wait();
            tmem_ld32(t_main + 128, vb);
#pragma unroll
            for (int j = 0; j < 16; ++j)
                out2[j] = fma_f32x2(mul_f32x2(da2[j], dw2), (uint64_t)va[2 * j] | ((uint64_t)va[2 * j + 1] << 32), out2[j]);
            tmem_ld_wait();
            tmem_ld32(t_main + 32, va);
#pragma unroll
            for (int j = 0; j < 16; ++j)
                out2[j] = fma_f32x2(mul_f32x2(da2[j], ndmin2), (uint64_t)vb[2 * j] | ((uint64_t)vb[2 * j + 1] << 32), out2[j]);
            tmem_ld_wait();
            tmem_ld32(t_main + 128 + 32, vb);
#pragma unroll
            for (int j = 0; j < 16; ++j)
                out2[16 + j] = fma_f32x2(mul_f32x2(da2[16 + j], dw2), (uint64_t)va[2 * j] | ((uint64_t)va[2 * j + 1] << 32), out2[16 + j]);
            tmem_ld_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(&min_free[mb]);               // local producer: the scale tile is free
                mbar_arrive_cluster(&pair_empty[buf], 0);  // leader's MMA issuer: this warp's accumulators are drained
            }
            if (warp == 0) G2_MARK(1, b, 2);
#pragma unroll
            for (int j = 0; j < 16; ++j)
                out2[16 + j] = fma_f32x2(mul_f32x2(da2[16 + j], ndmin2), (uint64_t)vb[2 * j] | ((uint64_t)vb[2 * j + 1] << 32), out2[16 + j]);
        }
        if (ok && row_ok) {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
                const int mrow = m0 + half * 64 + 2 * j;
                if (mrow < p.m) p.y[(int64_t)mrow * p.ldy + n] = __uint_as_float((uint32_t)(out2[j] & 0xffffffffu));
                if (mrow + 1 < p.m) p.y[(int64_t)(mrow + 1) * p.ldy + n] = __uint_as_float((uint32_t)(out2[j] >> 32));
            }
        }
    } else if (warp == kGemmEpiWarps) {
        // ------------------------------ operand tiles: bulk copies (own A rows, own half of B) ------------------------------
        const uint8_t *aimg = p.scratch + lay.aimg + (int64_t)nt * (p.k / 64) * kGemmAtomBytes;
        const uint8_t *mina = p.scratch + lay.mina + (int64_t)nt * nb * kGemmMinBytes;
        const uint8_t *bimg = p.scratch + lay.bimg + (int64_t)mt * (p.k / 64) * kGemmAtomBytes + rank * (kGemmAtomBytes / 2);
        const uint8_t *minb = p.scratch + lay.minb + (int64_t)mt * nb * kGemmMinBytes + rank * k2MinB;
        const uint8_t *dat = p.scratch + lay.dat + (int64_t)mt * nb * kGemmDaBytes;
        bool ok = true;
        for (int b = 0; b < nb && ok; ++b) {
            for (int h = 0; h < 2 && ok; ++h) {
                const int it = b * 2 + h, s = it % k2Stages;
                if (it >= k2Stages) ok = mbar_wait_abortable_cluster<32>(&empty[s], ((it / k2Stages) - 1) & 1, abort_flag);
                if (!ok) break;
                G2_MARK(2, b, h);
                if (lane == 0) {
                    mbar_arrive_expect_tx(&full[s], k2StageA + k2StageB);
                    bulk_g2s(smem + k2OffA + s * k2StageA, aimg + (int64_t)it * k2StageA, k2StageA, &full[s]);
                    bulk_g2s(smem + k2OffB + s * k2StageB, bimg + (int64_t)(2 * it) * kGemmAtomBytes, kGemmAtomBytes / 2, &full[s]);
                    bulk_g2s(smem + k2OffB + s * k2StageB + kGemmAtomBytes / 2, bimg + (int64_t)(2 * it + 1) * kGemmAtomBytes,
                             kGemmAtomBytes / 2, &full[s]);
                }
                __syncwarp();
            }
            if (!ok) break;
            const int mb = b % k2MinBufs;
            // the buffer is free after the Mn MMA of b-4 (commit) and the local epilogue of b-4 (scales read)
            if (b >= k2MinBufs) ok = mbar_wait_abortable_cluster<32>(&min_free[mb], ((b / k2MinBufs) - 1) & 1, abort_flag);
            if (!ok) break;
            G2_MARK(2, b, 2);
            if (lane == 0) {
                mbar_arrive_expect_tx(&min_full[mb], kGemmMinBytes + k2MinB + kGemmDaBytes);
                bulk_g2s(smem + k2OffMinA + mb * kGemmMinBytes, mina + (int64_t)b * kGemmMinBytes, kGemmMinBytes, &min_full[mb]);
                bulk_g2s(smem + k2OffMinB + mb * k2MinB, minb + (int64_t)b * kGemmMinBytes, k2MinB, &min_full[mb]);
                bulk_g2s(smem + k2OffDa + mb * kGemmDaBytes, dat + (int64_t)b * kGemmDaBytes, kGemmDaBytes, &min_full[mb]);
            }
            __syncwarp();
        }
    } else if (warp == kGemmEpiWarps + 1) {
        // ------------------------------ MMA issuer (leader CTA only) ------------------------------
        if (rank == 0) {
            // instruction descriptor: D = f32, A = B = f16, both K-major, N = 128, M = 256 over the pair
            const uint32_t idesc = (1u << 4) | ((uint32_t)(kGemmBM >> 3) << 17) | ((uint32_t)((2 * kGemmBN) >> 4) << 24);
            bool ok = true;
            for (int b = 0; b < nb && ok; ++b) {
                const int buf = b & 1;
                if (b >= 2) ok = mbar_wait_abortable_cluster<0>(&pair_empty[buf], ((b >> 1) - 1) & 1, abort_flag);
                if (!ok) break;
                tc_fence_after();
                G2_MARK(0, b, 0);
                const uint32_t d_main = tmem_base + (uint32_t)(buf * 256), d_min = d_main + 128;
                for (int h = 0; h < 2 && ok; ++h) {
                    const int it = b * 2 + h, s = it % k2Stages;
                    const uint32_t fpar = (it / k2Stages) & 1;
                    ok = mbar_wait_abortable<0>(&full[s], fpar, abort_flag);
                    G2_MARK(0, b, 1 + 3 * h);
                    ok = ok && mbar_wait_abortable_cluster<0>(&peer_full[s], fpar, abort_flag);
                    if (!ok) break;
                    tc_fence_after();
                    G2_MARK(0, b, 2 + 3 * h);
                    if (lane == 0) {
                        const uint32_t a_addr = smem_u32(smem + k2OffA + s * k2StageA);
                        const uint32_t b_addr = smem_u32(smem + k2OffB + s * k2StageB);
#pragma unroll
                        for (int kk = 0; kk < 8; ++kk) {  // K = 16 per instruction: atom kk/4, 32 bytes along its swizzled row
                            const uint32_t a_off = (uint32_t)((kk >> 2) * kGemmAtomBytes + (kk & 3) * 32);
                            const uint32_t b_off = (uint32_t)((kk >> 2) * (kGemmAtomBytes / 2) + (kk & 3) * 32);
                            umma_f16_2sm(d_main, umma_desc(a_addr + a_off, 16, 1024, 2), umma_desc(b_addr + b_off, 16, 1024, 2),
                                         idesc, (h | kk) != 0 ? 1u : 0u);
                        }
                        umma_commit_pair(&empty[s]);
                    }
                    __syncwarp();
                    G2_MARK(0, b, 3 + 3 * h);
                }
                if (!ok) break;
                const int mb = b % k2MinBufs;
                const uint32_t mpar = (b / k2MinBufs) & 1;
                ok = mbar_wait_abortable<0>(&min_full[mb], mpar, abort_flag) &&
                     mbar_wait_abortable_cluster<0>(&peer_min_full[mb], mpar, abort_flag);
                if (!ok) break;
                tc_fence_after();
                if (lane == 0) {
                    const uint64_t mad = umma_desc(smem_u32(smem + k2OffMinA + mb * kGemmMinBytes), 128, 256, 0);
                    const uint64_t mbd = umma_desc(smem_u32(smem + k2OffMinB + mb * k2MinB), 128, 256, 0);
                    umma_f16_2sm(d_min, mad, mbd, idesc, 0u);
                    umma_commit_pair(&acc_full[buf]);
                    umma_commit_pair(&min_free[mb]);
                }
                __syncwarp();
                G2_MARK(0, b, 7);
            }
        }
    } else {
        // ------------------------------ relay (peer CTA only): local arrivals -> leader's barriers ------------------------------
        if (rank == 1) {
            bool ok = true;
            for (int b = 0; b < nb && ok; ++b) {
                for (int h = 0; h < 2 && ok; ++h) {
                    const int it = b * 2 + h, s = it % k2Stages;
                    ok = mbar_wait_abortable<20>(&full[s], (it / k2Stages) & 1, abort_flag);
                    if (!ok) break;
                    if (lane == 0) mbar_arrive_cluster(&peer_full[s], 0);
                    __syncwarp();
                }
                if (!ok) break;
                const int mb = b % k2MinBufs;
                ok = mbar_wait_abortable<20>(&min_full[mb], (b / k2MinBufs) & 1, abort_flag);
                if (!ok) break;
                if (lane == 0) mbar_arrive_cluster(&peer_min_full[mb], 0);
                __syncwarp();
            }
        }
    }
    // ------------------------------ teardown ------------------------------
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();  // neither CTA frees tensor memory or exits while the other may still use the pair's resources
    if (warp == kGemmEpiWarps + 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
    }
}

// Launches the CTA-pair kernel when LLOOM_GEMM_2SM=1.  Off by default: on [14336, 4096] x 2048 rows it is
// parity-green but measures 469 us per forward against the one-SM kernel's 388 us.  Clock stamps of its roles
// show why: per superblock the pair needs ~1.5 us on an idle L2 (the issuing thread's waits, commits and the
// relay hop leave the tensor pipe idle between bursts) and ~2.2 us once all SMs stream operands, where the
// one-SM kernel needs 1.8 us; what the pair saves in shared-memory traffic it loses to the coupling of two
// CTAs (each MMA waits for the slower CTA's copies, each accumulator hand-back for the slower epilogue).
inline cudaError_t gemm_launch_pair_kernel(const GemmParams &p, int max_smem, cudaStream_t stream, bool &launched) {
    launched = false;
    static const bool enabled = []() { const char *e = getenv("LLOOM_GEMM_2SM"); return e && e[0] == '1'; }();
    if (!enabled || k2SmemBytes > max_smem) return cudaSuccess;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_q4k_2sm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, k2SmemBytes);
        if (e != cudaSuccess) return e;
        configured = true;
    }
    const int pairs = (p.n_tiles + 1) / 2;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(2 * pairs * p.m_tiles));
    cfg.blockDim = dim3(k2Threads);
    cfg.dynamicSmemBytes = k2SmemBytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    launched = true;
    return cudaLaunchKernelEx(&cfg, gemm_q4k_2sm_kernel, p);
}

}  // namespace lloom
