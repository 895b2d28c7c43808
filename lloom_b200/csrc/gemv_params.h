// Launch parameters and shared-memory sizing of the decode GEMV kernels: the part of gemv.cuh / gemv_mma.cuh
// that the host-side planner (lloom_b200.cu) and the kernels' translation units both need.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/lloom_b200.h"

namespace lloom {

constexpr int kQ8KUnitStride = 256 + 16;
constexpr int kQ8_0UnitStride = 64 + 16;
constexpr int kMaxStages = 8;
constexpr int kMaxPeers = 8;  // GPUs of one node
constexpr int kMaxGroup = LLOOM_B200_MAX_GROUP;  // weight matrices one grouped launch streams

__host__ __device__ inline int64_t round16(int64_t v) { return (v + 15) / 16 * 16; }

// Activation planes in shared memory, built once per CTA (layouts: gemv.cuh).  Formats dotted with Q8_0
// activations work on units of 64 elements, the k-quants on 256-element superblocks.
__host__ __device__ inline bool act_is_q8_0(int w_dtype) {
    return w_dtype == LLOOM_Q8_0 || w_dtype == LLOOM_Q4_0 || w_dtype == LLOOM_Q5_0;
}
__host__ __device__ inline int64_t act_qs_bytes(int w_dtype, int64_t m, int64_t k) {
    return act_is_q8_0(w_dtype) ? m * (k / 64) * kQ8_0UnitStride : m * (k / 256) * kQ8KUnitStride;
}
__host__ __device__ inline int64_t act_plane_bytes(int w_dtype, int64_t m, int64_t k) {
    const int64_t qs = act_qs_bytes(w_dtype, m, k);
    const int64_t d = act_is_q8_0(w_dtype) ? m * (k / 32) * 4 : m * (k / 256) * 4;
    const int64_t sums = act_is_q8_0(w_dtype) ? (w_dtype == LLOOM_Q8_0 ? 0 : m * (k / 32) * 4)
                                              : (w_dtype == LLOOM_Q6_K ? m * (k / 16) * 2 : m * (k / 32) * 2);
    return round16(qs) + round16(d) + round16(sums);
}

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
    int chunk_units;     // dp4a kernel, nchunks > 1: units (superblocks / pairs of 32-element blocks) of a row per piece
    int unit_bytes;      // dp4a kernel: bytes of a unit
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
    // Fused gather, barrier folded into the GEMV (publish != 0): the last CTA to finish advances this GPU's call
    // counter and stores it in slot [peer_rank] of every GPU's flag array (lloom_b200_qmatmul_fwd_gather_sync).
    // wait_flags != nullptr: the activations came out of an earlier fused gather whose flag array (this GPU's)
    // this is; the kernel waits for all `wait_peers` slots to reach that gather's count before it reads them.
    unsigned int *peer_flags[kMaxPeers];
    const unsigned int *wait_flags;
    int wait_peers;
    int publish;
    int peer_rank;
    float *y_peer[kMaxPeers];
    // Grouped launch (n_group > 1): matrices of one dtype and k that share the activations, streamed by one launch.
    // The kernel walks the concatenation of their rows; `n` is the total.  Matrix g: rows [goff[g], goff[g+1]).
    int n_group;
    const uint8_t *gw[kMaxGroup];
    float *gy[kMaxGroup];
    int64_t gldy[kMaxGroup];
    int goff[kMaxGroup + 1];
    int gstore[kMaxGroup];
    // Routed experts (moe_ids != nullptr, grouped launches only): matrix g is expert moe_ids[g] of the stacked
    // tensor at `w` (every expert has as many rows as the group's matrices); the ids are device data, read after the
    // stream predecessor is done.
    const uint32_t *moe_ids;
    int moe_experts;
};

// ---- tensor-core GEMV (gemv_mma.cuh) ----
constexpr int kMmaTileRows = 16;
constexpr int kMmaWarps = 16;  // consumer warps; SPLIT of them share a tile, warp j of a team takes superblocks j, j+SPLIT, ...
constexpr int kMmaRedBytes = 2 * kMmaWarps * 32 * 16;  // double-buffered partial sums, one float4 per lane
constexpr int kMmaBarBytes = 128;      // empty[8], one barrier for the activation image
constexpr int kMmaMaxTiles = 512;      // per CTA; one 8-byte barrier each

// Pitch in bytes (a multiple of 16, >= bytes) that is `want_words` 32-bit words modulo the 32 banks.
__host__ __device__ inline int64_t bank_pitch(int64_t bytes, int want_words) {
    const int64_t words = (bytes + 3) / 4;
    int64_t pad = (want_words - words % 32 + 32) % 32;
    while ((words + pad) % 4 != 0) pad += 32;  // never taken when bytes % 16 == 0 and want_words % 4 == 0
    return (words + pad) * 4;
}
__host__ __device__ inline int64_t mma_act_pitch(int64_t k) { return bank_pitch((k / 256) * 256, 16); }
__host__ __device__ inline int64_t mma_act_bytes(int64_t m, int64_t k) {
    return round16(m * mma_act_pitch(k) + m * (k / 256) * 16 + m * (k / 256) * 4);
}

// ---- launchers exported by the kernels' translation units ----
// dp4a GEMV, one unit per weight format.  rw: rows per lane (1 or 2).
cudaError_t launch_gemv_dp4a_q8_0(const GemvParams &p, int grid, int smem, bool overlap, int rw, cudaStream_t stream);
cudaError_t launch_gemv_dp4a_q4k(const GemvParams &p, int grid, int smem, bool overlap, int rw, cudaStream_t stream);
cudaError_t launch_gemv_dp4a_q6k(const GemvParams &p, int grid, int smem, bool overlap, int rw, cudaStream_t stream);
cudaError_t launch_gemv_dp4a_q5k(const GemvParams &p, int grid, int smem, bool overlap, int rw, cudaStream_t stream);
cudaError_t launch_gemv_dp4a_q4_0(const GemvParams &p, int grid, int smem, bool overlap, int rw, cudaStream_t stream);
cudaError_t launch_gemv_dp4a_q5_0(const GemvParams &p, int grid, int smem, bool overlap, int rw, cudaStream_t stream);
// tensor-core GEMV (Q4_K, 2..8 rows) and the quantizer that writes its activation image
cudaError_t launch_gemv_mma(const GemvParams &p, int grid, int smem, bool overlap, cudaStream_t stream);
cudaError_t launch_quantize_q8k_planes(const float *x, uint8_t *out, int m, int nb, int act_pitch, cudaStream_t stream);

}  // namespace lloom
