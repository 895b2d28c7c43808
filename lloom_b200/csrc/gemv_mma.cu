// Tensor-core decode GEMV (Q4_K, 2..8 activation rows): kernel instances, launcher, plane quantizer.
#include "gemv_mma.cuh"

namespace lloom {

LLOOM_TU_REGISTER()

template <int SPLIT, int EPI>
static cudaError_t launch_gemv_mma_inst(const GemvParams &p, int grid, int smem, bool overlap, cudaStream_t stream) {
    auto kern = gemv_mma_q4k_kernel<SPLIT, EPI>;
    static FuncSmemConfig cfg;
    cudaError_t e = ensure_smem(kern, cfg, smem, false);
    if (e != cudaSuccess) return e;
    return launch_with_overlap(kern, p, grid, 32 * (kMmaWarps + 1), smem, overlap, stream);
}

cudaError_t launch_gemv_mma(const GemvParams &p, int grid, int smem, bool overlap, cudaStream_t stream) {
    // whole rows per stage: four teams of four warps, a tile each; rows cut into pieces: one team of sixteen, so
    // that a piece is consumed (and its stage handed back) as fast as possible
    if (gemv_needs_epi(p)) {
        if (p.nchunks > 1) return launch_gemv_mma_inst<16, 1>(p, grid, smem, overlap, stream);
        return launch_gemv_mma_inst<4, 1>(p, grid, smem, overlap, stream);
    }
    if (p.nchunks > 1) return launch_gemv_mma_inst<16, 0>(p, grid, smem, overlap, stream);
    return launch_gemv_mma_inst<4, 0>(p, grid, smem, overlap, stream);
}

cudaError_t launch_quantize_q8k_planes(const float *x, uint8_t *out, int m, int nb, int act_pitch, cudaStream_t stream) {
    quantize_q8k_planes_kernel<<<(unsigned)ceil_div64((int64_t)m * nb * 32, 256), 256, 0, stream>>>(x, out, m, nb, act_pitch);
    return cudaGetLastError();
}

}  // namespace lloom
