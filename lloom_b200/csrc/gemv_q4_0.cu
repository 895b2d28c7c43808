// dp4a decode GEMV, Q4_0 weights: the kernel instances of this format and their launcher.
#include "gemv.cuh"

namespace lloom {

LLOOM_TU_REGISTER()

cudaError_t launch_gemv_dp4a_q4_0(const GemvParams &p, int grid, int smem, bool overlap, int rw, cudaStream_t stream) {
    return launch_gemv_format<FmtQ4_0>(p, grid, smem, overlap, rw, stream);
}

}  // namespace lloom
