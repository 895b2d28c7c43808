// Prefill GEMM for Q4_K weights on tcgen05 tensor cores (placeholder: not yet taken).
#pragma once

#include "common.cuh"

namespace lloom {

inline int64_t gemm_scratch_bytes(int /*w_dtype*/, int64_t /*m*/, int64_t /*n*/, int64_t /*k*/) { return 0; }

inline int gemm_launch(int /*w_dtype*/, const void * /*w*/, const void * /*act*/, float * /*y*/, int64_t /*m*/,
                       int64_t /*n*/, int64_t /*k*/, int64_t /*ldy*/, void * /*workspace*/, int /*sm_count*/,
                       int /*max_smem*/, cudaStream_t /*stream*/, bool &handled, int & /*cuda_err*/) {
    handled = false;
    return LLOOM_OK;
}

}  // namespace lloom
