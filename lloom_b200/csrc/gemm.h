// Host-side interface of the prefill GEMM translation unit (gemm.cu).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace lloom {

// Whether a tensor-core GEMM exists for this weight type and shape (else the caller runs slabs of the decode GEMV).
bool gemm_supported(int w_dtype, int64_t m, int64_t k, int max_smem);
// Bytes of the f16 operand images of a whole [n, k] weight matrix (what lloom_b200_weight_image_build writes).
int64_t gemm_weight_image_bytes(int w_dtype, int64_t n, int64_t k);
// Scratch of one GEMM call after the canonical activation blocks: the activation images, plus -- unless the caller
// brings a prebuilt weight image -- room for the weight images of one slab of rows.
int64_t gemm_scratch_bytes(int w_dtype, int64_t m, int64_t n, int64_t k, bool have_image);
cudaError_t gemm_weight_image_build(int w_dtype, const void *w, int64_t n, int64_t k, void *image, cudaStream_t stream);
// Whether gemm_forward takes f32 activations directly for this weight type (it then quantizes them itself, in the pass
// that builds the operand images).
bool gemm_takes_f32(int w_dtype);
// y[m, n] from canonical activation blocks `act`, or -- where gemm_takes_f32 -- from the f32 activations `x` [m, k]
// (exactly one of the two is non-null); w_image may be null (images are then built per call, slab by slab).
cudaError_t gemm_forward(int w_dtype, const void *w_blocks, const void *w_image, const void *act, const float *x, float *y,
                         int64_t m, int64_t n, int64_t k, int64_t ldy, void *scratch, cudaStream_t stream);

}  // namespace lloom
