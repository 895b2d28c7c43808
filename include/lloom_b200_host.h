/*
 * C view of the C++ host layer (lloom_b200/csrc/host/qcuda_storage.hpp): QTensor / QMatMul objects
 * behind opaque handles, for drivers that cannot call C++ (the Python tests and the benchmark).
 * A Rust integration does not need this header: it keeps its own QTensor / QCudaStorage and binds
 * the kernel-level entry points of lloom_b200.h directly.
 *
 * Unlike lloom_b200.h, these functions own device memory (cudaMalloc / cudaFree) the way
 * QCudaStorage does in the reference (lloom-tensor/src/quantized/cuda.rs:624-637, 1005-1024), and keep
 * one grow-only scratch buffer per device (fast_mmvq.rs:44-81).  All return 0 on success, else a
 * lloom_b200 status or -1; lloom_b200_host_last_error() describes the last failure on this thread.
 */
#ifndef LLOOM_B200_HOST_H
#define LLOOM_B200_HOST_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

const char *lloom_b200_host_last_error(void);

/* CPU weight quantizer, T::from_float per row (k_quants.rs:738-767, 1622-1680, 2174-2244): what
 * QCudaStorage::quantize runs before uploading (cuda.rs:720-741).  Host pointers. */
int lloom_b200_host_quantize_rows(int dtype, const float *x, void *blocks, int64_t rows, int64_t k, int nthreads);

/* T::from_float_imatrix per row (k_quants.rs:1682-1745, 1959-2041, 2246-2325): importance-weighted quantization,
 * `imatrix` holds k weights (one per column); Q4_K, Q5_K and Q6_K only, other types fail as in the reference. */
int lloom_b200_host_quantize_rows_imatrix(int dtype, const float *x, const float *imatrix, void *blocks, int64_t rows,
                                          int64_t k, int nthreads);
/* QTensor::quantize_imatrix / quantize_imatrix_onto (mod.rs:940-1020, cuda.rs:743-790). */
int lloom_b200_host_qtensor_quantize_imatrix(int device, void *stream, const float *src, const float *imatrix, int64_t n,
                                             int64_t k, int dtype, int nthreads, void **out);
/* QTensor::quantize (mod.rs:919-938): host f32 [n,k] -> packed blocks on `device`. */
int lloom_b200_host_qtensor_quantize(int device, void *stream, const float *src, int64_t n, int64_t k, int dtype,
                                     int nthreads, void **out);
/* QStorage::from_data + load_quantized (mod.rs:136-223, cuda.rs:1005-1024): raw GGUF block bytes. */
int lloom_b200_host_qtensor_from_data(int device, void *stream, const void *bytes, int64_t nbytes, int dtype,
                                      int64_t n, int64_t k, void **out);
void lloom_b200_host_qtensor_free(void *qtensor);
int64_t lloom_b200_host_qtensor_nbytes(void *qtensor);           /* storage_size_in_bytes */
const void *lloom_b200_host_qtensor_device_ptr(void *qtensor);   /* device_ptr */
int lloom_b200_host_qtensor_data(void *qtensor, void *out, int64_t capacity); /* data(): exact packed bytes */

/* QMatMul::forward (mod.rs:2022-2026): x f32 [m,k] on the device -> y f32 [m,n] on the device. */
int lloom_b200_host_qmatmul_forward(void *qtensor, const float *x_dev, int64_t m, float *y_dev);
/* QTensor::dequantize / dequantize_f16 (mod.rs:1065-1086) into a device buffer of n*k elements. */
int lloom_b200_host_qtensor_dequantize(void *qtensor, void *out_dev, int f16);
/* QTensor::embedding (mod.rs:1101-1144): ids u32 on the device -> f32 [n_ids, k] on the device. */
int lloom_b200_host_qtensor_embedding(void *qtensor, const uint32_t *ids_dev, int64_t n_ids, float *out_dev);

#ifdef __cplusplus
}
#endif
#endif
