// Host side of the CUDA slot, in C++ because the reference's host language (Rust) has no toolchain
// here.  Mirrors lloom-tensor's types for this path: GgmlDType (quantized/mod.rs:404-716),
// QCudaStorage (quantized/cuda.rs:586-1024), QTensor (mod.rs:94-101, 908-1666) and QMatMul
// (mod.rs:1698-1752, 2022-2069).  All device work goes through the C ABI in include/lloom_b200.h;
// this layer owns memory (cudaMalloc / cudaFree), shapes and errors, like the Rust side does.
#pragma once

#include <cstdint>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

namespace lloom {
namespace host {

enum class GgmlDType : int { Q4_0 = 2, Q5_0 = 6, Q8_0 = 8, Q4K = 12, Q5K = 13, Q6K = 14, Q8K = 15 };

int64_t block_size(GgmlDType t);  // elements per block
int64_t type_size(GgmlDType t);   // bytes per block

// Errors carry the library status (or -1 for host-side refusals) like lloom_tensor::Error::Cuda / Msg.
struct Error : public std::runtime_error {
    int status;
    Error(int s, const std::string &what) : std::runtime_error(what), status(s) {}
};

// One device + the stream every launch of this storage is enqueued on (the reference keeps one
// stream per CudaDevice, cuda_backend/device.rs:59-68).
struct CudaDevice {
    int ordinal = 0;
    void *stream = nullptr;  // cudaStream_t; null = the legacy default stream
};

// CPU weight quantizers, T::from_float (k_quants.rs:738-767, 1622-1680, 2174-2244 with
// utils.rs:62-224, 227-284).  The reference's CUDA slot quantizes weights on the CPU and uploads
// (cuda.rs:720-741); so does this one.  rows x k floats -> rows x (k/block) blocks, rows in parallel.
// imatrix != nullptr: T::from_float_imatrix with one importance weight per column (k_quants.rs:1682, 1959, 2246;
// Q4K, Q5K and Q6K only, like the reference).
void quantize_rows(GgmlDType t, const float *x, void *blocks, int64_t rows, int64_t k, int nthreads,
                   const float *imatrix = nullptr);

class QCudaStorage {
  public:
    QCudaStorage(const QCudaStorage &) = delete;
    QCudaStorage &operator=(const QCudaStorage &) = delete;
    ~QCudaStorage();

    // cuda.rs:624-637
    static std::unique_ptr<QCudaStorage> zeros(const CudaDevice &dev, int64_t el_count, GgmlDType dtype);
    // cuda.rs:1005-1024: raw GGUF block bytes, one H2D copy, zero tail padding, no repack.
    static std::unique_ptr<QCudaStorage> load_quantized(const CudaDevice &dev, const void *data, int64_t nbytes,
                                                        GgmlDType dtype);
    // cuda.rs:720-741 quantize_onto: CPU quantizer over host f32, then upload.
    void quantize_onto(const float *host_src, int64_t el_count, int64_t k, int nthreads);
    // cuda.rs:743-790 quantize_imatrix / quantize_imatrix_onto: the same with importance weights, one per column
    void quantize_imatrix_onto(const float *host_src, int64_t el_count, const float *imatrix_weights, int64_t n_per_row,
                               int nthreads);

    GgmlDType dtype() const { return dtype_; }
    const CudaDevice &device() const { return dev_; }
    int64_t storage_size_in_bytes() const { return len_; }
    const uint8_t *device_ptr() const { return data_; }
    std::vector<uint8_t> data() const;  // cuda.rs:894-900: the exact packed bytes

    // cuda.rs:647-718; `out` is a device buffer of elem_count f32 / f16
    void dequantize(int64_t elem_count, void *out, bool f16) const;
    // cuda.rs:828-860; ids u32 on device, out f32 [n_ids, hidden] on device
    void embedding(int64_t rows, int64_t hidden, const uint32_t *ids, int64_t n_ids, float *out) const;
    // cuda.rs:862-894; weight [n,k], x f32 [m,k] contiguous on device, y f32 with row stride ldy
    // store: LLOOM_STORE_PLAIN, or a block on the GEMV's store (m <= 8): LLOOM_STORE_SILU, LLOOM_STORE_MUL_INTO
    void fwd(int64_t n, int64_t k, const float *x, int64_t m, float *y, int64_t ldy, int store = 0) const;

  private:
    QCudaStorage(const CudaDevice &dev, GgmlDType dtype) : dev_(dev), dtype_(dtype) {}
    CudaDevice dev_;
    GgmlDType dtype_;
    uint8_t *data_ = nullptr;
    int64_t len_ = 0;
    int64_t padded_ = 0;
};

class QTensor {
  public:
    QTensor(std::unique_ptr<QCudaStorage> storage, std::vector<int64_t> shape);  // mod.rs:909-917 + check_shape
    // mod.rs:919-938: quantize host f32 [.., k] with the CPU quantizer and move it to the device
    static std::shared_ptr<QTensor> quantize(const CudaDevice &dev, const float *src, std::vector<int64_t> shape,
                                             GgmlDType dtype, int nthreads);
    // mod.rs:940-1020 quantize_imatrix / quantize_imatrix_onto: imatrix_len must equal the last dim
    static std::shared_ptr<QTensor> quantize_imatrix(const CudaDevice &dev, const float *src, const float *imatrix_weights,
                                                     int64_t imatrix_len, std::vector<int64_t> shape, GgmlDType dtype,
                                                     int nthreads);
    static std::shared_ptr<QTensor> from_data(const CudaDevice &dev, const void *bytes, int64_t nbytes,
                                              GgmlDType dtype, std::vector<int64_t> shape);
    GgmlDType dtype() const { return storage_->dtype(); }
    const std::vector<int64_t> &shape() const { return shape_; }
    int64_t elem_count() const;
    const QCudaStorage &storage() const { return *storage_; }

  private:
    std::unique_ptr<QCudaStorage> storage_;
    std::vector<int64_t> shape_;
};

class QMatMul {
  public:
    explicit QMatMul(std::shared_ptr<QTensor> w) : w_(std::move(w)) {}
    static QMatMul from_arc(std::shared_ptr<QTensor> w) { return QMatMul(std::move(w)); }  // mod.rs:1714-1729
    // Module::forward (mod.rs:2022-2026): xs dims [.., k] contiguous f32 on device -> y dims [.., n]
    void forward(const float *xs, const std::vector<int64_t> &xs_dims, float *y) const;
    // mod.rs:2105-2155: silu(W.x) / gate <- gate * (W.x) on the GEMV's store.  false where the store block does not
    // serve (more than 8 rows): the caller composes, as with the reference's None.
    bool forward_silu(const float *xs, const std::vector<int64_t> &xs_dims, float *y) const;
    bool forward_mul_into(const float *xs, const std::vector<int64_t> &xs_dims, float *gate) const;
    const QTensor &weight() const { return *w_; }

  private:
    bool forward_store(const float *xs, const std::vector<int64_t> &xs_dims, float *y, int store) const;
    std::shared_ptr<QTensor> w_;
};

}  // namespace host
}  // namespace lloom
