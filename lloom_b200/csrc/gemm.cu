// Prefill GEMM (m > 8): the tcgen05 kernels' translation unit -- planning of the operand images, their build
// kernels and the launches.  Q4_K: gemm_q4k.cuh; Q8_0 and Q6_K: gemm_planes.cuh.
#include "gemm.h"

#include <mutex>

#include "gemm_planes.cuh"

namespace lloom {

LLOOM_TU_REGISTER()

namespace {

using CfgQ8_0 = PlanesCfg<32, 1, 128>;
using CfgQ6K = PlanesCfg<256, 2, 256>;      // more than 128 activation rows
using CfgQ6KSmall = PlanesCfg<256, 2, 128>;  // up to 128: a 256-row tile would fetch and multiply empty rows

// activation rows per tile of the Q6_K GEMM for a call of m rows
int q6k_bm(int64_t m) { return m <= 128 ? CfgQ6KSmall::kBM : CfgQ6K::kBM; }

// Weight images of more than this are built and consumed slab by slab (whole 128-row tiles), so that the
// caller's workspace stays bounded whatever the matrix (a Q6_K lm_head image is 2.1 GB).
constexpr int64_t kSlabImageBytes = 256ll << 20;

struct OnceSmem {  // dynamic shared memory opt-in, per device
    std::mutex mu;
    bool done[64] = {false};
};

template <class Kern>
cudaError_t opt_in_smem(Kern kern, OnceSmem &st, int bytes) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    std::lock_guard<std::mutex> lock(st.mu);
    if (st.done[dev]) return cudaSuccess;
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e == cudaSuccess) st.done[dev] = true;
    return e;
}

int64_t image_bytes_for_rows(int w_dtype, int64_t rows, int64_t k) {
    switch (w_dtype) {
    case LLOOM_Q4_K:
    case LLOOM_Q5_K: return gemm_weight_layout(rows, k).total;
    case LLOOM_Q8_0:
    case LLOOM_Q4_0:
    case LLOOM_Q5_0: return planes_weight_bytes(rows, k, 1);
    case LLOOM_Q6_K: return planes_weight_bytes(rows, k, 2);
    }
    return 0;
}

int64_t act_image_bytes(int w_dtype, int64_t m, int64_t k) {
    switch (w_dtype) {
    case LLOOM_Q4_K:
    case LLOOM_Q5_K: return gemm_act_layout(m, k).total;
    case LLOOM_Q8_0:
    case LLOOM_Q4_0:
    case LLOOM_Q5_0: return planes_act_layout(m, k, 32, CfgQ8_0::kBM).total;
    case LLOOM_Q6_K: return planes_act_layout(m, k, 256, q6k_bm(m)).total;
    }
    return 0;
}

constexpr int kExpandSmem = 4 * kGemmAtomBytes + kGemmMinBytes;

cudaError_t build_image(int w_dtype, const uint8_t *w, int64_t rows, int64_t k, uint8_t *image, cudaStream_t stream) {
    const int64_t nt = (rows + kGemmBN - 1) / kGemmBN;
    if (w_dtype == LLOOM_Q4_K) {
        static OnceSmem once;
        cudaError_t e = opt_in_smem(gemm_expand_kernel<false>, once, kExpandSmem);
        if (e != cudaSuccess) return e;
        gemm_expand_kernel<false><<<(unsigned)(nt * (k / 256)), 128, kExpandSmem, stream>>>(w, (int)rows, (int)k, image);
    } else if (w_dtype == LLOOM_Q5_K) {
        static OnceSmem once;
        cudaError_t e = opt_in_smem(gemm_expand_kernel<true>, once, kExpandSmem);
        if (e != cudaSuccess) return e;
        gemm_expand_kernel<true><<<(unsigned)(nt * (k / 256)), 128, kExpandSmem, stream>>>(w, (int)rows, (int)k, image);
    } else if (w_dtype == LLOOM_Q8_0) {
        planes_expand_q8_0_kernel<<<(unsigned)(nt * (k / 64)), 128, 0, stream>>>(w, 0, (int)rows, (int)k, image);
    } else if (w_dtype == LLOOM_Q4_0) {
        planes_expand_q4or5_0_kernel<false><<<(unsigned)(nt * (k / 64)), 128, 0, stream>>>(w, 0, (int)rows, (int)k, image);
    } else if (w_dtype == LLOOM_Q5_0) {
        planes_expand_q4or5_0_kernel<true><<<(unsigned)(nt * (k / 64)), 128, 0, stream>>>(w, 0, (int)rows, (int)k, image);
    } else if (w_dtype == LLOOM_Q6_K) {
        planes_expand_q6k_kernel<<<(unsigned)(nt * (k / 64)), 128, 0, stream>>>(w, 0, (int)rows, (int)k, image);
    } else {
        return cudaErrorInvalidValue;
    }
    return cudaGetLastError();
}

template <class Cfg>
cudaError_t launch_planes(const PlanesParams &p, cudaStream_t stream) {
    static OnceSmem once;
    cudaError_t e = opt_in_smem(gemm_planes_kernel<Cfg>, once, Cfg::kSmemBytes);
    if (e != cudaSuccess) return e;
    gemm_planes_kernel<Cfg><<<(unsigned)(p.n_tiles * p.m_tiles), Cfg::kThreads, Cfg::kSmemBytes, stream>>>(p);
    return cudaGetLastError();
}

}  // namespace

bool gemm_supported(int w_dtype, int64_t m, int64_t k, int max_smem) {
    if (m <= 8) return false;
    switch (w_dtype) {
    case LLOOM_Q4_K:
    case LLOOM_Q5_K: return k % 256 == 0 && kGemmSmemBytes <= max_smem;
    case LLOOM_Q6_K: return k % 256 == 0 && CfgQ6K::kSmemBytes <= max_smem && CfgQ6KSmall::kSmemBytes <= max_smem;
    case LLOOM_Q8_0:
    case LLOOM_Q4_0:
    case LLOOM_Q5_0: return k % 128 == 0 && CfgQ8_0::kSmemBytes <= max_smem;  // a pipeline stage is 128 of K
    }
    return false;
}

int64_t gemm_weight_image_bytes(int w_dtype, int64_t n, int64_t k) { return image_bytes_for_rows(w_dtype, n, k); }

int64_t gemm_slab_rows(int w_dtype, int64_t n, int64_t k) {
    const int64_t per_tile = image_bytes_for_rows(w_dtype, kGemmBN, k);
    if (per_tile <= 0) return 0;
    int64_t tiles = kSlabImageBytes / per_tile;
    if (tiles < 1) tiles = 1;
    const int64_t all = (n + kGemmBN - 1) / kGemmBN;
    return (tiles < all ? tiles : all) * kGemmBN;
}

int64_t gemm_scratch_bytes(int w_dtype, int64_t m, int64_t n, int64_t k, bool have_image) {
    if (m <= 8) return 0;
    const int64_t act = act_image_bytes(w_dtype, m, k);
    if (act <= 0) return 0;
    if (have_image) return act;
    const int64_t rows = gemm_slab_rows(w_dtype, n, k);
    return act + (image_bytes_for_rows(w_dtype, rows, k) + 255) / 256 * 256;
}

cudaError_t gemm_weight_image_build(int w_dtype, const void *w, int64_t n, int64_t k, void *image, cudaStream_t stream) {
    return build_image(w_dtype, (const uint8_t *)w, n, k, (uint8_t *)image, stream);
}

bool gemm_takes_f32(int w_dtype) {
    return w_dtype == LLOOM_Q4_K || w_dtype == LLOOM_Q5_K || w_dtype == LLOOM_Q6_K || w_dtype == LLOOM_Q8_0 || w_dtype == LLOOM_Q4_0 ||
           w_dtype == LLOOM_Q5_0;
}

cudaError_t gemm_forward(int w_dtype, const void *w_blocks, const void *w_image, const void *act, const float *x, float *y,
                         int64_t m, int64_t n, int64_t k, int64_t ldy, void *scratch, cudaStream_t stream) {
    if ((act == nullptr) == (x == nullptr) || (x && !gemm_takes_f32(w_dtype))) return cudaErrorInvalidValue;
    const uint8_t *w = (const uint8_t *)w_blocks;
    uint8_t *act_img = (uint8_t *)scratch;
    const int64_t mt = w_dtype == LLOOM_Q6_K ? (m + q6k_bm(m) - 1) / q6k_bm(m) : gemm_m_tiles(m);
    // activation side, once per call
    const bool q4k_frame = w_dtype == LLOOM_Q4_K || w_dtype == LLOOM_Q5_K;
    const bool q8_0_frame = w_dtype == LLOOM_Q8_0 || w_dtype == LLOOM_Q4_0 || w_dtype == LLOOM_Q5_0;
    if (q4k_frame && x) {
        gemm_prep_f32_kernel<<<(unsigned)(mt * kGemmBM * (k / 256) / 8), 256, 0, stream>>>(x, (int)m, (int)k, act_img);
    } else if (q4k_frame) {
        gemm_prep_kernel<<<(unsigned)(mt * (k / 256) * 4), 256, 0, stream>>>((const uint8_t *)act, (int)m, (int)k, act_img);
    } else if (q8_0_frame && x) {
        planes_prep_f32_kernel<true, CfgQ8_0::kBM><<<(unsigned)(mt * CfgQ8_0::kBM * ((k + 255) / 256) / 8), 256, 0, stream>>>(x, (int)m, (int)k, act_img);
    } else if (w_dtype == LLOOM_Q6_K && x) {
        if (q6k_bm(m) == CfgQ6K::kBM)
            planes_prep_f32_kernel<false, CfgQ6K::kBM><<<(unsigned)(mt * CfgQ6K::kBM * (k / 256) / 8), 256, 0, stream>>>(x, (int)m, (int)k, act_img);
        else
            planes_prep_f32_kernel<false, CfgQ6KSmall::kBM><<<(unsigned)(mt * CfgQ6KSmall::kBM * (k / 256) / 8), 256, 0, stream>>>(x, (int)m, (int)k, act_img);
    } else if (q8_0_frame) {
        planes_prep_kernel<true, CfgQ8_0::kBM><<<(unsigned)(mt * (k / 64)), CfgQ8_0::kBM, 0, stream>>>((const uint8_t *)act, (int)m, (int)k, act_img);
    } else if (w_dtype == LLOOM_Q6_K) {
        if (q6k_bm(m) == CfgQ6K::kBM)
            planes_prep_kernel<false, CfgQ6K::kBM><<<(unsigned)(mt * (k / 64)), CfgQ6K::kBM, 0, stream>>>((const uint8_t *)act, (int)m, (int)k, act_img);
        else
            planes_prep_kernel<false, CfgQ6KSmall::kBM><<<(unsigned)(mt * (k / 64)), CfgQ6KSmall::kBM, 0, stream>>>((const uint8_t *)act, (int)m, (int)k, act_img);
    } else {
        return cudaErrorInvalidValue;
    }
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    const int64_t row_bytes = k / lloom_b200_block_elems(w_dtype) * lloom_b200_block_bytes(w_dtype);
    const int64_t slab = w_image ? n : gemm_slab_rows(w_dtype, n, k);
    uint8_t *slab_img = act_img + act_image_bytes(w_dtype, m, k);
    for (int64_t row0 = 0; row0 < n; row0 += slab) {
        const int64_t rows = n - row0 < slab ? n - row0 : slab;
        const uint8_t *w_slab = w + row0 * row_bytes;
        const uint8_t *img = (const uint8_t *)w_image;
        if (!img) {  // same stream: the previous slab's GEMM has read the buffer before this build overwrites it
            e = build_image(w_dtype, w_slab, rows, k, slab_img, stream);
            if (e != cudaSuccess) return e;
            img = slab_img;
        }
        const int n_tiles = (int)((rows + kGemmBN - 1) / kGemmBN);
        if (q4k_frame) {
            static OnceSmem once;
            e = opt_in_smem(gemm_q4k_kernel, once, kGemmSmemBytes);
            if (e != cudaSuccess) return e;
            GemmParams p;
            p.w = w_slab;
            p.act_img = act_img;
            p.w_img = img;
            p.y = y + row0;
            p.ldy = ldy;
            p.row_bytes = row_bytes;
            p.m = (int)m;
            p.n = (int)rows;
            p.k = (int)k;
            p.n_tiles = n_tiles;
            p.m_tiles = (int)mt;
            p.blk_bytes = (int)lloom_b200_block_bytes(w_dtype);
            gemm_q4k_kernel<<<(unsigned)(n_tiles * mt), kQ4kThreads, kGemmSmemBytes, stream>>>(p);
            e = cudaGetLastError();
        } else {
            PlanesParams p;
            p.w = w_slab;
            p.act_img = act_img;
            p.w_img = img;
            p.y = y + row0;
            p.ldy = ldy;
            p.row_bytes = row_bytes;
            p.row0 = 0;
            p.m = (int)m;
            p.n_end = (int)rows;
            p.k = (int)k;
            p.n_tiles = n_tiles;
            p.m_tiles = (int)mt;
            if (q8_0_frame) {
                p.scale_stride = (int)lloom_b200_block_bytes(w_dtype);  // the f16 scale opens every 32-element block
                p.scale_off = 0;
                e = launch_planes<CfgQ8_0>(p, stream);
            } else {
                p.scale_stride = Q6K_BYTES;
                p.scale_off = 208;
                e = q6k_bm(m) == CfgQ6K::kBM ? launch_planes<CfgQ6K>(p, stream) : launch_planes<CfgQ6KSmall>(p, stream);
            }
        }
        if (e != cudaSuccess) return e;
    }
    return cudaSuccess;
}

}  // namespace lloom
