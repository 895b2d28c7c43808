// C ABI of the library (see include/lloom_b200.h).  One translation unit: the kernels live in the
// headers included below.  No entry point allocates, frees or synchronises.
#include "common.cuh"
#include "dequant.cuh"
#include "gemm_q4k_2sm.cuh"
#include "gemv.cuh"
#include "gemv_mma.cuh"
#include "quantize_act.cuh"

#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>

namespace lloom {

static thread_local int t_last_cuda_error = 0;

static int launch_status(cudaError_t e) {
    if (e == cudaSuccess) return LLOOM_OK;
    t_last_cuda_error = (int)e;
    return LLOOM_ERR_LAUNCH;
}

static bool supported_weight(int dtype) { return dtype == LLOOM_Q8_0 || dtype == LLOOM_Q4_K || dtype == LLOOM_Q6_K; }

struct DeviceInfo {
    int sm_count = 0;
    int max_smem_optin = 0;   // per block
    int smem_per_sm = 0;      // per multiprocessor
    int smem_reserved = 0;    // per block, taken by the driver
    int cc_major = 0;
    bool ok = false;
};

// Launch overlap (programmatic dependent launch); off until lloom_b200_set_launch_overlap(1).
static std::atomic<int> g_launch_overlap{0};

// Per-device attributes, queried once (the reference caches the same facts, fast_mmq.rs device-info cache).
static int device_info(DeviceInfo &out) {
    static std::mutex mu;
    static DeviceInfo cache[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return LLOOM_ERR_DEVICE;
    std::lock_guard<std::mutex> lock(mu);
    DeviceInfo &c = cache[dev];
    if (!c.ok) {
        if (cudaDeviceGetAttribute(&c.sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return LLOOM_ERR_DEVICE;
        if (cudaDeviceGetAttribute(&c.max_smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev) != cudaSuccess)
            return LLOOM_ERR_DEVICE;
        if (cudaDeviceGetAttribute(&c.smem_per_sm, cudaDevAttrMaxSharedMemoryPerMultiprocessor, dev) != cudaSuccess)
            return LLOOM_ERR_DEVICE;
        if (cudaDeviceGetAttribute(&c.smem_reserved, cudaDevAttrReservedSharedMemoryPerBlock, dev) != cudaSuccess)
            return LLOOM_ERR_DEVICE;
        if (cudaDeviceGetAttribute(&c.cc_major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) return LLOOM_ERR_DEVICE;
        if (c.cc_major != 10) return LLOOM_ERR_DEVICE;  // sm_100a code only
        c.ok = true;
    }
    out = c;
    return LLOOM_OK;
}

static int64_t weight_row_bytes(int dtype, int64_t k) {
    return k / lloom_b200_block_elems(dtype) * lloom_b200_block_bytes(dtype);
}

// ---- GEMV launch planning ----

// EPI = 1 instances carry the store blocks and the fused gather; the plain forward uses the EPI = 0 instances.
static bool gemv_needs_epi(const GemvParams &p) { return p.n_peers != 0 || p.store_mode != LLOOM_STORE_PLAIN; }

template <class Item, int M, int RW, int CW, bool PIECES, int EPI>
static cudaError_t launch_gemv_inst2(const GemvParams &p, int grid, int smem, bool overlap, cudaStream_t stream) {
    auto kern = gemv_kernel<Item, M, RW, CW, PIECES, EPI>;
    static int configured_smem[64] = {0};
    int dev = 0;
    cudaGetDevice(&dev);
    if (configured_smem[dev] < smem) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return e;
        // ask for the largest shared-memory carve-out, so that two half-size CTAs really fit side by side
        e = cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        if (e != cudaSuccess) return e;
        configured_smem[dev] = smem;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(32u * (unsigned)(p.n_cwarps + 1));
    cfg.dynamicSmemBytes = (size_t)smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = overlap ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, p);
}

template <class Item, int M, int RW, int CW = 8, bool PIECES = false>
static cudaError_t launch_gemv_inst(const GemvParams &p, int grid, int smem, bool overlap, cudaStream_t stream) {
    if (gemv_needs_epi(p)) return launch_gemv_inst2<Item, M, RW, CW, PIECES, 1>(p, grid, smem, overlap, stream);
    return launch_gemv_inst2<Item, M, RW, CW, PIECES, 0>(p, grid, smem, overlap, stream);
}

template <class Fmt, int RW>
static cudaError_t launch_gemv_m(const GemvParams &p, int grid, int smem, bool overlap, cudaStream_t stream) {
    if (RW == 1 && p.nchunks > 1) {  // rows cut into pieces: side-by-side shapes with eight consumer warps, m <= 2 only
        if (p.n_cwarps > 8) return cudaErrorInvalidValue;
        if (p.m == 1) return launch_gemv_inst<Fmt, 1, 1, 8, true>(p, grid, smem, overlap, stream);
        if (p.m == 2) return launch_gemv_inst<Fmt, 2, 1, 8, true>(p, grid, smem, overlap, stream);
        return cudaErrorInvalidValue;
    }
    if (RW == 1 && p.n_cwarps > 8) {  // twelve-consumer-warp instances exist for m <= 2 only
        if (p.m == 1) return launch_gemv_inst<Fmt, 1, 1, 12>(p, grid, smem, overlap, stream);
        if (p.m == 2) return launch_gemv_inst<Fmt, 2, 1, 12>(p, grid, smem, overlap, stream);
        return cudaErrorInvalidValue;
    }
    switch (p.m) {
    case 1: return launch_gemv_inst<Fmt, 1, RW>(p, grid, smem, overlap, stream);
    case 2: return launch_gemv_inst<Fmt, 2, RW>(p, grid, smem, overlap, stream);
    case 3: return launch_gemv_inst<Fmt, 3, RW>(p, grid, smem, overlap, stream);
    case 4: return launch_gemv_inst<Fmt, 4, RW>(p, grid, smem, overlap, stream);
    case 5: return launch_gemv_inst<Fmt, 5, RW>(p, grid, smem, overlap, stream);
    case 6: return launch_gemv_inst<Fmt, 6, RW>(p, grid, smem, overlap, stream);
    case 7: return launch_gemv_inst<Fmt, 7, RW>(p, grid, smem, overlap, stream);
    case 8: return launch_gemv_inst<Fmt, 8, RW>(p, grid, smem, overlap, stream);
    }
    return cudaErrorInvalidValue;
}

template <int RW>
static cudaError_t launch_gemv_fmt(const GemvParams &p, int grid, int smem, bool overlap, cudaStream_t stream) {
    switch (p.w_dtype) {
    case LLOOM_Q8_0: return launch_gemv_m<FmtQ8_0, RW>(p, grid, smem, overlap, stream);
    case LLOOM_Q4_K: return launch_gemv_m<FmtQ4K, RW>(p, grid, smem, overlap, stream);
    case LLOOM_Q6_K: return launch_gemv_m<FmtQ6K, RW>(p, grid, smem, overlap, stream);
    }
    return cudaErrorInvalidValue;
}

// Development knob: LLOOM_GEMV_SHAPE="<consumer warps>,<rows per lane>" pins the tile shape.
static bool gemv_shape_override(int &cw, int &rw) {
    static int cached = -1, ccw = 0, crw = 0;
    if (cached < 0) {
        const char *e = getenv("LLOOM_GEMV_SHAPE");
        cached = (e && sscanf(e, "%d,%d", &ccw, &crw) == 2 && ccw >= 1 && ccw <= 12 && (crw == 1 || crw == 2) &&
                  (ccw <= 8 || crw == 1))
                     ? 1
                     : 0;
    }
    cw = ccw;
    rw = crw;
    return cached == 1;
}

template <int SPLIT, int EPI>
static cudaError_t launch_gemv_mma_inst(const GemvParams &p, int grid, int smem, bool overlap, cudaStream_t stream) {
    auto kern = gemv_mma_q4k_kernel<SPLIT, EPI>;
    static int configured_smem[64] = {0};
    int dev = 0;
    cudaGetDevice(&dev);
    if (configured_smem[dev] < smem) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return e;
        configured_smem[dev] = smem;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(32u * (kMmaWarps + 1));
    cfg.dynamicSmemBytes = (size_t)smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = overlap ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, p);
}

static cudaError_t launch_gemv_mma(const GemvParams &p, int grid, int smem, bool overlap, cudaStream_t stream) {
    // whole rows per stage: four teams of four warps, a tile each; rows cut into pieces: one team of sixteen, so
    // that a piece is consumed (and its stage handed back) as fast as possible
    if (gemv_needs_epi(p)) {
        if (p.nchunks > 1) return launch_gemv_mma_inst<16, 1>(p, grid, smem, overlap, stream);
        return launch_gemv_mma_inst<4, 1>(p, grid, smem, overlap, stream);
    }
    if (p.nchunks > 1) return launch_gemv_mma_inst<16, 0>(p, grid, smem, overlap, stream);
    return launch_gemv_mma_inst<4, 0>(p, grid, smem, overlap, stream);
}

// Development knob: LLOOM_GEMV_MMA=0 keeps 2 <= m <= 8 on the dp4a kernel.
static bool gemv_mma_enabled() {
    static int cached = -1;
    if (cached < 0) {
        const char *e = getenv("LLOOM_GEMV_MMA");
        cached = (e && e[0] == '0') ? 0 : 1;
    }
    return cached == 1;
}

// Whether the tensor-core GEMV quantizes the activations itself (as its prologue): up to two rows, and few enough
// 256-element blocks that a CTA's sixteen warps get through them in two rounds.
static bool gemv_mma_fused(int64_t m, int64_t k) { return m <= kMmaFusedMaxM && m * (k / QK_K) <= 32; }

// Shared-memory plan of the tensor-core GEMV: a stage holds `chunk_sb` superblocks of 16 rows -- whole rows when two
// such stages fit beside the activation planes, else the rows are cut into `nchunks` pieces of equal length
// (K = 14336: planes and whole-row stages would need 250 KB).
struct MmaPlan {
    bool ok = false;
    int chunk_sb = 0, nchunks = 0;
    int64_t bar_bytes = 0, row_pitch = 0, stage = 0, room = 0;
};

static MmaPlan gemv_mma_plan(const DeviceInfo &di, int w_dtype, int64_t m, int64_t n, int64_t k) {
    MmaPlan pl;
    if (w_dtype != LLOOM_Q4_K || m < 2 || m > 8 || !gemv_mma_enabled()) return pl;
    const int64_t nb = k / QK_K;
    const int64_t total = (n + kMmaTileRows - 1) / kMmaTileRows;
    const int64_t grid = total < di.sm_count ? total : di.sm_count;
    const int64_t tiles = (total + grid - 1) / grid;
    for (int64_t nchunks = 1; nchunks <= nb && nchunks <= 16; ++nchunks) {
        const int64_t chunk = (nb + nchunks - 1) / nchunks;
        const int64_t bars = round16(tiles * nchunks * 8);
        if (tiles * nchunks > kMmaMaxTiles) return pl;
        const int64_t pitch = bank_pitch(chunk * Q4K_BYTES, 8);
        const int64_t stage = (int64_t)kMmaTileRows * pitch;
        const int64_t room = (int64_t)di.max_smem_optin - kMmaBarBytes - kMmaRedBytes - bars - mma_act_bytes(m, k);
        if (room >= 2 * stage) {
            // (a single row stays on the dp4a kernel even at K = 14336, where this kernel alone would be faster --
            // 11.8 us against 14.9 us: the quantizer launch in front of it breaks the chain of overlapping
            // launches, and a 225-matmul decode step got 8 % slower with it)
            pl.ok = true;
            pl.chunk_sb = (int)chunk;
            pl.nchunks = (int)((nb + chunk - 1) / chunk);
            pl.bar_bytes = bars;
            pl.row_pitch = pitch;
            pl.stage = stage;
            pl.room = room;
            return pl;
        }
    }
    return pl;
}

// Whether the tensor-core GEMV takes this shape: Q4_K, 2..8 activation rows, a plan exists.
static bool gemv_mma_fits(const DeviceInfo &di, int w_dtype, int64_t m, int64_t n, int64_t k) {
    return gemv_mma_plan(di, w_dtype, m, n, k).ok;
}

// Launches the GEMV.  Exactly one of `act` (canonical activation blocks) and `x` (f32 activations,
// quantized in the kernel's prologue) is non-null.
struct PeerFlags {  // one flag array per GPU: kMaxPeers slots written by the peers + this GPU's call counter
    unsigned int *f[kMaxPeers];
};

struct PeerOut {  // fused gather: output buffers of all GPUs (own included), already offset to this shard's column
    int n = 0;
    float *y[kMaxPeers] = {};
    int store = LLOOM_STORE_PLAIN;  // block on the store (also used alone, with n == 0)
};

static int gemv_launch(int w_dtype, const void *w, const void *act, const float *x, float *y, int64_t m, int64_t n,
                       int64_t k, int64_t ldy, cudaStream_t stream, bool act_planes = false,
                       const PeerOut *peers = nullptr) {
    DeviceInfo di;
    int rc = device_info(di);
    if (rc != LLOOM_OK) return rc;
    if (act_planes && !gemv_mma_fits(di, w_dtype, m, n, k)) return LLOOM_ERR_SHAPE;
    GemvParams p;
    p.w = (const uint8_t *)w;
    p.act = (const uint8_t *)act;
    p.x = x;
    p.y = y;
    p.ldy = ldy;
    p.row_bytes = weight_row_bytes(w_dtype, k);
    p.w_bytes = n * p.row_bytes;
    p.n = (int)n;
    p.k = (int)k;
    p.m = (int)m;
    p.w_dtype = w_dtype;
    p.act_bytes = (int)act_plane_bytes(w_dtype, m, k);
    p.row_pitch = 0;
    p.act_pitch = 0;
    p.act_planes = 0;
    p.tile_bar_bytes = 0;
    p.chunk_sb = 0;
    p.nchunks = 1;
    p.chunk_units = 0;
    p.unit_bytes = w_dtype == LLOOM_Q4_K ? Q4K_BYTES : w_dtype == LLOOM_Q6_K ? Q6K_BYTES : 2 * Q8_0_BYTES;
    p.n_peers = peers ? peers->n : 0;
    p.out_bytes = 0;
    p.out_pitch = 0;
    p.store_mode = peers ? peers->store : LLOOM_STORE_PLAIN;
    for (int g = 0; g < kMaxPeers; ++g) p.y_peer[g] = (peers && g < peers->n) ? peers->y[g] : nullptr;
    // lanes per row: one lane per unit (superblock, or pair of Q8_0 blocks), rounded up to a power of two
    const int64_t units = k / (w_dtype == LLOOM_Q8_0 ? 64 : 256);
    int lpr_log2 = 0;
    while ((1 << lpr_log2) < units && lpr_log2 < 5) ++lpr_log2;
    p.lpr_log2 = lpr_log2;
    const int groups = 32 >> lpr_log2;
    // A stage holds one tile of rows, widened to 16-byte boundaries, plus slack for the word-wide
    // over-read of the unaligned loaders.
    const int64_t pad = (p.row_bytes % 16 == 0) ? 16 : 48;
    int grid = di.sm_count;
    if ((int64_t)grid > n) grid = (int)n;
    const bool overlap_on = g_launch_overlap.load(std::memory_order_relaxed) != 0;
    // Fused gather: room to stage a CTA's output rows (so that they leave for the peers in whole lines), if small
    auto staging = [&](int64_t rows_per_cta, int &pitch) -> int64_t {
        if (p.n_peers == 0) return 0;
        pitch = (int)((rows_per_cta + 3) / 4 * 4);
        const int64_t bytes = (int64_t)m * pitch * 4;
        return bytes <= 32 * 1024 ? bytes : 0;
    };
    // 3..8 activation rows of Q4_K: the tensor-core kernel, if two 16-row stages fit beside the activations
    const MmaPlan plan = gemv_mma_plan(di, w_dtype, m, n, k);
    if (plan.ok && (x == nullptr || gemv_mma_fused(m, k))) {
        const int64_t stage = plan.stage;
        p.act_bytes = (int)mma_act_bytes(m, k);
        p.act_pitch = (int)mma_act_pitch(k);
        p.act_planes = act_planes ? 1 : 0;
        p.row_pitch = (int)plan.row_pitch;
        p.tile_bar_bytes = (int)plan.bar_bytes;
        p.chunk_sb = plan.chunk_sb;
        p.nchunks = plan.nchunks;
        const int64_t room = plan.room;
        {
            const int64_t total_tiles = (n + kMmaTileRows - 1) / kMmaTileRows;
            const int64_t g = total_tiles < grid ? total_tiles : grid;
            int pitch = 0;
            const int64_t want = staging((total_tiles + g - 1) / g * kMmaTileRows, pitch);
            if (want > 0 && room - want >= 2 * stage) {
                p.out_bytes = (int)want;
                p.out_pitch = pitch;
            }
        }
        int64_t stages = (room - p.out_bytes) / stage;
        if (stages > kMaxStages) stages = kMaxStages;
        p.n_cwarps = kMmaWarps;
        p.stages = (int)stages;
        p.stage_bytes = (int)stage;
        const int smem = kMmaBarBytes + kMmaRedBytes + p.tile_bar_bytes + p.act_bytes + p.out_bytes + (int)(stages * stage);
        const int64_t total_tiles = (n + kMmaTileRows - 1) / kMmaTileRows;
        if (grid > total_tiles) grid = (int)total_tiles;
        return launch_status(launch_gemv_mma(p, grid, smem, overlap_on, stream));
    }
    // Tile shapes {consumer warps, rows per lane}, widest first (after an optional pinned shape); the
    // first that leaves room for at least two stages wins.  With launch overlap on, m <= 2 tries shapes
    // that fit two CTAs per SM first, so that consecutive launches can sit side by side.
    struct Shape { int cw, rw; bool half; };
    Shape shapes[12];
    int ns = 0, ocw = 0, orw = 0;
    const bool overlap = g_launch_overlap.load(std::memory_order_relaxed) != 0;
    if (gemv_shape_override(ocw, orw)) shapes[ns++] = {ocw, orw, overlap && orw == 1};
    if (overlap && m <= 2) {  // HBM-bound batch sizes only: wider batches need the registers and the row tiling
        // twelve consumer warps pay off for Q8_0 (cheap units, more of them per row); the k-quants are best at eight
        if (w_dtype == LLOOM_Q8_0) shapes[ns++] = {12, 1, true};
        const int half_cw[4] = {8, 4, 2, 1};
        for (int c : half_cw) shapes[ns++] = {c, 1, true};
    }
    const int full[5][2] = {{8, 2}, {8, 1}, {4, 1}, {2, 1}, {1, 1}};
    for (auto &f : full) shapes[ns++] = {f[0], f[1], false};
    int out_pitch = 0;
    const int64_t out_want = staging((n + grid - 1) / grid, out_pitch);
    for (int si = 0; si < ns; ++si) {
        const int cw = shapes[si].cw, rw = shapes[si].rw;
        const int64_t per_block = shapes[si].half ? (int64_t)(di.smem_per_sm - 2 * di.smem_reserved) / 2 / 16 * 16
                                                  : (int64_t)di.max_smem_optin;
        int64_t budget = per_block - 128 - p.act_bytes;
        int64_t stage = round16((int64_t)cw * groups * rw * p.row_bytes + pad);
        p.nchunks = 1;
        p.chunk_units = 0;
        p.lpr_log2 = lpr_log2;
        if (budget < 2 * stage) {
            // Long rows in a side-by-side shape: cut the rows into pieces of 16 units (32 for Q8_0), so that a stage
            // is 16 (8) rows x one piece -- the tile the kernel streams at K = 4096 -- instead of giving up the
            // overlap between consecutive launches for a one-CTA-per-SM shape.
            if (!shapes[si].half || cw > 8 || p.row_bytes % 16 != 0) continue;
            const int cu = w_dtype == LLOOM_Q8_0 ? 32 : 16;
            if (units <= cu || ((int64_t)cu * p.unit_bytes) % 16 != 0) continue;
            const int cl = w_dtype == LLOOM_Q8_0 ? 5 : 4;
            const int64_t pstage = round16((int64_t)cw * (32 >> cl) * rw * cu * p.unit_bytes + pad);
            if (budget < 2 * pstage) continue;
            stage = pstage;
            p.nchunks = (int)((units + cu - 1) / cu);
            p.chunk_units = cu;
            p.lpr_log2 = cl;
        }
        p.out_bytes = 0;
        p.out_pitch = 0;
        if (out_want > 0 && budget - out_want >= 2 * stage) {
            p.out_bytes = (int)out_want;
            p.out_pitch = out_pitch;
            budget -= out_want;
        }
        int64_t stages = budget / stage;
        if (stages > kMaxStages) stages = kMaxStages;
        p.n_cwarps = cw;
        p.stages = (int)stages;
        p.stage_bytes = (int)stage;
        const int smem = 128 + p.act_bytes + p.out_bytes + (int)(stages * stage);
        cudaError_t e = (rw == 2) ? launch_gemv_fmt<2>(p, grid, smem, overlap, stream)
                                  : launch_gemv_fmt<1>(p, grid, smem, overlap, stream);
        return launch_status(e);
    }
    return LLOOM_ERR_SHAPE;  // one row of weights plus the activations does not fit in shared memory
}

static int check_common(int w_dtype, int64_t m, int64_t n, int64_t k) {
    if (!supported_weight(w_dtype)) return LLOOM_ERR_DTYPE;
    if (m <= 0 || n <= 0 || k <= 0) return LLOOM_ERR_SHAPE;
    if (k % lloom_b200_block_elems(w_dtype) != 0) return LLOOM_ERR_SHAPE;
    if (k % 64 != 0) return LLOOM_ERR_SHAPE;  // kernels work on 64-element items
    if (m > (1 << 24) || n > (1 << 30) || k > (1 << 24)) return LLOOM_ERR_SHAPE;
    return LLOOM_OK;
}

static bool aligned(const void *p, uintptr_t a) { return ((uintptr_t)p & (a - 1)) == 0; }

// ---- built-in scratch of lloom_b200_qmatmul_fwd_static ----
// Lives in every device's copy of this module until the process exits.  In host code the name
// below is only a host-side stand-in for the symbol, never a device address: the address a kernel
// may use is the one cudaGetSymbolAddress returns, looked up once per device.
static __device__ __align__(256) uint8_t g_static_scratch[LLOOM_B200_STATIC_SCRATCH_BYTES];

static int static_scratch_ptr(void **out) {
    static std::mutex mu;
    static void *cache[64] = {nullptr};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return LLOOM_ERR_DEVICE;
    std::lock_guard<std::mutex> lock(mu);
    if (!cache[dev]) {
        void *p = nullptr;
        const cudaError_t e = cudaGetSymbolAddress(&p, g_static_scratch);  // `dev` is current here
        if (e != cudaSuccess) return launch_status(e);
        if (!p) return LLOOM_ERR_DEVICE;
        cache[dev] = p;
    }
    *out = cache[dev];
    return LLOOM_OK;
}

// Decode forward (m <= 8) after argument checks: quantizer + GEMV, outputs to `y` or to the peers' buffers.
static int decode_fwd(int w_dtype, const void *w_blocks, const float *x, float *y, int64_t m, int64_t n, int64_t k,
                      int64_t ldy, void *workspace, int64_t need, void *stream, const PeerOut *peers) {
    int rc;
    {
        DeviceInfo di;
        rc = device_info(di);
        if (rc != LLOOM_OK) return rc;
        const bool mma = gemv_mma_fits(di, w_dtype, m, n, k);
        // up to two rows: one launch, the activation quantizer is the GEMV's prologue (the workspace stays
        // unused).  From three rows on, every CTA re-quantizing all rows costs more than one small kernel does.
        if ((m <= 2 && !mma) || (mma && gemv_mma_fused(m, k)))
            return gemv_launch(w_dtype, w_blocks, nullptr, x, y, m, n, k, ldy, (cudaStream_t)stream, false, peers);
        // Q4_K batches for the tensor-core GEMV: the quantizer writes the kernel's own activation image (same
        // codes, scales and sums as the canonical blocks, laid out for its fragment loads)
        if (mma && mma_act_bytes(m, k) <= need) {
            const int nb = (int)(k / QK_K);
            quantize_q8k_planes_kernel<<<(unsigned)ceil_div64(m * nb * 32, 256), 256, 0, (cudaStream_t)stream>>>(
                x, (uint8_t *)workspace, (int)m, nb, (int)mma_act_pitch(k));
            rc = launch_status(cudaGetLastError());
            if (rc != LLOOM_OK) return rc;
            return gemv_launch(w_dtype, w_blocks, workspace, nullptr, y, m, n, k, ldy, (cudaStream_t)stream, true, peers);
        }
    }
    rc = lloom_b200_quantize_act(w_dtype, x, m, k, workspace, stream);
    if (rc != LLOOM_OK) return rc;
    return gemv_launch(w_dtype, w_blocks, workspace, nullptr, y, m, n, k, ldy, (cudaStream_t)stream, false, peers);
}


}  // namespace lloom

using namespace lloom;

extern "C" {

int lloom_b200_version(void) { return LLOOM_B200_VERSION; }

const char *lloom_b200_error_string(int status) {
    switch (status) {
    case LLOOM_OK: return "ok";
    case LLOOM_ERR_DTYPE: return "unsupported GgmlDType (only Q8_0, Q4_K, Q6_K weights)";
    case LLOOM_ERR_SHAPE: return "bad shape";
    case LLOOM_ERR_ALIGN: return "misaligned pointer";
    case LLOOM_ERR_NULL: return "null pointer";
    case LLOOM_ERR_WORKSPACE: return "workspace missing or too small";
    case LLOOM_ERR_LAUNCH: return "CUDA launch error";
    case LLOOM_ERR_TIMEOUT: return "device-side wait timed out";
    case LLOOM_ERR_DEVICE: return "not an sm_100 device";
    case LLOOM_ERR_STATIC_LIMIT: return "request exceeds the built-in scratch (m <= 8 and m * act_row_bytes <= 256 KiB)";
    }
    return "unknown status";
}

int lloom_b200_last_cuda_error(void) { return t_last_cuda_error; }

int lloom_b200_set_launch_overlap(int enable) {
    return g_launch_overlap.exchange(enable ? 1 : 0, std::memory_order_relaxed);
}

int lloom_b200_device_status(int *status_out) {
    if (!status_out) return LLOOM_ERR_NULL;
    int v = 0;
    cudaError_t e = cudaMemcpyFromSymbol(&v, g_device_status, sizeof(int));
    if (e != cudaSuccess) return launch_status(e);
    if (v != 0) {
        int zero = 0;
        e = cudaMemcpyToSymbol(g_device_status, &zero, sizeof(int));
        if (e != cudaSuccess) return launch_status(e);
    }
    *status_out = v;
    return LLOOM_OK;
}

int64_t lloom_b200_block_elems(int dtype) {
    switch (dtype) {
    case LLOOM_Q8_0: return QK8_0;
    case LLOOM_Q4_K: case LLOOM_Q6_K: case LLOOM_Q8_K: return QK_K;
    }
    return 0;
}

int64_t lloom_b200_block_bytes(int dtype) {
    switch (dtype) {
    case LLOOM_Q8_0: return Q8_0_BYTES;
    case LLOOM_Q4_K: return Q4K_BYTES;
    case LLOOM_Q6_K: return Q6K_BYTES;
    case LLOOM_Q8_K: return Q8K_BYTES;
    }
    return 0;
}

int lloom_b200_act_dtype(int w_dtype) {
    switch (w_dtype) {
    case LLOOM_Q8_0: return LLOOM_Q8_0;
    case LLOOM_Q4_K: case LLOOM_Q6_K: return LLOOM_Q8_K;
    }
    return 0;
}

int64_t lloom_b200_act_row_bytes(int w_dtype, int64_t k) {
    const int adt = lloom_b200_act_dtype(w_dtype);
    if (!adt || k <= 0 || k % lloom_b200_block_elems(adt) != 0) return 0;
    return k / lloom_b200_block_elems(adt) * lloom_b200_block_bytes(adt);
}

int64_t lloom_b200_workspace_bytes(int w_dtype, int64_t m, int64_t n, int64_t k) {
    if (check_common(w_dtype, m, n, k) != LLOOM_OK) return 0;
    int64_t act = (m * lloom_b200_act_row_bytes(w_dtype, k) + 255) / 256 * 256;
    return act + gemm_scratch_bytes(w_dtype, m, n, k);
}

int lloom_b200_quantize_act(int w_dtype, const float *x, int64_t m, int64_t k, void *act_blocks, void *stream) {
    int rc = check_common(w_dtype, m, 1, k);
    if (rc != LLOOM_OK) return rc;
    if (!x || !act_blocks) return LLOOM_ERR_NULL;
    if (!aligned(x, 16) || !aligned(act_blocks, 4)) return LLOOM_ERR_ALIGN;
    return launch_status(launch_quantize_act(w_dtype, x, m, k, act_blocks, (cudaStream_t)stream));
}

int lloom_b200_gemv(int w_dtype, const void *w_blocks, const void *act_blocks, float *y, int64_t m, int64_t n,
                    int64_t k, int64_t ldy, void *stream) {
    int rc = check_common(w_dtype, m, n, k);
    if (rc != LLOOM_OK) return rc;
    if (m > 8 || ldy < n) return LLOOM_ERR_SHAPE;
    if (!w_blocks || !act_blocks || !y) return LLOOM_ERR_NULL;
    if (!aligned(w_blocks, 16) || !aligned(act_blocks, 4) || !aligned(y, 4)) return LLOOM_ERR_ALIGN;
    return gemv_launch(w_dtype, w_blocks, act_blocks, nullptr, y, m, n, k, ldy, (cudaStream_t)stream);
}

int lloom_b200_gemm(int w_dtype, const void *w_blocks, const void *act_blocks, float *y, int64_t m, int64_t n,
                    int64_t k, int64_t ldy, void *workspace, int64_t workspace_bytes, void *stream) {
    int rc = check_common(w_dtype, m, n, k);
    if (rc != LLOOM_OK) return rc;
    if (ldy < n) return LLOOM_ERR_SHAPE;
    if (!w_blocks || !act_blocks || !y) return LLOOM_ERR_NULL;
    if (!aligned(w_blocks, 16) || !aligned(act_blocks, 4) || !aligned(y, 4)) return LLOOM_ERR_ALIGN;
    const int64_t need = gemm_scratch_bytes(w_dtype, m, n, k);
    if (need > 0 && (!workspace || workspace_bytes < need)) return LLOOM_ERR_WORKSPACE;
    if (need > 0 && !aligned(workspace, 256)) return LLOOM_ERR_ALIGN;
    DeviceInfo di;
    rc = device_info(di);
    if (rc != LLOOM_OK) return rc;
    bool handled = false;
    rc = gemm_launch(w_dtype, w_blocks, act_blocks, y, m, n, k, ldy, workspace, di.sm_count, di.max_smem_optin,
                     (cudaStream_t)stream, handled, t_last_cuda_error);
    if (handled) return rc;
    // Shapes the tensor-core kernel does not take: slabs of up to 8 activation rows through the GEMV.
    const int64_t arow = lloom_b200_act_row_bytes(w_dtype, k);
    for (int64_t r = 0; r < m; r += 8) {
        const int64_t mm = (m - r < 8) ? (m - r) : 8;
        rc = gemv_launch(w_dtype, w_blocks, (const uint8_t *)act_blocks + r * arow, nullptr, y + r * ldy, mm, n, k, ldy,
                         (cudaStream_t)stream);
        if (rc != LLOOM_OK) return rc;
    }
    return LLOOM_OK;
}

int lloom_b200_qmatmul_fwd(int w_dtype, const void *w_blocks, const float *x, float *y, int64_t m, int64_t n,
                           int64_t k, int64_t ldy, void *workspace, int64_t workspace_bytes, void *stream) {
    int rc = check_common(w_dtype, m, n, k);
    if (rc != LLOOM_OK) return rc;
    if (ldy < n) return LLOOM_ERR_SHAPE;
    if (!w_blocks || !x || !y) return LLOOM_ERR_NULL;
    const int64_t need = lloom_b200_workspace_bytes(w_dtype, m, n, k);
    if (!workspace || workspace_bytes < need) return LLOOM_ERR_WORKSPACE;
    if (!aligned(workspace, 256) || !aligned(w_blocks, 16) || !aligned(x, 16) || !aligned(y, 4)) return LLOOM_ERR_ALIGN;
    if (m <= 8) return decode_fwd(w_dtype, w_blocks, x, y, m, n, k, ldy, workspace, need, stream, nullptr);
    rc = lloom_b200_quantize_act(w_dtype, x, m, k, workspace, stream);
    if (rc != LLOOM_OK) return rc;
    const int64_t act = (m * lloom_b200_act_row_bytes(w_dtype, k) + 255) / 256 * 256;
    return lloom_b200_gemm(w_dtype, w_blocks, workspace, y, m, n, k, ldy, (uint8_t *)workspace + act,
                           workspace_bytes - act, stream);
}

int lloom_b200_qmatmul_fwd_store(int w_dtype, const void *w_blocks, const float *x, float *y, int64_t m, int64_t n,
                                 int64_t k, int64_t ldy, int store, void *workspace, int64_t workspace_bytes,
                                 void *stream) {
    int rc = check_common(w_dtype, m, n, k);
    if (rc != LLOOM_OK) return rc;
    if (m > 8 || ldy < n || store < LLOOM_STORE_PLAIN || store > LLOOM_STORE_MUL_INTO) return LLOOM_ERR_SHAPE;
    if (!w_blocks || !x || !y) return LLOOM_ERR_NULL;
    const int64_t need = lloom_b200_workspace_bytes(w_dtype, m, n, k);
    if (!workspace || workspace_bytes < need) return LLOOM_ERR_WORKSPACE;
    if (!aligned(workspace, 256) || !aligned(w_blocks, 16) || !aligned(x, 16) || !aligned(y, 4)) return LLOOM_ERR_ALIGN;
    PeerOut out;
    out.store = store;
    return decode_fwd(w_dtype, w_blocks, x, y, m, n, k, ldy, workspace, need, stream, &out);
}

int lloom_b200_qmatmul_fwd_gather(int w_dtype, const void *w_shard, const float *x, int64_t m, int64_t n_shard, int64_t k,
                                  int64_t ldy, int64_t col0, float *const *y_peers, int n_peers, void *workspace,
                                  int64_t workspace_bytes, void *stream) {
    int rc = check_common(w_dtype, m, n_shard, k);
    if (rc != LLOOM_OK) return rc;
    if (m > 8 || n_peers < 1 || n_peers > kMaxPeers || col0 < 0 || ldy < col0 + n_shard) return LLOOM_ERR_SHAPE;
    if (!w_shard || !x || !y_peers) return LLOOM_ERR_NULL;
    const int64_t need = lloom_b200_workspace_bytes(w_dtype, m, n_shard, k);
    if (!workspace || workspace_bytes < need) return LLOOM_ERR_WORKSPACE;
    if (!aligned(workspace, 256) || !aligned(w_shard, 16) || !aligned(x, 16)) return LLOOM_ERR_ALIGN;
    PeerOut peers;
    peers.n = n_peers;
    for (int g = 0; g < n_peers; ++g) {
        if (!y_peers[g]) return LLOOM_ERR_NULL;
        if (!aligned(y_peers[g], 4)) return LLOOM_ERR_ALIGN;
        peers.y[g] = y_peers[g] + col0;
    }
    return decode_fwd(w_dtype, w_shard, x, peers.y[0], m, n_shard, k, ldy, workspace, need, stream, &peers);
}

// Cross-GPU barrier after a fused gather: one small kernel per GPU.  Each GPU bumps its own epoch, publishes it in
// slot [rank] of every GPU's flag array (system-scope release: the gather's stores, finished with the previous
// kernel on this stream, are visible before it) and waits until all slots of its own array have reached the
// epoch.  The wait is bounded in time; on a time-out the status word is set and the kernel returns.
__global__ void peer_barrier_kernel(int rank, int n_peers, PeerFlags flags) {
    __shared__ unsigned int s_epoch;
    // launched with programmatic serialization when launch overlap is on: resident early, it waits here for the
    // GEMV before it (and that GEMV's peer stores) to finish
    asm volatile("griddepcontrol.wait;" ::: "memory");
    unsigned int *mine = flags.f[rank];
    if (threadIdx.x == 0) {
        s_epoch = mine[kMaxPeers] + 1;  // slot kMaxPeers: this GPU's call counter
        mine[kMaxPeers] = s_epoch;
        __threadfence_system();
    }
    __syncthreads();
    const unsigned int epoch = s_epoch;
    const int g = threadIdx.x;
    if (g >= n_peers) return;
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(flags.f[g] + rank), "r"(epoch) : "memory");
    unsigned long long t0 = 0;
    for (uint32_t i = 0; i < kMaxSpins; ++i) {
        unsigned int seen;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(mine + g) : "memory");
        if ((int)(seen - epoch) >= 0) return;
        if ((i & 63) == 63) {
            const unsigned long long now = global_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > kMaxWaitNs) break;
        }
        __nanosleep(100);
    }
    atomicExch(&g_device_status, LLOOM_ERR_TIMEOUT);
}

int lloom_b200_peer_barrier(int rank, int n_peers, unsigned int *const *flag_peers, void *stream) {
    if (n_peers < 1 || n_peers > kMaxPeers || rank < 0 || rank >= n_peers) return LLOOM_ERR_SHAPE;
    if (!flag_peers) return LLOOM_ERR_NULL;
    PeerFlags flags;
    for (int g = 0; g < kMaxPeers; ++g) {
        flags.f[g] = g < n_peers ? flag_peers[g] : nullptr;
        if (g < n_peers && !flags.f[g]) return LLOOM_ERR_NULL;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(1);
    cfg.blockDim = dim3(32);
    cfg.stream = (cudaStream_t)stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_launch_overlap.load(std::memory_order_relaxed) != 0 ? 1 : 0;
    return launch_status(cudaLaunchKernelEx(&cfg, peer_barrier_kernel, rank, n_peers, flags));
}

// Set-up helpers for buffers that other processes of the node map (CUDA IPC); not on the forward path.
int lloom_b200_peer_alloc(int64_t bytes, void **ptr) {
    if (!ptr || bytes <= 0) return LLOOM_ERR_NULL;
    cudaError_t e = cudaMalloc(ptr, (size_t)bytes);
    if (e == cudaSuccess) e = cudaMemset(*ptr, 0, (size_t)bytes);
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    return launch_status(e);
}
int lloom_b200_peer_free(void *ptr) { return launch_status(cudaFree(ptr)); }
int lloom_b200_peer_export(const void *ptr, unsigned char *handle64) {
    if (!ptr || !handle64) return LLOOM_ERR_NULL;
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    cudaIpcMemHandle_t h;
    cudaError_t e = cudaIpcGetMemHandle(&h, const_cast<void *>(ptr));
    if (e == cudaSuccess) memcpy(handle64, &h, 64);
    return launch_status(e);
}
int lloom_b200_peer_open(const unsigned char *handle64, void **ptr) {
    if (!ptr || !handle64) return LLOOM_ERR_NULL;
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, 64);
    return launch_status(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess));
}
int lloom_b200_peer_close(void *ptr) { return launch_status(cudaIpcCloseMemHandle(ptr)); }

int lloom_b200_qmatmul_fwd_static(int w_dtype, const void *w_blocks, const float *x, float *y, int64_t m, int64_t n,
                                  int64_t k, int64_t ldy, void *stream) {
    int rc = check_common(w_dtype, m, n, k);
    if (rc != LLOOM_OK) return rc;
    if (ldy < n) return LLOOM_ERR_SHAPE;
    if (!w_blocks || !x || !y) return LLOOM_ERR_NULL;
    if (!aligned(w_blocks, 16) || !aligned(x, 16) || !aligned(y, 4)) return LLOOM_ERR_ALIGN;
    if (m > 8 || m * lloom_b200_act_row_bytes(w_dtype, k) > (int64_t)LLOOM_B200_STATIC_SCRATCH_BYTES)
        return LLOOM_ERR_STATIC_LIMIT;
    void *scratch = nullptr;
    rc = static_scratch_ptr(&scratch);  // first call per device: cudaGetSymbolAddress (keep it out of captures)
    if (rc != LLOOM_OK) return rc;
    // The quantizer writes every byte of the m activation rows the GEMV then reads; the rest of the
    // array (left over from earlier calls) is never touched.
    rc = launch_status(launch_quantize_act(w_dtype, x, m, k, scratch, (cudaStream_t)stream));
    if (rc != LLOOM_OK) return rc;
    return gemv_launch(w_dtype, w_blocks, scratch, nullptr, y, m, n, k, ldy, (cudaStream_t)stream);
}

#ifdef LLOOM_TRACE
int lloom_b200_read_trace(unsigned long long *out, unsigned int *cnt) {  // development build only
    cudaMemcpyFromSymbol(cnt, g_trace_cnt, sizeof(g_trace_cnt));
    return (int)cudaMemcpyFromSymbol(out, g_trace, sizeof(g_trace));
}
int lloom_b200_read_gemm2_trace(long long *out) {  // development build only
    return (int)cudaMemcpyFromSymbol(out, g_gemm2_trace, sizeof(g_gemm2_trace));
}

#endif

int lloom_b200_dequantize(int dtype, const void *blocks, int64_t elem_count, void *out, int out_is_f16,
                          void *stream) {
    if (!supported_weight(dtype)) return LLOOM_ERR_DTYPE;
    if (elem_count <= 0 || elem_count % lloom_b200_block_elems(dtype) != 0) return LLOOM_ERR_SHAPE;
    if (!blocks || !out) return LLOOM_ERR_NULL;
    if (!aligned(blocks, 16) || !aligned(out, 16)) return LLOOM_ERR_ALIGN;
    const int64_t threads = elem_count / 4;
    const unsigned grid = (unsigned)ceil_div64(threads, 256);
    if (out_is_f16)
        dequantize_kernel<true><<<grid, 256, 0, (cudaStream_t)stream>>>(dtype, (const uint8_t *)blocks, elem_count, out);
    else
        dequantize_kernel<false><<<grid, 256, 0, (cudaStream_t)stream>>>(dtype, (const uint8_t *)blocks, elem_count, out);
    return launch_status(cudaGetLastError());
}

int lloom_b200_get_rows(int dtype, const void *blocks, int64_t rows, int64_t hidden, const uint32_t *ids,
                        int64_t n_ids, float *out, void *stream) {
    if (!supported_weight(dtype)) return LLOOM_ERR_DTYPE;
    if (rows <= 0 || hidden <= 0 || n_ids <= 0 || hidden % lloom_b200_block_elems(dtype) != 0) return LLOOM_ERR_SHAPE;
    if (!blocks || !ids || !out) return LLOOM_ERR_NULL;
    if (!aligned(blocks, 16) || !aligned(out, 16) || !aligned(ids, 4)) return LLOOM_ERR_ALIGN;
    const int64_t threads = n_ids * (hidden / 4);
    get_rows_kernel<<<(unsigned)ceil_div64(threads, 256), 256, 0, (cudaStream_t)stream>>>(
        dtype, (const uint8_t *)blocks, rows, hidden, weight_row_bytes(dtype, hidden), ids, n_ids, out);
    return launch_status(cudaGetLastError());
}

}  // extern "C"
