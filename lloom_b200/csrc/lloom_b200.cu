// C ABI of the library (see include/lloom_b200.h): argument checks, launch planning and dispatch.  The kernels live
// in translation units of their own (gemv_*.cu, gemv_mma.cu, gemm.cu); this one holds the small ones (activation
// quantizers, dequantize, the peer barrier).  No entry point on the forward path allocates, frees or synchronises.
#include "common.cuh"
#include "dequant.cuh"
#include "gemm.h"
#include "gemv_params.h"
#include "quantize_act.cuh"

#include <algorithm>
#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <vector>

namespace lloom {

LLOOM_TU_REGISTER()

// ---- translation-unit registry: every unit has its own device-side status word and wait limit ----
namespace {
struct TuRegistry {
    std::mutex mu;
    std::vector<TuHooks> hooks;
};
TuRegistry &tu_registry() {
    static TuRegistry r;
    return r;
}
}  // namespace

void register_tu(const TuHooks &hooks) {
    TuRegistry &r = tu_registry();
    std::lock_guard<std::mutex> lock(r.mu);
    r.hooks.push_back(hooks);
}

static thread_local int t_last_cuda_error = 0;

static int launch_status(cudaError_t e) {
    if (e == cudaSuccess) return LLOOM_OK;
    t_last_cuda_error = (int)e;
    return LLOOM_ERR_LAUNCH;
}

static bool supported_weight(int dtype) {
    switch (dtype) {
    case LLOOM_Q8_0: case LLOOM_Q4_K: case LLOOM_Q6_K: case LLOOM_Q4_0: case LLOOM_Q5_0: case LLOOM_Q5_K: return true;
    }
    return false;
}

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

static cudaError_t launch_gemv_dp4a(const GemvParams &p, int grid, int smem, bool overlap, int rw, cudaStream_t stream) {
    switch (p.w_dtype) {
    case LLOOM_Q8_0: return launch_gemv_dp4a_q8_0(p, grid, smem, overlap, rw, stream);
    case LLOOM_Q4_K: return launch_gemv_dp4a_q4k(p, grid, smem, overlap, rw, stream);
    case LLOOM_Q6_K: return launch_gemv_dp4a_q6k(p, grid, smem, overlap, rw, stream);
    case LLOOM_Q5_K: return launch_gemv_dp4a_q5k(p, grid, smem, overlap, rw, stream);
    case LLOOM_Q4_0: return launch_gemv_dp4a_q4_0(p, grid, smem, overlap, rw, stream);
    case LLOOM_Q5_0: return launch_gemv_dp4a_q5_0(p, grid, smem, overlap, rw, stream);
    }
    return cudaErrorInvalidValue;
}

// Whether the tensor-core GEMV quantizes the activations itself (as its prologue, every CTA all rows): up to 48
// 256-element blocks, three per warp.  Measured per forward on [14336, 4096], prologue against separate quantizer
// kernel: 3 rows 10.5 / 11.1 us, 4 rows 11.4 / 11.1 us, 8 rows 14.7 / 11.2 us; [4096, 14336], 2 rows: 13.1 / 11.8 us.
static bool gemv_mma_fused(int64_t m, int64_t k) { return m * (k / QK_K) <= 48; }

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
    if (w_dtype != LLOOM_Q4_K || m > 8) return pl;
    // One row always runs on the dp4a kernel.  Back to back with itself this kernel (quantizer as prologue) is the
    // faster one on long rows -- [4096, 14336] 10.9 against 12.5 us, [4096, 11008] 8.9 / 10.0 us, [14336, 5120] 10.9 /
    // 12.7 us ([8192, 8192]: 12.0 / 10.5 us) -- but it fills an SM alone, so its neighbours in a decode step's chain of
    // launches cannot start beside it: a 225-matmul step took 1.55 ms with it against 1.43 ms without.
    if (m < 2) return pl;
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
        if (room >= 2 * stage) {  // (asking for three or more stages of shorter pieces measured equal or slower)
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

struct PeerFlags {  // one flag array per GPU: kMaxPeers slots written by the peers + this GPU's call counter
    unsigned int *f[kMaxPeers];
};

// Where the outputs go, beyond the plain y: the fused gather (output buffers of all GPUs, own included, already offset
// to this shard's column), a block on the store, and the flag traffic of a gather with its barrier folded in.
struct GemvOut {
    int n_peers = 0;
    float *y[kMaxPeers] = {};
    int store = LLOOM_STORE_PLAIN;
    int rank = 0;
    bool publish = false;
    unsigned int *flags[kMaxPeers] = {};
    const unsigned int *wait_flags = nullptr;
    int wait_peers = 0;
};

// Several matrices of one dtype and k behind one launch (the activations are shared).
struct GemvGroup {
    int count = 0;
    const uint8_t *w[kMaxGroup] = {};
    float *y[kMaxGroup] = {};
    int64_t n[kMaxGroup] = {};
    int64_t ldy[kMaxGroup] = {};
    int store[kMaxGroup] = {};
    const uint32_t *moe_ids = nullptr;  // routed experts: matrix g = expert moe_ids[g] of the stack at `w` of the launch
    int moe_experts = 0;
};

// Launches the GEMV.  Exactly one of `act` (canonical activation blocks) and `x` (f32 activations,
// quantized in the kernel's prologue) is non-null.  With a group, w / y / n / ldy are ignored (n = total rows).
static int gemv_launch(int w_dtype, const void *w, const void *act, const float *x, float *y, int64_t m, int64_t n,
                       int64_t k, int64_t ldy, cudaStream_t stream, bool act_planes = false,
                       const GemvOut *out = nullptr, const GemvGroup *group = nullptr) {
    DeviceInfo di;
    int rc = device_info(di);
    if (rc != LLOOM_OK) return rc;
    if (act_planes && !gemv_mma_fits(di, w_dtype, m, n, k)) return LLOOM_ERR_SHAPE;
    GemvParams p;
    memset(&p, 0, sizeof(p));
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
    p.nchunks = 1;
    p.unit_bytes = (int)((act_is_q8_0(w_dtype) ? 2 : 1) * lloom_b200_block_bytes(w_dtype));
    p.n_peers = out ? out->n_peers : 0;
    p.store_mode = out ? out->store : LLOOM_STORE_PLAIN;
    if (out) {
        p.publish = out->publish ? 1 : 0;
        p.peer_rank = out->rank;
        p.wait_flags = out->wait_flags;
        p.wait_peers = out->wait_peers;
        for (int g = 0; g < kMaxPeers; ++g) {
            p.y_peer[g] = g < out->n_peers ? out->y[g] : nullptr;
            p.peer_flags[g] = g < out->n_peers ? out->flags[g] : nullptr;
        }
    }
    if (group) {
        p.n_group = group->count;
        int64_t off = 0;
        for (int g = 0; g < group->count; ++g) {
            p.gw[g] = group->w[g];
            p.gy[g] = group->y[g];
            p.gldy[g] = group->ldy[g];
            p.gstore[g] = group->store[g];
            p.goff[g] = (int)off;
            off += group->n[g];
        }
        p.goff[group->count] = (int)off;
        p.n = (int)off;
        n = off;
        p.moe_ids = group->moe_ids;
        p.moe_experts = group->moe_experts;
    }
    // lanes per row: one lane per unit (superblock, or pair of 32-element blocks), rounded up to a power of two
    const int64_t units = k / (act_is_q8_0(w_dtype) ? 64 : 256);
    int lpr_log2 = 0;
    while ((1 << lpr_log2) < units && lpr_log2 < 5) ++lpr_log2;
    p.lpr_log2 = lpr_log2;
    const int groups = 32 >> lpr_log2;
    // A stage holds one tile of rows, widened to 16-byte boundaries, plus slack for the word-wide
    // over-read of the unaligned loaders.
    const int64_t pad = (p.row_bytes % 16 == 0) ? 16 : 48;
    int grid = di.sm_count;
    if ((int64_t)grid > n) grid = (int)n;
    const bool overlap = g_launch_overlap.load(std::memory_order_relaxed) != 0;
    // Fused gather: room to stage a CTA's output rows (so that they leave for the peers in whole lines), if small
    auto staging = [&](int64_t rows_per_cta, int &pitch) -> int64_t {
        if (p.n_peers == 0) return 0;
        pitch = (int)((rows_per_cta + 3) / 4 * 4);
        const int64_t bytes = (int64_t)m * pitch * 4;
        return bytes <= 32 * 1024 ? bytes : 0;
    };
    // 2..8 activation rows of Q4_K: the tensor-core kernel, if two 16-row stages fit beside the activations
    const MmaPlan plan = group ? MmaPlan() : gemv_mma_plan(di, w_dtype, m, n, k);
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
        const int64_t total_tiles = (n + kMmaTileRows - 1) / kMmaTileRows;
        {
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
        if (grid > total_tiles) grid = (int)total_tiles;
        return launch_status(launch_gemv_mma(p, grid, smem, overlap, stream));
    }
    // Tile shapes {consumer warps, rows per lane}, widest first; the first that leaves room for at least two stages
    // wins.  With launch overlap on, m <= 2 tries shapes that fit two CTAs per SM first, so that consecutive
    // launches can sit side by side.  A grouped launch runs the eight-warp, one-row-per-lane shapes only.
    struct Shape { int cw, rw; bool half; };
    Shape shapes[12];
    int ns = 0;
    if (group) {
        if (overlap) shapes[ns++] = {8, 1, true};
        shapes[ns++] = {8, 1, false};
    } else {
        if (overlap && m <= 2) {  // HBM-bound batch sizes only: wider batches need the registers and the row tiling
            // twelve consumer warps pay off for Q8_0 (cheap units, more of them per row); the k-quants are best at eight
            if (w_dtype == LLOOM_Q8_0) shapes[ns++] = {12, 1, true};
            const int half_cw[4] = {8, 4, 2, 1};
            for (int c : half_cw) shapes[ns++] = {c, 1, true};
        }
        const int full[5][2] = {{8, 2}, {8, 1}, {4, 1}, {2, 1}, {1, 1}};
        for (auto &f : full) shapes[ns++] = {f[0], f[1], false};
    }
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
            // Long rows in a side-by-side shape: cut the rows into pieces of 16 units (32 for 64-element units), so
            // that a stage is 16 (8) rows x one piece -- the tile the kernel streams at K = 4096 -- instead of giving
            // up the overlap between consecutive launches for a one-CTA-per-SM shape.
            if ((group && m != 1) || !shapes[si].half || cw > 8 || p.row_bytes % 16 != 0) continue;
            const int cu = act_is_q8_0(w_dtype) ? 32 : 16, cl = act_is_q8_0(w_dtype) ? 5 : 4;
            if (units <= cu || ((int64_t)cu * p.unit_bytes) % 16 != 0) continue;
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
        return launch_status(launch_gemv_dp4a(p, grid, smem, overlap, rw, stream));
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

static int64_t act_blocks_bytes(int w_dtype, int64_t m, int64_t k) {
    return (m * lloom_b200_act_row_bytes(w_dtype, k) + 255) / 256 * 256;
}

// Decode forward (m <= 8) after argument checks: quantizer + GEMV, outputs to `y` or to the peers' buffers.
static int decode_fwd(int w_dtype, const void *w_blocks, const float *x, float *y, int64_t m, int64_t n, int64_t k,
                      int64_t ldy, void *workspace, int64_t need, void *stream, const GemvOut *out) {
    int rc;
    {
        DeviceInfo di;
        rc = device_info(di);
        if (rc != LLOOM_OK) return rc;
        // activations that an earlier fused gather delivers may only be read by the kernel that waits for that gather
        const bool must_fuse = out && out->wait_flags;
        const bool mma = gemv_mma_fits(di, w_dtype, m, n, k) && (!must_fuse || gemv_mma_fused(m, k));
        // up to two rows: one launch, the activation quantizer is the GEMV's prologue (the workspace stays
        // unused).  From three rows on, every CTA re-quantizing all rows costs more than one small kernel does.
        if ((m <= 2 && !mma) || (mma && gemv_mma_fused(m, k)))
            return gemv_launch(w_dtype, w_blocks, nullptr, x, y, m, n, k, ldy, (cudaStream_t)stream, false, out);
        // Q4_K batches for the tensor-core GEMV: the quantizer writes the kernel's own activation image (same
        // codes, scales and sums as the canonical blocks, laid out for its fragment loads)
        if (mma && mma_act_bytes(m, k) <= need) {
            rc = launch_status(launch_quantize_q8k_planes(x, (uint8_t *)workspace, (int)m, (int)(k / QK_K),
                                                          (int)mma_act_pitch(k), (cudaStream_t)stream));
            if (rc != LLOOM_OK) return rc;
            return gemv_launch(w_dtype, w_blocks, workspace, nullptr, y, m, n, k, ldy, (cudaStream_t)stream, true, out);
        }
    }
    rc = lloom_b200_quantize_act(w_dtype, x, m, k, workspace, stream);
    if (rc != LLOOM_OK) return rc;
    return gemv_launch(w_dtype, w_blocks, workspace, nullptr, y, m, n, k, ldy, (cudaStream_t)stream, false, out);
}

// Prefill forward (m > 8) after argument checks.  Activations: canonical blocks in `act`, or f32 in `x` with `act_ws` the
// place to quantize them to where a kernel needs canonical blocks (the Q4_K / Q5_K GEMM takes the f32 itself).
// `scratch` follows the activation blocks in the caller's workspace.
static int gemm_dispatch(int w_dtype, const void *w_blocks, const void *w_image, const void *act, const float *x, void *act_ws,
                         float *y, int64_t m, int64_t n, int64_t k, int64_t ldy, void *scratch, void *stream) {
    DeviceInfo di;
    int rc = device_info(di);
    if (rc != LLOOM_OK) return rc;
    const bool tensor = gemm_supported(w_dtype, m, k, di.max_smem_optin);
    if (tensor && !act && gemm_takes_f32(w_dtype))
        return launch_status(gemm_forward(w_dtype, w_blocks, w_image, nullptr, x, y, m, n, k, ldy, scratch, (cudaStream_t)stream));
    if (!act) {
        rc = lloom_b200_quantize_act(w_dtype, x, m, k, act_ws, stream);
        if (rc != LLOOM_OK) return rc;
        act = act_ws;
    }
    if (tensor)
        return launch_status(gemm_forward(w_dtype, w_blocks, w_image, act, nullptr, y, m, n, k, ldy, scratch, (cudaStream_t)stream));
    // Shapes no tensor-core kernel takes: slabs of up to 8 activation rows through the GEMV.
    const int64_t arow = lloom_b200_act_row_bytes(w_dtype, k);
    for (int64_t r = 0; r < m; r += 8) {
        const int64_t mm = (m - r < 8) ? (m - r) : 8;
        rc = gemv_launch(w_dtype, w_blocks, (const uint8_t *)act + r * arow, nullptr, y + r * ldy, mm, n, k, ldy,
                         (cudaStream_t)stream);
        if (rc != LLOOM_OK) return rc;
    }
    return LLOOM_OK;
}

static int fwd_checks(int w_dtype, const void *w_blocks, const float *x, const float *y, int64_t m, int64_t n, int64_t k,
                      int64_t ldy, const void *workspace, int64_t workspace_bytes, int64_t need) {
    int rc = check_common(w_dtype, m, n, k);
    if (rc != LLOOM_OK) return rc;
    if (ldy < n) return LLOOM_ERR_SHAPE;
    if (!w_blocks || !x || !y) return LLOOM_ERR_NULL;
    if (!workspace || workspace_bytes < need) return LLOOM_ERR_WORKSPACE;
    if (!aligned(workspace, 256) || !aligned(w_blocks, 16) || !aligned(x, 16) || !aligned(y, 4)) return LLOOM_ERR_ALIGN;
    return LLOOM_OK;
}

}  // namespace lloom

using namespace lloom;

extern "C" {

int lloom_b200_version(void) { return LLOOM_B200_VERSION; }

const char *lloom_b200_error_string(int status) {
    switch (status) {
    case LLOOM_OK: return "ok";
    case LLOOM_ERR_DTYPE: return "unsupported GgmlDType (weights: Q4_0, Q5_0, Q8_0, Q4_K, Q5_K, Q6_K)";
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
    TuRegistry &r = tu_registry();
    std::lock_guard<std::mutex> lock(r.mu);  // one reader at a time: the fetch goes through a per-unit landing word
    int status = 0;
    for (const TuHooks &h : r.hooks) {
        int v = 0;
        const cudaError_t e = h.fetch_status(&v, nullptr);  // device-side atomic exchange, then a synchronous read
        if (e != cudaSuccess) return launch_status(e);
        if (v != 0) status = v;
    }
    *status_out = status;
    return LLOOM_OK;
}

int lloom_b200_set_wait_limit_ns(uint64_t ns) {
    if (ns == 0) ns = kDefaultWaitNs;
    TuRegistry &r = tu_registry();
    std::lock_guard<std::mutex> lock(r.mu);
    for (const TuHooks &h : r.hooks) {
        const cudaError_t e = h.set_wait_limit((unsigned long long)ns);
        if (e != cudaSuccess) return launch_status(e);
    }
    return LLOOM_OK;
}

int64_t lloom_b200_block_elems(int dtype) {
    switch (dtype) {
    case LLOOM_Q8_0: case LLOOM_Q4_0: case LLOOM_Q5_0: return QK8_0;
    case LLOOM_Q4_K: case LLOOM_Q5_K: case LLOOM_Q6_K: case LLOOM_Q8_K: return QK_K;
    }
    return 0;
}

int64_t lloom_b200_block_bytes(int dtype) {
    switch (dtype) {
    case LLOOM_Q8_0: return Q8_0_BYTES;
    case LLOOM_Q4_K: return Q4K_BYTES;
    case LLOOM_Q6_K: return Q6K_BYTES;
    case LLOOM_Q8_K: return Q8K_BYTES;
    case LLOOM_Q4_0: return Q4_0_BYTES;
    case LLOOM_Q5_0: return Q5_0_BYTES;
    case LLOOM_Q5_K: return Q5K_BYTES;
    }
    return 0;
}

int lloom_b200_act_dtype(int w_dtype) {
    switch (w_dtype) {
    case LLOOM_Q8_0: case LLOOM_Q4_0: case LLOOM_Q5_0: return LLOOM_Q8_0;
    case LLOOM_Q4_K: case LLOOM_Q5_K: case LLOOM_Q6_K: return LLOOM_Q8_K;
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
    return act_blocks_bytes(w_dtype, m, k) + gemm_scratch_bytes(w_dtype, m, n, k, false);
}

int64_t lloom_b200_workspace_bytes_with_image(int w_dtype, int64_t m, int64_t n, int64_t k) {
    if (check_common(w_dtype, m, n, k) != LLOOM_OK) return 0;
    return act_blocks_bytes(w_dtype, m, k) + gemm_scratch_bytes(w_dtype, m, n, k, true);
}

int64_t lloom_b200_weight_image_bytes(int w_dtype, int64_t n, int64_t k) {
    if (check_common(w_dtype, 1, n, k) != LLOOM_OK) return 0;
    if (!gemm_supported(w_dtype, 9, k, 1 << 30)) return 0;
    return gemm_weight_image_bytes(w_dtype, n, k);
}

int lloom_b200_weight_image_build(int w_dtype, const void *w_blocks, int64_t n, int64_t k, void *image, int64_t image_bytes,
                                  void *stream) {
    int rc = check_common(w_dtype, 1, n, k);
    if (rc != LLOOM_OK) return rc;
    const int64_t need = lloom_b200_weight_image_bytes(w_dtype, n, k);
    if (need <= 0) return LLOOM_ERR_SHAPE;
    if (!w_blocks || !image) return LLOOM_ERR_NULL;
    if (image_bytes < need) return LLOOM_ERR_WORKSPACE;
    if (!aligned(w_blocks, 16) || !aligned(image, 1024)) return LLOOM_ERR_ALIGN;
    return launch_status(gemm_weight_image_build(w_dtype, w_blocks, n, k, image, (cudaStream_t)stream));
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
    const int64_t need = gemm_scratch_bytes(w_dtype, m, n, k, false);
    if (need > 0 && (!workspace || workspace_bytes < need)) return LLOOM_ERR_WORKSPACE;
    if (need > 0 && !aligned(workspace, 256)) return LLOOM_ERR_ALIGN;
    return gemm_dispatch(w_dtype, w_blocks, nullptr, act_blocks, nullptr, nullptr, y, m, n, k, ldy, workspace, stream);
}

int lloom_b200_qmatmul_fwd(int w_dtype, const void *w_blocks, const float *x, float *y, int64_t m, int64_t n,
                           int64_t k, int64_t ldy, void *workspace, int64_t workspace_bytes, void *stream) {
    const int64_t need = lloom_b200_workspace_bytes(w_dtype, m, n, k);
    int rc = fwd_checks(w_dtype, w_blocks, x, y, m, n, k, ldy, workspace, workspace_bytes, need);
    if (rc != LLOOM_OK) return rc;
    if (m <= 8) return decode_fwd(w_dtype, w_blocks, x, y, m, n, k, ldy, workspace, need, stream, nullptr);
    return gemm_dispatch(w_dtype, w_blocks, nullptr, nullptr, x, workspace, y, m, n, k, ldy,
                         (uint8_t *)workspace + act_blocks_bytes(w_dtype, m, k), stream);
}

int lloom_b200_qmatmul_fwd_image(int w_dtype, const void *w_blocks, const void *w_image, const float *x, float *y,
                                 int64_t m, int64_t n, int64_t k, int64_t ldy, void *workspace, int64_t workspace_bytes,
                                 void *stream) {
    if (!w_image) return lloom_b200_qmatmul_fwd(w_dtype, w_blocks, x, y, m, n, k, ldy, workspace, workspace_bytes, stream);
    const int64_t need = lloom_b200_workspace_bytes_with_image(w_dtype, m, n, k);
    int rc = fwd_checks(w_dtype, w_blocks, x, y, m, n, k, ldy, workspace, workspace_bytes, need);
    if (rc != LLOOM_OK) return rc;
    if (!aligned(w_image, 1024)) return LLOOM_ERR_ALIGN;
    if (m <= 8) return decode_fwd(w_dtype, w_blocks, x, y, m, n, k, ldy, workspace, need, stream, nullptr);
    if (lloom_b200_weight_image_bytes(w_dtype, n, k) <= 0) return LLOOM_ERR_SHAPE;  // no image exists for this shape
    return gemm_dispatch(w_dtype, w_blocks, w_image, nullptr, x, workspace, y, m, n, k, ldy,
                         (uint8_t *)workspace + act_blocks_bytes(w_dtype, m, k), stream);
}

int lloom_b200_qmatmul_fwd_store(int w_dtype, const void *w_blocks, const float *x, float *y, int64_t m, int64_t n,
                                 int64_t k, int64_t ldy, int store, void *workspace, int64_t workspace_bytes,
                                 void *stream) {
    const int64_t need = lloom_b200_workspace_bytes(w_dtype, m, n, k);
    int rc = fwd_checks(w_dtype, w_blocks, x, y, m, n, k, ldy, workspace, workspace_bytes, need);
    if (rc != LLOOM_OK) return rc;
    if (m > 8 || store < LLOOM_STORE_PLAIN || store > LLOOM_STORE_MUL_INTO) return LLOOM_ERR_SHAPE;
    GemvOut out;
    out.store = store;
    return decode_fwd(w_dtype, w_blocks, x, y, m, n, k, ldy, workspace, need, stream, &out);
}

int lloom_b200_qmatmul_fwd_group(int w_dtype, int n_mats, const void *const *w_blocks, const float *x, float *const *ys,
                                 const int64_t *ns, const int64_t *ldys, const int *stores, int64_t m, int64_t k,
                                 void *workspace, int64_t workspace_bytes, void *stream) {
    if (n_mats < 1 || n_mats > kMaxGroup) return LLOOM_ERR_SHAPE;
    if (!w_blocks || !x || !ys || !ns || !ldys) return LLOOM_ERR_NULL;
    if (m > 8) return LLOOM_ERR_SHAPE;
    GemvGroup group;
    group.count = n_mats;
    int64_t n_max = 0, n_total = 0;
    for (int g = 0; g < n_mats; ++g) {
        int rc = check_common(w_dtype, m, ns[g], k);
        if (rc != LLOOM_OK) return rc;
        if (ldys[g] < ns[g]) return LLOOM_ERR_SHAPE;
        if (!w_blocks[g] || !ys[g]) return LLOOM_ERR_NULL;
        if (!aligned(w_blocks[g], 16) || !aligned(ys[g], 4)) return LLOOM_ERR_ALIGN;
        const int store = stores ? stores[g] : LLOOM_STORE_PLAIN;
        if (store < LLOOM_STORE_PLAIN || store > LLOOM_STORE_MUL_INTO) return LLOOM_ERR_SHAPE;
        group.w[g] = (const uint8_t *)w_blocks[g];
        group.y[g] = ys[g];
        group.n[g] = ns[g];
        group.ldy[g] = ldys[g];
        group.store[g] = store;
        if (ns[g] > n_max) n_max = ns[g];
        n_total += ns[g];
    }
    if (n_total > (1ll << 30)) return LLOOM_ERR_SHAPE;
    const int64_t need = lloom_b200_workspace_bytes(w_dtype, m, n_max, k);
    if (!workspace || workspace_bytes < need) return LLOOM_ERR_WORKSPACE;
    if (!aligned(workspace, 256) || !aligned(x, 16)) return LLOOM_ERR_ALIGN;
    DeviceInfo di;
    int rc = device_info(di);
    if (rc != LLOOM_OK) return rc;
    // One launch for the whole group where the dp4a kernel with its quantizer prologue is the decode path anyway
    // (one row; two rows of the formats without a tensor-core GEMV) and whole rows fit its stages.
    // (where a forward of its own would take the tensor-core kernel, so does every matrix here: same bits either way)
    const bool one_launch = n_mats > 1 && m <= 2 && !gemv_mma_fits(di, w_dtype, m, n_max, k);
    if (one_launch) {
        rc = gemv_launch(w_dtype, nullptr, nullptr, x, nullptr, m, 0, k, 0, (cudaStream_t)stream, false, nullptr, &group);
        if (rc != LLOOM_ERR_SHAPE) return rc;  // rows too long for whole-row stages: matrix by matrix below
    }
    // Otherwise the activations are quantized once and every matrix gets its own GEMV launch.
    const bool mma = gemv_mma_fits(di, w_dtype, m, n_max, k);
    bool all_mma = mma;
    for (int g = 0; g < n_mats && all_mma; ++g) all_mma = gemv_mma_fits(di, w_dtype, m, ns[g], k);
    if (all_mma && mma_act_bytes(m, k) <= need) {
        rc = launch_status(launch_quantize_q8k_planes(x, (uint8_t *)workspace, (int)m, (int)(k / QK_K), (int)mma_act_pitch(k),
                                                      (cudaStream_t)stream));
    } else {
        all_mma = false;
        rc = lloom_b200_quantize_act(w_dtype, x, m, k, workspace, stream);
    }
    if (rc != LLOOM_OK) return rc;
    for (int g = 0; g < n_mats; ++g) {
        GemvOut out;
        out.store = group.store[g];
        rc = gemv_launch(w_dtype, group.w[g], workspace, nullptr, group.y[g], m, group.n[g], k, group.ldy[g],
                         (cudaStream_t)stream, all_mma, &out);
        if (rc != LLOOM_OK) return rc;
    }
    return LLOOM_OK;
}

int lloom_b200_indexed_moe_forward(int w_dtype, const void *w_experts, int64_t n_experts, int64_t n, int64_t k,
                                   const float *x, int64_t batch, int64_t in_dim1, const uint32_t *ids, int64_t topk,
                                   float *out, void *workspace, int64_t workspace_bytes, void *stream) {
    int rc = check_common(w_dtype, 1, n, k);
    if (rc != LLOOM_OK) return rc;
    if (n_experts <= 0 || n_experts > (1 << 20) || batch <= 0 || topk <= 0 || (in_dim1 != 1 && in_dim1 != topk))
        return LLOOM_ERR_SHAPE;
    if (!w_experts || !x || !ids || !out) return LLOOM_ERR_NULL;
    if (n_experts * n > (1ll << 30)) return LLOOM_ERR_SHAPE;
    if (!aligned(w_experts, 16) || !aligned(x, 16) || !aligned(ids, 4) || !aligned(out, 4)) return LLOOM_ERR_ALIGN;
    const int64_t need = lloom_b200_workspace_bytes(w_dtype, 1, n, k);
    if (!workspace || workspace_bytes < need) return LLOOM_ERR_WORKSPACE;
    if (!aligned(workspace, 256)) return LLOOM_ERR_ALIGN;
    const bool share_x = in_dim1 == 1 && topk <= kMaxGroup;
    for (int64_t b = 0; b < batch; ++b) {
        for (int64_t t0 = 0; t0 < topk; t0 += share_x ? topk : 1) {
            GemvGroup group;
            group.count = share_x ? (int)topk : 1;
            for (int g = 0; g < group.count; ++g) {
                group.w[g] = (const uint8_t *)w_experts;  // replaced on the device by the routed expert
                group.y[g] = out + ((b * topk + t0 + g) * n);
                group.n[g] = n;
                group.ldy[g] = n;
                group.store[g] = LLOOM_STORE_PLAIN;
            }
            group.moe_ids = ids + b * topk + t0;
            group.moe_experts = (int)n_experts;
            const float *xrow = x + (b * in_dim1 + (in_dim1 == 1 ? 0 : t0)) * k;
            rc = gemv_launch(w_dtype, w_experts, nullptr, xrow, nullptr, 1, 0, k, 0, (cudaStream_t)stream, false, nullptr, &group);
            if (rc != LLOOM_OK) return rc;
        }
    }
    return LLOOM_OK;
}

static int gather_common(int w_dtype, const void *w_shard, const float *x, int64_t m, int64_t n_shard, int64_t k,
                         int64_t ldy, int64_t col0, float *const *y_peers, int n_peers, void *workspace,
                         int64_t workspace_bytes, void *stream, GemvOut &peers) {
    int rc = check_common(w_dtype, m, n_shard, k);
    if (rc != LLOOM_OK) return rc;
    if (m > 8 || n_peers < 1 || n_peers > kMaxPeers || col0 < 0 || ldy < col0 + n_shard) return LLOOM_ERR_SHAPE;
    if (!w_shard || !x || !y_peers) return LLOOM_ERR_NULL;
    const int64_t need = lloom_b200_workspace_bytes(w_dtype, m, n_shard, k);
    if (!workspace || workspace_bytes < need) return LLOOM_ERR_WORKSPACE;
    if (!aligned(workspace, 256) || !aligned(w_shard, 16) || !aligned(x, 16)) return LLOOM_ERR_ALIGN;
    peers.n_peers = n_peers;
    for (int g = 0; g < n_peers; ++g) {
        if (!y_peers[g]) return LLOOM_ERR_NULL;
        if (!aligned(y_peers[g], 4)) return LLOOM_ERR_ALIGN;
        peers.y[g] = y_peers[g] + col0;
    }
    return decode_fwd(w_dtype, w_shard, x, peers.y[0], m, n_shard, k, ldy, workspace, need, stream, &peers);
}

int lloom_b200_qmatmul_fwd_gather(int w_dtype, const void *w_shard, const float *x, int64_t m, int64_t n_shard, int64_t k,
                                  int64_t ldy, int64_t col0, float *const *y_peers, int n_peers, void *workspace,
                                  int64_t workspace_bytes, void *stream) {
    GemvOut peers;
    return gather_common(w_dtype, w_shard, x, m, n_shard, k, ldy, col0, y_peers, n_peers, workspace, workspace_bytes, stream,
                         peers);
}

int lloom_b200_qmatmul_fwd_gather_sync(int w_dtype, const void *w_shard, const float *x, int64_t m, int64_t n_shard,
                                       int64_t k, int64_t ldy, int64_t col0, float *const *y_peers, int n_peers, int rank,
                                       unsigned int *const *flag_peers, const unsigned int *wait_flags, void *workspace,
                                       int64_t workspace_bytes, void *stream) {
    if (n_peers < 1 || n_peers > kMaxPeers || rank < 0 || rank >= n_peers) return LLOOM_ERR_SHAPE;
    if (!flag_peers) return LLOOM_ERR_NULL;
    if (wait_flags && m > 2) return LLOOM_ERR_SHAPE;  // the wait sits in the GEMV's own quantizer prologue (m <= 2)
    GemvOut peers;
    peers.publish = true;
    peers.rank = rank;
    for (int g = 0; g < n_peers; ++g) {
        if (!flag_peers[g]) return LLOOM_ERR_NULL;
        if (!aligned(flag_peers[g], 4)) return LLOOM_ERR_ALIGN;
        peers.flags[g] = flag_peers[g];
    }
    peers.wait_flags = wait_flags;
    peers.wait_peers = wait_flags ? n_peers : 0;
    return gather_common(w_dtype, w_shard, x, m, n_shard, k, ldy, col0, y_peers, n_peers, workspace, workspace_bytes, stream,
                         peers);
}

int lloom_b200_qmatmul_fwd_after_gather(int w_dtype, const void *w_blocks, const float *x, float *y, int64_t m, int64_t n,
                                        int64_t k, int64_t ldy, const unsigned int *wait_flags, int n_peers,
                                        void *workspace, int64_t workspace_bytes, void *stream) {
    const int64_t need = lloom_b200_workspace_bytes(w_dtype, m, n, k);
    int rc = fwd_checks(w_dtype, w_blocks, x, y, m, n, k, ldy, workspace, workspace_bytes, need);
    if (rc != LLOOM_OK) return rc;
    if (m > 2 || n_peers < 1 || n_peers > kMaxPeers) return LLOOM_ERR_SHAPE;  // served where the quantizer is the GEMV's prologue
    if (!wait_flags) return LLOOM_ERR_NULL;
    GemvOut out;
    out.wait_flags = wait_flags;
    out.wait_peers = n_peers;
    return decode_fwd(w_dtype, w_blocks, x, y, m, n, k, ldy, workspace, need, stream, &out);
}

// Waits (bounded) until every slot of this GPU's flag array has reached the GPU's own call counter: the gathered
// rows of the last lloom_b200_qmatmul_fwd_gather_sync on this stream are complete.  One warp, lane g polls slot g.
__global__ void peer_wait_kernel(int n_peers, const unsigned int *flags) {
    // let the stream's next kernel become resident (a GEMV starts streaming its weights) while this one waits for
    // the GEMV before it and then for the peers; that kernel's own griddepcontrol.wait holds it until this one is done
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int g = threadIdx.x;
    if (g >= n_peers) return;
    unsigned int want;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(want) : "l"(flags + kMaxPeers) : "memory");
    unsigned long long t0 = 0;
    for (uint32_t i = 0; i < kMaxSpins; ++i) {
        unsigned int seen;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(flags + g) : "memory");
        if ((int)(seen - want) >= 0) return;
        if ((i & 63) == 63) {
            const unsigned long long now = global_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > wait_limit_ns()) break;
        }
        __nanosleep(100);
    }
    atomicExch(&g_device_status, LLOOM_ERR_TIMEOUT);
}

// Cross-GPU barrier after a fused gather: one small kernel per GPU.  Each GPU bumps its own epoch, publishes it in
// slot [rank] of every GPU's flag array (system-scope release: the gather's stores, finished with the previous
// kernel on this stream, are visible before it) and waits until all slots of its own array have reached the
// epoch.  The wait is bounded in time; on a time-out the status word is set and the kernel returns.
__global__ void peer_barrier_kernel(int rank, int n_peers, PeerFlags flags) {
    __shared__ unsigned int s_epoch;
    // launched with programmatic serialization when launch overlap is on: resident early, it waits here for the
    // GEMV before it (and that GEMV's peer stores) to finish; the kernel behind it may become resident meanwhile
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
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
            else if (now - t0 > wait_limit_ns()) break;
        }
        __nanosleep(100);
    }
    atomicExch(&g_device_status, LLOOM_ERR_TIMEOUT);
}

static cudaError_t launch_one_warp(void (*kern)(int, const unsigned int *), int a, const unsigned int *b, cudaStream_t stream) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(1);
    cfg.blockDim = dim3(32);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_launch_overlap.load(std::memory_order_relaxed) != 0 ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, a, b);
}

int lloom_b200_peer_wait(int n_peers, const unsigned int *flags_own, void *stream) {
    if (n_peers < 1 || n_peers > kMaxPeers) return LLOOM_ERR_SHAPE;
    if (!flags_own) return LLOOM_ERR_NULL;
    return launch_status(launch_one_warp(peer_wait_kernel, n_peers, flags_own, (cudaStream_t)stream));
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
