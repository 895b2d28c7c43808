/*
 * lloom_b200 -- C ABI of the B200 (sm_100a) quantized-weight matmul library.
 *
 * This is the boundary a lloom maintainer binds from Rust (`extern "C"`) inside
 * `QCudaStorage` (lloom-tensor/src/quantized/cuda.rs): plain pointers and sizes,
 * CUDA stream as `void*` exactly like the launchers it replaces
 * (candle-kernels/src/ffi.rs).  Every entry point
 *   - returns an `int` status (0 = ok) instead of the reference's `void`,
 *   - enqueues on the caller's stream and never synchronises the host,
 *   - never allocates or frees device memory: scratch comes from the caller
 *     (`lloom_b200_workspace_bytes`), outputs are caller buffers.
 *
 * Arithmetic contract: the CPU path of the reference (`k_quants::matmul`), i.e.
 * activations quantized to Q8_0 (for Q8_0 weights) or Q8_K (for Q4_K / Q6_K
 * weights), bit-exact with `BlockQ8_0::from_float` / `BlockQ8K::from_float`;
 * exact integer block dot products; f32 scale application in the reference's
 * algebraic form.  Only the f32 summation order across blocks differs.
 *
 * dtype codes are the reference's GGUF type ids (lloom-tensor/src/quantized/mod.rs:505-568).
 * Weight layout is the canonical GGUF block stream, row-major [n][k / block]:
 * the bytes `QTensor::data()` returns.  Device weight pointers must be 16-byte aligned.
 */
#ifndef LLOOM_B200_H
#define LLOOM_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define LLOOM_B200_VERSION 100

/* GgmlDType ids (mod.rs:505-568): only these are implemented; anything else returns LLOOM_ERR_DTYPE. */
#define LLOOM_Q4_0 2
#define LLOOM_Q5_0 6
#define LLOOM_Q8_0 8
#define LLOOM_Q4_K 12
#define LLOOM_Q5_K 13
#define LLOOM_Q6_K 14
#define LLOOM_Q8_K 15 /* activation-only */

enum {
    LLOOM_OK = 0,
    LLOOM_ERR_DTYPE = 1,     /* unsupported GgmlDType (no fallback exists) */
    LLOOM_ERR_SHAPE = 2,     /* k not a multiple of the block size, m/n/k <= 0, ldy < n, ... */
    LLOOM_ERR_ALIGN = 3,     /* pointer alignment (weights 16 B; f32 buffers 4 B; act blocks 4 B) */
    LLOOM_ERR_NULL = 4,      /* null pointer */
    LLOOM_ERR_WORKSPACE = 5, /* workspace missing or smaller than lloom_b200_workspace_bytes */
    LLOOM_ERR_LAUNCH = 6,    /* CUDA reported an error at launch (see lloom_b200_last_cuda_error) */
    LLOOM_ERR_TIMEOUT = 7,   /* a bounded device-side wait ran out (reported by lloom_b200_device_status) */
    LLOOM_ERR_DEVICE = 8,    /* not an sm_100 device / attribute query failed */
    LLOOM_ERR_STATIC_LIMIT = 9 /* request exceeds the built-in scratch of lloom_b200_qmatmul_fwd_static */
};

/* Library version (LLOOM_B200_VERSION of the build). */
int lloom_b200_version(void);
/* Static description of a status code. */
const char *lloom_b200_error_string(int status);
/* The cudaError_t of the last LLOOM_ERR_LAUNCH on this thread (0 if none). */
int lloom_b200_last_cuda_error(void);
/* Reads and clears (one atomic exchange on the device, then a synchronous copy) the status word of the
 * current device: 0, or LLOOM_ERR_TIMEOUT when a bounded wait inside a kernel gave up since the last call.
 * One word per device serves every stream.  For tests and post-mortems; safe to call from several host threads. */
int lloom_b200_device_status(int *status_out);
/* Time limit of every bounded device-side wait (mbarrier waits inside the kernels, the cross-GPU flag waits) on the
 * current device, in nanoseconds; 0 restores the default of 2 s.  A wait that runs out sets the status word to
 * LLOOM_ERR_TIMEOUT and the kernel unwinds by itself (no trap; the context stays usable).  Synchronous; call it
 * between launches.  (The reference has no counterpart: its kernels never wait on one another.) */
int lloom_b200_set_wait_limit_ns(uint64_t ns);

/* Launch overlap for the decode GEMV (off by default; returns the previous setting).  When on, GEMV
 * launches carry the programmatic-stream-serialization attribute: a GEMV may start streaming its
 * weights while the kernel before it in the stream is still finishing, and waits for that kernel
 * only before it reads activations or writes outputs.  Turn it on once weights are resident; the one
 * rule it adds is that the kernel launched immediately before a GEMV on the same stream must not be
 * the one that writes that GEMV's weight blocks (copies and earlier kernels are fine).  Results are
 * unchanged. */
int lloom_b200_set_launch_overlap(int enable);

/* GgmlDType::block_size / type_size (mod.rs:663-715): 32|256 elements, 34|144|210|292 bytes; 0 if unsupported. */
int64_t lloom_b200_block_elems(int dtype);
int64_t lloom_b200_block_bytes(int dtype);
/* Activation block type a weight type is dotted with (GgmlType::VecDotType, k_quants.rs:717,1507,2082). */
int lloom_b200_act_dtype(int w_dtype);
/* Bytes of one quantized activation row of k elements for this weight type. */
int64_t lloom_b200_act_row_bytes(int w_dtype, int64_t k);

/* Scratch lloom_b200_qmatmul_fwd needs for an [m,k] x [n,k]^T product (quantized activations
 * plus the GEMM's per-call planes).  Replaces the grow-only per-device scratch of
 * fast_mmvq.rs:44-81 / fast_mmq.rs:135-174; the caller owns it.  256-byte aligned. */
int64_t lloom_b200_workspace_bytes(int w_dtype, int64_t m, int64_t n, int64_t k);

/* ---- Prebuilt weight images for the prefill GEMM ----
 * The tensor-core GEMM reads the weights as f16 operand images (exact integers: scale x code).  By default every
 * call with m > 8 builds them in its workspace, slab by slab; a caller that runs many prefill calls on the same
 * weights can build the image once into a buffer it owns (about 3.6x the Q4_K bytes, 3.8x Q8_0, 4.9x Q6_K) and
 * pass it to lloom_b200_qmatmul_fwd_image, which then needs only lloom_b200_workspace_bytes_with_image.
 * (The reference re-quantizes activations per call but keeps no second weight form; 180 GB of HBM per GPU is
 * what makes the second form affordable here.)  image: 1024-byte aligned.  0 bytes = no GEMM for this type/shape. */
int64_t lloom_b200_weight_image_bytes(int w_dtype, int64_t n, int64_t k);
int lloom_b200_weight_image_build(int w_dtype, const void *w_blocks, int64_t n, int64_t k, void *image, int64_t image_bytes,
                                  void *stream);
int64_t lloom_b200_workspace_bytes_with_image(int w_dtype, int64_t m, int64_t n, int64_t k);
/* lloom_b200_qmatmul_fwd with the weight image prebuilt (w_image == NULL: exactly lloom_b200_qmatmul_fwd). */
int lloom_b200_qmatmul_fwd_image(int w_dtype, const void *w_blocks, const void *w_image, const float *x, float *y,
                                 int64_t m, int64_t n, int64_t k, int64_t ldy, void *workspace, int64_t workspace_bytes,
                                 void *stream);

/* Activation quantizer: x f32 [m,k] contiguous -> canonical Q8_0 / Q8_K blocks [m][k/block],
 * bit-exact with BlockQ8_0::from_float (k_quants.rs:738-767) / BlockQ8K::from_float
 * (k_quants.rs:2400-2438).  Replaces launch_mmvq_gguf_quantize_q8_1_f32 (ffi.rs:412) and
 * launch_mmq_quantize_q8_1_* (ffi.rs:424-454), which quantize to Q8_1 instead. */
int lloom_b200_quantize_act(int w_dtype, const float *x, int64_t m, int64_t k, void *act_blocks, void *stream);

/* Decode GEMV, 1 <= m <= 8: y[r*ldy + c] = vec_dot(W[c], A[r]) for c < n
 * (GgmlType::vec_dot, k_quants.rs:800-818, 1540-1620, 2115-2172 through matmul :2587-2637).
 * Replaces launch_mmvq_gguf_{q8_0,q4_k,q6_k}_f32_plain (ffi.rs:217,250,272). */
int lloom_b200_gemv(int w_dtype, const void *w_blocks, const void *act_blocks, float *y, int64_t m, int64_t n,
                    int64_t k, int64_t ldy, void *stream);

/* Prefill GEMM, any m >= 1 (meant for m > 8): same result definition as the GEMV
 * (matmul m > 1 arm, k_quants.rs:2518-2585).  All six formats run on tcgen05 tensor cores (the 32-element-block
 * formats Q8_0, Q4_0, Q5_0 for k a multiple of 128); other shapes fall to slabs of eight rows through the GEMV.
 * Replaces launch_mmq_gguf_* (ffi.rs:583).  `workspace`: lloom_b200_workspace_bytes minus the activation blocks
 * (passing a buffer of the full lloom_b200_workspace_bytes is always enough). */
int lloom_b200_gemm(int w_dtype, const void *w_blocks, const void *act_blocks, float *y, int64_t m, int64_t n,
                    int64_t k, int64_t ldy, void *workspace, int64_t workspace_bytes, void *stream);

/* QCudaStorage::fwd equivalent (cuda.rs:862-894): quantize x [m,k] f32, then GEMV (m <= 8) or GEMM.
 * Weight shape [n,k]; y f32 with row stride ldy >= n.  A GPU holding only weight rows
 * [n0, n0+n) of a larger matrix passes its shard as w_blocks and y + n0 with the full row stride:
 * per-row arithmetic does not depend on the shard, so sharded == unsharded bit for bit. */
int lloom_b200_qmatmul_fwd(int w_dtype, const void *w_blocks, const float *x, float *y, int64_t m, int64_t n,
                           int64_t k, int64_t ldy, void *workspace, int64_t workspace_bytes, void *stream);

/* Decode forward for callers that have no way to provide scratch memory.  (No counterpart in the
 * reference: its CUDA path always allocates its Q8_1 scratch through cudarc.)
 *
 * Who needs it: code that runs where device allocation is off limits -- a host thread that must not
 * call cudaMalloc because allocation synchronises the device or is reserved to another component,
 * a plugin handed only input and output buffers by its framework, a tight decode loop that wants
 * zero allocator traffic.  Same result as lloom_b200_qmatmul_fwd for 1 <= m <= 8 (bit for bit: the
 * same kernels run), but the quantized activations live in a fixed array inside the library
 * instead of a caller workspace.
 *
 * Limits and rules:
 *   - m <= 8 and m * lloom_b200_act_row_bytes(w_dtype, k) <= LLOOM_B200_STATIC_SCRATCH_BYTES
 *     (256 KiB: e.g. m = 8 with k up to 28672 for Q4_K / Q6_K); anything larger returns
 *     LLOOM_ERR_STATIC_LIMIT and launches nothing.
 *   - Every GPU that loads the library holds that array until the process exits.
 *   - The first call on each device looks up the array's device address (one cudaGetSymbolAddress,
 *     with that device current).  Make that first call outside any stream capture.
 *   - All calls on a device share the one array, and it keeps whatever the previous call wrote.  Each call
 *     overwrites every byte it later reads, so nothing needs clearing, but two calls whose kernels
 *     overlap on the GPU (different streams, no ordering) race on it: serialise them.
 *   - It calls no cudaMalloc / cudaFree and no allocating library routine. */
#define LLOOM_B200_STATIC_SCRATCH_BYTES (256 * 1024)
int lloom_b200_qmatmul_fwd_static(int w_dtype, const void *w_blocks, const float *x, float *y, int64_t m, int64_t n,
                                  int64_t k, int64_t ldy, void *stream);

/* QCudaStorage::dequantize / dequantize_f16 (cuda.rs:647-718; CPU T::to_float k_quants.rs:720-736,
 * 1747-1774, 2327-2358): elem_count elements (a multiple of the block size) to f32 or f16. */
int lloom_b200_dequantize(int dtype, const void *blocks, int64_t elem_count, void *out, int out_is_f16,
                          void *stream);

/* QCudaStorage::embedding / get_rows (cuda.rs:225-316, 828-860): out[i, :] = to_float(row ids[i]),
 * table [rows][hidden/block] blocks, ids u32 on device, out f32 [n_ids, hidden].  Ids >= rows yield zeros. */
int lloom_b200_get_rows(int dtype, const void *blocks, int64_t rows, int64_t hidden, const uint32_t *ids,
                        int64_t n_ids, float *out, void *stream);

/* ---- Blocks on the GEMV's store: the reference's MvStore (mod.rs:1668-1696) ----
 * QMatMul::forward_silu (mod.rs:2105-2122): y = silu(W.x), SiLU as v / (1 + exp(-v)) in f32 (op.rs:755-757).
 * QMatMul::forward_mul_into (mod.rs:2124-2155): y <- y * (W.x) in y's own buffer, the SwiGLU's up projection
 * landing as silu(g) * u.  One launch each (plus the quantizer kernel for 3..8 rows), no extra pass over y.
 * Like the reference's store blocks they serve the matvec path only: m <= 8, else LLOOM_ERR_SHAPE and the caller
 * composes.  Other arguments as lloom_b200_qmatmul_fwd. */
#define LLOOM_STORE_PLAIN 0
#define LLOOM_STORE_SILU 1
#define LLOOM_STORE_MUL_INTO 2
int lloom_b200_qmatmul_fwd_store(int w_dtype, const void *w_blocks, const float *x, float *y, int64_t m, int64_t n,
                                 int64_t k, int64_t ldy, int store, void *workspace, int64_t workspace_bytes,
                                 void *stream);

/* ---- Grouped decode forward: several weight matrices that share one activation, one launch ----
 * The reference's callers run gate|up (lloom/src/models/quantized_lfm2.rs:20-23) and q|k|v as separate
 * QMatMul::forward calls on the same input; each pays a launch and re-quantizes the activations.  This entry
 * streams up to LLOOM_B200_MAX_GROUP matrices of one dtype and one k, in the order given, with one activation read:
 * for one activation row (and two rows of the formats without a tensor-core GEMV) a single persistent launch walks
 * the concatenated rows; for wider batches the activations are quantized once and each matrix gets its GEMV launch.
 * ys[g] f32 [m][ldys[g]], ns[g] rows of matrix g, stores[g] one of LLOOM_STORE_* (NULL = all plain; MUL_INTO reads
 * and writes ys[g]).  Each matrix's result is bit-identical to its own lloom_b200_qmatmul_fwd.  m <= 8.
 * workspace: lloom_b200_workspace_bytes(w_dtype, m, max ns, k). */
#define LLOOM_B200_MAX_GROUP 8
int lloom_b200_qmatmul_fwd_group(int w_dtype, int n_mats, const void *const *w_blocks, const float *x, float *const *ys,
                                 const int64_t *ns, const int64_t *ldys, const int *stores, int64_t m, int64_t k,
                                 void *workspace, int64_t workspace_bytes, void *stream);

/* ---- Routed mixture-of-experts forward: QCudaStorage::indexed_moe_forward (cuda.rs:505-622) ----
 * w_experts: [n_experts][n][k / block] canonical blocks (one stacked tensor, 16-byte aligned); x f32 [batch][in_dim1][k] with in_dim1 == 1 or topk; ids u32 [batch][topk] ON THE DEVICE;
 * out f32 [batch][topk][n]:  out[b][t] = W[ids[b][t]] . x[b][in_dim1 == 1 ? 0 : t].
 * Each (token, expert) product is bit-identical to lloom_b200_qmatmul_fwd of that expert's matrix on that row (the
 * activations are quantized to Q8_0 / Q8_K as on the dense path, where the reference's CUDA arm uses Q8_1).  One
 * persistent launch per token walks that token's topk experts behind one activation read (in_dim1 == 1; topk <=
 * LLOOM_B200_MAX_GROUP), else one launch per (token, expert); the expert ids are read on the device, after the
 * kernel before this one in the stream has finished.  An id >= n_experts is clamped to the last expert and sets the
 * device status word to LLOOM_ERR_SHAPE (lloom_b200_device_status).  Meant for decode-sized batches.
 * workspace: lloom_b200_workspace_bytes(w_dtype, 1, n, k). */
int lloom_b200_indexed_moe_forward(int w_dtype, const void *w_experts, int64_t n_experts, int64_t n, int64_t k,
                                   const float *x, int64_t batch, int64_t in_dim1, const uint32_t *ids, int64_t topk,
                                   float *out, void *workspace, int64_t workspace_bytes, void *stream);

/* ---- Row-sharded forward with the all-gather fused into the GEMV (one node, up to 8 GPUs) ----
 *
 * The reference shards nothing on this path; the sharded layer here (rank g owns rows [g*ceil(n/G), ...), the
 * logits are concatenated) normally ends in an NCCL all-gather.  This entry replaces that collective for decode
 * batches: the GEMV stores every output value straight into the output buffer of each GPU (peer memory over
 * NVLink), so the exchange overlaps the computation and costs no extra launch except the barrier below.
 *
 *   y_peers   host array of n_peers device pointers: the [m][ldy] f32 output buffer of every GPU of the group,
 *             own buffer included, all mapped into this process (lloom_b200_peer_open); index = rank
 *   col0      first output column of this shard (its first weight row in the unsharded matrix)
 *   m <= 8; other arguments as lloom_b200_qmatmul_fwd.
 * After it, lloom_b200_peer_barrier on the same stream; the gathered rows are complete on this GPU when that
 * kernel has finished.  A buffer may be written again only after every GPU has finished reading it (alternate
 * two buffers, as the Python layer does). */
int lloom_b200_qmatmul_fwd_gather(int w_dtype, const void *w_shard, const float *x, int64_t m, int64_t n_shard, int64_t k,
                                  int64_t ldy, int64_t col0, float *const *y_peers, int n_peers, void *workspace,
                                  int64_t workspace_bytes, void *stream);
/* flag_peers: host array of n_peers device pointers, the flag array (LLOOM_B200_PEER_FLAG_WORDS u32, zeroed once)
 * of every GPU, mapped into this process.  Bounded wait: LLOOM_ERR_TIMEOUT shows in lloom_b200_device_status. */
#define LLOOM_B200_PEER_FLAG_WORDS 16
int lloom_b200_peer_barrier(int rank, int n_peers, unsigned int *const *flag_peers, void *stream);
/* The same gather with the barrier folded into the GEMV: the last CTA to finish on each GPU publishes that GPU's
 * call counter into slot [rank] of every GPU's flag array (after a system-scope fence behind its peer stores), so no
 * barrier kernel runs between the GEMV and its consumer.  The consumer waits (bounded) until all n_peers slots of its
 * own flag array have reached its own counter: either lloom_b200_peer_wait on the same stream, or the next forward
 * on the gathered rows itself -- pass the gather's own-GPU flag array as `wait_flags` to the next
 * lloom_b200_qmatmul_fwd_gather_sync / lloom_b200_qmatmul_fwd_after_gather (m <= 2: the wait then sits in the GEMV's
 * quantizer prologue, behind its weight prefetch).  A flag array serves one gathered buffer pair on one stream; words
 * [8] and [9] of it are the GPU's call counter and CTA arrival counter.  flag_peers as for lloom_b200_peer_barrier
 * (do not mix the two protocols on one flag array).  wait_flags may be NULL. */
int lloom_b200_qmatmul_fwd_gather_sync(int w_dtype, const void *w_shard, const float *x, int64_t m, int64_t n_shard,
                                       int64_t k, int64_t ldy, int64_t col0, float *const *y_peers, int n_peers, int rank,
                                       unsigned int *const *flag_peers, const unsigned int *wait_flags, void *workspace,
                                       int64_t workspace_bytes, void *stream);
/* An ordinary (replicated) decode forward whose activations are the output of a gather_sync: waits on that gather's
 * flags in its prologue.  m <= 2. */
int lloom_b200_qmatmul_fwd_after_gather(int w_dtype, const void *w_blocks, const float *x, float *y, int64_t m, int64_t n,
                                        int64_t k, int64_t ldy, const unsigned int *wait_flags, int n_peers,
                                        void *workspace, int64_t workspace_bytes, void *stream);
/* One-warp kernel that waits (bounded) for the last gather_sync on this stream to be complete on this GPU. */
int lloom_b200_peer_wait(int n_peers, const unsigned int *flags_own, void *stream);
/* Set-up helpers (not on the forward path; these do allocate / synchronise): a zeroed device buffer other processes
 * of the node can map, its 64-byte CUDA IPC handle, mapping a peer's handle, and the matching releases. */
int lloom_b200_peer_alloc(int64_t bytes, void **ptr);
int lloom_b200_peer_free(void *ptr);
int lloom_b200_peer_export(const void *ptr, unsigned char *handle64);
int lloom_b200_peer_open(const unsigned char *handle64, void **ptr);
int lloom_b200_peer_close(void *ptr);

#ifdef __cplusplus
}
#endif
#endif
