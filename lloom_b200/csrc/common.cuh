// Shared device helpers: GGUF block layouts, mbarrier / bulk-copy PTX wrappers, status word.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/lloom_b200.h"

namespace lloom {

constexpr int QK8_0 = 32;
constexpr int QK_K = 256;
constexpr int Q8_0_BYTES = 34;
constexpr int Q4K_BYTES = 144;
constexpr int Q6K_BYTES = 210;
constexpr int Q8K_BYTES = 292;
constexpr int Q4_0_BYTES = 18;
constexpr int Q5_0_BYTES = 22;
constexpr int Q5K_BYTES = 176;

// Field offsets inside the canonical blocks (lloom-tensor/src/quantized/k_quants.rs:155-159, 217-223, 255-261, 265-270).
// Q8_0 : f16 d @0, i8 qs[32] @2
// Q4_K : f16 d @0, f16 dmin @2, u8 scales[12] @4, u8 qs[128] @16
// Q6_K : u8 ql[128] @0, u8 qh[64] @128, i8 scales[16] @192, f16 d @208
// Q8_K : f32 d @0, i8 qs[256] @4, i16 bsums[16] @260
// Q4_0 : f16 d @0, u8 qs[16] @2                                   (k_quants.rs:84-91)
// Q5_0 : f16 d @0, u8 qh[4] @2, u8 qs[16] @6                      (k_quants.rs:117-125)
// Q5_K : f16 d @0, f16 dmin @2, u8 scales[12] @4, u8 qh[32] @16, u8 qs[128] @48   (k_quants.rs:184-192)

// Device-side status word: 0, or LLOOM_ERR_TIMEOUT once a bounded wait gave up, and the time limit of those
// waits.  The library is several translation units compiled without relocatable device code, so each unit has
// its own copy of both; LLOOM_TU_REGISTER (below) hands the host-side accessors of a unit's copies to the ABI
// unit, which reads / writes all of them (lloom_b200_device_status, lloom_b200_set_wait_limit_ns).
static __device__ int g_device_status = 0;
static __device__ int g_status_fetch = 0;  // landing place of the atomic read-and-clear
constexpr unsigned long long kDefaultWaitNs = 2000000000ull;  // 2 s
static __device__ unsigned long long g_wait_limit_ns = kDefaultWaitNs;

struct TuHooks {
    cudaError_t (*fetch_status)(int *status, cudaStream_t stream);  // read-and-clear, atomic on the device
    cudaError_t (*set_wait_limit)(unsigned long long ns);
};
void register_tu(const TuHooks &hooks);  // lloom_b200.cu

static __global__ void status_fetch_kernel() { g_status_fetch = atomicExch(&g_device_status, 0); }

#define LLOOM_TU_REGISTER()                                                                                    \
    namespace {                                                                                                \
    cudaError_t tu_fetch_status(int *status, cudaStream_t stream) {                                            \
        status_fetch_kernel<<<1, 1, 0, stream>>>();                                                            \
        cudaError_t e = cudaGetLastError();                                                                    \
        if (e != cudaSuccess) return e;                                                                        \
        return cudaMemcpyFromSymbol(status, g_status_fetch, sizeof(int));                                      \
    }                                                                                                          \
    cudaError_t tu_set_wait_limit(unsigned long long ns) {                                                     \
        return cudaMemcpyToSymbol(g_wait_limit_ns, &ns, sizeof(ns));                                           \
    }                                                                                                          \
    const int tu_registered = (::lloom::register_tu({tu_fetch_status, tu_set_wait_limit}), 0);                 \
    }

__host__ __device__ inline int64_t ceil_div64(int64_t a, int64_t b) { return (a + b - 1) / b; }

// ---- mbarrier / bulk async copy (TMA engine, untiled) ----

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
// Makes `v` a value the compiler must have computed at this point of the program (no instruction of its own).  Used
// before a shared-memory stage is handed back to the bulk-copy engine: when every running sum the stage's loads feed
// has been computed, those loads have returned -- the hardware only issues an instruction whose operands have arrived,
// and issues in program order -- so the release that follows cannot overtake them.  (A consumer that released a
// buffer while a load from it was still in flight read the next copy's bytes: seen in the GEMM epilogue, whose
// scale-tile reads are therefore fenced with fence.proxy.async.)
__device__ __forceinline__ void pin_value(float &v) { asm volatile("" : "+f"(v)); }
__device__ __forceinline__ void pin_value(int &v) { asm volatile("" : "+r"(v)); }

__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait: every spin in this library is limited both in polls and in wall time (a single
// mbarrier.try_wait may itself suspend the thread for a while, so a poll count alone is not a time
// bound).  On expiry the status word is set and false is returned; the caller unwinds (no trap, the
// context stays usable).
constexpr uint32_t kMaxSpins = 1u << 24;
__device__ __forceinline__ unsigned long long wait_limit_ns() { return *(volatile unsigned long long *)&g_wait_limit_ns; }
__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity) {
    unsigned long long t0 = 0;
    for (uint32_t i = 0; i < kMaxSpins; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 255) == 255) {
            const unsigned long long now = global_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > wait_limit_ns()) break;
            __nanosleep(64);
        }
    }
    atomicExch(&g_device_status, LLOOM_ERR_TIMEOUT);
    return false;
}

// global -> shared bulk copy; src, dst and bytes are multiples of 16.  Completion is signalled on `bar`.
__device__ __forceinline__ void bulk_g2s(void *dst_smem, const void *src_gmem, uint32_t bytes, uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
            smem_u32(dst_smem)),
        "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}

// ---- small arithmetic helpers ----

__device__ __forceinline__ float f16_bits_to_f32(uint32_t h) {
    return __half2float(__ushort_as_half((unsigned short)h));
}

// utils.rs:50-60 get_scale_min_k4 on the 12 scale bytes held as three little-endian words.
__device__ __forceinline__ void q4k_scale_min(const uint32_t s[3], int j, int &sc, int &mn) {
    // byte i of the 12: (s[i>>2] >> (8*(i&3))) & 0xff
    auto byte_at = [&](int i) -> uint32_t { return (s[i >> 2] >> (8 * (i & 3))) & 0xffu; };
    if (j < 4) {
        sc = byte_at(j) & 63;
        mn = byte_at(j + 4) & 63;
    } else {
        sc = (byte_at(j + 4) & 0xF) | ((byte_at(j - 4) >> 6) << 4);
        mn = (byte_at(j + 4) >> 4) | ((byte_at(j) >> 6) << 4);
    }
}

}  // namespace lloom
