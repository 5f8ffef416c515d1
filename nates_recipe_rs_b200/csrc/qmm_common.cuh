// Shared device/host helpers for libqmm (sm_100a only).
#pragma once
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include "../../include/qmm.h"

namespace qmm {

constexpr int QK8 = 32;
constexpr int QKK = 256;
constexpr int Q8_0_BYTES = 34;
constexpr int Q8_1_BYTES = 36;
constexpr int Q4_K_BYTES = 144;
constexpr int Q6_K_BYTES = 210;

// Device status word: a kernel that gives up on a bounded wait stores a non-zero
// code here and returns; the host reads it through qmm_device_status().
enum DeviceStatus : int {
    DEV_OK = 0,
    DEV_TIMEOUT_FULL = 1,   // consumer gave up waiting for a staged tile
    DEV_TIMEOUT_EMPTY = 2,  // producer gave up waiting for a free stage
    DEV_TIMEOUT_DRAIN = 3,  // producer gave up waiting for its own copies at exit
    DEV_TIMEOUT_MMA = 4,    // GEMM: gave up waiting for tensor-core completion
    DEV_TIMEOUT_PEER = 5,   // allreduce: gave up waiting for a peer's flag
};
// (libqmm is built as ONE translation unit, so this is a single word per device.)
static __device__ int g_device_status = 0;

// thread-local record of the last failing CUDA runtime call
void set_last_cuda_error(cudaError_t e);
inline int cuda_fail(cudaError_t e) {
    set_last_cuda_error(e);
    return QMM_ERR_CUDA;
}
#define QMM_CUDA_TRY(expr)                                  \
    do {                                                    \
        cudaError_t _e = (expr);                            \
        if (_e != cudaSuccess) return ::qmm::cuda_fail(_e); \
    } while (0)

int sm_count();           // SM count of the current device (cached per device)
bool overlap_enabled();   // programmatic dependent launch on/off

static inline cudaStream_t as_stream(void* s) { return reinterpret_cast<cudaStream_t>(s); }

// ------------------------------------------------------------------ device
#ifdef __CUDACC__

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ float f16_bits_to_f32(uint32_t h) {
    return __half2float(__ushort_as_half(static_cast<unsigned short>(h)));
}

__device__ __forceinline__ uint64_t globaltimer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// ---- mbarrier (shared::cta, 64-bit) ----
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("{ .reg .b64 st; mbarrier.arrive.shared::cta.b64 st, [%0]; }" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("{ .reg .b64 st; mbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1; }" ::"r"(bar), "r"(bytes)
                 : "memory");
}
// One potentially-blocking probe of a phase: the hardware parks the thread until the
// phase completes or a short time slice ends, so a waiting warp costs almost no issue
// slots (a test_wait polling loop was measured to execute 4x more instructions than
// the arithmetic of the whole kernel).
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

// Non-blocking probe of a phase
__device__ __forceinline__ bool mbar_test_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{ .reg .pred p; mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

// Bounded wait: polls the barrier; gives up after WAIT_LIMIT_CYCLES of the SM clock
// (about 2 s at the boost clock, longer at lower clocks, never unbounded) or at once
// when another thread of the CTA has already given up; the caller then records a
// status code and unwinds without touching the data.  The SM cycle counter is used
// because it is a plain register read; the global nanosecond timer is not.
constexpr long long WAIT_LIMIT_CYCLES = 4000000000ll;
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity, volatile int* cta_abort) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 256; ++i)
            if (mbar_try_wait(bar, parity)) return true;
        if (*cta_abort) return false;
        if (clock64() - t0 > WAIT_LIMIT_CYCLES) return false;
    }
}

// 1-D bulk async copy global -> shared, completion counted on an mbarrier.
// Both addresses 16-byte aligned, bytes a multiple of 16.
__device__ __forceinline__ void bulk_g2s(uint32_t smem_dst, const void* gsrc, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_dst),
                 "l"(gsrc), "r"(bytes), "r"(bar)
                 : "memory");
}

// Programmatic dependent launch controls (no-ops when the launch does not use it)
__device__ __forceinline__ void pdl_wait_prior_grids() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_release_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__device__ __forceinline__ int dp4a_ss(int a, int b, int c) { return __dp4a(a, b, c); }

// 32-bit word at a 2-byte aligned shared-memory address
__device__ __forceinline__ uint32_t lds_u32_align2(const uint8_t* p) {
    const uintptr_t a = reinterpret_cast<uintptr_t>(p);
    const uint32_t* q = reinterpret_cast<const uint32_t*>(a & ~uintptr_t(3));
    const uint32_t sh = (a & 2u) * 8u;
    return __funnelshift_r(q[0], q[1], sh);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

#endif  // __CUDACC__
}  // namespace qmm
