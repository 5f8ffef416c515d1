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

// ---- tensor-parallel exchange: a sum of partial outputs over the ranks of one box, pushed ----
// Every rank owns an exchange area that all its peers have mapped (cudaIpc): two alternating buffers,
// each with one slot array per source rank.  A partial output travels as ONE 64-bit word per value,
// {float bits, sequence number of the exchange}, stored straight into every rank's area (the own one
// included) by the kernel that produced it; the consumer polls its LOCAL area until the word carries the
// expected sequence number, so there is no separate flag, no fence and no remote read on the critical path.
// The sequence number of the next exchange is (completed exchanges + 1), kept in device memory and advanced
// by the last CTA of the consuming kernel, so graph replays stay in step; the buffer is (sequence & 1).  A
// buffer is rewritten two exchanges later, which a rank can only reach after every peer has finished
// reading it (a peer's words of the exchange in between are stored after its own read completed).
constexpr int QMM_TP_MAX = 8;
struct TpPush {                          // by value in the matvec kernels' parameters; tp == 0: plain stores to y
    unsigned long long* dst[QMM_TP_MAX];  // dst[r]: this rank's slot array in rank r's area (buffer 0)
    const unsigned* counter;              // exchanges completed on this rank
    long buf_words;                       // words from buffer 0 to buffer 1
    long word0;                           // slot index of y[0][0]; y[mi][row] goes to word0 + mi * y_stride + row
    int tp;
};
struct TpRecv {                          // the consuming side
    const unsigned long long* base;       // own area, buffer 0, source rank 0
    unsigned* counter;                    // exchanges completed (advanced by the last CTA of the consumer)
    unsigned* ticket;                     // CTAs of the consumer that have finished
    long buf_words, src_words;            // words between the buffers, and between the slot arrays of two source ranks
    int tp;
};
__device__ __forceinline__ unsigned ld_volatile_u32(const unsigned* p) {
    unsigned v;
    asm volatile("ld.volatile.global.u32 %0, [%1];" : "=r"(v) : "l"(p));
    return v;
}
__device__ __forceinline__ unsigned tp_next_seq(const unsigned* counter) { return ld_volatile_u32(counter) + 1u; }
__device__ __forceinline__ void tp_push_word(const TpPush& s, unsigned seq, long word, float v) {
    const unsigned long long bits = ((unsigned long long)seq << 32) | (unsigned long long)__float_as_uint(v);
    const long off = ((seq & 1u) ? s.buf_words : 0) + word;
#pragma unroll
    for (int r = 0; r < QMM_TP_MAX; ++r)
        if (r < s.tp) asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(s.dst[r] + off), "l"(bits) : "memory");
}
// one output of a matvec: an ordinary store, or the push to every rank
__device__ __forceinline__ void tp_store_out(const TpPush& s, unsigned seq, float* y, long y_stride, int mi, long row, float v) {
    if (s.tp > 0)
        tp_push_word(s, seq, s.word0 + (long)mi * y_stride + row, v);
    else
        y[(size_t)mi * y_stride + row] = v;
}
// Polls the word of source rank r (bounded): true and the value once it carries `seq`.
__device__ __forceinline__ bool tp_poll_word(const TpRecv& rcv, unsigned seq, int r, long word, float& v, volatile int* give_up) {
    const unsigned long long* p = rcv.base + ((seq & 1u) ? rcv.buf_words : 0) + (long)r * rcv.src_words + word;
    unsigned long long bits;
    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(bits) : "l"(p) : "memory");
    if ((unsigned)(bits >> 32) != seq) {
        const long long t0 = clock64();
        for (;;) {
            asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(bits) : "l"(p) : "memory");
            if ((unsigned)(bits >> 32) == seq) break;
            if (*give_up || clock64() - t0 > WAIT_LIMIT_CYCLES) {
                *give_up = 1;
                return false;
            }
        }
    }
    v = __uint_as_float((unsigned)bits);
    return true;
}
// End of the consuming kernel (one thread per CTA, after the CTA's last read): the last CTA advances the counter.
__device__ __forceinline__ void tp_consumer_done(const TpRecv& rcv, unsigned seq, unsigned n_ctas) {
    __threadfence();
    if (atomicAdd(rcv.ticket, 1u) == n_ctas - 1u) {
        *rcv.ticket = 0u;
        __threadfence();
        *reinterpret_cast<volatile unsigned*>(rcv.counter) = seq;
    }
}

#endif  // __CUDACC__
}  // namespace qmm
