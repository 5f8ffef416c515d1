// Prefill dequant-GEMM on the 5th-generation tensor cores:
//     y(m,n) = bf16( sum_k x(m,k) * bf16(dequant(w(n,k))) ),   x, y bf16, w Q4_K, fp32 accumulate.
// The dense-contraction counterpart of the decode matvec; it replaces the same upstream
// pair (widen window + gpu_gemm_bt_f64_into, gpu-core/src/infer_ops.rs:85-101, 224-240) when
// m is in the hundreds.
//
// One CTA owns 128 weight rows for up to 512 rows of x.  The WEIGHTS are the M = 128 operand of the
// instruction and 256 rows of x its N: a tcgen05.mma costs the issuing thread about 70 ns whatever its N
// (measured: M128 N64/N128/N256 K16 all 63-72 ns back to back, a commit about as much again), so only N = 256
// reaches the tensor cores' rate, and the accumulator is the TRANSPOSED output tile (weight row = TMEM lane,
// row of x = TMEM column).  Warp roles:
//   warp 0      TMA producer: x tiles (256 rows x 64 k, 128-byte swizzle), one or two per k-step
//   warp 18     TMA producer: the packed super-blocks of the 128 weight rows (128 x 144 bytes, four k-steps),
//               one super-block ahead (the unpack threads make no global loads: the proxy fence they need
//               after every tile would otherwise wait for their own prefetches)
//   warps 1, 19 one lane each issues the tcgen05.mma (128x256x16, bf16 -> f32 in TMEM) of ONE block of 256 rows
//               of x and one tcgen05.commit per k-step, on a barrier that frees the weight slot and the x slot
//               together.  The issuing thread is the critical path (its waits, fence and commit add to the
//               ~130 cycles each instruction takes to issue), so each block has its own; warp 1 also owns
//               the TMEM allocation
//   warps 2..17 unpack one 32-byte group of qs per row and k-step (= 64 weights = one 128-byte
//               swizzled row of the weight tile) into a 3-slot ring, then run the epilogue
// A k-step is 64 elements: exactly one group of a Q4_K super-block, so the tile row of a
// weight row is one group of that row's current super-block.
// Accumulators: one or two 128x256 f32 blocks = up to all 512 TMEM columns; the epilogue reads them
// with tcgen05.ld (32 lanes x 32 columns per warp), rounds to bf16 and stores (the 32 lanes of a warp
// write 32 consecutive outputs of one row of y).
// Every wait is bounded; on expiry the CTA records a status code, drains its copies, frees
// its TMEM and returns.
#include "qmm_formats.cuh"
#include <cuda.h>

namespace qmm {

constexpr int GEMM_BW = 128;   // weight rows per CTA: the M of the instruction
constexpr int GEMM_BX = 256;   // rows of x per block: the N of the instruction
constexpr int GEMM_BK = 64, GEMM_NB_MAX = 2;
constexpr int GEMM_SW = 3;     // weight-tile slots
constexpr int GEMM_ND = 4;     // barriers that track finished k-steps (at least as many as any ring has slots)
constexpr int GEMM_XT = 4;     // x tiles in the ring: GEMM_XT / (blocks per CTA) k-steps
constexpr int GEMM_SP = 2;     // packed super-block slots
constexpr int GEMM_P_BYTES = GEMM_BW * Q4_K_BYTES;   // 18 KB: 128 rows x one super-block
constexpr int GEMM_W_BYTES = GEMM_BW * GEMM_BK * 2;  // 16 KB: 128 rows x 128 bytes
constexpr int GEMM_X_BYTES = GEMM_BX * GEMM_BK * 2;  // 32 KB: 256 rows x 128 bytes
constexpr int GEMM_DEQ_WARPS = 16;
constexpr int GEMM_THREADS = (4 + GEMM_DEQ_WARPS) * 32;
constexpr int GEMM_WARP_PACKED = 2 + GEMM_DEQ_WARPS, GEMM_WARP_MMA1 = 3 + GEMM_DEQ_WARPS;
constexpr uint32_t GEMM_TMEM_COLS = 512;
// instruction descriptor: D f32, A bf16, B bf16, both K-major, N = 256, M = 128
constexpr uint32_t GEMM_IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((GEMM_BX >> 3) << 17) | ((GEMM_BW >> 4) << 24);

struct GemmParams {
    const uint8_t* w;     // Q4_K rows (n, k)
    __nv_bfloat16* y;     // (m, n) bf16, may be null when yf is given
    float* yf;            // optional (m, n) f32 copy of the accumulators
    int m, n, k;
    int row_bytes;
    int probe;            // tuning aid: 0 normal, 1 = unpack arithmetic skipped, 2 = tensor-core work skipped
    int nb_per_cta;       // 256-row blocks of x per CTA (1..GEMM_NB_MAX)
    int ksplit;           // CTAs of a cluster that share one output tile, each with a contiguous part of K (1 or 2)
    int w_bf16;           // 1: the weights are bf16 rows (n, k) and reach the weight ring by TMA; nothing is unpacked
};

struct __align__(16) GemmSmemHeader {
    uint64_t w_full[GEMM_SW];   // a weight tile is unpacked (one arrival per unpack warp)
    uint64_t x_full[GEMM_XT];   // the x tiles of a k-step have landed
    uint64_t done[GEMM_ND];     // the tensor-core work of k-step ks (ks % GEMM_ND) has retired: both its slots are free
    uint64_t p_full[GEMM_SP];   // a packed super-block has landed
    uint64_t p_empty[GEMM_SP];  // ... and every unpack warp has read it
    uint64_t acc_full;
    uint32_t tmem_base;
    int abort_flag;
};

__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr) {
    // K-major, 128-byte swizzle: rows of 128 bytes, 8-row groups 1024 bytes apart
    return (uint64_t)((smem_addr & 0x3FFFFu) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) |
           ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{ .reg .pred p; setp.ne.b32 p, %4, 0; tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p; }" ::"r"(d_tmem),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// barrier over all threads of all CTAs of the cluster, with release/acquire ordering of (distributed) shared memory
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tma_load_2d(uint32_t smem_dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
                     smem_dst),
                 "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar)
                 : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, "
        "%18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n\t"
        "tcgen05.wait::ld.sync.aligned;"  // in the same statement: the registers must not be read before the wait
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]),
          "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]),
          "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}

// 8 weights of one sub-block from two words holding one nibble per byte:
// value = (ds*q) - off with each operation rounded, then pairs rounded to bf16 (RNE) = one 16-byte chunk.
__device__ __forceinline__ uint4 q4k_to_bf16x8(uint32_t t0, uint32_t t1, float ds, float off) {
    uint32_t o[4];
    const uint32_t t[2] = {t0, t1};
#pragma unroll
    for (int w = 0; w < 2; ++w) {
        float v[4];
#pragma unroll
        for (int b = 0; b < 4; ++b) v[b] = __fsub_rn(__fmul_rn(ds, byte_to_float(t[w], b)), off);
        const __nv_bfloat162 p0 = __floats2bfloat162_rn(v[0], v[1]), p1 = __floats2bfloat162_rn(v[2], v[3]);
        o[2 * w] = *reinterpret_cast<const uint32_t*>(&p0);
        o[2 * w + 1] = *reinterpret_cast<const uint32_t*>(&p1);
    }
    return make_uint4(o[0], o[1], o[2], o[3]);
}

__global__ void __launch_bounds__(GEMM_THREADS, 1) qgemm_q4k_kernel(const __grid_constant__ CUtensorMap xmap, const __grid_constant__ CUtensorMap wmap,
                                                                    const GemmParams p) {
    extern __shared__ __align__(1024) uint8_t gsm[];
    // layout: [weight ring: SW x 16 KB][x ring: XT x 32 KB][packed ring: SP x 18 KB][header]; the base is aligned to 1024 by hand
    const uint32_t raw = smem_u32(gsm);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t* sm = gsm + (base - raw);
    uint8_t* w_ring = sm;
    uint8_t* x_ring = sm + GEMM_SW * GEMM_W_BYTES;
    uint8_t* p_ring = x_ring + GEMM_XT * GEMM_X_BYTES;
    GemmSmemHeader* hdr = reinterpret_cast<GemmSmemHeader*>(p_ring + GEMM_SP * GEMM_P_BYTES);
    volatile int* cta_abort = &hdr->abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = blockIdx.x * GEMM_BW;
    const int m0 = blockIdx.y * (GEMM_BX * p.nb_per_cta);
    const int nb = min(p.nb_per_cta, (p.m - m0 + GEMM_BX - 1) / GEMM_BX);
    const int xs_slots = GEMM_XT / p.nb_per_cta;  // k-steps of x in the ring
    // K range of this CTA: whole super-blocks; blockIdx.z is the rank in the cluster of p.ksplit CTAs
    const int split = (int)blockIdx.z;
    const int sb0 = split * (p.k / QKK) / p.ksplit, n_sb = (split + 1) * (p.k / QKK) / p.ksplit - sb0;
    const int kt = n_sb * (QKK / GEMM_BK), ks0 = sb0 * (QKK / GEMM_BK);

    if (threadIdx.x == 0) {
        for (int s = 0; s < GEMM_SW; ++s) mbar_init(smem_u32(&hdr->w_full[s]), p.w_bf16 ? 1 : GEMM_DEQ_WARPS);
        for (int s = 0; s < GEMM_ND; ++s) mbar_init(smem_u32(&hdr->done[s]), nb);  // one commit per block and k-step
        for (int s = 0; s < GEMM_XT; ++s) mbar_init(smem_u32(&hdr->x_full[s]), 1);
        for (int s = 0; s < GEMM_SP; ++s) mbar_init(smem_u32(&hdr->p_full[s]), 1), mbar_init(smem_u32(&hdr->p_empty[s]), GEMM_DEQ_WARPS);
        mbar_init(smem_u32(&hdr->acc_full), nb);
        hdr->abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&hdr->tmem_base)),
                     "r"(GEMM_TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = hdr->tmem_base;

    auto give_up = [&](int code) {
        if (!*cta_abort) {
            atomicExch(&g_device_status, code);
            *cta_abort = 1;
        }
    };
    // k-step ks has retired on the tensor cores (its commit has arrived)
    auto wait_done = [&](int ks) { return mbar_wait_bounded(smem_u32(&hdr->done[ks % GEMM_ND]), (ks / GEMM_ND) & 1, cta_abort); };
    bool role_ok = true;  // unpack warps: the main loop ran to its end

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer (x tiles)
        if (lane == 0) {
            int issued = 0;
            for (int ks = 0; ks < kt; ++ks, ++issued) {
                if (ks >= xs_slots && !wait_done(ks - xs_slots)) {
                    give_up(DEV_TIMEOUT_EMPTY);
                    break;
                }
                const int slot = ks % xs_slots;
                const uint32_t bar = smem_u32(&hdr->x_full[slot]);
                mbar_arrive_expect_tx(bar, (uint32_t)nb * GEMM_X_BYTES);
                for (int b = 0; b < nb; ++b)  // rows past m are filled with zeros
                    tma_load_2d(smem_u32(x_ring + (slot * p.nb_per_cta + b) * GEMM_X_BYTES), &xmap, (ks0 + ks) * GEMM_BK, m0 + b * GEMM_BX, bar);
            }
            if (*cta_abort) {
                // copies that were issued but perhaps not consumed: wait (bounded) for them to land
                for (int i = max(0, issued - xs_slots); i < issued; ++i) {
                    const long long t0 = clock64();
                    while (!mbar_try_wait(smem_u32(&hdr->x_full[i % xs_slots]), (i / xs_slots) & 1)) {
                        if (clock64() - t0 > WAIT_LIMIT_CYCLES) {
                            atomicExch(&g_device_status, DEV_TIMEOUT_DRAIN);
                            break;
                        }
                    }
                }
            }
        }
    } else if (warp == 1 || warp == GEMM_WARP_MMA1) {
        // ------------------------------------------------------------ MMA issuers: block b of the CTA's rows of x
        const int b = warp == 1 ? 0 : 1;
        if (lane == 0 && b < nb) {
            const uint32_t d_tmem = tmem_base + (uint32_t)b * GEMM_BX;
            for (int ks = 0; ks < kt; ++ks) {
                const int sw = ks % GEMM_SW, sx = ks % xs_slots;
                if (!mbar_wait_bounded(smem_u32(&hdr->x_full[sx]), (ks / xs_slots) & 1, cta_abort) ||
                    !mbar_wait_bounded(smem_u32(&hdr->w_full[sw]), (ks / GEMM_SW) & 1, cta_abort)) {
                    give_up(DEV_TIMEOUT_FULL);
                    break;
                }
                tc_fence_after();
                const uint64_t wdesc = umma_desc_sw128(smem_u32(w_ring + sw * GEMM_W_BYTES));
                const uint64_t xdesc = umma_desc_sw128(smem_u32(x_ring + (sx * p.nb_per_cta + b) * GEMM_X_BYTES));
#pragma unroll
                for (int k16 = 0; k16 < GEMM_BK / 16; ++k16)  // 32 bytes of K per instruction: +2 in 16-byte units
                    if (p.probe != 2) umma_bf16(d_tmem, wdesc + 2 * k16, xdesc + 2 * k16, GEMM_IDESC, (ks > 0 || k16 > 0) ? 1u : 0u);
                umma_commit(smem_u32(&hdr->done[ks % GEMM_ND]));  // frees the weight slot and the x slot when these MMAs retire
            }
            umma_commit(smem_u32(&hdr->acc_full));  // also on the give-up path, so the epilogue warps are released
        }
    } else if (warp == GEMM_WARP_PACKED) {
        // ------------------------------------------------------------ TMA producer (packed super-blocks, or bf16 weight tiles)
        if (lane == 0 && p.w_bf16) {
            // plain bf16 weights: one 128 x 64 tile per k-step straight into the weight ring (128-byte swizzle, as x)
            int issued = 0;
            for (int ks = 0; ks < kt; ++ks, ++issued) {
                if (ks >= GEMM_SW && !wait_done(ks - GEMM_SW)) {
                    give_up(DEV_TIMEOUT_EMPTY);
                    break;
                }
                const uint32_t bar = smem_u32(&hdr->w_full[ks % GEMM_SW]);
                mbar_arrive_expect_tx(bar, GEMM_W_BYTES);
                tma_load_2d(smem_u32(w_ring + (ks % GEMM_SW) * GEMM_W_BYTES), &wmap, (ks0 + ks) * GEMM_BK, n0, bar);  // rows past n: zeros
            }
            if (*cta_abort) {
                for (int i = max(0, issued - GEMM_SW); i < issued; ++i) {
                    const long long t0 = clock64();
                    while (!mbar_try_wait(smem_u32(&hdr->w_full[i % GEMM_SW]), (i / GEMM_SW) & 1)) {
                        if (clock64() - t0 > WAIT_LIMIT_CYCLES) {
                            atomicExch(&g_device_status, DEV_TIMEOUT_DRAIN);
                            break;
                        }
                    }
                }
            }
        } else if (lane == 0) {
            int issued = 0;
            for (int sb = 0; sb < n_sb; ++sb, ++issued) {
                const int slot = sb % GEMM_SP;
                if (sb >= GEMM_SP && !mbar_wait_bounded(smem_u32(&hdr->p_empty[slot]), ((sb / GEMM_SP) - 1) & 1, cta_abort)) {
                    give_up(DEV_TIMEOUT_EMPTY);
                    break;
                }
                const uint32_t bar = smem_u32(&hdr->p_full[slot]);
                mbar_arrive_expect_tx(bar, GEMM_P_BYTES);
                tma_load_2d(smem_u32(p_ring + slot * GEMM_P_BYTES), &wmap, (sb0 + sb) * Q4_K_BYTES, n0, bar);  // rows past n: zeros
            }
            if (*cta_abort) {
                for (int i = max(0, issued - GEMM_SP); i < issued; ++i) {
                    const long long t0 = clock64();
                    while (!mbar_try_wait(smem_u32(&hdr->p_full[i % GEMM_SP]), (i / GEMM_SP) & 1)) {
                        if (clock64() - t0 > WAIT_LIMIT_CYCLES) {
                            atomicExch(&g_device_status, DEV_TIMEOUT_DRAIN);
                            break;
                        }
                    }
                }
            }
        }
    } else {
        // ------------------------------------------------------------ unpack warps, then epilogue
        // thread = (weight row of the tile, which 8 bytes of the 32-byte group): consecutive lanes take
        // consecutive rows, so the eight lanes of a store phase hit eight different swizzle positions
        const int t = threadIdx.x - 64;          // 0..511
        const int row = t & 127, part = t >> 7;  // part 0..3
        const uint32_t row_off = (uint32_t)row * 128u, swz = (uint32_t)(row & 7);
        bool ok = true;
        for (int sb = 0; sb < (p.w_bf16 ? 0 : n_sb) && ok; ++sb) {
            // this row's super-block from the packed ring: header and this thread's 8 bytes of each group
            const int ps = sb % GEMM_SP;
            if (!mbar_wait_bounded(smem_u32(&hdr->p_full[ps]), (sb / GEMM_SP) & 1, cta_abort)) {
                if (lane == 0) give_up(DEV_TIMEOUT_FULL);
                ok = false;
                break;
            }
            const uint8_t* blk = p_ring + ps * GEMM_P_BYTES + row * Q4_K_BYTES;
            const uint4 hd = *reinterpret_cast<const uint4*>(blk);
            uint2 qv[4];
#pragma unroll
            for (int g = 0; g < 4; ++g) qv[g] = *reinterpret_cast<const uint2*>(blk + 16 + 32 * g + 8 * part);
            // 6-bit scale / min codes, one per byte: A = sub-blocks 0..3, B = 4..7
            const uint32_t scA = hd.y & 0x3F3F3F3Fu, mA = hd.z & 0x3F3F3F3Fu;
            const uint32_t scB = (hd.w & 0x0F0F0F0Fu) | ((hd.y >> 2) & 0x30303030u);
            const uint32_t mB = ((hd.w >> 4) & 0x0F0F0F0Fu) | ((hd.z >> 2) & 0x30303030u);
            const float d = f16_bits_to_f32(hd.x & 0xFFFFu), dmin = f16_bits_to_f32(hd.x >> 16);
#pragma unroll
            for (int g = 0; g < 4; ++g) {
                const int ks = sb * 4 + g;
                // sub-blocks 2g (low nibbles) and 2g+1 (high nibbles)
                const uint32_t sc4 = g < 2 ? scA : scB, m4 = g < 2 ? mA : mB;
                const uint32_t i0 = (uint32_t)(2 * g) & 3u;
                const float ds0 = __fmul_rn(d, byte_to_float(sc4, i0)), off0 = __fmul_rn(dmin, byte_to_float(m4, i0));
                const float ds1 = __fmul_rn(d, byte_to_float(sc4, i0 + 1)), off1 = __fmul_rn(dmin, byte_to_float(m4, i0 + 1));
                // bytes 8*part .. 8*part+7 of the group: low nibbles = elements 8*part.. (chunk part),
                // high nibbles = elements 32+8*part.. (chunk 4+part)
                const uint2 qs = qv[g];
                uint4 c_lo, c_hi;
                if (p.probe != 1) {
                    c_lo = q4k_to_bf16x8(qs.x & 0x0F0F0F0Fu, qs.y & 0x0F0F0F0Fu, ds0, off0);
                    c_hi = q4k_to_bf16x8((qs.x >> 4) & 0x0F0F0F0Fu, (qs.y >> 4) & 0x0F0F0F0Fu, ds1, off1);
                } else {
                    c_lo = make_uint4(qs.x, qs.y, hd.x, hd.y);
                    c_hi = c_lo;
                }
                const int sw = ks % GEMM_SW;
                if (ks >= GEMM_SW && !wait_done(ks - GEMM_SW)) {
                    if (lane == 0) give_up(DEV_TIMEOUT_EMPTY);
                    ok = false;
                    break;
                }
                uint8_t* tile = w_ring + sw * GEMM_W_BYTES + row_off;
                *reinterpret_cast<uint4*>(tile + ((((uint32_t)part + 0) ^ swz) << 4)) = c_lo;
                *reinterpret_cast<uint4*>(tile + ((((uint32_t)part + 4) ^ swz) << 4)) = c_hi;
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic-proxy stores -> tensor-core reads
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(smem_u32(&hdr->w_full[sw]));
                    if (g == 0) mbar_arrive(smem_u32(&hdr->p_empty[ps]));  // the super-block is in registers: its slot may be refilled
                }
            }
        }
        role_ok = ok;
    }

    // ---- epilogue (the unpack warps): TMEM -> registers -> bf16 -> global.  Lane = weight row, column = row of x.
    const bool is_unpack = warp >= 2 && warp < 2 + GEMM_DEQ_WARPS;
    bool acc_ok = false;
    if (is_unpack) {
        acc_ok = role_ok && mbar_wait_bounded(smem_u32(&hdr->acc_full), 0, cta_abort) && !*cta_abort;
        if (!acc_ok && role_ok && lane == 0) give_up(DEV_TIMEOUT_MMA);
        tc_fence_after();
    }
    const int q = warp & 3;                 // TMEM lane quarter this warp may read
    const int cq = (warp - 2) >> 2;         // the four warps of a quarter split the columns
    const int cols_w = nb * GEMM_BX / 4;    // columns per warp: 64 or 128
    const int wrow_l = 32 * q + lane;       // this lane's weight row within the tile
    if (p.ksplit > 1) {
        // Split K: the CTAs of the cluster hold partial sums of the same tile.  Once every CTA's tensor-core work
        // has retired (first cluster barrier: the rings are idle everywhere) rank 1 stores its accumulators into
        // rank 0's x ring (128 KB = 128 x 256 floats) through distributed shared memory; after the second barrier
        // rank 0 adds them to its own (fixed order: reruns are bit identical) and writes the tile.  Every thread of
        // the cluster reaches both barriers on every path (a failed wait only skips work).
        cluster_sync_all();
        if (is_unpack && split != 0 && acc_ok) {
            uint32_t remote;
            asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(x_ring)), "r"(0));
            for (int c = cq * cols_w; c < (cq + 1) * cols_w; c += 32) {
                if (m0 + c >= p.m) break;
                uint32_t r[32];
                tmem_ld32(tmem_base + ((uint32_t)(32 * q) << 16) + (uint32_t)c, r);
                const uint32_t rowb = remote + (uint32_t)(((c >> 5) * GEMM_BW + wrow_l) * 128);
#pragma unroll
                for (int j = 0; j < 8; ++j)  // 16-byte pieces, rotated by the row so that eight lanes hit eight bank groups
                    asm volatile("st.shared::cluster.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(rowb + (uint32_t)((j ^ (wrow_l & 7)) << 4)), "r"(r[4 * j]),
                                 "r"(r[4 * j + 1]), "r"(r[4 * j + 2]), "r"(r[4 * j + 3])
                                 : "memory");
            }
        }
        cluster_sync_all();
    }
    if (is_unpack && split == 0) {
        if (acc_ok) {
            const int gcol = n0 + wrow_l;    // this lane's output column of y
            // bf16 output with rows of y a multiple of 16 bytes: the warp turns its 32 x 32 block through a
            // private 2 KB of the (now idle) weight ring, so a lane stores 16 bytes = 8 outputs of one row
            const bool wide = p.y && !p.yf && p.n % 8 == 0 && reinterpret_cast<uintptr_t>(p.y) % 16 == 0;
            uint8_t* stg = w_ring + (warp - 2) * 2048;
            for (int c = cq * cols_w; c < (cq + 1) * cols_w; c += 32) {
                if (m0 + c >= p.m) break;  // rows of x past m (the blocks of a CTA are consecutive, so are their columns)
                uint32_t r[32];
                tmem_ld32(tmem_base + ((uint32_t)(32 * q) << 16) + (uint32_t)c, r);
                if (p.ksplit > 1) {
                    const uint8_t* rowp = x_ring + ((c >> 5) * GEMM_BW + wrow_l) * 128;
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const float4 v = *reinterpret_cast<const float4*>(rowp + ((j ^ (wrow_l & 7)) << 4));
                        r[4 * j] = __float_as_uint(__uint_as_float(r[4 * j]) + v.x);
                        r[4 * j + 1] = __float_as_uint(__uint_as_float(r[4 * j + 1]) + v.y);
                        r[4 * j + 2] = __float_as_uint(__uint_as_float(r[4 * j + 2]) + v.z);
                        r[4 * j + 3] = __float_as_uint(__uint_as_float(r[4 * j + 3]) + v.w);
                    }
                }
                if (wide) {
                    __nv_bfloat16* st = reinterpret_cast<__nv_bfloat16*>(stg);
#pragma unroll
                    for (int i = 0; i < 32; ++i) st[i * 32 + lane] = __float2bfloat16_rn(__uint_as_float(r[i]));
                    __syncwarp();
#pragma unroll
                    for (int it = 0; it < 4; ++it) {
                        const int pc = lane + 32 * it, mm = pc >> 2, j = pc & 3;  // row of the block, 16-byte piece of its 64 bytes
                        const int ncol = n0 + 32 * q + 8 * j;
                        if (m0 + c + mm < p.m && ncol < p.n)
                            *reinterpret_cast<uint4*>(p.y + (size_t)(m0 + c + mm) * p.n + ncol) = *reinterpret_cast<const uint4*>(stg + mm * 64 + j * 16);
                    }
                    __syncwarp();
                } else if (gcol < p.n) {
                    const size_t o = (size_t)(m0 + c) * p.n + gcol;
                    if (p.yf) {
#pragma unroll
                        for (int i = 0; i < 32; ++i)
                            if (m0 + c + i < p.m) p.yf[o + (size_t)i * p.n] = __uint_as_float(r[i]);
                    }
                    if (p.y) {
#pragma unroll
                        for (int i = 0; i < 32; ++i)
                            if (m0 + c + i < p.m) p.y[o + (size_t)i * p.n] = __float2bfloat16_rn(__uint_as_float(r[i]));
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(GEMM_TMEM_COLS) : "memory");
    }
}

// ------------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(ptr);
    }
    return fn;
}

static int g_gemm_probe = 0;
void gemm_set_probe(int v) { g_gemm_probe = v; }
static int g_gemm_ksplit = 0;  // tunable "gemm_ksplit": 0 = automatic, 1, 2
int gemm_set_ksplit(int v) {
    if (v < 0 || v > 2) return QMM_ERR_UNSUPPORTED;
    g_gemm_ksplit = v;
    return QMM_OK;
}
static int g_gemm_mb = 0;  // tunable "gemm_mb": 256-row blocks of x per CTA, 0 = automatic
int gemm_set_mb(int v) {
    if (v < 0 || v > GEMM_NB_MAX) return QMM_ERR_UNSUPPORTED;
    g_gemm_mb = v;
    return QMM_OK;
}

static int gemm_launch(const void* w, bool w_bf16, const void* x, void* y, float* yf, int m, int n, int k, cudaStream_t stream) {
    if (!w || !x || (!y && !yf)) return QMM_ERR_NULL;
    if (m <= 0 || n <= 0 || k <= 0 || k % 256 != 0) return QMM_ERR_SHAPE;
    if (reinterpret_cast<uintptr_t>(w) % 16 != 0 || reinterpret_cast<uintptr_t>(x) % 16 != 0 ||
        reinterpret_cast<uintptr_t>(y) % 2 != 0 || reinterpret_cast<uintptr_t>(yf) % 4 != 0)
        return QMM_ERR_ALIGN;
    EncodeTiledFn enc = encode_tiled_fn();
    if (!enc) return cuda_fail(cudaErrorNotSupported);
    CUtensorMap map;
    const cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)m};
    const cuuint64_t strides[1] = {(cuuint64_t)k * 2};
    const cuuint32_t box[2] = {GEMM_BK, GEMM_BX};
    const cuuint32_t estr[2] = {1, 1};
    if (enc(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(x), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return cuda_fail(cudaErrorInvalidValue);

    // the packed weights as a 2-D byte tensor (row bytes, rows): one box = one super-block of 128 rows; bf16 weights as
    // a (k, n) bf16 tensor: one box = one 128 x 64 tile, swizzled like the x tiles
    CUtensorMap wmap;
    if (w_bf16) {
        const cuuint64_t wdims[2] = {(cuuint64_t)k, (cuuint64_t)n};
        const cuuint64_t wstrides[1] = {(cuuint64_t)k * 2};
        const cuuint32_t wbox[2] = {GEMM_BK, GEMM_BW};
        if (enc(&wmap, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(w), wdims, wstrides, wbox, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return cuda_fail(cudaErrorInvalidValue);
    } else {
        const cuuint64_t wdims[2] = {(cuuint64_t)(k / 256 * Q4_K_BYTES), (cuuint64_t)n};
        const cuuint64_t wstrides[1] = {(cuuint64_t)(k / 256 * Q4_K_BYTES)};
        const cuuint32_t wbox[2] = {Q4_K_BYTES, GEMM_BW};
        if (enc(&wmap, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(w), wdims, wstrides, wbox, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return cuda_fail(cudaErrorInvalidValue);
    }

    GemmParams p;
    p.w = static_cast<const uint8_t*>(w);
    p.y = static_cast<__nv_bfloat16*>(y);
    p.yf = yf;
    p.m = m, p.n = n, p.k = k;
    p.row_bytes = k / 256 * Q4_K_BYTES;
    p.probe = g_gemm_probe;
    p.w_bf16 = w_bf16 ? 1 : 0;
    const size_t smem = (size_t)GEMM_SW * GEMM_W_BYTES + (size_t)GEMM_XT * GEMM_X_BYTES + (size_t)GEMM_SP * GEMM_P_BYTES + sizeof(GemmSmemHeader) + 1024;
    static bool configured[64] = {};
    int dev = 0;
    QMM_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        QMM_CUDA_TRY(cudaFuncSetAttribute(qgemm_q4k_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    // Blocks of 256 rows of x per CTA.  Measured on B200: a CTA takes about 0.71 us per 64-wide k-step with one
    // block and 1.0 us with two (shared-memory traffic: the x tiles written by the copies, the weight tile written
    // by the unpack warps, and both read by every instruction), plus about 9 us of prologue and epilogue; the grid
    // runs in waves of one CTA per SM.  Take the count with the smaller modelled time ("gemm_mb" overrides).
    const int col_tiles = (n + GEMM_BW - 1) / GEMM_BW, x_blocks = (m + GEMM_BX - 1) / GEMM_BX;
    int nbc = 1;
    double best = 0.0;
    for (int cand = 1; cand <= GEMM_NB_MAX && cand <= x_blocks; ++cand) {
        const long ctas = (long)col_tiles * ((x_blocks + cand - 1) / cand);
        const double t = (double)((ctas + sm_count() - 1) / sm_count()) * ((cand == 1 ? 0.71 : 1.0) * (k / GEMM_BK) + 9.0);
        if (cand == 1 || t < best) best = t, nbc = cand;
    }
    if (g_gemm_mb >= 1 && g_gemm_mb <= GEMM_NB_MAX) nbc = g_gemm_mb;
    p.nb_per_cta = nbc;
    // Few tiles (a narrow matrix at a few hundred rows): two CTAs per tile, each with half of K, joined through
    // distributed shared memory.  Only with one block of x per CTA (the partial tile must fit the x ring).
    const long ctas = (long)col_tiles * ((x_blocks + nbc - 1) / nbc);
    int ksplit = (nbc == 1 && 2 * ctas <= sm_count() && k >= 8 * QKK) ? 2 : 1;
    if (g_gemm_ksplit == 1 || (g_gemm_ksplit == 2 && nbc == 1 && k >= 2 * QKK)) ksplit = g_gemm_ksplit;
    p.ksplit = ksplit;
    const dim3 grid(col_tiles, (x_blocks + nbc - 1) / nbc, ksplit);
    if (ksplit == 1) {
        qgemm_q4k_kernel<<<grid, GEMM_THREADS, smem, stream>>>(map, wmap, p);
        QMM_CUDA_TRY(cudaGetLastError());
        return QMM_OK;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(GEMM_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = (unsigned)ksplit;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    QMM_CUDA_TRY(cudaLaunchKernelEx(&cfg, qgemm_q4k_kernel, map, wmap, p));
    return QMM_OK;
}

int qgemm_q4k_launch(const void* w, const void* x, void* y, float* yf, int m, int n, int k, cudaStream_t stream) {
    return gemm_launch(w, false, x, y, yf, m, n, k, stream);
}
// out(m, n) = a(m, k) . b(n, k)^T with a and b bf16: the upstream's gemm_bt on a decoded (bf16) weight window
int gemm_bt_bf16_launch(const void* a, const void* b, void* y, float* yf, int m, int n, int k, cudaStream_t stream) {
    return gemm_launch(b, true, a, y, yf, m, n, k, stream);
}

}  // namespace qmm
