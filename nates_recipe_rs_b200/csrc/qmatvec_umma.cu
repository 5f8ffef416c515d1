// Small-batch matvec on the 5th-generation tensor cores, integer form: Q4_K weights, 9..32 activation rows.
//     y(m,n) = sum over 32-element sub-blocks j of  d*sc_j * dx_j * (q_j . xq_j)  -  dmin*m_j * s_j
// the operator of qmatvec.cu / qmatvec_mma.cu (the upstream's gpu_gemm_bt_f64_into at a handful of rows,
// gpu-core/src/infer_ops.rs:224-240) for the batch sizes where the per-instruction work of mma.sync (31 warp
// instructions around every m16n8k32) is what a launch costs.  Here the integer dot products of 128 weight rows x
// NC activation rows x one sub-block are ONE tcgen05.mma (kind::i8, M = 128, N = NC, K = 32) with the int32 result
// in tensor memory; the scales are applied by epilogue warps that read the sums back (tcgen05.ld), lane = weight row.
//
// A CTA owns 128 weight rows.  A k-step is 128 elements of K (four sub-blocks = half a super-block = one 128-byte
// swizzled row of int8).  Warp roles:
//   warp 0       TMA producer: the packed super-blocks of the 128 rows (128 x 144 bytes), four slots
//   warp 1       one lane issues the four tcgen05.mma of a k-step (each into its own NC columns, no accumulation)
//                and one tcgen05.commit; owns the TMEM allocation
//   warp 2       TMA producer: the Q8_1 blocks of a k-step (NC rows x 144 bytes; rows past m are filled with zeros),
//                eight k-steps ahead (they come from L2: a k-step is shorter than that round trip)
//   warp 3       activations: the raw blocks -> int8 tile (NC rows x 128 bytes, swizzled) + the blocks' d and s as f32
//   warps 4..7   unpack: nibbles -> int8 tile of the weights (128 rows x 128 bytes, swizzled) + d*sc_j and
//                dmin*m_j of every row as f32
//   warps 8..15  epilogue, two groups of four warps taking alternate k-steps: int32 sums -> f32 (exact, by the
//                2^23 trick), times the weight and activation scales, minus the min term, into NC f32 sums per
//                thread; at the end the groups (and, with K split over a cluster, the CTAs) add their sums in a
//                fixed order and store y.
// Four stages everywhere (weight tile, activation tile, scale arrays, accumulator columns).  Every wait is bounded;
// on expiry the CTA records a status code, drains its copies, frees its TMEM and returns.
#include "qmm_formats.cuh"
#include <cuda.h>

namespace qmm {

constexpr int UMV_BW = 128;
constexpr int UMV_KS = 128;
constexpr int UMV_ST = 4;
constexpr int UMV_SP = 4;
constexpr int UMV_P_BYTES = UMV_BW * Q4_K_BYTES;  // 18 KB
constexpr int UMV_W_BYTES = UMV_BW * UMV_KS;      // 16 KB
constexpr int UMV_X_BYTES = 32 * UMV_KS;          // 4 KB (NC <= 32 rows of 128 bytes)
constexpr int UMV_XS_BYTES = 2 * 4 * 32 * 4;      // d and s of 4 sub-blocks x 32 columns
constexpr int UMV_XR = 8;                         // raw activation slots
constexpr int UMV_XR_BYTES = 32 * 4 * Q8_1_BYTES; // 4608: NC <= 32 rows x four Q8_1 blocks
constexpr int UMV_WS_BYTES = UMV_BW * 32;         // 8 floats per weight row
constexpr int UMV_X_WARPS = 2, UMV_UNPACK_WARPS = 4, UMV_EPI_WARPS = 8;
constexpr int UMV_WARP_X = 2, UMV_WARP_UNPACK = UMV_WARP_X + UMV_X_WARPS, UMV_WARP_EPI = UMV_WARP_UNPACK + UMV_UNPACK_WARPS;
constexpr int UMV_THREADS = (UMV_WARP_EPI + UMV_EPI_WARPS) * 32;
constexpr int UMV_KSPLIT_MAX = 4;

struct UmvParams {
    const uint8_t* xq;  // (m, k/32) Q8_1 blocks
    float* y;
    long y_stride;
    int m, n, k;
    int xq_row_bytes;
    int ksplit;         // CTAs of a cluster that share a tile of rows, each with a contiguous part of K
    TpPush push;        // tensor parallel: the outputs go to every rank's exchange area instead of y
};

struct __align__(16) UmvSmemHeader {
    uint64_t p_full[UMV_SP], p_empty[UMV_SP];
    uint64_t w_full[UMV_ST], x_full[UMV_ST];
    uint64_t xr_full[UMV_XR], xr_empty[UMV_XR];
    uint64_t done[UMV_ST];       // the tensor-core work of a k-step has retired
    uint64_t acc_empty[UMV_ST];  // ... and its epilogue group has read the sums and the scales: the stage is free
    uint32_t tmem_base;
    int abort_flag;
};

__device__ __forceinline__ void umma_i8(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc) {
    asm volatile("{ .reg .pred p; setp.ne.b32 p, 0, 0; tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p; }" ::"r"(d_tmem), "l"(adesc),
                 "l"(bdesc), "r"(idesc)
                 : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];\n\t"
        "tcgen05.wait::ld.sync.aligned;"  // in the same statement: the registers must not be read before the wait
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
// The same load without the wait, and the wait as a statement that "writes" the registers, so that nothing reads them
// between the two.
__device__ __forceinline__ void tmem_ld16_issue(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait16(uint32_t (&r)[16]) {
    asm volatile("tcgen05.wait::ld.sync.aligned;"
                 : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]), "+r"(r[8]), "+r"(r[9]),
                   "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15])
                 :
                 : "memory");
}
__device__ __forceinline__ void epi_bar_sync() { asm volatile("bar.sync 1, %0;" ::"n"(UMV_EPI_WARPS * 32) : "memory"); }

// NC: activation rows the instruction covers (16 or 32; rows past m are zeros)
template <int NC>
__global__ void __launch_bounds__(UMV_THREADS, 1) qmv_umma_kernel(const __grid_constant__ CUtensorMap wmap, const __grid_constant__ CUtensorMap xmap,
                                                                   const UmvParams p) {
    extern __shared__ __align__(1024) uint8_t usm[];
    const uint32_t raw = smem_u32(usm);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t* sm = usm + (base - raw);
    uint8_t* w_ring = sm;                                   // UMV_ST x 16 KB
    uint8_t* x_ring = w_ring + UMV_ST * UMV_W_BYTES;        // UMV_ST x 4 KB
    uint8_t* p_ring = x_ring + UMV_ST * UMV_X_BYTES;        // UMV_SP x 18 KB
    uint8_t* xs_ring = p_ring + UMV_SP * UMV_P_BYTES;       // UMV_ST x 1 KB: [d: 4 x 32][s: 4 x 32] floats
    uint8_t* ws_ring = xs_ring + UMV_ST * UMV_XS_BYTES;     // UMV_ST x 4 KB: per row {ds0, ds1, dm0, dm1, ds2, ds3, dm2, dm3}
    uint8_t* xr_ring = ws_ring + UMV_ST * UMV_WS_BYTES;     // UMV_XR x 4.5 KB: raw Q8_1 blocks, [column][4 blocks]
    UmvSmemHeader* hdr = reinterpret_cast<UmvSmemHeader*>(xr_ring + UMV_XR * UMV_XR_BYTES);
    volatile int* cta_abort = &hdr->abort_flag;
    constexpr int CS = 32;                           // TMEM columns between the sums of consecutive sub-blocks
    constexpr uint32_t TMEM_COLS = UMV_ST * 4 * CS;  // 512
    // instruction descriptor: D s32, A and B signed 8-bit (the weight codes are 0..15), both K-major, N = NC, M = 128
    constexpr uint32_t IDESC = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(NC >> 3) << 17) | ((uint32_t)(UMV_BW >> 4) << 24);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = blockIdx.x * UMV_BW;
    const int split = (int)blockIdx.z;
    const int sb_all = p.k / QKK;
    const int sb0 = split * sb_all / p.ksplit, n_sb = (split + 1) * sb_all / p.ksplit - sb0;
    const int kt = n_sb * 2, ks0 = sb0 * 2;  // k-steps of this CTA, first k-step

    if (threadIdx.x == 0) {
        for (int s = 0; s < UMV_SP; ++s) mbar_init(smem_u32(&hdr->p_full[s]), 1), mbar_init(smem_u32(&hdr->p_empty[s]), UMV_UNPACK_WARPS);
        for (int s = 0; s < UMV_ST; ++s) {
            mbar_init(smem_u32(&hdr->w_full[s]), UMV_UNPACK_WARPS);
            mbar_init(smem_u32(&hdr->x_full[s]), 1);
            mbar_init(smem_u32(&hdr->done[s]), 1);
            mbar_init(smem_u32(&hdr->acc_empty[s]), UMV_EPI_WARPS / 2);
        }
        for (int s = 0; s < UMV_XR; ++s) mbar_init(smem_u32(&hdr->xr_full[s]), 1), mbar_init(smem_u32(&hdr->xr_empty[s]), 1);
        hdr->abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&hdr->tmem_base)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    pdl_release_dependents();
    const uint32_t tmem_base = hdr->tmem_base;

    auto give_up = [&](int code) {
        if (!*cta_abort) {
            atomicExch(&g_device_status, code);
            *cta_abort = 1;
        }
    };
    // stage of k-step ks is free again: the epilogue of k-step ks - UMV_ST has finished (ks >= UMV_ST)
    auto wait_stage_free = [&](int ks) { return mbar_wait_bounded(smem_u32(&hdr->acc_empty[ks % UMV_ST]), ((ks / UMV_ST) - 1) & 1, cta_abort); };

    float acc[NC];         // epilogue threads: this thread's weight row against the NC activation rows
    uint64_t acc2[NC / 2];  // ... as packed pairs while the k-steps run
#pragma unroll
    for (int c = 0; c < NC / 2; ++c) acc2[c] = 0ull;  // (+0.f, +0.f)
    bool epi_ok = true;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer (packed super-blocks; model data:
        // not ordered after the preceding kernel)
        if (lane == 0) {
            int issued = 0;
            for (int sb = 0; sb < n_sb; ++sb, ++issued) {
                const int slot = sb % UMV_SP;
                if (sb >= UMV_SP && !mbar_wait_bounded(smem_u32(&hdr->p_empty[slot]), ((sb / UMV_SP) - 1) & 1, cta_abort)) {
                    give_up(DEV_TIMEOUT_EMPTY);
                    break;
                }
                const uint32_t bar = smem_u32(&hdr->p_full[slot]);
                mbar_arrive_expect_tx(bar, UMV_P_BYTES);
                tma_load_2d(smem_u32(p_ring + slot * UMV_P_BYTES), &wmap, (sb0 + sb) * Q4_K_BYTES, n0, bar);  // rows past n: zeros
            }
            if (*cta_abort) {
                for (int i = max(0, issued - UMV_SP); i < issued; ++i) {
                    const long long t0 = clock64();
                    while (!mbar_try_wait(smem_u32(&hdr->p_full[i % UMV_SP]), (i / UMV_SP) & 1)) {
                        if (clock64() - t0 > WAIT_LIMIT_CYCLES) {
                            atomicExch(&g_device_status, DEV_TIMEOUT_DRAIN);
                            break;
                        }
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            for (int ks = 0; ks < kt; ++ks) {
                const int st = ks % UMV_ST;
                const uint32_t ph = (ks / UMV_ST) & 1;
                if ((ks >= UMV_ST && !wait_stage_free(ks)) || !mbar_wait_bounded(smem_u32(&hdr->x_full[st]), ph, cta_abort) ||
                    !mbar_wait_bounded(smem_u32(&hdr->w_full[st]), ph, cta_abort)) {
                    give_up(DEV_TIMEOUT_FULL);
                    break;
                }
                tc_fence_after();
                const uint64_t wdesc = umma_desc_sw128(smem_u32(w_ring + st * UMV_W_BYTES));
                const uint64_t xdesc = umma_desc_sw128(smem_u32(x_ring + st * UMV_X_BYTES));
#pragma unroll
                for (int j = 0; j < 4; ++j)  // sub-block j: 32 bytes of K (+2 in 16-byte units), its own NC columns
                    umma_i8(tmem_base + (uint32_t)(st * 4 * CS + j * CS), wdesc + 2 * j, xdesc + 2 * j, IDESC);
                umma_commit(smem_u32(&hdr->done[st]));
            }
        }
    } else if (warp == UMV_WARP_X) {
        // ------------------------------------------------------------ TMA producer (raw activation blocks)
        if (lane == 0) {
            pdl_wait_prior_grids();  // the activations come from the preceding kernel
            int issued = 0;
            for (int ks = 0; ks < kt; ++ks, ++issued) {
                const int slot = ks % UMV_XR;
                if (ks >= UMV_XR && !mbar_wait_bounded(smem_u32(&hdr->xr_empty[slot]), ((ks / UMV_XR) - 1) & 1, cta_abort)) {
                    give_up(DEV_TIMEOUT_EMPTY);
                    break;
                }
                const uint32_t bar = smem_u32(&hdr->xr_full[slot]);
                mbar_arrive_expect_tx(bar, NC * 4 * Q8_1_BYTES);
                tma_load_2d(smem_u32(xr_ring + slot * UMV_XR_BYTES), &xmap, (ks0 + ks) * 4 * Q8_1_BYTES, 0, bar);  // rows past m: zeros
            }
            if (*cta_abort) {
                for (int i = max(0, issued - UMV_XR); i < issued; ++i) {
                    const long long t0 = clock64();
                    while (!mbar_try_wait(smem_u32(&hdr->xr_full[i % UMV_XR]), (i / UMV_XR) & 1)) {
                        if (clock64() - t0 > WAIT_LIMIT_CYCLES) {
                            atomicExch(&g_device_status, DEV_TIMEOUT_DRAIN);
                            break;
                        }
                    }
                }
            }
        }
    } else if (warp < UMV_WARP_UNPACK) {
        // ------------------------------------------------------------ activations: raw Q8_1 blocks -> int8 tile + scales
        // lane handles blocks id = lane + 32 b: column c = id / 4, sub-block j = id % 4 of the k-step
        constexpr int BPT = NC * 4 / 32;  // 2 (NC = 16) or 4 (NC = 32)
        for (int ks = 0; ks < kt; ++ks) {
            const int st = ks % UMV_ST, slot = ks % UMV_XR;
            if (!mbar_wait_bounded(smem_u32(&hdr->xr_full[slot]), (ks / UMV_XR) & 1, cta_abort)) {
                if (lane == 0) give_up(DEV_TIMEOUT_FULL);
                break;
            }
            uint32_t blk[BPT][9];
#pragma unroll
            for (int b = 0; b < BPT; ++b) {
                const int id = lane + 32 * b;
                const uint32_t* src = reinterpret_cast<const uint32_t*>(xr_ring + slot * UMV_XR_BYTES + id * Q8_1_BYTES);  // [c][j] blocks back to back
#pragma unroll
                for (int i = 0; i < 9; ++i) blk[b][i] = src[i];
            }
            if (ks >= UMV_ST && !wait_stage_free(ks)) {
                if (lane == 0) give_up(DEV_TIMEOUT_EMPTY);
                break;
            }
            uint8_t* tile = x_ring + st * UMV_X_BYTES;
            float* xd = reinterpret_cast<float*>(xs_ring + st * UMV_XS_BYTES);
#pragma unroll
            for (int b = 0; b < BPT; ++b) {
                const int id = lane + 32 * b, c = id >> 2, j = id & 3;
                uint8_t* rowp = tile + c * 128;
                const uint32_t swz = (uint32_t)(c & 7);
                *reinterpret_cast<uint4*>(rowp + ((((uint32_t)(2 * j)) ^ swz) << 4)) = make_uint4(blk[b][1], blk[b][2], blk[b][3], blk[b][4]);
                *reinterpret_cast<uint4*>(rowp + ((((uint32_t)(2 * j + 1)) ^ swz) << 4)) = make_uint4(blk[b][5], blk[b][6], blk[b][7], blk[b][8]);
                xd[j * 32 + c] = f16_bits_to_f32(blk[b][0] & 0xFFFFu);
                xd[128 + j * 32 + c] = f16_bits_to_f32(blk[b][0] >> 16);
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();  // every lane's values are stored (and fenced): the tile is complete, the raw slot may be refilled
            if (lane == 0) mbar_arrive(smem_u32(&hdr->x_full[st])), mbar_arrive(smem_u32(&hdr->xr_empty[slot]));
        }
    } else if (warp < UMV_WARP_EPI) {
        // ------------------------------------------------------------ unpack: thread = weight row of the tile
        const int row = threadIdx.x - UMV_WARP_UNPACK * 32;
        const uint32_t swz = (uint32_t)(row & 7);
        bool ok = true;
        for (int sb = 0; sb < n_sb && ok; ++sb) {
            const int ps = sb % UMV_SP;
            if (!mbar_wait_bounded(smem_u32(&hdr->p_full[ps]), (sb / UMV_SP) & 1, cta_abort)) {
                if (lane == 0) give_up(DEV_TIMEOUT_FULL);
                break;
            }
            const uint8_t* blk = p_ring + ps * UMV_P_BYTES + row * Q4_K_BYTES;
            const uint4 hd = *reinterpret_cast<const uint4*>(blk);
            uint4 qv[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) qv[i] = *reinterpret_cast<const uint4*>(blk + 16 + 16 * i);
            // 6-bit scale / min codes, one per byte: A = sub-blocks 0..3, B = 4..7
            const uint32_t scA = hd.y & 0x3F3F3F3Fu, mA = hd.z & 0x3F3F3F3Fu;
            const uint32_t scB = (hd.w & 0x0F0F0F0Fu) | ((hd.y >> 2) & 0x30303030u);
            const uint32_t mB = ((hd.w >> 4) & 0x0F0F0F0Fu) | ((hd.z >> 2) & 0x30303030u);
            const float d = f16_bits_to_f32(hd.x & 0xFFFFu), dmin = f16_bits_to_f32(hd.x >> 16);
#pragma unroll
            for (int h = 0; h < 2; ++h) {  // the two k-steps of the super-block: sub-blocks 4h..4h+3 = groups 2h, 2h+1
                const int ks = sb * 2 + h, st = ks % UMV_ST;
                if (ks >= UMV_ST && !wait_stage_free(ks)) {
                    if (lane == 0) give_up(DEV_TIMEOUT_EMPTY);
                    ok = false;
                    break;
                }
                uint8_t* tile = w_ring + st * UMV_W_BYTES + row * 128;
                const uint32_t sc4 = h == 0 ? scA : scB, m4 = h == 0 ? mA : mB;
                float4 sA, sB;  // {ds, ds, dm, dm} of the sub-blocks of group 2h, then of group 2h+1
                sA.x = __fmul_rn(d, byte_to_float(sc4, 0)), sA.y = __fmul_rn(d, byte_to_float(sc4, 1));
                sA.z = __fmul_rn(dmin, byte_to_float(m4, 0)), sA.w = __fmul_rn(dmin, byte_to_float(m4, 1));
                sB.x = __fmul_rn(d, byte_to_float(sc4, 2)), sB.y = __fmul_rn(d, byte_to_float(sc4, 3));
                sB.z = __fmul_rn(dmin, byte_to_float(m4, 2)), sB.w = __fmul_rn(dmin, byte_to_float(m4, 3));
#pragma unroll
                for (int gi = 0; gi < 2; ++gi) {  // group 2h+gi: low nibbles = sub-block 2gi of the k-step, high = 2gi+1
                    const uint4 a = qv[(2 * h + gi) * 2], b = qv[(2 * h + gi) * 2 + 1];
                    const uint32_t M = 0x0F0F0F0Fu;
                    const uint32_t c0 = (uint32_t)(4 * gi);  // first 16-byte chunk of sub-block 2gi
                    *reinterpret_cast<uint4*>(tile + (((c0 + 0) ^ swz) << 4)) = make_uint4(a.x & M, a.y & M, a.z & M, a.w & M);
                    *reinterpret_cast<uint4*>(tile + (((c0 + 1) ^ swz) << 4)) = make_uint4(b.x & M, b.y & M, b.z & M, b.w & M);
                    *reinterpret_cast<uint4*>(tile + (((c0 + 2) ^ swz) << 4)) = make_uint4((a.x >> 4) & M, (a.y >> 4) & M, (a.z >> 4) & M, (a.w >> 4) & M);
                    *reinterpret_cast<uint4*>(tile + (((c0 + 3) ^ swz) << 4)) = make_uint4((b.x >> 4) & M, (b.y >> 4) & M, (b.z >> 4) & M, (b.w >> 4) & M);
                }
                float4* wsr = reinterpret_cast<float4*>(ws_ring + st * UMV_WS_BYTES + row * 32);
                wsr[0] = sA;
                wsr[1] = sB;
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&hdr->w_full[st]));
            }
            __syncwarp();
            // only now: released right after the loads above, the slot was refilled while loads of this warp were still
            // outstanding (observed as wrong sums for a few of a tile's first rows); here every loaded value has been used
            if (lane == 0) mbar_arrive(smem_u32(&hdr->p_empty[ps]));
        }
    } else {
        // ------------------------------------------------------------ epilogue: group g takes k-steps g, g+2, ...
        const int g = (warp - UMV_WARP_EPI) >> 2, q = warp & 3;
        const int row = 32 * q + lane;
        for (int ks = g; ks < kt; ks += 2) {
            const int st = ks % UMV_ST;
            const uint32_t ph = (ks / UMV_ST) & 1;
            // the tensor-core work has retired; the scale arrays come from the unpack and activation warps directly
            if (!mbar_wait_bounded(smem_u32(&hdr->done[st]), ph, cta_abort) || !mbar_wait_bounded(smem_u32(&hdr->x_full[st]), ph, cta_abort) ||
                !mbar_wait_bounded(smem_u32(&hdr->w_full[st]), ph, cta_abort)) {
                if (lane == 0) give_up(DEV_TIMEOUT_MMA);
                epi_ok = false;
                break;
            }
            tc_fence_after();
            const float4* wsr = reinterpret_cast<const float4*>(ws_ring + st * UMV_WS_BYTES + row * 32);
            const float4 sA = wsr[0], sB = wsr[1];
            const float wds[4] = {sA.x, sA.y, sB.x, sB.y}, wdm[4] = {sA.z, sA.w, sB.z, sB.w};
            const float* xd = reinterpret_cast<const float*>(xs_ring + st * UMV_XS_BYTES);
            // The sums come in chunks of 16 columns, the next chunk's tcgen05.ld in flight under the current chunk's
            // arithmetic (the load takes a few hundred cycles).  Chunk i: sub-block j = i / CPS, columns 16 (i % CPS)...
            constexpr int CPS = NC / 16, CHUNKS = 4 * CPS;
            const uint32_t tstage = tmem_base + ((uint32_t)(32 * q) << 16) + (uint32_t)(st * 4 * CS);
            uint32_t r[2][16];
            tmem_ld16_issue(tstage, r[0]);
            const uint64_t magic2 = pack_f2(-12582912.f, -12582912.f);
#pragma unroll
            for (int i = 0; i < CHUNKS; ++i) {
                const int j = i / CPS, c0 = 16 * (i % CPS);
                tmem_ld_wait16(r[i & 1]);
                if (i + 1 < CHUNKS) tmem_ld16_issue(tstage + (uint32_t)(((i + 1) / CPS) * CS + 16 * ((i + 1) % CPS)), r[(i + 1) & 1]);
                const uint64_t wd2 = pack_f2(wds[j], wds[j]), nwm2 = pack_f2(-wdm[j], -wdm[j]);
#pragma unroll
                for (int c = 0; c < 16; c += 4) {
                    const float4 dx = *reinterpret_cast<const float4*>(xd + j * 32 + c0 + c);
                    const float4 sx = *reinterpret_cast<const float4*>(xd + 128 + j * 32 + c0 + c);
                    // int32 -> f32, exact for |i| < 2^22: the bits of 2^23 + 2^22 + i, minus 2^23 + 2^22
                    const uint64_t f01 = add_f2(pack_b64(r[i & 1][c] + 0x4B400000u, r[i & 1][c + 1] + 0x4B400000u), magic2);
                    const uint64_t f23 = add_f2(pack_b64(r[i & 1][c + 2] + 0x4B400000u, r[i & 1][c + 3] + 0x4B400000u), magic2);
                    uint64_t a01 = acc2[(c0 + c) >> 1], a23 = acc2[((c0 + c) >> 1) + 1];
                    a01 = fma_f2(mul_f2(f01, wd2), pack_f2(dx.x, dx.y), a01);
                    a23 = fma_f2(mul_f2(f23, wd2), pack_f2(dx.z, dx.w), a23);
                    acc2[(c0 + c) >> 1] = fma_f2(nwm2, pack_f2(sx.x, sx.y), a01);
                    acc2[((c0 + c) >> 1) + 1] = fma_f2(nwm2, pack_f2(sx.z, sx.w), a23);
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&hdr->acc_empty[st]));
        }
#pragma unroll
        for (int c = 0; c < NC / 2; ++c) unpack_f2(acc2[c], acc[2 * c], acc[2 * c + 1]);
        // every k-step's sums are read: all tensor-core work of the CTA has retired and the rings are idle.
        // Group 1 hands its sums to group 0 through the first 16 KB of the weight ring (row-major, NC floats per row,
        // 16-byte pieces rotated by the row).
        epi_bar_sync();
        float* stg = reinterpret_cast<float*>(w_ring);
        if (g == 1) {
#pragma unroll
            for (int c = 0; c < NC; c += 4)
                *reinterpret_cast<float4*>(stg + row * NC + (((c >> 2) ^ (row & (NC / 4 - 1))) << 2)) = make_float4(acc[c], acc[c + 1], acc[c + 2], acc[c + 3]);
        }
        epi_bar_sync();
        if (g == 0) {
#pragma unroll
            for (int c = 0; c < NC; c += 4) {
                const float4 v = *reinterpret_cast<const float4*>(stg + row * NC + (((c >> 2) ^ (row & (NC / 4 - 1))) << 2));
                acc[c] += v.x, acc[c + 1] += v.y, acc[c + 2] += v.z, acc[c + 3] += v.w;
            }
        }
    }

    const bool is_epi0 = warp >= UMV_WARP_EPI && warp < UMV_WARP_EPI + 4;
    const int row = 32 * (warp & 3) + lane;
    if (p.ksplit > 1) {
        // Split K: after the first cluster barrier every CTA's rings are idle; ranks 1.. store their sums into rank 0's
        // weight ring (16 KB per rank, from 16 KB on) through distributed shared memory; after the second barrier rank 0
        // adds them in rank order.  Every thread of the cluster reaches both barriers on every path.
        cluster_sync_all();
        if (is_epi0 && split != 0) {
            uint32_t remote;
            asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(w_ring + split * UMV_W_BYTES)), "r"(0));
#pragma unroll
            for (int c = 0; c < NC; c += 4)
                asm volatile("st.shared::cluster.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(remote + (uint32_t)((row * NC + (((c >> 2) ^ (row & (NC / 4 - 1))) << 2)) * 4)),
                             "r"(__float_as_uint(acc[c])), "r"(__float_as_uint(acc[c + 1])), "r"(__float_as_uint(acc[c + 2])), "r"(__float_as_uint(acc[c + 3]))
                             : "memory");
        }
        cluster_sync_all();
        if (is_epi0 && split == 0) {
            for (int r = 1; r < p.ksplit; ++r) {
                const float* part = reinterpret_cast<const float*>(w_ring + r * UMV_W_BYTES);
#pragma unroll
                for (int c = 0; c < NC; c += 4) {
                    const float4 v = *reinterpret_cast<const float4*>(part + row * NC + (((c >> 2) ^ (row & (NC / 4 - 1))) << 2));
                    acc[c] += v.x, acc[c + 1] += v.y, acc[c + 2] += v.z, acc[c + 3] += v.w;
                }
            }
        }
    }
    if (is_epi0 && split == 0 && epi_ok && !*cta_abort) {
        pdl_wait_prior_grids();  // y may still be read by the preceding kernel; the exchange counter belongs to it too
        const unsigned push_seq = p.push.tp > 0 ? tp_next_seq(p.push.counter) : 0u;
        if (n0 + row < p.n) {
#pragma unroll
            for (int c = 0; c < NC; ++c)
                if (c < p.m) tp_store_out(p.push, push_seq, p.y, p.y_stride, c, (long)n0 + row, acc[c]);  // a warp: 32 consecutive outputs
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

static int g_umv_min_m = 17;  // tunable "umma_min_m": activation rows from which Q4_K takes this kernel (0 = never)
int umv_set_min_m(int v) {
    if (v < 0 || v > 33) return QMM_ERR_UNSUPPORTED;
    g_umv_min_m = v;
    return QMM_OK;
}
int umv_min_m() { return g_umv_min_m; }
static int g_umv_min_k = 4096;  // tunable "umma_min_k": shortest rows (elements) that take this kernel
int umv_set_min_k(int v) {
    if (v < QKK || v % QKK) return QMM_ERR_UNSUPPORTED;
    g_umv_min_k = v;
    return QMM_OK;
}
int umv_min_k() { return g_umv_min_k; }
static int g_umv_ksplit = 0;  // tunable "umma_ksplit": 0 = automatic
int umv_set_ksplit(int v) {
    if (v < 0 || v > UMV_KSPLIT_MAX || v == 3) return QMM_ERR_UNSUPPORTED;
    g_umv_ksplit = v;
    return QMM_OK;
}

// Q4_K rows back to back, up to 32 activation rows, k a multiple of 256; QMM_ERR_UNSUPPORTED for anything else
// (the caller falls back to the mma.sync kernel).  push (tensor parallel): as in the other matvec kernels.
int qmatvec_umma_launch(const void* w, const void* xq, float* y, long y_stride, int m, int n, int k, const TpPush* push, cudaStream_t stream) {
    if (m <= 0 || m > 32 || k % QKK != 0 || reinterpret_cast<uintptr_t>(w) % 16 != 0 || reinterpret_cast<uintptr_t>(xq) % 16 != 0) return QMM_ERR_UNSUPPORTED;
    EncodeTiledFn enc = encode_tiled_fn();
    if (!enc) return QMM_ERR_UNSUPPORTED;
    const int row_bytes = k / QKK * Q4_K_BYTES;
    CUtensorMap wmap;
    const cuuint64_t wdims[2] = {(cuuint64_t)row_bytes, (cuuint64_t)n};
    const cuuint64_t wstrides[1] = {(cuuint64_t)row_bytes};
    const cuuint32_t wbox[2] = {Q4_K_BYTES, UMV_BW};
    const cuuint32_t estr[2] = {1, 1};
    if (enc(&wmap, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(w), wdims, wstrides, wbox, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return cuda_fail(cudaErrorInvalidValue);
    // the Q8_1 rows as a 2-D byte tensor: one box = the four blocks of a k-step for 16 or 32 rows (rows past m: zeros)
    const int wide = m > 16 ? 1 : 0;
    CUtensorMap xmap;
    const cuuint64_t xdims[2] = {(cuuint64_t)(k / QK8 * Q8_1_BYTES), (cuuint64_t)m};
    const cuuint64_t xstrides[1] = {(cuuint64_t)(k / QK8 * Q8_1_BYTES)};
    const cuuint32_t xbox[2] = {4 * Q8_1_BYTES, wide ? 32u : 16u};
    if (enc(&xmap, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(xq), xdims, xstrides, xbox, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return cuda_fail(cudaErrorInvalidValue);
    UmvParams p;
    p.xq = static_cast<const uint8_t*>(xq);
    p.y = y;
    p.y_stride = y_stride;
    p.m = m, p.n = n, p.k = k;
    p.push = TpPush{};
    if (push) p.push = *push;
    p.xq_row_bytes = k / QK8 * Q8_1_BYTES;
    const int tiles = (n + UMV_BW - 1) / UMV_BW;
    // few tiles: split K over a cluster so that most SMs have a CTA (each part at least four super-blocks)
    int ksplit = 1;
    while (ksplit < UMV_KSPLIT_MAX && tiles * ksplit * 2 <= sm_count() && (k / QKK) / (ksplit * 2) >= 4) ksplit *= 2;
    if (g_umv_ksplit && (k / QKK) >= g_umv_ksplit) ksplit = g_umv_ksplit;
    p.ksplit = ksplit;
    const size_t smem = (size_t)UMV_ST * (UMV_W_BYTES + UMV_X_BYTES + UMV_XS_BYTES + UMV_WS_BYTES) + (size_t)UMV_SP * UMV_P_BYTES +
                        (size_t)UMV_XR * UMV_XR_BYTES + sizeof(UmvSmemHeader) + 1024;
    static bool configured[64][2] = {};
    int dev = 0;
    QMM_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !configured[dev][wide]) {
        if (wide) QMM_CUDA_TRY(cudaFuncSetAttribute(qmv_umma_kernel<32>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        else QMM_CUDA_TRY(cudaFuncSetAttribute(qmv_umma_kernel<16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        if (dev >= 0 && dev < 64) configured[dev][wide] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(tiles, 1, ksplit);
    cfg.blockDim = dim3(UMV_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int na = 0;
    if (overlap_enabled()) {
        attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[na].val.programmaticStreamSerializationAllowed = 1;
        ++na;
    }
    if (ksplit > 1) {
        attr[na].id = cudaLaunchAttributeClusterDimension;
        attr[na].val.clusterDim.x = 1;
        attr[na].val.clusterDim.y = 1;
        attr[na].val.clusterDim.z = (unsigned)ksplit;
        ++na;
    }
    cfg.attrs = attr;
    cfg.numAttrs = na;
    if (wide) QMM_CUDA_TRY(cudaLaunchKernelEx(&cfg, qmv_umma_kernel<32>, wmap, xmap, p));
    else QMM_CUDA_TRY(cudaLaunchKernelEx(&cfg, qmv_umma_kernel<16>, wmap, xmap, p));
    return QMM_OK;
}

}  // namespace qmm
