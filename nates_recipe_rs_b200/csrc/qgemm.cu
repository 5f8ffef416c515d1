// Prefill dequant-GEMM on the 5th-generation tensor cores:
//     y(m,n) = bf16( sum_k x(m,k) * bf16(dequant(w(n,k))) ),   x, y bf16, w Q4_K, fp32 accumulate.
// The dense-contraction counterpart of the decode matvec; it replaces the same upstream
// pair (widen window + gpu_gemm_bt_f64_into, gpu-core/src/infer_ops.rs:85-101, 224-240) when
// m is in the hundreds.
//
// One CTA owns a 128-column tile of the output for up to 512 rows of x, so every weight is
// unpacked once per 512 tokens.  Warp roles:
//   warp 0      TMA producer: x tiles (128 rows x 64 k, 128-byte swizzle) through a 6-slot ring
//   warp 1      TMEM allocation; one lane issues tcgen05.mma (128x128x16, bf16 -> f32 in TMEM)
//   warps 2..17 unpack one 32-byte group of qs per row and k-step (= 64 weights = one 128-byte
//               swizzled row of the B tile) into a 6-slot ring, then run the epilogue
// A k-step is 64 elements: exactly one group of a Q4_K super-block, so the B tile row of a
// weight row is one group of that row's current super-block.
// Accumulators: up to four 128x128 f32 blocks = all 512 TMEM columns; the epilogue reads them
// with tcgen05.ld (32 lanes x 32 columns per warp), rounds to bf16 and stores.
// Every wait is bounded; on expiry the CTA records a status code, drains its copies, frees
// its TMEM and returns.
#include "qmm_formats.cuh"
#include <cuda.h>

namespace qmm {

constexpr int GEMM_BN = 128, GEMM_BK = 64, GEMM_MB_MAX = 4;
constexpr int GEMM_SA = 6, GEMM_SB = 6;
constexpr int GEMM_TILE_BYTES = 128 * GEMM_BK * 2;  // 16 KB: 128 rows x 128 bytes
constexpr int GEMM_DEQ_WARPS = 16;
constexpr int GEMM_THREADS = (2 + GEMM_DEQ_WARPS) * 32;
constexpr uint32_t GEMM_TMEM_COLS = 512;
// instruction descriptor: D f32, A bf16, B bf16, both K-major, N = 128, M = 128
constexpr uint32_t GEMM_IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((GEMM_BN >> 3) << 17) | ((128u >> 4) << 24);

struct GemmParams {
    const uint8_t* w;     // Q4_K rows (n, k)
    __nv_bfloat16* y;     // (m, n) bf16, may be null when yf is given
    float* yf;            // optional (m, n) f32 copy of the accumulators
    int m, n, k;
    int row_bytes;
    int probe;            // tuning aid: 0 normal, 1 = unpack arithmetic skipped, 2 = tensor-core work skipped
    int mb_per_cta;       // 128-row blocks of x per CTA (1..GEMM_MB_MAX): fewer when the column tiles alone do not fill the GPU
};

struct __align__(16) GemmSmemHeader {
    uint64_t a_full[GEMM_SA], a_empty[GEMM_SA];
    uint64_t b_full[GEMM_SB], b_empty[GEMM_SB];
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
        "%18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]),
          "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]),
          "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
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

__global__ void __launch_bounds__(GEMM_THREADS, 1) qgemm_q4k_kernel(const __grid_constant__ CUtensorMap xmap, const GemmParams p) {
    extern __shared__ __align__(1024) uint8_t gsm[];
    // layout: [A ring: SA x 16 KB][B ring: SB x 16 KB][header]; the base is aligned to 1024 by hand
    const uint32_t raw = smem_u32(gsm);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t* sm = gsm + (base - raw);
    uint8_t* a_ring = sm;
    uint8_t* b_ring = sm + GEMM_SA * GEMM_TILE_BYTES;
    GemmSmemHeader* hdr = reinterpret_cast<GemmSmemHeader*>(sm + (GEMM_SA + GEMM_SB) * GEMM_TILE_BYTES);
    volatile int* cta_abort = &hdr->abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = blockIdx.x * GEMM_BN;
    const int m0 = blockIdx.y * (128 * p.mb_per_cta);
    const int mb_count = min(p.mb_per_cta, (p.m - m0 + 127) / 128);
    const int kt = p.k / GEMM_BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < GEMM_SA; ++s) mbar_init(smem_u32(&hdr->a_full[s]), 1), mbar_init(smem_u32(&hdr->a_empty[s]), 1);
        for (int s = 0; s < GEMM_SB; ++s)
            mbar_init(smem_u32(&hdr->b_full[s]), GEMM_DEQ_WARPS), mbar_init(smem_u32(&hdr->b_empty[s]), 1);
        mbar_init(smem_u32(&hdr->acc_full), 1);
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

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer (x tiles)
        if (lane == 0) {
            int issued = 0;
            bool ok = true;
            for (int ks = 0; ks < kt && ok; ++ks) {
                for (int mb = 0; mb < mb_count; ++mb, ++issued) {
                    const int slot = issued % GEMM_SA, use = issued / GEMM_SA;
                    if (use > 0 && !mbar_wait_bounded(smem_u32(&hdr->a_empty[slot]), (use - 1) & 1, cta_abort)) {
                        give_up(DEV_TIMEOUT_EMPTY);
                        ok = false;
                        break;
                    }
                    const uint32_t bar = smem_u32(&hdr->a_full[slot]);
                    mbar_arrive_expect_tx(bar, GEMM_TILE_BYTES);
                    tma_load_2d(smem_u32(a_ring + slot * GEMM_TILE_BYTES), &xmap, ks * GEMM_BK, m0 + mb * 128, bar);
                }
            }
            if (!ok) {
                // copies that were issued but perhaps not consumed: wait (bounded) for them to land
                for (int i = max(0, issued - GEMM_SA); i < issued; ++i) {
                    const long long t0 = clock64();
                    while (!mbar_try_wait(smem_u32(&hdr->a_full[i % GEMM_SA]), (i / GEMM_SA) & 1)) {
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
            int a_it = 0;
            bool ok = true;
            for (int ks = 0; ks < kt && ok; ++ks) {
                const int sb = ks % GEMM_SB;
                if (!mbar_wait_bounded(smem_u32(&hdr->b_full[sb]), (ks / GEMM_SB) & 1, cta_abort)) {
                    give_up(DEV_TIMEOUT_FULL);
                    break;
                }
                tc_fence_after();
                const uint64_t bdesc = umma_desc_sw128(smem_u32(b_ring + sb * GEMM_TILE_BYTES));
                for (int mb = 0; mb < mb_count; ++mb, ++a_it) {
                    const int sa = a_it % GEMM_SA;
                    if (!mbar_wait_bounded(smem_u32(&hdr->a_full[sa]), (a_it / GEMM_SA) & 1, cta_abort)) {
                        give_up(DEV_TIMEOUT_FULL);
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint64_t adesc = umma_desc_sw128(smem_u32(a_ring + sa * GEMM_TILE_BYTES));
#pragma unroll
                    for (int k16 = 0; k16 < GEMM_BK / 16; ++k16)  // 32 bytes of K per instruction: +2 in 16-byte units
                        if (p.probe != 2) umma_bf16(tmem_base + (uint32_t)mb * GEMM_BN, adesc + 2 * k16, bdesc + 2 * k16, GEMM_IDESC,
                                  (ks > 0 || k16 > 0) ? 1u : 0u);
                    umma_commit(smem_u32(&hdr->a_empty[sa]));  // frees the x slot when these MMAs retire
                }
                umma_commit(smem_u32(&hdr->b_empty[sb]));
            }
            umma_commit(smem_u32(&hdr->acc_full));  // also on the give-up path, so the epilogue warps are released
        }
    } else {
        // ------------------------------------------------------------ unpack warps, then epilogue
        // thread = (weight row of the tile, which 8 bytes of the 32-byte group): consecutive lanes take
        // consecutive rows, so the eight lanes of a store phase hit eight different swizzle positions
        const int t = threadIdx.x - 64;          // 0..511
        const int row = t & 127, part = t >> 7;  // part 0..3
        const int wrow = min(n0 + row, p.n - 1); // rows past n are unpacked from the last row and never stored
        const uint8_t* wr = p.w + (size_t)wrow * p.row_bytes;
        const uint32_t row_off = (uint32_t)row * 128u, swz = (uint32_t)(row & 7);
        // two k-steps of packed words in flight ahead of the one being unpacked
        // A super-block serves four k-steps: its header and this thread's four 8-byte pieces are fetched
        // together, one whole super-block (four k-steps) ahead of their use.
        struct Packed {
            uint4 hdr;
            uint2 q[4];
        };
        auto fetch = [&](int sbi, Packed& pk) {
            const uint8_t* blk = wr + (size_t)sbi * Q4_K_BYTES;
            pk.hdr = *reinterpret_cast<const uint4*>(blk);
#pragma unroll
            for (int g = 0; g < 4; ++g) pk.q[g] = *reinterpret_cast<const uint2*>(blk + 16 + 32 * g + 8 * part);
        };
        Packed cur, nxt;
        fetch(0, cur);
        nxt = cur;
        bool ok = true;
        for (int ks = 0; ks < kt; ++ks) {
            if ((ks & 3) == 0) {
                if (ks > 0) cur = nxt;
                if (ks + 4 < kt) fetch((ks >> 2) + 1, nxt);
            }
            const uint4 hd = cur.hdr;
            const int gsel = ks & 3;
            const uint2 qs = gsel == 0 ? cur.q[0] : (gsel == 1 ? cur.q[1] : (gsel == 2 ? cur.q[2] : cur.q[3]));
            // scale / min codes of sub-blocks 2g (low nibbles) and 2g+1 (high nibbles); g is uniform over the CTA
            const int g = ks & 3;
            const uint32_t scA = hd.y & 0x3F3F3F3Fu, mA = hd.z & 0x3F3F3F3Fu;
            const uint32_t scB = (hd.w & 0x0F0F0F0Fu) | ((hd.y >> 2) & 0x30303030u);
            const uint32_t mB = ((hd.w >> 4) & 0x0F0F0F0Fu) | ((hd.z >> 2) & 0x30303030u);
            const uint32_t sc4 = g < 2 ? scA : scB, m4 = g < 2 ? mA : mB;
            const uint32_t i0 = (uint32_t)(2 * g) & 3u;
            const float d = f16_bits_to_f32(hd.x & 0xFFFFu), dmin = f16_bits_to_f32(hd.x >> 16);
            const float ds0 = __fmul_rn(d, byte_to_float(sc4, i0)), off0 = __fmul_rn(dmin, byte_to_float(m4, i0));
            const float ds1 = __fmul_rn(d, byte_to_float(sc4, i0 + 1)), off1 = __fmul_rn(dmin, byte_to_float(m4, i0 + 1));
            // bytes 8*part .. 8*part+7 of the group: low nibbles = elements 8*part.. (chunk part),
            // high nibbles = elements 32+8*part.. (chunk 4+part)
            uint4 c_lo, c_hi;
            if (p.probe != 1) {
                c_lo = q4k_to_bf16x8(qs.x & 0x0F0F0F0Fu, qs.y & 0x0F0F0F0Fu, ds0, off0);
                c_hi = q4k_to_bf16x8((qs.x >> 4) & 0x0F0F0F0Fu, (qs.y >> 4) & 0x0F0F0F0Fu, ds1, off1);
            } else {
                c_lo = make_uint4(qs.x, qs.y, hd.x, hd.y);
                c_hi = c_lo;
            }

            const int sb = ks % GEMM_SB, use = ks / GEMM_SB;
            if (use > 0 && !mbar_wait_bounded(smem_u32(&hdr->b_empty[sb]), (use - 1) & 1, cta_abort)) {
                if (lane == 0) give_up(DEV_TIMEOUT_EMPTY);
                ok = false;
                break;
            }
            uint8_t* tile = b_ring + sb * GEMM_TILE_BYTES + row_off;
            *reinterpret_cast<uint4*>(tile + ((((uint32_t)part + 0) ^ swz) << 4)) = c_lo;
            *reinterpret_cast<uint4*>(tile + ((((uint32_t)part + 4) ^ swz) << 4)) = c_hi;
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic-proxy stores -> tensor-core reads
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&hdr->b_full[sb]));
        }
        // ---- epilogue: TMEM -> registers -> bf16 -> global
        if (ok && mbar_wait_bounded(smem_u32(&hdr->acc_full), 0, cta_abort) && !*cta_abort) {
            tc_fence_after();
            const int q = warp & 3;                 // TMEM lane quarter this warp may read
            const int cq = (warp - 2) >> 2;         // the four warps of a quarter take 32 columns each
            for (int mb = 0; mb < mb_count; ++mb) {
                const int grow = m0 + mb * 128 + 32 * q + lane;
                {
                    const int col = 32 * cq;
                    uint32_t r[32];
                    tmem_ld32(tmem_base + ((uint32_t)(32 * q) << 16) + (uint32_t)(mb * GEMM_BN + col), r);
                    if (grow < p.m) {
                        const int gcol = n0 + col;
                        if (p.yf) {
                            float* dst = p.yf + (size_t)grow * p.n + gcol;
#pragma unroll
                            for (int i = 0; i < 32; ++i)
                                if (gcol + i < p.n) dst[i] = __uint_as_float(r[i]);
                        }
                        if (p.y) {
                            __nv_bfloat16* dst = p.y + (size_t)grow * p.n + gcol;
                            if (gcol + 32 <= p.n && (((size_t)grow * p.n + gcol) & 7) == 0) {
#pragma unroll
                                for (int i = 0; i < 32; i += 8) {
                                    uint32_t o[4];
#pragma unroll
                                    for (int j = 0; j < 4; ++j) {
                                        const __nv_bfloat162 pr =
                                            __floats2bfloat162_rn(__uint_as_float(r[i + 2 * j]), __uint_as_float(r[i + 2 * j + 1]));
                                        o[j] = *reinterpret_cast<const uint32_t*>(&pr);
                                    }
                                    *reinterpret_cast<uint4*>(dst + i) = make_uint4(o[0], o[1], o[2], o[3]);
                                }
                            } else {
#pragma unroll
                                for (int i = 0; i < 32; ++i)
                                    if (gcol + i < p.n) dst[i] = __float2bfloat16_rn(__uint_as_float(r[i]));
                            }
                        }
                    }
                }
            }
        } else if (ok && lane == 0) {
            give_up(DEV_TIMEOUT_MMA);
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
static int g_gemm_mb = 0;  // tunable "gemm_mb": row blocks per CTA, 0 = automatic
int gemm_set_mb(int v) {
    if (v < 0 || v > GEMM_MB_MAX || v == 3) return QMM_ERR_UNSUPPORTED;
    g_gemm_mb = v;
    return QMM_OK;
}

int qgemm_q4k_launch(const void* w, const void* x, void* y, float* yf, int m, int n, int k, cudaStream_t stream) {
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
    const cuuint32_t box[2] = {GEMM_BK, 128};
    const cuuint32_t estr[2] = {1, 1};
    if (enc(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(x), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return cuda_fail(cudaErrorInvalidValue);

    GemmParams p;
    p.w = static_cast<const uint8_t*>(w);
    p.y = static_cast<__nv_bfloat16*>(y);
    p.yf = yf;
    p.m = m, p.n = n, p.k = k;
    p.row_bytes = k / 256 * Q4_K_BYTES;
    p.probe = g_gemm_probe;
    const size_t smem = (size_t)(GEMM_SA + GEMM_SB) * GEMM_TILE_BYTES + sizeof(GemmSmemHeader) + 1024;
    static bool configured[64] = {};
    int dev = 0;
    QMM_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        QMM_CUDA_TRY(cudaFuncSetAttribute(qgemm_q4k_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    // Row blocks of x per CTA.  Measured on B200 at K = 4096: a CTA takes about 36 us (its whole weight tile is
    // unpacked whatever the rows) plus 18.5 us per row block (the tensor-core side), and the grid runs in waves
    // of one CTA per SM; take the count with the smallest modelled time ("gemm_mb" overrides).
    const int col_tiles = (n + GEMM_BN - 1) / GEMM_BN, row_blocks = (m + 127) / 128;
    int mb = GEMM_MB_MAX;
    double best = 0.0;
    for (int cand = GEMM_MB_MAX; cand >= 1; cand /= 2) {
        const long ctas = (long)col_tiles * ((row_blocks + cand - 1) / cand);
        const double t = (double)((ctas + sm_count() - 1) / sm_count()) * (36.0 + 18.5 * cand);
        if (cand == GEMM_MB_MAX || t < best) best = t, mb = cand;
    }
    if (g_gemm_mb >= 1 && g_gemm_mb <= GEMM_MB_MAX) mb = g_gemm_mb;
    p.mb_per_cta = mb;
    const dim3 grid(col_tiles, (row_blocks + mb - 1) / mb);
    qgemm_q4k_kernel<<<grid, GEMM_THREADS, smem, stream>>>(map, p);
    QMM_CUDA_TRY(cudaGetLastError());
    return QMM_OK;
}

}  // namespace qmm
