// Small-batch decode matvec on the int8 tensor cores:  y(m,n) = xq(m,k) . w(n,k)^T  for 5..16
// activation rows per launch, w in Q4_K super-blocks, xq in Q8_1 blocks.
//
// The dp4a kernel (qmatvec.cu) pays its integer dot products once per activation row; from a
// handful of rows on it is bound by instruction issue and re-streams the weights for every four
// rows.  Here one warp-level mma.sync.m16n8k32 (u8 x s8 -> s32) multiplies a sub-block (32 weights)
// of 16 weight rows with 8 activation rows, so the weights stream once for up to 16 rows:
//
//   * one persistent CTA per SM owns a contiguous range of 16-row tiles; the K axis is cut into
//     chunks of CW super-block columns (CW = consumer warps).  A ring stage holds the pieces
//     (16 rows x CW super-blocks) of one tile and one chunk, fetched with one 1-D bulk copy per row
//     (cp.async.bulk + mbarrier, issued by warp 0 between its tiles); the row pitch in shared
//     memory is chosen so that the 8-byte fragment loads of a half-warp touch 32 different banks;
//   * consumer warp c owns super-block column c of the chunk and keeps the Q8_1 words, scales
//     and sums of that column for all activation rows in registers, already in B-fragment order
//     (reloaded once per chunk); the 4-bit weights are masked straight into A fragments;
//   * the per-sub-block integer sums are scaled in float (6-bit scale as an integer multiply-add
//     onto a magic constant, then the activation scale), the mins term  sum_j m_j * s_j  of a
//     super-block is one f16 mma (6-bit mins and the fp16 sums of Q8_1 are exact in f16);
//   * the CW partial tiles of a stage are added in a fixed order after a named barrier (no atomics);
//     with several chunks the running sums wait in shared memory until the last chunk.
#include "qmm_formats.cuh"

namespace qmm {

struct MmaParams {
    const uint8_t* w;
    const uint8_t* xq;
    float* y;
    long y_stride;
    int m, n;
    int k_blocks;      // super-blocks per weight row
    int row_bytes, xq_row_bytes;
    int cw;            // consumer warps = super-block columns per chunk
    int n_chunks;
    int pitch;         // bytes between the row pieces of a stage
    int nst;           // ring stages
    int stage_bytes;   // 16 * pitch
    int tiles_total;   // ceil(n / 16)
    int part_off, yacc_off, ring_off;
};

constexpr int MMA_MAX_STAGES = 8;
constexpr int MMA_MAX_CW = 16;

struct __align__(16) MmaSmemHeader {
    uint64_t full[MMA_MAX_STAGES];
    int abort_flag;
};

__device__ __forceinline__ void mma_u8s8_k32(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                             uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}
// k = 16 with the upper eight k zero on both sides
__device__ __forceinline__ void mma_f16_k16_lo(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%6}, {%7,%6}, {%8,%8,%8,%8};"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a0), "r"(a1), "r"(0), "r"(b0), "f"(0.f));
}
__device__ __forceinline__ void named_bar_sync(int id, int threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}
// exact float of sum * scale for |sum * scale| < 2^22: integer multiply-add onto 1.5 * 2^23, then subtract it
__device__ __forceinline__ float scaled_sum_to_float(int sum, int scale) {
    return __int_as_float(sum * scale + 0x4B400000) - 12582912.f;
}
// two 6-bit codes (bytes 0 and 1 of v) as f16x2: 0x6400 | c is 1024 + c
__device__ __forceinline__ uint32_t codes_to_half2(uint32_t v) {
    const uint32_t biased = __byte_perm(v, 0x64646464u, 0x4140);
    const __half2 r = __hsub2(*reinterpret_cast<const __half2*>(&biased), __float2half2_rn(1024.f));
    return *reinterpret_cast<const uint32_t*>(&r);
}

__device__ __forceinline__ bool mma_wait(uint32_t bar, uint32_t parity, volatile int* cta_abort) {
    if (*cta_abort) return false;
    return mbar_wait_bounded(bar, parity, cta_abort);
}

// NT: activation rows in tiles of eight (1: m <= 8, 2: m <= 16)
template <int NT>
__global__ void __launch_bounds__(MMA_MAX_CW * 32, 1) qmv_mma_q4k_kernel(const MmaParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    MmaSmemHeader* hdr = reinterpret_cast<MmaSmemHeader*>(smem);
    float* part = reinterpret_cast<float*>(smem + p.part_off);   // [2][cw][128*NT]
    float* yacc = reinterpret_cast<float*>(smem + p.yacc_off);   // [tiles][128*NT], several chunks only
    uint8_t* ring = smem + p.ring_off;
    volatile int* cta_abort = &hdr->abort_flag;
    constexpr int OUTS = 128 * NT;  // values of one 16 x (8*NT) output tile, in fragment order

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t_begin = (int)((long)blockIdx.x * p.tiles_total / gridDim.x);
    const int t_end = (int)((long)(blockIdx.x + 1) * p.tiles_total / gridDim.x);
    const int tiles = t_end - t_begin;
    const int row0 = t_begin * 16;
    const int rows_cta = min(p.n, t_end * 16) - row0;
    const int n_it = p.n_chunks * tiles;

    if (threadIdx.x == 0) {
        for (int s = 0; s < p.nst; ++s) mbar_init(smem_u32(&hdr->full[s]), 1);
        hdr->abort_flag = 0;
        mbar_fence_init();
    }
    __syncthreads();
    pdl_release_dependents();

    // Stage `it` = (chunk it / tiles, tile it % tiles).  Warp 0 issues the copies: the named barrier that
    // every warp passes once per stage (below) also tells it that the slot of the stage just finished
    // is free, so the ring needs no second set of barriers and no warp of its own.
    auto issue = [&](int it) {
        const int slot = it % p.nst;
        const int c = it / tiles, ti = it - c * tiles;
        const int cols = min(p.cw, p.k_blocks - c * p.cw);
        const uint32_t piece = (uint32_t)cols * Q4_K_BYTES;
        const int nr = min(16, rows_cta - ti * 16);
        const uint32_t bar = smem_u32(&hdr->full[slot]);
        if (lane == 0) mbar_arrive_expect_tx(bar, (uint32_t)nr * piece);
        __syncwarp();
        if (lane < nr)
            bulk_g2s(smem_u32(ring + (size_t)slot * p.stage_bytes + (size_t)lane * p.pitch),
                     p.w + (size_t)(row0 + ti * 16 + lane) * p.row_bytes + (size_t)c * p.cw * Q4_K_BYTES, piece, bar);
    };
    int issued = 0;
    if (warp == 0)
        for (; issued < n_it && issued < p.nst; ++issued) issue(issued);

    // Every warp passes every stage and every named barrier, also after a timeout (it then skips
    // the waits and the arithmetic), so no warp is left behind at a barrier.
    const int q = lane >> 2, pq = lane & 3;
    const int tid = threadIdx.x;
    pdl_wait_prior_grids();  // activations come from the preceding kernel, y may still be read by it

    uint32_t xb0[NT][8], xb1[NT][8];  // B fragments: sub-block j, activation row 8t+q, elements 8pq.. and 8pq+4..
    uint32_t xdh[NT][8];              // NT == 2: fp16 scales of activation rows 8t+2pq (low half) and 8t+2pq+1
    float xda[NT][8], xdb[NT][8];     // NT == 1: the same scales as floats
    uint32_t xsf[NT];                 // f16x2: Q8_1 sums of sub-blocks 2pq, 2pq+1 of activation row 8t+q

    for (int c = 0; c < p.n_chunks; ++c) {
        const int col = c * p.cw + warp;
        const bool active = col < p.k_blocks;
        const int cols = min(p.cw, p.k_blocks - c * p.cw);
        if (active) {
#pragma unroll
            for (int t = 0; t < NT; ++t) {
                const int bq = 8 * t + q, ba = 8 * t + 2 * pq;
                const uint8_t* rq = p.xq + (size_t)bq * p.xq_row_bytes + (size_t)col * 8 * Q8_1_BYTES;
                const uint8_t* ra = p.xq + (size_t)ba * p.xq_row_bytes + (size_t)col * 8 * Q8_1_BYTES;
                const uint8_t* rb = ra + p.xq_row_bytes;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    uint32_t w0 = 0, w1 = 0, da = 0, db = 0;
                    if (bq < p.m) {
                        const uint32_t* qs = reinterpret_cast<const uint32_t*>(rq + j * Q8_1_BYTES + 4 + 8 * pq);
                        w0 = qs[0], w1 = qs[1];
                    }
                    if (ba < p.m) da = *reinterpret_cast<const uint16_t*>(ra + j * Q8_1_BYTES);
                    if (ba + 1 < p.m) db = *reinterpret_cast<const uint16_t*>(rb + j * Q8_1_BYTES);
                    xb0[t][j] = w0, xb1[t][j] = w1;
                    if constexpr (NT == 1) {
                        xda[t][j] = f16_bits_to_f32(da), xdb[t][j] = f16_bits_to_f32(db);
                    } else {
                        xdh[t][j] = da | (db << 16);
                    }
                }
                uint32_t s = 0;
                if (bq < p.m) {
                    const uint32_t s0 = *reinterpret_cast<const uint16_t*>(rq + (2 * pq) * Q8_1_BYTES + 2);
                    const uint32_t s1 = *reinterpret_cast<const uint16_t*>(rq + (2 * pq + 1) * Q8_1_BYTES + 2);
                    s = s0 | (s1 << 16);
                }
                xsf[t] = s;
            }
        }

        for (int ti = 0; ti < tiles; ++ti) {
            const int it = c * tiles + ti, slot = it % p.nst;
            bool ok = mma_wait(smem_u32(&hdr->full[slot]), (it / p.nst) & 1, cta_abort);
            if (!ok && lane == 0 && !*cta_abort) {
                atomicExch(&g_device_status, DEV_TIMEOUT_FULL);
                *cta_abort = 1;
            }
            float* my_part = part + ((size_t)(it & 1) * p.cw + warp) * OUTS + lane;
            if (ok && active) {
                const uint8_t* r0 = ring + (size_t)slot * p.stage_bytes + (size_t)q * p.pitch + (size_t)warp * Q4_K_BYTES;
                const uint8_t* r1 = r0 + 8 * (size_t)p.pitch;
                const uint4 h0 = *reinterpret_cast<const uint4*>(r0);
                const uint4 h1 = *reinterpret_cast<const uint4*>(r1);
                // 6-bit codes, one per byte: A = sub-blocks 0..3, B = 4..7
                const uint32_t scA0 = h0.y & 0x3F3F3F3Fu, scB0 = (h0.w & 0x0F0F0F0Fu) | ((h0.y >> 2) & 0x30303030u);
                const uint32_t scA1 = h1.y & 0x3F3F3F3Fu, scB1 = (h1.w & 0x0F0F0F0Fu) | ((h1.y >> 2) & 0x30303030u);
                const uint32_t mA0 = h0.z & 0x3F3F3F3Fu, mB0 = ((h0.w >> 4) & 0x0F0F0F0Fu) | ((h0.z >> 2) & 0x30303030u);
                const uint32_t mA1 = h1.z & 0x3F3F3F3Fu, mB1 = ((h1.w >> 4) & 0x0F0F0F0Fu) | ((h1.z >> 2) & 0x30303030u);
                // mins of sub-blocks 2pq, 2pq+1 of both rows as f16x2 A fragments
                const uint32_t sh = 16u * (pq & 1);
                const uint32_t ma0 = codes_to_half2(((pq < 2) ? mA0 : mB0) >> sh);
                const uint32_t ma1 = codes_to_half2(((pq < 2) ? mA1 : mB1) >> sh);
                float cm[NT][4], acc[NT][4];
#pragma unroll
                for (int t = 0; t < NT; ++t) {
                    mma_f16_k16_lo(cm[t], ma0, ma1, xsf[t]);
#pragma unroll
                    for (int i = 0; i < 4; ++i) acc[t][i] = 0.f;
                }
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                    const uint2 w0 = *reinterpret_cast<const uint2*>(r0 + 16 + 32 * g + 8 * pq);
                    const uint2 w1 = *reinterpret_cast<const uint2*>(r1 + 16 + 32 * g + 8 * pq);
#pragma unroll
                    for (int hi = 0; hi < 2; ++hi) {
                        const int j = 2 * g + hi;
                        const uint32_t a0 = (hi ? (w0.x >> 4) : w0.x) & 0x0F0F0F0Fu, a2 = (hi ? (w0.y >> 4) : w0.y) & 0x0F0F0F0Fu;
                        const uint32_t a1 = (hi ? (w1.x >> 4) : w1.x) & 0x0F0F0F0Fu, a3 = (hi ? (w1.y >> 4) : w1.y) & 0x0F0F0F0Fu;
                        const int sc0 = (int)(((j < 4 ? scA0 : scB0) >> (8 * (j & 3))) & 0xFFu);
                        const int sc1 = (int)(((j < 4 ? scA1 : scB1) >> (8 * (j & 3))) & 0xFFu);
#pragma unroll
                        for (int t = 0; t < NT; ++t) {
                            int d[4];
                            mma_u8s8_k32(d, a0, a1, a2, a3, xb0[t][j], xb1[t][j]);
                            float da, db;
                            if constexpr (NT == 1) {
                                da = xda[t][j], db = xdb[t][j];
                            } else {
                                const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&xdh[t][j]));
                                da = f.x, db = f.y;
                            }
                            acc[t][0] += da * scaled_sum_to_float(d[0], sc0);
                            acc[t][1] += db * scaled_sum_to_float(d[1], sc0);
                            acc[t][2] += da * scaled_sum_to_float(d[2], sc1);
                            acc[t][3] += db * scaled_sum_to_float(d[3], sc1);
                        }
                    }
                }
                const float d0 = f16_bits_to_f32(h0.x & 0xFFFFu), dmin0 = f16_bits_to_f32(h0.x >> 16);
                const float d1 = f16_bits_to_f32(h1.x & 0xFFFFu), dmin1 = f16_bits_to_f32(h1.x >> 16);
#pragma unroll
                for (int t = 0; t < NT; ++t) {
                    my_part[(4 * t + 0) * 32] = d0 * acc[t][0] - dmin0 * cm[t][0];
                    my_part[(4 * t + 1) * 32] = d0 * acc[t][1] - dmin0 * cm[t][1];
                    my_part[(4 * t + 2) * 32] = d1 * acc[t][2] - dmin1 * cm[t][2];
                    my_part[(4 * t + 3) * 32] = d1 * acc[t][3] - dmin1 * cm[t][3];
                }
            }
            named_bar_sync(1, p.cw * 32);
            if (warp == 0 && it + p.nst < n_it && !*cta_abort) {
                issue(it + p.nst);
                issued = it + p.nst + 1;
            }
            // fold: thread tid owns value tid of the tile (fragment order: register tid/32 of lane tid%32)
            if (tid < OUTS && !*cta_abort) {
                const float* src = part + (size_t)(it & 1) * p.cw * OUTS + tid;
                float s = 0.f;
                for (int wv = 0; wv < cols; ++wv) s += src[(size_t)wv * OUTS];
                if (p.n_chunks > 1) {
                    float* ya = yacc + (size_t)ti * OUTS + tid;
                    if (c > 0) s += *ya;
                    if (c + 1 < p.n_chunks) *ya = s;
                }
                if (c + 1 == p.n_chunks) {
                    const int i = tid >> 5, l = tid & 31;
                    const int row = ti * 16 + (l >> 2) + 8 * ((i >> 1) & 1);
                    const int b = 8 * (i >> 2) + 2 * (l & 3) + (i & 1);
                    if (row < rows_cta && b < p.m) p.y[(size_t)b * p.y_stride + row0 + row] = s;
                }
            }
        }
    }
    if (warp == 0 && lane == 0 && *cta_abort) {
        // wait (bounded) for copies still in flight before the CTA's shared memory is released
        for (int it = max(0, issued - p.nst); it < issued; ++it) {
            const long long t0 = clock64();
            while (!mbar_try_wait(smem_u32(&hdr->full[it % p.nst]), (it / p.nst) & 1)) {
                if (clock64() - t0 > WAIT_LIMIT_CYCLES) {
                    atomicExch(&g_device_status, DEV_TIMEOUT_DRAIN);
                    break;
                }
            }
        }
    }
}

// ------------------------------------------------------------------- host side
static int g_mma_min_m = 3;  // fewest activation rows that take this path (0: never)
int mma_set_min_m(int v) {
    if (v < 0 || v > 16) return QMM_ERR_UNSUPPORTED;
    g_mma_min_m = v;
    return QMM_OK;
}
int mma_min_m() { return g_mma_min_m; }

template <int NT>
static int mma_launch_inst(const MmaParams& p, int grid, int threads, size_t smem, cudaStream_t stream) {
    auto kern = qmv_mma_q4k_kernel<NT>;
    static size_t configured[64] = {};
    int dev = 0;
    QMM_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || smem > configured[dev]) {
        QMM_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        if (dev >= 0 && dev < 64) configured[dev] = smem;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(threads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = overlap_enabled() ? 1 : 0;
    QMM_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, p));
    return QMM_OK;
}

// Returns QMM_ERR_UNSUPPORTED (nothing launched) when the shape does not fit this kernel; the caller
// then uses the dp4a kernel.  m <= 16.
int qmatvec_mma_launch(int type, const void* w, const void* xq, float* y, long y_stride, int m, int n, int k, cudaStream_t stream) {
    if (type != QMM_TYPE_Q4_K || m < 1 || m > 16 || k % QKK != 0) return QMM_ERR_UNSUPPORTED;
    MmaParams p = {};
    p.w = static_cast<const uint8_t*>(w);
    p.xq = static_cast<const uint8_t*>(xq);
    p.y = y;
    p.y_stride = y_stride;
    p.m = m;
    p.n = n;
    p.k_blocks = k / QKK;
    p.row_bytes = p.k_blocks * Q4_K_BYTES;
    p.xq_row_bytes = k / QK8 * Q8_1_BYTES;
    const int nt = m > 8 ? 2 : 1;
    // consumer warps: a divisor of the super-blocks per row in 12..16 if there is one (no ragged last chunk)
    int cw = p.k_blocks < MMA_MAX_CW ? p.k_blocks : MMA_MAX_CW;
    for (int c = MMA_MAX_CW; c >= 12; --c)
        if (p.k_blocks >= c && p.k_blocks % c == 0) {
            cw = c;
            break;
        }
    if (cw < 4 * nt) return QMM_ERR_UNSUPPORTED;  // the fold needs 128*nt threads
    p.cw = cw;
    p.n_chunks = (p.k_blocks + cw - 1) / cw;
    const int piece = cw * Q4_K_BYTES;
    p.pitch = piece + ((32 - piece % 128) + 128) % 128;  // pitch % 128 == 32: conflict-free 8-byte fragment loads
    p.stage_bytes = 16 * p.pitch;
    p.tiles_total = (n + 15) / 16;
    const int sms = sm_count();
    const int grid = p.tiles_total < sms ? p.tiles_total : sms;
    const int tiles_max = (p.tiles_total + grid - 1) / grid;
    constexpr size_t SMEM_LIMIT = 200 * 1024;
    p.part_off = 256;
    const size_t part_bytes = (size_t)2 * cw * 128 * nt * sizeof(float);
    p.yacc_off = (int)(p.part_off + part_bytes);
    const size_t yacc_bytes = p.n_chunks > 1 ? (size_t)tiles_max * 128 * nt * sizeof(float) : 0;
    p.ring_off = (int)((p.yacc_off + yacc_bytes + 127) & ~size_t(127));
    if ((size_t)p.ring_off + 2 * (size_t)p.stage_bytes > SMEM_LIMIT) return QMM_ERR_UNSUPPORTED;
    p.nst = (int)((SMEM_LIMIT - p.ring_off) / p.stage_bytes);
    if (p.nst > MMA_MAX_STAGES) p.nst = MMA_MAX_STAGES;
    const size_t smem = (size_t)p.ring_off + (size_t)p.nst * p.stage_bytes;
    const int threads = cw * 32;
    return nt == 1 ? mma_launch_inst<1>(p, grid, threads, smem, stream) : mma_launch_inst<2>(p, grid, threads, smem, stream);
}

}  // namespace qmm
