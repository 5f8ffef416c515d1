// Small-batch decode matvec on the int8 tensor cores:  y(m,n) = xq(m,k) . w(n,k)^T  for 3..32
// activation rows per launch, w in Q4_K or Q6_K super-blocks, xq in Q8_1 blocks.
//
// The dp4a kernel (qmatvec.cu) pays its integer dot products once per activation row; from a
// handful of rows on it is bound by instruction issue and re-streams the weights for every four
// rows.  Here one warp-level mma.sync.m16n8k32 (u8 x s8 -> s32) multiplies a sub-block (32 weights)
// of 16 weight rows with 8 activation rows, so the weights stream once for up to 32 rows:
//
//   * one persistent CTA per SM owns a contiguous range of 16-row tiles; the K axis is cut into
//     chunks of CW super-block columns (CW = warps).  A ring stage holds the pieces
//     (16 rows x CW super-blocks) of one tile and one chunk, fetched with one 3-D tensor copy
//     (cp.async.bulk.tensor + mbarrier) whose box is a little wider than the columns, which makes the
//     row pitch in shared memory one that spreads the 8-byte fragment loads of a half-warp over all banks;
//   * warp c owns super-block column c of the chunk and keeps the Q8_1 words, scales
//     and sums of that column for all activation rows in registers, already in B-fragment order
//     (reloaded once per chunk through a small staging area filled a chunk ahead); the 4-bit weights are
//     masked straight into A fragments;
//   * the per-sub-block integer sums are scaled in float (6-bit scale as an integer multiply-add
//     onto a magic constant, then the activation scale), the mins term  sum_j m_j * s_j  of a
//     super-block is one f16 mma (6-bit mins and the fp16 sums of Q8_1 are exact in f16);
//   * a warp keeps the sums of its column for TP tiles in REGISTERS over all the K chunks: a pass walks
//     (chunk, tile) with the tile innermost, so the activations of a column serve TP stages per reload, and
//     the warps meet only at the end of a pass, where every warp writes its TP tiles to shared memory, a
//     barrier joins them, and the tiles are added in warp order (fixed order, no atomics) by threads that
//     each own one (activation row, weight row) output, weight rows running along the lanes.  (A first form
//     of this kernel added the warps' partial tiles after EVERY stage, through shared memory and an
//     mbarrier: that cost more instructions than the arithmetic of the stage, 56 per mma.)
//   * the warps wait for the data of a stage and nothing else; each makes one arrival per stage on the
//     slot's release barrier, and the warp whose arrival completes it refills the slot (no producer warp:
//     registers are handed out per four warps, a ninth warp would cost every thread a quarter of them).
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
    int cw;            // warps = super-block columns per chunk
    int n_chunks;
    int pitch;         // bytes between the row pieces of a stage
    int chunk_groups;  // 96- or 48-byte groups per chunk of columns
    int nst;           // ring stages
    int stage_bytes;   // 16 * pitch
    int tiles_total;   // ceil(n / 16)
    int tiles_q, tiles_r;  // tiles_total / grid and tiles_total % grid
    int part_off, ring_off, xstage_off;
    TpPush push;       // tensor parallel: the outputs go to every rank's exchange area instead of y
};

constexpr int MMA_MAX_STAGES = 8;
constexpr int MMA_MAX_CW = 16;
#ifndef MMA_WAIT_SLEEP_NS
#define MMA_WAIT_SLEEP_NS 100
#endif

__device__ __forceinline__ void mma_u8s8_k32(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                             uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}
// k = 16, accumulating onto c: one 16-element scale group of Q6_K
__device__ __forceinline__ void mma_u8s8_k16(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t b0, const int (&c)[4]) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%8,%9,%10};"
                 : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
                 : "r"(a0), "r"(a1), "r"(b0), "r"(c[0]), "r"(c[1]), "r"(c[2]), "r"(c[3]));
}
// the same with signed weights and every accumulator input equal to c
__device__ __forceinline__ void mma_s8s8_k16(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t b0, int c) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%7,%7,%7};"
                 : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
                 : "r"(a0), "r"(a1), "r"(b0), "r"(c));
}
// k = 16 with the upper eight k zero on both sides
__device__ __forceinline__ void mma_f16_k16_lo(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%6}, {%7,%6}, {%8,%8,%8,%8};"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a0), "r"(a1), "r"(0), "r"(b0), "f"(0.f));
}
// two 6-bit codes (bytes 0 and 1 of v) as f16x2: 0x6400 | c is 1024 + c
__device__ __forceinline__ uint32_t codes_to_half2(uint32_t v) {
    const uint32_t biased = __byte_perm(v, 0x64646464u, 0x4140);
    const __half2 r = __hsub2(*reinterpret_cast<const __half2*>(&biased), __float2half2_rn(1024.f));
    return *reinterpret_cast<const uint32_t*>(&r);
}

// packed pairs of floats (one 64-bit register): d = a * b + c and d = a + b on both halves
__device__ __forceinline__ uint64_t pack_b64(uint32_t lo, uint32_t hi) {
    uint64_t d;
    asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "r"(lo), "r"(hi));
    return d;
}
__device__ __forceinline__ void unpack_f2(uint64_t v, float& lo, float& hi) {
    uint32_t a, b;
    asm("mov.b64 {%0, %1}, %2;" : "=r"(a), "=r"(b) : "l"(v));
    lo = __uint_as_float(a), hi = __uint_as_float(b);
}
__device__ __forceinline__ uint64_t pack_f2(float lo, float hi) { return pack_b64(__float_as_uint(lo), __float_as_uint(hi)); }
__device__ __forceinline__ uint64_t fma_f2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ uint64_t mul_f2(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ uint64_t add_f2(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
// shared-memory accesses by 32-bit shared address (no 64-bit address arithmetic in the inner loops)
__device__ __forceinline__ uint4 lds_v4(uint32_t a) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
    return v;
}
__device__ __forceinline__ uint2 lds_v2(uint32_t a) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(a));
    return v;
}
// the same with a compile-time byte offset folded into the instruction
template <int OFF>
__device__ __forceinline__ uint2 lds_v2_at(uint32_t a) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2+%3];" : "=r"(v.x), "=r"(v.y) : "r"(a), "n"(OFF));
    return v;
}
__device__ __forceinline__ uint32_t lds_u32(uint32_t a) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ uint32_t lds_u16(uint32_t a) {
    uint32_t v;
    asm volatile("{ .reg .b16 h; ld.shared.u16 h, [%1]; cvt.u32.u16 %0, h; }" : "=r"(v) : "r"(a));
    return v;
}
// two 16-bit loads (addresses a and a+8) packed into one word: bytes a, a+1, a+8, a+9
template <int OFF>
__device__ __forceinline__ uint32_t lds_u16_at(uint32_t a) {
    uint32_t v;
    asm volatile("{ .reg .b16 h; ld.shared.u16 h, [%1+%2]; cvt.u32.u16 %0, h; }" : "=r"(v) : "r"(a), "n"(OFF));
    return v;
}
// bytes a+OFF, a+OFF+1, a+OFF+8, a+OFF+9 in one word
template <int OFF>
__device__ __forceinline__ uint32_t lds_h2_at(uint32_t a) { return __byte_perm(lds_u16_at<OFF>(a), lds_u16_at<OFF + 8>(a), 0x5410); }
__device__ __forceinline__ uint32_t lds_h2(uint32_t a) { return __byte_perm(lds_u16(a), lds_u16(a + 8), 0x5410); }
__device__ __forceinline__ float lds_f32(uint32_t a) {
    float v;
    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ void sts_f32(uint32_t a, float v) { asm volatile("st.shared.f32 [%0], %1;" ::"r"(a), "f"(v) : "memory"); }
__device__ __forceinline__ uint32_t byte_n(uint32_t v, int n) { return __byte_perm(v, 0, 0x4440 + n); }

// Bounded wait of this kernel: a warp whose barrier is not ready sleeps between polls, leaving the issue
// slots to the warps that have work.
__device__ __forceinline__ bool mma_wait(uint32_t bar, uint32_t parity, volatile int* cta_abort) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 256; ++i) {
            __nanosleep(MMA_WAIT_SLEEP_NS);
            if (mbar_try_wait(bar, parity)) return true;
        }
        if (*cta_abort) return false;
        if (clock64() - t0 > WAIT_LIMIT_CYCLES) return false;
    }
}

struct __align__(16) MmaSmemHeader {
    uint64_t full[MMA_MAX_STAGES];
    uint64_t empty[MMA_MAX_STAGES];
    int abort_flag;
    int refill_next;  // first stage whose ring slot has not been handed back to the copies yet
};

// TYPE: Q4_K or Q6_K.  NT: activation rows in tiles of eight.  TP: 16-row weight tiles per pass.
// MAXW: most consumer warps (the register budget per thread follows from it).
template <int TYPE, int NT, int TP, int MAXW>
__global__ void __launch_bounds__(MAXW * 32, 1) qmv_mma_kernel(const __grid_constant__ CUtensorMap wmap, const MmaParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    MmaSmemHeader* hdr = reinterpret_cast<MmaSmemHeader*>(smem);
    volatile int* cta_abort = &hdr->abort_flag;
    constexpr int BLOCK_BYTES = TYPE == QMM_TYPE_Q4_K ? Q4_K_BYTES : Q6_K_BYTES;
    constexpr uint32_t X_COL_BYTES = 8 * Q8_1_BYTES;  // one super-block column of one activation row
    constexpr bool XD_HALF = NT > 2;                  // activation scales kept as f16 pairs (registers)
    const uint32_t part_s = smem_u32(smem + p.part_off);  // [cw][TP][NT][128] floats
    const uint32_t ring_s = (smem_u32(smem + p.ring_off) + 127u) & ~127u;  // tensor copies land on 128-byte boundaries
    const uint32_t full_s = smem_u32(&hdr->full[0]), empty_s = smem_u32(&hdr->empty[0]);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int bx = (int)blockIdx.x;
    const int t_begin = bx * p.tiles_q + min(bx, p.tiles_r);
    const int tiles = p.tiles_q + (bx < p.tiles_r ? 1 : 0);
    const int row0 = t_begin * 16;
    const int rows_cta = min(p.n, (t_begin + tiles) * 16) - row0;
    const int n_pass = (tiles + TP - 1) / TP;
    const int n_it = p.n_chunks * tiles;

    if (threadIdx.x == 0) {
        for (int s = 0; s < p.nst; ++s) mbar_init(full_s + 8 * s, 1), mbar_init(empty_s + 8 * s, p.cw);
        hdr->abort_flag = 0;
        hdr->refill_next = 0;
        mbar_fence_init();
    }
    __syncthreads();
    pdl_release_dependents();

    auto give_up = [&](int code) {
        if (lane == 0 && !*cta_abort) {
            atomicExch(&g_device_status, code);
            *cta_abort = 1;
        }
    };

    // Stage `it` of pass ps is (chunk c, tile ti), the tile innermost.  One 3-D tensor copy of 16 rows x pitch
    // bytes per stage, the row as (96- or 48-byte groups, group index); the box is wider than the chunk's
    // columns so that the rows land pitch bytes apart (what it fetches beyond them is never read).
    auto issue = [&](int slot, int ps, int c, int ti) {
        const uint32_t bar = full_s + 8 * slot;
        mbar_arrive_expect_tx(bar, (uint32_t)p.stage_bytes);
        asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];" ::"r"(
                         ring_s + (uint32_t)slot * p.stage_bytes),
                     "l"(reinterpret_cast<uint64_t>(&wmap)), "r"(0), "r"(c * p.chunk_groups), "r"(row0 + (ps * TP + ti) * 16), "r"(bar)
                     : "memory");
    };
    // coordinates of the stage p.nst ahead of the current one (the one that refills the current slot),
    // advanced with the stages
    int r_ps = 0, r_c = 0, r_ti = 0, r_tp = min(TP, tiles);
    auto r_advance = [&]() {
        if (++r_ti == r_tp) {
            r_ti = 0;
            if (++r_c == p.n_chunks) r_c = 0, ++r_ps, r_tp = min(TP, tiles - r_ps * TP);
        }
    };
    for (int s = 0; s < p.nst && s < n_it; ++s) {
        if (warp == 0 && lane == 0) issue(s, r_ps, r_c, r_ti);
        r_advance();
    }

    const int q = lane >> 2, pq = lane & 3;
    const int cthreads = p.cw * 32;
    pdl_wait_prior_grids();  // activations come from the preceding kernel, y may still be read by it
    unsigned push_seq = 0u;
    if (p.push.tp > 0) push_seq = tp_next_seq(p.push.counter);

    // Activations of a warp's column reach its registers through a private staging area: NT*8 rows x 288
    // bytes fetched with 16-byte asynchronous copies, requested one chunk ahead, then read in fragment order
    // (one bulk copy per row onto a barrier of the warp's own measured 7 % slower).
    const uint32_t xst_s = smem_u32(smem + p.xstage_off) + (uint32_t)warp * (NT * 8 * X_COL_BYTES);
    auto stage_x = [&](int col) {
        for (int i = lane; i < NT * 8 * 18; i += 32) {
            const int r = i / 18, piece = i - r * 18;
            if (r < p.m) {
                const uint8_t* src = p.xq + (size_t)r * p.xq_row_bytes + (size_t)col * X_COL_BYTES + piece * 16;
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(xst_s + r * X_COL_BYTES + piece * 16), "l"(src) : "memory");
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    if (warp < p.k_blocks) stage_x(warp);

    uint2 xb[NT][8];                       // B fragments: sub-block j, activation row 8t+q, elements 8pq.. (x) and 8pq+4.. (y)
    uint64_t xdf[XD_HALF ? 1 : NT][8];     // scales of activation rows 8t+2pq, 8t+2pq+1 as a pair of floats
    uint32_t xdh[XD_HALF ? NT : 1][8];     // or as an f16 pair
    uint32_t xsf[NT];                      // f16x2: Q8_1 sums of sub-blocks 2pq, 2pq+1 of activation row 8t+q
    auto load_b = [&]() {
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncwarp();
#pragma unroll
        for (int t = 0; t < NT; ++t) {
            const int bq = 8 * t + q, ba = 8 * t + 2 * pq;
            const uint32_t rq = xst_s + (uint32_t)bq * X_COL_BYTES, ra = xst_s + (uint32_t)ba * X_COL_BYTES;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                uint32_t w0 = 0, w1 = 0, da = 0, db = 0;
                if (bq < p.m) {
                    if constexpr (TYPE == QMM_TYPE_Q4_K) {
                        w0 = lds_u32(rq + j * Q8_1_BYTES + 4 + 8 * pq), w1 = lds_u32(rq + j * Q8_1_BYTES + 8 + 8 * pq);
                    } else {  // 16-element run s of the block: elements 2pq, 2pq+1, 8+2pq, 9+2pq of the run
                        w0 = lds_h2(rq + j * Q8_1_BYTES + 4 + 2 * pq), w1 = lds_h2(rq + j * Q8_1_BYTES + 4 + 16 + 2 * pq);
                    }
                }
                if (ba < p.m) da = lds_u16(ra + j * Q8_1_BYTES);
                if (ba + 1 < p.m) db = lds_u16(ra + X_COL_BYTES + j * Q8_1_BYTES);
                xb[t][j] = make_uint2(w0, w1);
                if constexpr (XD_HALF)
                    xdh[t][j] = da | (db << 16);
                else
                    xdf[t][j] = pack_f2(f16_bits_to_f32(da), f16_bits_to_f32(db));
            }
            uint32_t s = 0;
            if (TYPE == QMM_TYPE_Q4_K && bq < p.m) s = lds_u16(rq + (2 * pq) * Q8_1_BYTES + 2) | (lds_u16(rq + (2 * pq + 1) * Q8_1_BYTES + 2) << 16);
            xsf[t] = s;
        }
        __syncwarp();  // the staging area is overwritten next
    };
    auto scale_pair = [&](int t, int j) -> uint64_t {
        if constexpr (XD_HALF) {
            const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&xdh[t][j]));
            return pack_f2(f.x, f.y);
        } else {
            return xdf[t][j];
        }
    };

    const uint64_t minus_magic = pack_f2(-12582912.f, -12582912.f);
    const uint32_t sh_m = 16u * (pq & 1);
    const uint32_t my_row_off = (uint32_t)q * p.pitch + (uint32_t)warp * BLOCK_BYTES;

    // One stage: the warp's super-block of 16 weight rows against all activation rows, added to A01 (weight
    // row q: activation rows 2pq, 2pq+1 of every tile of eight) and A23 (weight row q+8).
    auto tile = [&](uint32_t r0, uint64_t (&A01)[NT], uint64_t (&A23)[NT]) {
        const uint32_t r1 = r0 + 8u * p.pitch;
        uint64_t acc01[NT], acc23[NT];
        if constexpr (TYPE == QMM_TYPE_Q4_K) {
            const uint32_t q0 = r0 + 8 * pq, q1 = r1 + 8 * pq;  // this lane's 8 bytes of every 32-byte group
            const uint4 h0 = lds_v4(r0), h1 = lds_v4(r1);
            // 6-bit codes, one per byte: A = sub-blocks 0..3, B = 4..7
            const uint32_t scA0 = h0.y & 0x3F3F3F3Fu, scB0 = (h0.w & 0x0F0F0F0Fu) | ((h0.y >> 2) & 0x30303030u);
            const uint32_t scA1 = h1.y & 0x3F3F3F3Fu, scB1 = (h1.w & 0x0F0F0F0Fu) | ((h1.y >> 2) & 0x30303030u);
            const uint32_t mA0 = h0.z & 0x3F3F3F3Fu, mB0 = ((h0.w >> 4) & 0x0F0F0F0Fu) | ((h0.z >> 2) & 0x30303030u);
            const uint32_t mA1 = h1.z & 0x3F3F3F3Fu, mB1 = ((h1.w >> 4) & 0x0F0F0F0Fu) | ((h1.z >> 2) & 0x30303030u);
            // mins of sub-blocks 2pq, 2pq+1 of both rows as f16x2 A fragments
            const uint32_t ma0 = codes_to_half2(((pq < 2) ? mA0 : mB0) >> sh_m);
            const uint32_t ma1 = codes_to_half2(((pq < 2) ? mA1 : mB1) >> sh_m);
            const float d0 = f16_bits_to_f32(h0.x & 0xFFFFu), dmin0 = f16_bits_to_f32(h0.x >> 16);
            const float d1 = f16_bits_to_f32(h1.x & 0xFFFFu), dmin1 = f16_bits_to_f32(h1.x >> 16);
            const uint64_t nm0 = pack_f2(-dmin0, -dmin0), nm1 = pack_f2(-dmin1, -dmin1);
#pragma unroll
            for (int t = 0; t < NT; ++t) {
                float cm[4];
                mma_f16_k16_lo(cm, ma0, ma1, xsf[t]);
                A01[t] = fma_f2(nm0, pack_f2(cm[0], cm[1]), A01[t]);
                A23[t] = fma_f2(nm1, pack_f2(cm[2], cm[3]), A23[t]);
                acc01[t] = 0, acc23[t] = 0;
            }
#pragma unroll
            for (int g = 0; g < 4; ++g) {
                const uint2 w0 = g == 0 ? lds_v2_at<16>(q0) : g == 1 ? lds_v2_at<48>(q0) : g == 2 ? lds_v2_at<80>(q0) : lds_v2_at<112>(q0);
                const uint2 w1 = g == 0 ? lds_v2_at<16>(q1) : g == 1 ? lds_v2_at<48>(q1) : g == 2 ? lds_v2_at<80>(q1) : lds_v2_at<112>(q1);
#pragma unroll
                for (int hi = 0; hi < 2; ++hi) {
                    const int j = 2 * g + hi;
                    const uint32_t a0 = (hi ? (w0.x >> 4) : w0.x) & 0x0F0F0F0Fu, a2 = (hi ? (w0.y >> 4) : w0.y) & 0x0F0F0F0Fu;
                    const uint32_t a1 = (hi ? (w1.x >> 4) : w1.x) & 0x0F0F0F0Fu, a3 = (hi ? (w1.y >> 4) : w1.y) & 0x0F0F0F0Fu;
                    const int sc0 = (int)byte_n(j < 4 ? scA0 : scB0, j & 3);
                    const int sc1 = (int)byte_n(j < 4 ? scA1 : scB1, j & 3);
#pragma unroll
                    for (int t = 0; t < NT; ++t) {
                        int d[4];
                        mma_u8s8_k32(d, a0, a1, a2, a3, xb[t][j].x, xb[t][j].y);
                        const uint64_t dab = scale_pair(t, j);
                        // sum * scale as exact floats: integer multiply-add onto 1.5 * 2^23, then subtract it
                        const uint64_t v01 = pack_b64((uint32_t)(d[0] * sc0 + 0x4B400000), (uint32_t)(d[1] * sc0 + 0x4B400000));
                        const uint64_t v23 = pack_b64((uint32_t)(d[2] * sc1 + 0x4B400000), (uint32_t)(d[3] * sc1 + 0x4B400000));
                        acc01[t] = fma_f2(dab, add_f2(v01, minus_magic), acc01[t]);
                        acc23[t] = fma_f2(dab, add_f2(v23, minus_magic), acc23[t]);
                    }
                }
            }
#pragma unroll
            for (int t = 0; t < NT; ++t) {
                A01[t] = fma_f2(pack_f2(d0, d0), acc01[t], A01[t]);
                A23[t] = fma_f2(pack_f2(d1, d1), acc23[t], A23[t]);
            }
        } else {
            // ---- Q6_K: sixteen runs of 16 weights with one int8 scale each, one k = 16 mma per run.
            // The codes stay unsigned (low nibble | two high bits); their offset of 32 enters through
            // a first mma of the constant -32 against the same activations, which also plants the
            // float magic 1.5 * 2^23 in the accumulator, so the result is the exact sum as a float.
            uint32_t sw0[4], sw1[4];  // the sixteen scales of both rows, biased to unsigned
#define QMM_Q6_SCALES(I)                                                                                                  \
    sw0[I] = __byte_perm(lds_u16_at<192 + 4 * I>(r0), lds_u16_at<194 + 4 * I>(r0), 0x5410) ^ 0x80808080u,                \
    sw1[I] = __byte_perm(lds_u16_at<192 + 4 * I>(r1), lds_u16_at<194 + 4 * I>(r1), 0x5410) ^ 0x80808080u
            QMM_Q6_SCALES(0);
            QMM_Q6_SCALES(1);
            QMM_Q6_SCALES(2);
            QMM_Q6_SCALES(3);
#undef QMM_Q6_SCALES
            const uint64_t minus_bias = pack_f2(-(12582912.f + 128.f), -(12582912.f + 128.f));
#pragma unroll
            for (int t = 0; t < NT; ++t) acc01[t] = 0, acc23[t] = 0;
            const uint32_t q0 = r0 + 2 * pq, q1 = r1 + 2 * pq;  // this lane's two bytes of every 8-byte piece
#pragma unroll
            for (int hs = 0; hs < 4; ++hs) {
                const int h = hs >> 1, s = hs & 1;
                uint32_t A0, B0, H0, A1, B1, H1;
                // ql at 64h + 16s (+32), qh at 128 + 32h + 16s; the offsets are instruction immediates
#define QMM_Q6_LOAD(HS)                                                                                                  \
    A0 = lds_h2_at<64 * (HS >> 1) + 16 * (HS & 1)>(q0), B0 = lds_h2_at<64 * (HS >> 1) + 16 * (HS & 1) + 32>(q0),         \
    H0 = lds_h2_at<128 + 32 * (HS >> 1) + 16 * (HS & 1)>(q0), A1 = lds_h2_at<64 * (HS >> 1) + 16 * (HS & 1)>(q1),        \
    B1 = lds_h2_at<64 * (HS >> 1) + 16 * (HS & 1) + 32>(q1), H1 = lds_h2_at<128 + 32 * (HS >> 1) + 16 * (HS & 1)>(q1)
                if (hs == 0) QMM_Q6_LOAD(0);
                else if (hs == 1) QMM_Q6_LOAD(1);
                else if (hs == 2) QMM_Q6_LOAD(2);
                else QMM_Q6_LOAD(3);
#undef QMM_Q6_LOAD
#pragma unroll
                for (int t4 = 0; t4 < 4; ++t4) {
                    const uint32_t s0 = (t4 & 1) ? B0 : A0, s1 = (t4 & 1) ? B1 : A1;
                    const uint32_t n0 = (t4 < 2 ? s0 : s0 >> 4) & 0x0F0F0F0Fu, n1 = (t4 < 2 ? s1 : s1 >> 4) & 0x0F0F0F0Fu;
                    const uint32_t g0 = t4 == 0 ? H0 << 4 : t4 == 1 ? H0 << 2 : t4 == 2 ? H0 : H0 >> 2;
                    const uint32_t g1 = t4 == 0 ? H1 << 4 : t4 == 1 ? H1 << 2 : t4 == 2 ? H1 : H1 >> 2;
                    const uint32_t qa0 = n0 | (g0 & 0x30303030u), qa1 = n1 | (g1 & 0x30303030u);
                    const int idx = 8 * h + 2 * t4 + s, j = 4 * h + t4;
                    // (scale + 128) as a float by byte insertion into the magic constant, twice in a pair
                    const uint32_t v0 = __byte_perm(sw0[idx >> 2], 0x4B400000u, 0x7640 + (idx & 3));
                    const uint32_t v1 = __byte_perm(sw1[idx >> 2], 0x4B400000u, 0x7640 + (idx & 3));
                    const uint64_t S0 = add_f2(pack_b64(v0, v0), minus_bias), S1 = add_f2(pack_b64(v1, v1), minus_bias);
#pragma unroll
                    for (int t = 0; t < NT; ++t) {
                        const uint32_t xw = s ? xb[t][j].y : xb[t][j].x;
                        int d1[4], d[4];
                        mma_s8s8_k16(d1, 0xE0E0E0E0u, 0xE0E0E0E0u, xw, 0x4B400000);
                        mma_u8s8_k16(d, qa0, qa1, xw, d1);
                        const uint64_t dab = scale_pair(t, j);
                        const uint64_t f01 = add_f2(pack_b64((uint32_t)d[0], (uint32_t)d[1]), minus_magic);
                        const uint64_t f23 = add_f2(pack_b64((uint32_t)d[2], (uint32_t)d[3]), minus_magic);
                        acc01[t] = fma_f2(mul_f2(dab, S0), f01, acc01[t]);
                        acc23[t] = fma_f2(mul_f2(dab, S1), f23, acc23[t]);
                    }
                }
            }
            const float d0 = f16_bits_to_f32(lds_u16_at<208>(r0)), d1f = f16_bits_to_f32(lds_u16_at<208>(r1));
#pragma unroll
            for (int t = 0; t < NT; ++t) {
                A01[t] = fma_f2(pack_f2(d0, d0), acc01[t], A01[t]);
                A23[t] = fma_f2(pack_f2(d1f, d1f), acc23[t], A23[t]);
            }
        }
    };

    int slot = 0, it = 0;
    uint32_t full_par = 0;
    bool dead = false, loaded = false;
    constexpr int ROWS_P = TP * 16;
    constexpr uint32_t WARP_PART_B = (uint32_t)TP * NT * 128 * 4;  // bytes between the partial tiles of two warps

    for (int ps = 0; ps < n_pass; ++ps) {
        const int tp_now = min(TP, tiles - ps * TP);
        uint64_t A01[TP][NT], A23[TP][NT];
#pragma unroll
        for (int ti = 0; ti < TP; ++ti)
#pragma unroll
            for (int t = 0; t < NT; ++t) A01[ti][t] = 0, A23[ti][t] = 0;

        for (int c = 0; c < p.n_chunks; ++c) {
            const int col = c * p.cw + warp;
            const bool active = col < p.k_blocks;
            // with one chunk the activations of the column stay in the registers for every pass
            if (active && (p.n_chunks > 1 || !loaded)) {
                load_b();
                loaded = true;
            }
            if (p.n_chunks > 1) {
                const bool wrap = c + 1 == p.n_chunks;
                const int ncol = wrap ? warp : col + p.cw;
                if ((!wrap || ps + 1 < n_pass) && ncol < p.k_blocks) stage_x(ncol);
            }
#pragma unroll
            for (int ti = 0; ti < TP; ++ti) {
                if (ti < tp_now) {
                    bool ok = !dead;  // after a timeout only the arrivals remain
                    if (ok && !mma_wait(full_s + 8 * slot, full_par, cta_abort)) {
                        give_up(DEV_TIMEOUT_FULL);
                        ok = false, dead = true;
                    }
                    if (ok && active) tile(ring_s + (uint32_t)slot * p.stage_bytes + my_row_off, A01[ti], A23[ti]);
                    __syncwarp();
                    // Once the arrivals of a stage are complete nobody reads its weights any more.  The warp that
                    // arrives last sees the phase complete at once and refills the slot; if two warps see it,
                    // the compare-and-swap picks one.  (The release barrier of a slot is in the same phase as
                    // its data barrier: both complete once per use of the slot.)
                    if (lane == 0) {
                        const uint32_t bar = empty_s + 8 * slot;
                        mbar_arrive(bar);
                        if (it + p.nst < n_it && !dead && mbar_test_wait(bar, full_par) && atomicCAS(&hdr->refill_next, it, it + 1) == it)
                            issue(slot, r_ps, r_c, r_ti);
                    }
                    r_advance();
                    ++it;
                    if (++slot == p.nst) slot = 0, full_par ^= 1;
                }
            }
        }

        // ---- end of the pass: the warps' tiles meet in shared memory
        {
            const uint32_t mp = part_s + (uint32_t)warp * WARP_PART_B + (uint32_t)lane * 4u;
#pragma unroll
            for (int ti = 0; ti < TP; ++ti)
#pragma unroll
                for (int t = 0; t < NT; ++t) {
                    float a, b, e, f;
                    unpack_f2(A01[ti][t], a, b);
                    unpack_f2(A23[ti][t], e, f);
                    const uint32_t at = mp + (uint32_t)((ti * NT + t) * 512);
                    sts_f32(at, a), sts_f32(at + 128, b), sts_f32(at + 256, e), sts_f32(at + 384, f);
                }
        }
        __syncthreads();
        if (!dead) {
            for (int o = (int)threadIdx.x; o < ROWS_P * 8 * NT; o += cthreads) {
                const int rr = o % ROWS_P, b = o / ROWS_P;
                const int ti = rr >> 4, row = rr & 15;
                const int grow = (ps * TP + ti) * 16 + row;
                if (ti < tp_now && b < p.m && grow < rows_cta) {
                    // register (row / 8) * 2 + (b & 1) of lane (row % 8) * 4 + (b % 8) / 2 in tile (ti, b / 8)
                    const int fi = (((ti * NT + (b >> 3)) * 4 + ((row >> 3) * 2 + (b & 1))) * 32) + ((row & 7) * 4 + ((b & 7) >> 1));
                    const uint32_t a = part_s + (uint32_t)fi * 4u;
                    float sum = 0.f;
                    for (int w = 0; w < p.cw; ++w) sum += lds_f32(a + (uint32_t)w * WARP_PART_B);
                    tp_store_out(p.push, push_seq, p.y, p.y_stride, b, (long)row0 + grow, sum);
                }
            }
        }
        if (ps + 1 < n_pass) __syncthreads();
    }
    asm volatile("cp.async.wait_all;" ::: "memory");  // a staged column that was never read
    __syncthreads();  // every warp is here (timed-out waits only skip work), so refill_next is final
    if (*cta_abort) {
        // wait (bounded) for copies still in flight before the CTA's shared memory is released
        if (warp == 0 && lane == 0) {
            const int issued = min(n_it, hdr->refill_next + p.nst);
            for (int s = max(0, issued - p.nst); s < issued; ++s) {
                const long long t0 = clock64();
                while (!mbar_try_wait(full_s + 8 * (s % p.nst), (s / p.nst) & 1)) {
                    if (clock64() - t0 > WAIT_LIMIT_CYCLES) {
                        atomicExch(&g_device_status, DEV_TIMEOUT_DRAIN);
                        break;
                    }
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

template <auto KERN>
static int mma_launch_kernel(const CUtensorMap& wmap, const MmaParams& p, int grid, int threads, size_t smem, cudaStream_t stream) {
    static size_t configured[64] = {};
    int dev = 0;
    QMM_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || smem > configured[dev]) {
        QMM_CUDA_TRY(cudaFuncSetAttribute(KERN, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
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
    QMM_CUDA_TRY(cudaLaunchKernelEx(&cfg, KERN, wmap, p));
    return QMM_OK;
}
// tunables (measured defaults: more tiles per pass = fewer reloads of the activations, as far as the registers go)
static int g_mma_acc_tp[3] = {8, 8, 4};  // weight tiles per pass for 1, 2 and 4 tiles of eight activation rows
static int g_mma_acc_w1 = 16;    // most warps for up to eight activation rows (8 or 16)
int mma_acc_set(const char* key, int v) {
    const std::string k(key);
    if (k == "mma_acc_w1") return (v == 8 || v == 16) ? (g_mma_acc_w1 = v, QMM_OK) : QMM_ERR_UNSUPPORTED;
    for (int i = 0; i < 3; ++i)
        if (k == std::string("mma_acc_tp") + char('0' + (1 << i))) return (v == 2 || v == 4 || v == 8) ? (g_mma_acc_tp[i] = v, QMM_OK) : QMM_ERR_UNSUPPORTED;
    return QMM_ERR_UNSUPPORTED;
}
int mma_group_rows() { return 32; }

static bool mma_tensor_map(CUtensorMap* wmap, const void* w, int group, long pitch_bytes, int n, int smem_pitch) {
    EncodeTiledFn enc = encode_tiled_fn();
    if (!enc) return false;
    const cuuint64_t dims[3] = {(cuuint64_t)(group / 4), (cuuint64_t)(pitch_bytes / group), (cuuint64_t)n};
    const cuuint64_t strides[2] = {(cuuint64_t)group, (cuuint64_t)pitch_bytes};
    const cuuint32_t box[3] = {(cuuint32_t)(group / 4), (cuuint32_t)(smem_pitch / group), 16};
    const cuuint32_t estr[3] = {1, 1, 1};
    return enc(wmap, CU_TENSOR_MAP_DATA_TYPE_UINT32, 3, const_cast<void*>(w), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
               CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int TYPE>
static int mma_dispatch(int nt, int tp, int maxw, const CUtensorMap& wmap, const MmaParams& p, int grid, int threads, size_t smem,
                            cudaStream_t stream) {
#define QMM_ACC_CASE(NT_, TP_, W_) \
    if (nt == NT_ && tp == TP_ && maxw == W_) return mma_launch_kernel<qmv_mma_kernel<TYPE, NT_, TP_, W_>>(wmap, p, grid, threads, smem, stream)
    QMM_ACC_CASE(1, 8, 16);
    QMM_ACC_CASE(1, 4, 16);
    QMM_ACC_CASE(1, 2, 16);
    QMM_ACC_CASE(1, 8, 8);
    QMM_ACC_CASE(1, 4, 8);
    QMM_ACC_CASE(1, 2, 8);
    QMM_ACC_CASE(2, 8, 8);
    QMM_ACC_CASE(2, 4, 8);
    QMM_ACC_CASE(2, 2, 8);
    QMM_ACC_CASE(4, 4, 8);
    QMM_ACC_CASE(4, 2, 8);
#undef QMM_ACC_CASE
    return QMM_ERR_UNSUPPORTED;
}

// m <= 32.  Returns QMM_ERR_UNSUPPORTED (nothing launched) when the type or shape does not fit.
static int qmatvec_mma_launch_one(int type, const void* w, long row_pitch, const void* xq, float* y, long y_stride, int m, int n, int k,
                                  int cta_limit, const TpPush* push, cudaStream_t stream) {
    if ((type != QMM_TYPE_Q4_K && type != QMM_TYPE_Q6_K) || m < 1 || m > 32 || k % QKK != 0) return QMM_ERR_UNSUPPORTED;
    if (reinterpret_cast<uintptr_t>(xq) % 16 != 0 || reinterpret_cast<uintptr_t>(w) % 16 != 0) return QMM_ERR_UNSUPPORTED;
    const bool q4 = type == QMM_TYPE_Q4_K;
    const int block_bytes = q4 ? Q4_K_BYTES : Q6_K_BYTES;
    MmaParams p = {};
    p.w = static_cast<const uint8_t*>(w);
    p.xq = static_cast<const uint8_t*>(xq);
    p.y = y;
    p.y_stride = y_stride;
    p.m = m;
    p.n = n;
    if (push) p.push = *push;
    p.k_blocks = k / QKK;
    p.row_bytes = p.k_blocks * block_bytes;
    p.xq_row_bytes = k / QK8 * Q8_1_BYTES;
    const long pitch_bytes = row_pitch ? row_pitch : p.row_bytes;
    if (pitch_bytes < p.row_bytes) return QMM_ERR_SHAPE;
    const int nt = m > 16 ? 4 : (m > 8 ? 2 : 1);
    const int maxw = nt == 1 ? g_mma_acc_w1 : 8;
    // tensor copies: a row and a chunk of columns are whole groups (Q4_K: 96 bytes, even column counts;
    // Q6_K: 48 bytes, multiples of eight columns)
    const int group = q4 ? 96 : 48;
    const int col_step = q4 ? 2 : 8;
    if (pitch_bytes % group != 0 || pitch_bytes % 16 != 0) return QMM_ERR_UNSUPPORTED;
    // consumer warps = columns per chunk: the largest divisor of the super-blocks per row within a quarter
    // of the most (no ragged last chunk), else the most; a short row takes the next multiple of col_step
    int cw = p.k_blocks < maxw ? (p.k_blocks + col_step - 1) / col_step * col_step : maxw;
    for (int c = maxw; c >= maxw - maxw / 4; c -= col_step)
        if (p.k_blocks >= c && p.k_blocks % c == 0) {
            cw = c;
            break;
        }
    if (cw > maxw) return QMM_ERR_UNSUPPORTED;
    p.cw = cw;
    p.n_chunks = (p.k_blocks + cw - 1) / cw;
    const int piece = cw * block_bytes;
    p.pitch = 0;
    for (int pad = 0; pad <= 8 * group; pad += group) {
        const int cand = piece + pad;
        if (q4 ? (pad > 0 && (cand % 128 == 32 || cand % 128 == 96)) : (cand % 32 == 16)) {
            p.pitch = cand;
            break;
        }
    }
    if (!p.pitch) return QMM_ERR_UNSUPPORTED;
    p.chunk_groups = piece / group;
    p.stage_bytes = 16 * p.pitch;
    CUtensorMap wmap;
    if (!mma_tensor_map(&wmap, w, group, pitch_bytes, n, p.pitch)) return cuda_fail(cudaErrorInvalidValue);
    p.tiles_total = (n + 15) / 16;
    int sms = sm_count();
    if (cta_limit > 0 && cta_limit < sms) sms = cta_limit;
    const int grid = p.tiles_total < sms ? p.tiles_total : sms;
    const int tiles_max = (p.tiles_total + grid - 1) / grid;
    p.tiles_q = p.tiles_total / grid, p.tiles_r = p.tiles_total % grid;
    // tiles per pass: the configured number, no more than a CTA has (the partial tiles take shared memory)
    int tp = g_mma_acc_tp[nt == 1 ? 0 : (nt == 2 ? 1 : 2)];
    if (nt == 4 && tp > 4) tp = 4;
    while (tp > 2 && tp / 2 >= tiles_max) tp /= 2;
    constexpr size_t SMEM_LIMIT = 220 * 1024;
    p.part_off = (sizeof(MmaSmemHeader) + 127) & ~127;
    p.xstage_off = p.part_off + cw * tp * nt * 512;
    p.ring_off = (p.xstage_off + cw * nt * 8 * 8 * Q8_1_BYTES + 127) & ~127;
    if ((size_t)p.ring_off + 128 + 2 * (size_t)p.stage_bytes > SMEM_LIMIT) return QMM_ERR_UNSUPPORTED;
    p.nst = (int)((SMEM_LIMIT - p.ring_off - 128) / p.stage_bytes);
    if (p.nst > MMA_MAX_STAGES) p.nst = MMA_MAX_STAGES;
    const size_t smem = (size_t)p.ring_off + 128 + (size_t)p.nst * p.stage_bytes;
    const int threads = cw * 32;
    return q4 ? mma_dispatch<QMM_TYPE_Q4_K>(nt, tp, maxw, wmap, p, grid, threads, smem, stream)
              : mma_dispatch<QMM_TYPE_Q6_K>(nt, tp, maxw, wmap, p, grid, threads, smem, stream);
}

// Returns QMM_ERR_UNSUPPORTED (nothing launched) when the type or shape does not fit this kernel; the
// caller then uses the dp4a kernel.  m <= 32.
int qmatvec_mma_launch(int type, const void* w, long row_pitch, const void* xq, float* y, long y_stride, int m, int n, int k, int cta_limit,
                       unsigned long long* /*trace*/, const TpPush* push, cudaStream_t stream) {
    return qmatvec_mma_launch_one(type, w, row_pitch, xq, y, y_stride, m, n, k, cta_limit, push, stream);
}

}  // namespace qmm
