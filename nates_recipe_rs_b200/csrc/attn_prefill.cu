// Attention over a whole sequence at once, the counterpart of the upstream's gpu_gqa_attn_into
// (gpu-core/src/infer_ops.rs:160-189 -> launch_gqa_masked_attn, gpu-core/src/kernels/f64_infer.hip:42-100):
// q (t, nqh*hd), k and v (t, nkv*hd), out (t, nqh*hd), query head h reads kv head h / (nqh / nkv); positions
// p < prefix are causal (attend sp <= p), positions p >= prefix attend the whole sequence; the scores are
// q.k * kq_scale (the upstream folds its scale into q and passes 1).  The upstream runs one block per
// (position, head) with the t scores in shared memory and one thread doing the softmax; here a CTA owns 64
// query positions of one head and walks the keys in tiles of 64 with a running softmax, scores and outputs on the
// f16 tensor cores (mma.sync.m16n8k16, f32 accumulation): q (scaled), k, v and the probabilities are rounded to
// f16, about 1e-3 relative, everything else is f32.  The t x t score matrix is never stored.  When two query heads
// share a kv head the CTA takes both (eight warps), so a tile of keys and values is fetched and converted once for
// the two: the kernel is bound by that traffic (f32 k and v from L2 for every tile of queries), not by the mma.
// KV16: k and v are already f16 (the rows of a KV cache, strides in halves): their tiles go from global to shared
// memory with cp.async, the next tile's copy in flight under the current tile's arithmetic (two stages), no
// conversion and half the traffic.
#include "qmm_formats.cuh"

namespace qmm {

constexpr int PF_BQ = 64, PF_BK = 64;

__device__ __forceinline__ uint32_t pack_h2(float a, float b) {
    const __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&h);
}

__device__ __forceinline__ void cp_async_16(uint32_t smem_dst, const void* gsrc) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_dst), "l"(gsrc) : "memory");
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}

// HD: head dimension (a multiple of 16 up to 256).  GH: query heads of one kv head per CTA (1 or 2), four warps each.
template <int HD, int GH, bool KV16>
__global__ void __launch_bounds__(128 * GH, (KV16 && HD <= 128) ? 2 : 1) attn_prefill_kernel(const float* __restrict__ q, const void* __restrict__ k_, const void* __restrict__ v_,
                                                                  float* __restrict__ out, int t, int nqh, int nkv, int prefix, float kq_scale,
                                                                  long q_stride, long k_stride, long v_stride, long o_stride,
                                                                  __nv_bfloat16* __restrict__ out_bf16, int t_kv, int q_pos0) {
    extern __shared__ __align__(16) uint8_t pf_raw[];
    constexpr int PITCH = HD + 8;  // halves: rows 16 bytes apart modulo 128, so the 8 rows of an ldmatrix hit all banks
    constexpr int PF_THREADS = 128 * GH;
    __half* qs_all = reinterpret_cast<__half*>(pf_raw);  // GH query tiles
    constexpr int KV_STAGES = KV16 ? 2 : 1;
    __half* ks_all = qs_all + GH * PF_BQ * PITCH;            // KV_STAGES key tiles, then as many value tiles
    __half* vs_all = ks_all + KV_STAGES * PF_BK * PITCH;
    const float* k = static_cast<const float*>(k_);
    const float* v = static_cast<const float*>(v_);
    const __half* k16 = static_cast<const __half*>(k_);
    const __half* v16 = static_cast<const __half*>(v_);
    const int tid = threadIdx.x, wall = tid >> 5, lane = tid & 31, qr = lane >> 2, pq = lane & 3;
    const int hl = wall >> 2, warp = wall & 3;  // head within the CTA, 16-row block of the query tile
    // Causal tiles of queries cost in proportion to their position, and CTAs start in grid order (x fastest): the grid is
    // (head group, tile of queries) with the LAST tile of queries first, so the long CTAs start first and the short ones
    // fill the end of the run (started in increasing order the longest CTAs would begin when most of the GPU is idle).
    const int hg = blockIdx.x, qt = gridDim.y - 1 - blockIdx.y;
    const int h = hg * GH + hl, kvh = (hg * GH) / (nqh / nkv);
    __half* qs = qs_all + hl * PF_BQ * PITCH;
    const size_t qd = (size_t)q_stride, kd = (size_t)k_stride, vd = (size_t)v_stride, od = (size_t)o_stride;  // floats between rows
    const int q0 = qt * PF_BQ;

    // the query tiles, scaled, as f16 (rows past t as zeros)
    for (int i = tid; i < GH * PF_BQ * (HD / 4); i += PF_THREADS) {
        const int hh = i / (PF_BQ * (HD / 4)), j = i - hh * (PF_BQ * (HD / 4));
        const int r = j / (HD / 4), c = (j - r * (HD / 4)) * 4;
        float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
        if (q0 + r < t) x = *reinterpret_cast<const float4*>(q + (size_t)(q0 + r) * qd + (size_t)(hg * GH + hh) * HD + c);
        *reinterpret_cast<uint2*>(qs_all + (hh * PF_BQ + r) * PITCH + c) = make_uint2(pack_h2(x.x * kq_scale, x.y * kq_scale), pack_h2(x.z * kq_scale, x.w * kq_scale));
    }

    // this thread's two query rows and their running softmax state
    // (row r of q and out is position q_pos0 + r of the sequence; the keys and values are positions 0 .. t_kv-1)
    const int r0 = q0 + 16 * warp + qr, r1 = r0 + 8;
    const int p0 = q_pos0 + r0, p1 = p0 + 8;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
    float o[HD / 8][4];
#pragma unroll
    for (int n = 0; n < HD / 8; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;

    // key tiles: a tile of queries that is causal throughout stops at its own diagonal tile
    const int n_kt = (t_kv + PF_BK - 1) / PF_BK;
    const int kt_end = (q_pos0 + q0 + PF_BQ <= prefix) ? min(n_kt, (q_pos0 + q0 + PF_BQ - 1) / PF_BK + 1) : n_kt;
    // Keys and values of a tile: float4 pieces, KV_IT per thread and matrix.  When a thread's pieces of a tile fit
    // its registers (KV_IT <= 8) the NEXT tile's loads are issued before the current tile's arithmetic, so their round
    // trip to L2 hides under the mma; otherwise a tile is loaded in chunks of eight pieces right before its use.
    constexpr int KV_IT = PF_BK * (HD / 4) / PF_THREADS;  // (whole: HD is a multiple of 32)
    constexpr bool PREFETCH = !KV16 && KV_IT <= 8;
    constexpr int KV_CH = KV_IT < 8 ? KV_IT : 8;
    float4 ka[KV_CH], va[KV_CH];
    auto load_kv = [&](int kt, int base) {
#pragma unroll
        for (int it = 0; it < KV_CH; ++it) {
            const int i = tid + (base + it) * PF_THREADS, r = i / (HD / 4), c = (i - r * (HD / 4)) * 4;
            const int sp = kt * PF_BK + r;
            ka[it] = va[it] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (sp < t_kv) {
                ka[it] = *reinterpret_cast<const float4*>(k + (size_t)sp * kd + (size_t)kvh * HD + c);
                va[it] = *reinterpret_cast<const float4*>(v + (size_t)sp * vd + (size_t)kvh * HD + c);
            }
        }
    };
    auto store_kv = [&](int base) {
#pragma unroll
        for (int it = 0; it < KV_CH; ++it) {
            const int i = tid + (base + it) * PF_THREADS, r = i / (HD / 4), c = (i - r * (HD / 4)) * 4;
            *reinterpret_cast<uint2*>(ks_all + r * PITCH + c) = make_uint2(pack_h2(ka[it].x, ka[it].y), pack_h2(ka[it].z, ka[it].w));
            *reinterpret_cast<uint2*>(vs_all + r * PITCH + c) = make_uint2(pack_h2(va[it].x, va[it].y), pack_h2(va[it].z, va[it].w));
        }
    };
    // KV16: 16-byte pieces (8 halves) of a key and a value tile straight into stage `stage`; rows past t as zeros
    auto copy_kv16 = [&](int kt, int stage) {
        __half* kd_s = ks_all + stage * PF_BK * PITCH;
        __half* vd_s = vs_all + stage * PF_BK * PITCH;
        for (int i = tid; i < PF_BK * (HD / 8); i += PF_THREADS) {
            const int r = i / (HD / 8), c = (i - r * (HD / 8)) * 8;
            const int sp = kt * PF_BK + r;
            if (sp < t_kv) {
                cp_async_16(smem_u32(kd_s + r * PITCH + c), k16 + (size_t)sp * kd + (size_t)kvh * HD + c);
                cp_async_16(smem_u32(vd_s + r * PITCH + c), v16 + (size_t)sp * vd + (size_t)kvh * HD + c);
            } else {
                *reinterpret_cast<uint4*>(kd_s + r * PITCH + c) = make_uint4(0u, 0u, 0u, 0u);
                *reinterpret_cast<uint4*>(vd_s + r * PITCH + c) = make_uint4(0u, 0u, 0u, 0u);
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    if (PREFETCH && kt_end > 0) load_kv(0, 0);
    if (KV16 && kt_end > 0) copy_kv16(0, 0);
    for (int kt = 0; kt < kt_end; ++kt) {
        if constexpr (KV16) {
            asm volatile("cp.async.wait_group 0;" ::: "memory");  // this thread's pieces of tile kt
            __syncthreads();  // everyone's pieces; and the tile before is consumed (first pass: the query tile is written)
            if (kt + 1 < kt_end) copy_kv16(kt + 1, (kt + 1) & 1);
        } else {
            __syncthreads();  // the previous tile is consumed (first pass: the query tile is written)
            if constexpr (PREFETCH) {
                store_kv(0);
            } else {
#pragma unroll 1
                for (int base = 0; base < KV_IT; base += KV_CH) {
                    load_kv(kt, base);
                    store_kv(base);
                }
            }
            __syncthreads();
            if (PREFETCH && kt + 1 < kt_end) load_kv(kt + 1, 0);
        }
        const __half* ks = ks_all + (KV16 ? (kt & 1) : 0) * PF_BK * PITCH;
        const __half* vs = vs_all + (KV16 ? (kt & 1) : 0) * PF_BK * PITCH;

        // scores of the warp's 16 query rows against the 64 keys: 8 n-tiles of 8 keys
        float s[PF_BK / 8][4];
#pragma unroll
        for (int n = 0; n < PF_BK / 8; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
        // fragments by ldmatrix.x4: lane l addresses row (l & 7) of 8x8 matrix l >> 3.  A (queries): matrices = (rows 0-7 |
        // 8-15) x (columns kk.. | kk+8..); B (keys): the two column halves of key rows 8n..8n+7, then of 8n+8..8n+15
        const uint32_t qa = smem_u32(qs + (16 * warp + (lane & 7) + ((lane >> 3) & 1) * 8) * PITCH + ((lane >> 4) & 1) * 8);
        const uint32_t kb = smem_u32(ks + ((lane & 7) + ((lane >> 4) & 1) * 8) * PITCH + ((lane >> 3) & 1) * 8);
#pragma unroll
        for (int kk = 0; kk < HD; kk += 16) {
            uint32_t a0, a1, a2, a3;
            ldmatrix_x4(a0, a1, a2, a3, qa + kk * 2);
#pragma unroll
            for (int n = 0; n < PF_BK / 8; n += 2) {
                uint32_t b0, b1, b2, b3;
                ldmatrix_x4(b0, b1, b2, b3, kb + (8 * n * PITCH + kk) * 2);
                mma_f16_k16(s[n], a0, a1, a2, a3, b0, b1);
                mma_f16_k16(s[n + 1], a0, a1, a2, a3, b2, b3);
            }
        }
        // mask (the upstream writes -1e30 into a masked score; a key past the end does not exist), running softmax
        // (only a tile that reaches past the end or past the diagonal of this warp's first row has anything to mask)
        const int w0 = q_pos0 + q0 + 16 * warp;
        if (kt * PF_BK + PF_BK > t_kv || (w0 < prefix && kt * PF_BK + PF_BK - 1 > w0)) {
#pragma unroll
            for (int n = 0; n < PF_BK / 8; ++n) {
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int sp = kt * PF_BK + 8 * n + 2 * pq + e;
                    if (sp >= t_kv) s[n][e] = -INFINITY, s[n][2 + e] = -INFINITY;
                    else {
                        if (p0 < prefix && sp > p0) s[n][e] = -1e30f;
                        if (p1 < prefix && sp > p1) s[n][2 + e] = -1e30f;
                    }
                }
            }
        }
        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int n = 0; n < PF_BK / 8; ++n) mx0 = fmaxf(mx0, fmaxf(s[n][0], s[n][1])), mx1 = fmaxf(mx1, fmaxf(s[n][2], s[n][3]));
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1)), mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1)), mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);  // finite: every tile holds at least one existing key
        const float c0 = __expf(m0 - mn0), c1 = __expf(m1 - mn1);
        m0 = mn0, m1 = mn1;
        float r0 = 0.f, r1 = 0.f;
        uint32_t pa[PF_BK / 16][4];  // the probabilities as A fragments: key block j = n-tiles 2j, 2j+1
#pragma unroll
        for (int n = 0; n < PF_BK / 8; ++n) {
            const float e0 = __expf(s[n][0] - mn0), e1 = __expf(s[n][1] - mn0), e2 = __expf(s[n][2] - mn1), e3 = __expf(s[n][3] - mn1);
            r0 += e0 + e1, r1 += e2 + e3;
            pa[n >> 1][(n & 1) * 2] = pack_h2(e0, e1);
            pa[n >> 1][(n & 1) * 2 + 1] = pack_h2(e2, e3);
        }
        r0 += __shfl_xor_sync(0xffffffffu, r0, 1), r0 += __shfl_xor_sync(0xffffffffu, r0, 2);
        r1 += __shfl_xor_sync(0xffffffffu, r1, 1), r1 += __shfl_xor_sync(0xffffffffu, r1, 2);
        l0 = l0 * c0 + r0, l1 = l1 * c1 + r1;
#pragma unroll
        for (int n = 0; n < HD / 8; ++n) o[n][0] *= c0, o[n][1] *= c0, o[n][2] *= c1, o[n][3] *= c1;
        // outputs: P (16 x 64) . V (64 x HD), V transposed on load
#pragma unroll
        for (int j = 0; j < PF_BK / 16; ++j) {
#pragma unroll
            for (int n = 0; n < HD / 8; n += 2) {  // (transposed: key rows 16j..16j+7 | +8..15 of columns 8n.., then of 8n+8..)
                const uint32_t addr = smem_u32(vs + (16 * j + (lane & 15)) * PITCH + 8 * n + ((lane >> 4) & 1) * 8);
                uint32_t b0, b1, b2, b3;
                asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(b0), "=r"(b1), "=r"(b2), "=r"(b3) : "r"(addr));
                mma_f16_k16(o[n], pa[j][0], pa[j][1], pa[j][2], pa[j][3], b0, b1);
                mma_f16_k16(o[n + 1], pa[j][0], pa[j][1], pa[j][2], pa[j][3], b2, b3);
            }
        }
    }
    const float i0 = l0 > 0.f ? 1.f / l0 : 0.f, i1 = l1 > 0.f ? 1.f / l1 : 0.f;
#pragma unroll
    for (int n = 0; n < HD / 8; ++n) {
        if (out_bf16) {  // the same layout as out, as bf16 (the input of a GEMM)
            if (r0 < t) *reinterpret_cast<__nv_bfloat162*>(out_bf16 + (size_t)r0 * od + (size_t)h * HD + 8 * n + 2 * pq) = __floats2bfloat162_rn(o[n][0] * i0, o[n][1] * i0);
            if (r1 < t) *reinterpret_cast<__nv_bfloat162*>(out_bf16 + (size_t)r1 * od + (size_t)h * HD + 8 * n + 2 * pq) = __floats2bfloat162_rn(o[n][2] * i1, o[n][3] * i1);
        } else {
            if (r0 < t) *reinterpret_cast<float2*>(out + (size_t)r0 * od + (size_t)h * HD + 8 * n + 2 * pq) = make_float2(o[n][0] * i0, o[n][1] * i0);
            if (r1 < t) *reinterpret_cast<float2*>(out + (size_t)r1 * od + (size_t)h * HD + 8 * n + 2 * pq) = make_float2(o[n][2] * i1, o[n][3] * i1);
        }
    }
}

template <int HD, int GH, bool KV16>
static int attn_prefill_inst(const float* q, const void* k, const void* v, float* out, int t, int nqh, int nkv, int prefix, float kq_scale,
                             long q_stride, long k_stride, long v_stride, long o_stride, __nv_bfloat16* out_bf16, int t_kv, int q_pos0, cudaStream_t s) {
    const size_t smem = (size_t)(GH * PF_BQ + (KV16 ? 4 : 2) * PF_BK) * (HD + 8) * sizeof(__half);
    static std::mutex mu;
    static bool configured[64] = {};
    int dev = 0;
    QMM_CUDA_TRY(cudaGetDevice(&dev));
    if (smem > 48 * 1024) {
        std::lock_guard<std::mutex> g(mu);
        if (dev < 0 || dev >= 64 || !configured[dev]) {
            QMM_CUDA_TRY(cudaFuncSetAttribute(attn_prefill_kernel<HD, GH, KV16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            if (dev >= 0 && dev < 64) configured[dev] = true;
        }
    }
    attn_prefill_kernel<HD, GH, KV16><<<dim3(nqh / GH, (t + PF_BQ - 1) / PF_BQ), 128 * GH, smem, s>>>(q, k, v, out, t, nqh, nkv, prefix, kq_scale, q_stride, k_stride,
                                                                                                 v_stride, o_stride, out_bf16, t_kv, q_pos0);
    QMM_CUDA_TRY(cudaGetLastError());
    return QMM_OK;
}

// q, k, v, out with their own row strides (floats; multiples of 4): the projections of a layer write [q | k] and v
// side by side
// (kv_f16: k and v are f16 rows, their strides in halves and multiples of 8)
int attn_prefill_launch(const float* q, const void* k, const void* v, float* out, int t, int n_q_heads, int n_kv_heads, int head_dim, int prefix,
                        float kq_scale, long q_stride, long k_stride, long v_stride, long o_stride, cudaStream_t s, __nv_bfloat16* out_bf16, bool kv_f16, int t_kv, int q_pos0) {
    if (!q || !k || !v || (!out && !out_bf16)) return QMM_ERR_NULL;
    if (t <= 0 || n_q_heads <= 0 || n_kv_heads <= 0 || n_q_heads % n_kv_heads != 0 || prefix < 0) return QMM_ERR_SHAPE;
    if (t_kv <= 0) t_kv = t;  // (0: as many keys as queries, the first query at position 0)
    if (q_pos0 < 0 || q_pos0 + t > t_kv) return QMM_ERR_SHAPE;  // every query position has its own key
    if (q_stride < (long)n_q_heads * head_dim || o_stride < (long)n_q_heads * head_dim || k_stride < (long)n_kv_heads * head_dim ||
        v_stride < (long)n_kv_heads * head_dim || q_stride % 4 || k_stride % (kv_f16 ? 8 : 4) || v_stride % (kv_f16 ? 8 : 4) || o_stride % 2)
        return QMM_ERR_SHAPE;
    if (out == q || static_cast<const void*>(out) == k || static_cast<const void*>(out) == v) return QMM_ERR_SHAPE;  // every CTA reads the whole sequence (as upstream)
    if (reinterpret_cast<uintptr_t>(q) % 16 || reinterpret_cast<uintptr_t>(k) % 16 || reinterpret_cast<uintptr_t>(v) % 16 ||
        reinterpret_cast<uintptr_t>(out) % 8 || reinterpret_cast<uintptr_t>(out_bf16) % 4)
        return QMM_ERR_ALIGN;
    const bool two = (n_q_heads / n_kv_heads) % 2 == 0;  // two query heads of a kv head per CTA
#define QMM_PF_CASE(HD_)                                                                                                                              \
    case HD_:                                                                                                                                          \
        if (kv_f16)                                                                                                                                    \
            return two ? attn_prefill_inst<HD_, 2, true>(q, k, v, out, t, n_q_heads, n_kv_heads, prefix, kq_scale, q_stride, k_stride, v_stride, o_stride, out_bf16, t_kv, q_pos0, s) \
                       : attn_prefill_inst<HD_, 1, true>(q, k, v, out, t, n_q_heads, n_kv_heads, prefix, kq_scale, q_stride, k_stride, v_stride, o_stride, out_bf16, t_kv, q_pos0, s); \
        return two ? attn_prefill_inst<HD_, 2, false>(q, k, v, out, t, n_q_heads, n_kv_heads, prefix, kq_scale, q_stride, k_stride, v_stride, o_stride, out_bf16, t_kv, q_pos0, s)   \
                   : attn_prefill_inst<HD_, 1, false>(q, k, v, out, t, n_q_heads, n_kv_heads, prefix, kq_scale, q_stride, k_stride, v_stride, o_stride, out_bf16, t_kv, q_pos0, s)
    switch (head_dim) {
        QMM_PF_CASE(32);
        QMM_PF_CASE(64);
        QMM_PF_CASE(96);
        QMM_PF_CASE(128);
        QMM_PF_CASE(256);
    }
#undef QMM_PF_CASE
    return QMM_ERR_UNSUPPORTED;
}

}  // namespace qmm

using namespace qmm;

extern "C" int launch_attn_prefill(const float* q, const float* k, const float* v, float* out, int t, int n_q_heads, int n_kv_heads, int head_dim,
                                   int prefix, float kq_scale, void* stream) {
    const long qd = (long)n_q_heads * head_dim, kd = (long)n_kv_heads * head_dim;
    if (!out) return QMM_ERR_NULL;
    return attn_prefill_launch(q, k, v, out, t, n_q_heads, n_kv_heads, head_dim, prefix, kq_scale, qd, kd, kd, qd, as_stream(stream), nullptr, false, 0, 0);
}

extern "C" int launch_attn_prefill_f16kv(const float* q, const void* k, const void* v, float* out, int t, int n_q_heads, int n_kv_heads, int head_dim,
                                         int prefix, float kq_scale, void* stream) {
    const long qd = (long)n_q_heads * head_dim, kd = (long)n_kv_heads * head_dim;
    if (!out) return QMM_ERR_NULL;
    return attn_prefill_launch(q, k, v, out, t, n_q_heads, n_kv_heads, head_dim, prefix, kq_scale, qd, kd, kd, qd, as_stream(stream), nullptr, true, 0, 0);
}

// Queries at positions q_pos0 .. q_pos0+t-1 of a sequence whose keys and values 0 .. t_kv-1 are f16 rows (a KV cache that
// already holds the earlier positions): the continuation of a prompt.  Row for row the same arithmetic as the whole
// sequence in one call.
extern "C" int launch_attn_prefill_f16kv_at(const float* q, const void* k, const void* v, float* out, int t, int t_kv, int q_pos0, int n_q_heads,
                                            int n_kv_heads, int head_dim, int prefix, float kq_scale, void* stream) {
    const long qd = (long)n_q_heads * head_dim, kd = (long)n_kv_heads * head_dim;
    if (!out) return QMM_ERR_NULL;
    if (t_kv <= 0) return QMM_ERR_SHAPE;
    return attn_prefill_launch(q, k, v, out, t, n_q_heads, n_kv_heads, head_dim, prefix, kq_scale, qd, kd, kd, qd, as_stream(stream), nullptr, true, t_kv, q_pos0);
}
