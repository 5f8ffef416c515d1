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
#include "qmm_formats.cuh"

namespace qmm {

constexpr int PF_BQ = 64, PF_BK = 64;

__device__ __forceinline__ uint32_t pack_h2(float a, float b) {
    const __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&h);
}

// HD: head dimension (a multiple of 16 up to 256).  GH: query heads of one kv head per CTA (1 or 2), four warps each.
template <int HD, int GH>
__global__ void __launch_bounds__(128 * GH) attn_prefill_kernel(const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v,
                                                                  float* __restrict__ out, int t, int nqh, int nkv, int prefix, float kq_scale,
                                                                  long q_stride, long k_stride, long v_stride, long o_stride,
                                                                  __nv_bfloat16* __restrict__ out_bf16) {
    extern __shared__ __align__(16) uint8_t pf_raw[];
    constexpr int PITCH = HD + 8;  // halves: rows 16 bytes apart modulo 128, so the 8 rows of an ldmatrix hit all banks
    constexpr int PF_THREADS = 128 * GH;
    __half* qs_all = reinterpret_cast<__half*>(pf_raw);  // GH query tiles
    __half* ks = qs_all + GH * PF_BQ * PITCH;
    __half* vs = ks + PF_BK * PITCH;
    const int tid = threadIdx.x, wall = tid >> 5, lane = tid & 31, qr = lane >> 2, pq = lane & 3;
    const int hl = wall >> 2, warp = wall & 3;  // head within the CTA, 16-row block of the query tile
    const int qt = blockIdx.x, h = blockIdx.y * GH + hl, kvh = (blockIdx.y * GH) / (nqh / nkv);
    __half* qs = qs_all + hl * PF_BQ * PITCH;
    const size_t qd = (size_t)q_stride, kd = (size_t)k_stride, vd = (size_t)v_stride, od = (size_t)o_stride;  // floats between rows
    const int q0 = qt * PF_BQ;

    // the query tiles, scaled, as f16 (rows past t as zeros)
    for (int i = tid; i < GH * PF_BQ * (HD / 4); i += PF_THREADS) {
        const int hh = i / (PF_BQ * (HD / 4)), j = i - hh * (PF_BQ * (HD / 4));
        const int r = j / (HD / 4), c = (j - r * (HD / 4)) * 4;
        float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
        if (q0 + r < t) x = *reinterpret_cast<const float4*>(q + (size_t)(q0 + r) * qd + (size_t)(blockIdx.y * GH + hh) * HD + c);
        *reinterpret_cast<uint2*>(qs_all + (hh * PF_BQ + r) * PITCH + c) = make_uint2(pack_h2(x.x * kq_scale, x.y * kq_scale), pack_h2(x.z * kq_scale, x.w * kq_scale));
    }

    // this thread's two query rows and their running softmax state
    const int p0 = q0 + 16 * warp + qr, p1 = p0 + 8;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
    float o[HD / 8][4];
#pragma unroll
    for (int n = 0; n < HD / 8; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;

    // key tiles: a tile of queries that is causal throughout stops at its own diagonal tile
    const int n_kt = (t + PF_BK - 1) / PF_BK;
    const int kt_end = (q0 + PF_BQ <= prefix) ? min(n_kt, qt + 1) : n_kt;
    // Keys and values of a tile: float4 pieces, KV_IT per thread and matrix.  When a thread's pieces of a tile fit
    // its registers (KV_IT <= 8) the NEXT tile's loads are issued before the current tile's arithmetic, so their round
    // trip to L2 hides under the mma; otherwise a tile is loaded in chunks of eight pieces right before its use.
    constexpr int KV_IT = PF_BK * (HD / 4) / PF_THREADS;  // (whole: HD is a multiple of 32)
    constexpr bool PREFETCH = KV_IT <= 8;
    constexpr int KV_CH = KV_IT < 8 ? KV_IT : 8;
    float4 ka[KV_CH], va[KV_CH];
    auto load_kv = [&](int kt, int base) {
#pragma unroll
        for (int it = 0; it < KV_CH; ++it) {
            const int i = tid + (base + it) * PF_THREADS, r = i / (HD / 4), c = (i - r * (HD / 4)) * 4;
            const int sp = kt * PF_BK + r;
            ka[it] = va[it] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (sp < t) {
                ka[it] = *reinterpret_cast<const float4*>(k + (size_t)sp * kd + (size_t)kvh * HD + c);
                va[it] = *reinterpret_cast<const float4*>(v + (size_t)sp * vd + (size_t)kvh * HD + c);
            }
        }
    };
    auto store_kv = [&](int base) {
#pragma unroll
        for (int it = 0; it < KV_CH; ++it) {
            const int i = tid + (base + it) * PF_THREADS, r = i / (HD / 4), c = (i - r * (HD / 4)) * 4;
            *reinterpret_cast<uint2*>(ks + r * PITCH + c) = make_uint2(pack_h2(ka[it].x, ka[it].y), pack_h2(ka[it].z, ka[it].w));
            *reinterpret_cast<uint2*>(vs + r * PITCH + c) = make_uint2(pack_h2(va[it].x, va[it].y), pack_h2(va[it].z, va[it].w));
        }
    };
    if (PREFETCH && kt_end > 0) load_kv(0, 0);
    for (int kt = 0; kt < kt_end; ++kt) {
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

        // scores of the warp's 16 query rows against the 64 keys: 8 n-tiles of 8 keys
        float s[PF_BK / 8][4];
#pragma unroll
        for (int n = 0; n < PF_BK / 8; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
        const __half* qa = qs + (16 * warp + qr) * PITCH + 2 * pq;
#pragma unroll
        for (int kk = 0; kk < HD; kk += 16) {
            const uint32_t a0 = *reinterpret_cast<const uint32_t*>(qa + kk), a1 = *reinterpret_cast<const uint32_t*>(qa + 8 * PITCH + kk);
            const uint32_t a2 = *reinterpret_cast<const uint32_t*>(qa + kk + 8), a3 = *reinterpret_cast<const uint32_t*>(qa + 8 * PITCH + kk + 8);
#pragma unroll
            for (int n = 0; n < PF_BK / 8; ++n) {
                const __half* kb = ks + (8 * n + qr) * PITCH + 2 * pq + kk;
                mma_f16_k16(s[n], a0, a1, a2, a3, *reinterpret_cast<const uint32_t*>(kb), *reinterpret_cast<const uint32_t*>(kb + 8));
            }
        }
        // mask (the upstream writes -1e30 into a masked score; a key past the end does not exist), running softmax
        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int n = 0; n < PF_BK / 8; ++n) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int sp = kt * PF_BK + 8 * n + 2 * pq + e;
                if (sp >= t) s[n][e] = -INFINITY, s[n][2 + e] = -INFINITY;
                else {
                    if (p0 < prefix && sp > p0) s[n][e] = -1e30f;
                    if (p1 < prefix && sp > p1) s[n][2 + e] = -1e30f;
                }
                mx0 = fmaxf(mx0, s[n][e]), mx1 = fmaxf(mx1, s[n][2 + e]);
            }
        }
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
            for (int n = 0; n < HD / 8; ++n) {
                const uint32_t addr = smem_u32(vs + (16 * j + (lane & 15)) * PITCH + 8 * n);
                uint32_t b0, b1;
                asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];" : "=r"(b0), "=r"(b1) : "r"(addr));
                mma_f16_k16(o[n], pa[j][0], pa[j][1], pa[j][2], pa[j][3], b0, b1);
            }
        }
    }
    const float i0 = l0 > 0.f ? 1.f / l0 : 0.f, i1 = l1 > 0.f ? 1.f / l1 : 0.f;
#pragma unroll
    for (int n = 0; n < HD / 8; ++n) {
        if (out_bf16) {  // the same layout as out, as bf16 (the input of a GEMM)
            if (p0 < t) *reinterpret_cast<__nv_bfloat162*>(out_bf16 + (size_t)p0 * od + (size_t)h * HD + 8 * n + 2 * pq) = __floats2bfloat162_rn(o[n][0] * i0, o[n][1] * i0);
            if (p1 < t) *reinterpret_cast<__nv_bfloat162*>(out_bf16 + (size_t)p1 * od + (size_t)h * HD + 8 * n + 2 * pq) = __floats2bfloat162_rn(o[n][2] * i1, o[n][3] * i1);
        } else {
            if (p0 < t) *reinterpret_cast<float2*>(out + (size_t)p0 * od + (size_t)h * HD + 8 * n + 2 * pq) = make_float2(o[n][0] * i0, o[n][1] * i0);
            if (p1 < t) *reinterpret_cast<float2*>(out + (size_t)p1 * od + (size_t)h * HD + 8 * n + 2 * pq) = make_float2(o[n][2] * i1, o[n][3] * i1);
        }
    }
}

template <int HD, int GH>
static int attn_prefill_inst(const float* q, const float* k, const float* v, float* out, int t, int nqh, int nkv, int prefix, float kq_scale,
                             long q_stride, long k_stride, long v_stride, long o_stride, __nv_bfloat16* out_bf16, cudaStream_t s) {
    const size_t smem = (size_t)(GH * PF_BQ + 2 * PF_BK) * (HD + 8) * sizeof(__half);
    static std::mutex mu;
    static bool configured[64] = {};
    int dev = 0;
    QMM_CUDA_TRY(cudaGetDevice(&dev));
    if (smem > 48 * 1024) {
        std::lock_guard<std::mutex> g(mu);
        if (dev < 0 || dev >= 64 || !configured[dev]) {
            QMM_CUDA_TRY(cudaFuncSetAttribute(attn_prefill_kernel<HD, GH>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            if (dev >= 0 && dev < 64) configured[dev] = true;
        }
    }
    attn_prefill_kernel<HD, GH><<<dim3((t + PF_BQ - 1) / PF_BQ, nqh / GH), 128 * GH, smem, s>>>(q, k, v, out, t, nqh, nkv, prefix, kq_scale, q_stride, k_stride,
                                                                                                 v_stride, o_stride, out_bf16);
    QMM_CUDA_TRY(cudaGetLastError());
    return QMM_OK;
}

// q, k, v, out with their own row strides (floats; multiples of 4): the projections of a layer write [q | k] and v
// side by side
int attn_prefill_launch(const float* q, const float* k, const float* v, float* out, int t, int n_q_heads, int n_kv_heads, int head_dim, int prefix,
                        float kq_scale, long q_stride, long k_stride, long v_stride, long o_stride, cudaStream_t s, __nv_bfloat16* out_bf16) {
    if (!q || !k || !v || (!out && !out_bf16)) return QMM_ERR_NULL;
    if (t <= 0 || n_q_heads <= 0 || n_kv_heads <= 0 || n_q_heads % n_kv_heads != 0 || prefix < 0) return QMM_ERR_SHAPE;
    if (q_stride < (long)n_q_heads * head_dim || o_stride < (long)n_q_heads * head_dim || k_stride < (long)n_kv_heads * head_dim ||
        v_stride < (long)n_kv_heads * head_dim || q_stride % 4 || k_stride % 4 || v_stride % 4 || o_stride % 2)
        return QMM_ERR_SHAPE;
    if (out == q || out == k || out == v) return QMM_ERR_SHAPE;  // every CTA reads the whole sequence (as upstream)
    if (reinterpret_cast<uintptr_t>(q) % 16 || reinterpret_cast<uintptr_t>(k) % 16 || reinterpret_cast<uintptr_t>(v) % 16 ||
        reinterpret_cast<uintptr_t>(out) % 8 || reinterpret_cast<uintptr_t>(out_bf16) % 4)
        return QMM_ERR_ALIGN;
    const bool two = (n_q_heads / n_kv_heads) % 2 == 0;  // two query heads of a kv head per CTA
#define QMM_PF_CASE(HD_)                                                                                                                              \
    case HD_:                                                                                                                                          \
        return two ? attn_prefill_inst<HD_, 2>(q, k, v, out, t, n_q_heads, n_kv_heads, prefix, kq_scale, q_stride, k_stride, v_stride, o_stride, out_bf16, s)   \
                   : attn_prefill_inst<HD_, 1>(q, k, v, out, t, n_q_heads, n_kv_heads, prefix, kq_scale, q_stride, k_stride, v_stride, o_stride, out_bf16, s)
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
    return attn_prefill_launch(q, k, v, out, t, n_q_heads, n_kv_heads, head_dim, prefix, kq_scale, qd, kd, kd, qd, as_stream(stream), nullptr);
}
