// Mixture-of-experts branch of a decode step, on the device.
//
// The upstream example routes on the host: it downloads the activations, computes the router logits, the
// softmax and the top-k per token in f64 loops, gathers the tokens of every chosen expert into a staging
// buffer, uploads it, runs the expert's gate_up and down projections one expert after the other and
// accumulates the weighted outputs on the host again (examples/gemma4.rs:684-742).  Here nothing leaves
// the device:
//   * moe_router_topk_kernel   RMS-normalises a token (no gain), scales it, applies the router's input gain,
//                              takes the router logits (one warp per expert), the softmax over the experts,
//                              the top-k (lowest index first on ties, as the upstream's stable sort) and
//                              renormalises the chosen probabilities to sum 1;
//   * the chosen experts' projections run as ONE job-list launch each (qmatvec_jobs.cu): a job takes its
//     matrix from the expert bank by a selector it reads on the device (bank + select[0] * stride), so the
//     host never learns the choice and nothing is gathered or copied;
//   * moe_combine_kernel       out[token] = sum over the chosen experts of weight * expert_scale * down output,
//                              in slot order (deterministic).
// Decode-sized token counts only: every (token, slot) pair is a job of its own, an expert chosen by several
// tokens is streamed once per token.
#include "qmm_formats.cuh"
#include <vector>

namespace qmm {

int qmatvec_jobs_launch(const qmm_matvec_job* jobs, int n_jobs, int m, cudaStream_t stream);

constexpr int MOE_MAX_EXPERTS = 256;
constexpr int MOE_MAX_TOPK = 8;
constexpr int MOE_ROUTER_THREADS = 256;

// One CTA per token.  x (hidden) f32; router_w (n_experts, hidden) f32 row-major.
__global__ void __launch_bounds__(MOE_ROUTER_THREADS) moe_router_topk_kernel(const float* __restrict__ x, const float* __restrict__ gain,
                                                                            const float* __restrict__ router_w, int hidden, int n_experts,
                                                                            int top_k, float scale, float eps, int* __restrict__ sel,
                                                                            float* __restrict__ weight, float* __restrict__ probs_out) {
    extern __shared__ float rin[];  // hidden floats: the router's input
    __shared__ float logit[MOE_MAX_EXPERTS];
    __shared__ float red[32];
    const int p = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    const float* xr = x + (size_t)p * hidden;
    float ss = 0.f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        const float v = xr[i];
        rin[i] = v;
        ss += v * v;
    }
    ss = warp_sum(ss);
    if (lane == 0) red[warp] = ss;
    __syncthreads();
    float tot = 0.f;
    for (int w = 0; w < nw; ++w) tot += red[w];
    const float inv = rsqrtf(tot / (float)hidden + eps) * scale;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) rin[i] = rin[i] * inv * (gain ? gain[i] : 1.f);
    __syncthreads();
    for (int e = warp; e < n_experts; e += nw) {  // one warp per expert row, fixed lane order
        const float* wr = router_w + (size_t)e * hidden;
        float acc = 0.f;
        for (int i = lane; i < hidden; i += 32) acc += wr[i] * rin[i];
        acc = warp_sum(acc);
        if (lane == 0) logit[e] = acc;
    }
    __syncthreads();
    if (warp == 0) {
        // softmax over the experts, then k rounds of (largest remaining, lowest index on ties)
        float mx = -INFINITY;
        for (int e = lane; e < n_experts; e += 32) mx = fmaxf(mx, logit[e]);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        float den = 0.f;
        for (int e = lane; e < n_experts; e += 32) {
            const float pe = __expf(logit[e] - mx);
            logit[e] = pe;
            den += pe;
        }
        den = warp_sum(den);
        __syncwarp();
        for (int e = lane; e < n_experts; e += 32) {
            logit[e] = logit[e] / den;
            if (probs_out) probs_out[(size_t)p * n_experts + e] = logit[e];
        }
        __syncwarp();
        float chosen_sum = 0.f;
        int my_sel = -1;      // lane j keeps choice j
        float my_prob = 0.f;
        for (int j = 0; j < top_k; ++j) {
            float bv = -1.f;
            int bi = 0x7fffffff;
            for (int e = lane; e < n_experts; e += 32) {
                const float v = logit[e];
                if (v > bv || (v == bv && e < bi)) bv = v, bi = e;
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
                const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
                if (ov > bv || (ov == bv && oi < bi)) bv = ov, bi = oi;
            }
            if (lane == j) my_sel = bi, my_prob = bv;
            chosen_sum += bv;
            if (lane == 0) logit[bi] = -2.f;  // taken
            __syncwarp();
        }
        if (lane < top_k) {
            sel[(size_t)p * top_k + lane] = my_sel;
            weight[(size_t)p * top_k + lane] = my_prob / chosen_sum;
        }
    }
}

// out(m, hidden) = sum_j weight[p][j] * expert_scale[sel[p][j]] * dv[p][j][:]   (slot order)
__global__ void moe_combine_kernel(const float* __restrict__ dv, const float* __restrict__ weight, const int* __restrict__ sel,
                                   const float* __restrict__ expert_scale, float* __restrict__ out, int top_k, int hidden) {
    const int p = blockIdx.y;
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= hidden) return;
    float acc = 0.f;
    for (int j = 0; j < top_k; ++j) {
        const float w = weight[(size_t)p * top_k + j] * (expert_scale ? expert_scale[sel[(size_t)p * top_k + j]] : 1.f);
        acc += w * dv[((size_t)p * top_k + j) * hidden + i];
    }
    out[(size_t)p * hidden + i] = acc;
}

}  // namespace qmm

using namespace qmm;

extern "C" {

int launch_moe_router_topk(const float* x, const float* gain, const float* router_w, int m, int hidden, int n_experts, int top_k, float scale,
                           float eps, int* sel, float* weight, float* probs, void* stream) {
    if (!x || !router_w || !sel || !weight) return QMM_ERR_NULL;
    if (m <= 0 || hidden <= 0 || n_experts <= 0 || top_k <= 0 || top_k > n_experts) return QMM_ERR_SHAPE;
    if (n_experts > MOE_MAX_EXPERTS || top_k > MOE_MAX_TOPK || (size_t)hidden * 4 > 160 * 1024) return QMM_ERR_UNSUPPORTED;
    const size_t smem = (size_t)hidden * sizeof(float);
    static size_t configured[64] = {};
    int dev = 0;
    QMM_CUDA_TRY(cudaGetDevice(&dev));
    if (smem > 48 * 1024 && (dev < 0 || dev >= 64 || smem > configured[dev])) {
        QMM_CUDA_TRY(cudaFuncSetAttribute(moe_router_topk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        if (dev >= 0 && dev < 64) configured[dev] = smem;
    }
    moe_router_topk_kernel<<<m, MOE_ROUTER_THREADS, smem, as_stream(stream)>>>(x, gain, router_w, hidden, n_experts, top_k, scale, eps, sel,
                                                                                weight, probs);
    QMM_CUDA_TRY(cudaGetLastError());
    return QMM_OK;
}

long qmm_moe_scratch_bytes(int m, int top_k, int hidden, int ffn_expert) {
    if (m <= 0 || top_k <= 0 || hidden <= 0 || ffn_expert <= 0 || ffn_expert % 32 != 0) return QMM_ERR_SHAPE;
    const long pairs = (long)m * top_k;
    long b = pairs * 2 * ffn_expert * 4;                                  // gate|up outputs, f32
    b += (pairs * (ffn_expert / 32) * Q8_1_BYTES + 255) & ~255l;          // activated values, Q8_1
    b += pairs * hidden * 4;                                              // down outputs, f32
    return b + 512;
}

// The expert branch for m tokens whose choices (sel, weight: (m, top_k)) are on the device:
//   for every (token, slot): gu = xq[token] . W_gu[sel]^T ; ea = Q8_1(act(gate) * up) ; dv = ea . W_dn[sel]^T
//   out[token] = sum over slots of weight * expert_scale[sel] * dv
// gate_up_bank: n_experts matrices (2 * ffn_expert, hidden) of type_gu, `gu_stride_bytes` apart;
// down_bank: n_experts matrices (hidden, ffn_expert) of type_dn, `dn_stride_bytes` apart.
int launch_moe_experts(int type_gu, const void* gate_up_bank, long gu_stride_bytes, int type_dn, const void* down_bank, long dn_stride_bytes,
                       const void* xq, const int* sel, const float* weight, const float* expert_scale, float* out, void* scratch, int m,
                       int top_k, int hidden, int ffn_expert, int act, void* stream) {
    if (!gate_up_bank || !down_bank || !xq || !sel || !weight || !out || !scratch) return QMM_ERR_NULL;
    if (m <= 0 || top_k <= 0 || top_k > MOE_MAX_TOPK || hidden <= 0 || ffn_expert <= 0 || ffn_expert % 32 != 0) return QMM_ERR_SHAPE;
    if (gu_stride_bytes % 16 != 0 || dn_stride_bytes % 16 != 0 || reinterpret_cast<uintptr_t>(scratch) % 16 != 0) return QMM_ERR_ALIGN;
    const long xq_row = qmm_row_bytes(QMM_TYPE_Q8_1, hidden);
    const long ea_row = qmm_row_bytes(QMM_TYPE_Q8_1, ffn_expert);
    if (xq_row < 0) return (int)xq_row;
    if (xq_row % 16 != 0 || ea_row % 16 != 0) return QMM_ERR_UNSUPPORTED;  // each token's activations start a bulk copy
    cudaStream_t s = as_stream(stream);
    const long pairs = (long)m * top_k;
    uint8_t* sc = static_cast<uint8_t*>(scratch);
    float* gu = reinterpret_cast<float*>(sc);
    uint8_t* ea = sc + pairs * 2 * ffn_expert * 4;
    float* dv = reinterpret_cast<float*>(ea + ((pairs * ea_row + 255) & ~255l));
    std::vector<qmm_matvec_job> jobs((size_t)pairs);
    for (int p = 0; p < m; ++p)
        for (int j = 0; j < top_k; ++j) {
            qmm_matvec_job& q = jobs[(size_t)p * top_k + j];
            q = qmm_matvec_job{};
            q.type = type_gu, q.n = 2 * ffn_expert, q.k = hidden;
            q.w = gate_up_bank, q.xq = static_cast<const uint8_t*>(xq) + (size_t)p * xq_row;
            q.y = gu + ((size_t)p * top_k + j) * 2 * ffn_expert;
            q.select = sel + (size_t)p * top_k + j, q.select_stride_bytes = gu_stride_bytes;
        }
    if (int st = qmatvec_jobs_launch(jobs.data(), (int)pairs, 1, s)) return st;
    if (int st = launch_glu_act_q8_1(gu, ea, nullptr, (int)pairs, ffn_expert, act, stream)) return st;
    for (int p = 0; p < m; ++p)
        for (int j = 0; j < top_k; ++j) {
            qmm_matvec_job& q = jobs[(size_t)p * top_k + j];
            q = qmm_matvec_job{};
            q.type = type_dn, q.n = hidden, q.k = ffn_expert;
            q.w = down_bank, q.xq = ea + ((size_t)p * top_k + j) * ea_row;
            q.y = dv + ((size_t)p * top_k + j) * hidden;
            q.select = sel + (size_t)p * top_k + j, q.select_stride_bytes = dn_stride_bytes;
        }
    if (int st = qmatvec_jobs_launch(jobs.data(), (int)pairs, 1, s)) return st;
    moe_combine_kernel<<<dim3((hidden + 255) / 256, m), 256, 0, s>>>(dv, weight, sel, expert_scale, out, top_k, hidden);
    QMM_CUDA_TRY(cudaGetLastError());
    return QMM_OK;
}

}  // extern "C"
