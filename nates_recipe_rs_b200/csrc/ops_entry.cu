// Stand-alone entry points for the small per-layer operators of the decode stack (the engine calls the same
// kernels directly).  Each one is the fp32 / Q8_1-producing counterpart of an upstream f64 operator:
//   launch_add_rmsnorm_q8_1   launch_normx_rmsnorm   gpu-core/src/kernels/normx.hip:135-159, gpu-core/src/infer_ops.rs:117-139
//   launch_rope_kv_append     launch_rope_partial    gpu-core/src/kernels/f64_infer.hip:107-132, infer_ops.rs:61-83
//   launch_glu_act_q8_1       launch_glu_gelu        gpu-core/src/kernels/f64_infer.hip:150-166, infer_ops.rs:206-222
//   launch_embed_rows         host-side embedding gather of the upstream example, examples/gemma4.rs:951-958
//   launch_argmax_rows        host-side pick of the next token, examples/gemma4.rs:1021-1046 (greedy here)
//   launch_scale_f32          launch_scale_f64       gpu-core/src/kernels/gemm_f64.hip:57-65, infer_ops.rs:242-248
//   launch_qdense             LayerKind::Dense of the upstream's forward pass: gpu_linear_into + one activation launch,
//                             recipe-infer/src/forward.rs:372-431, with the weight in packed blocks
#include "qmm_formats.cuh"

namespace qmm {

__global__ void scale_f32_kernel(float* __restrict__ x, float scalar, long n) {
    const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) x[i] = __fmul_rn(x[i], scalar);
}

constexpr int ARGMAX_ENTRY_PARTS = 256;

// y = act(y + bias) in place, the epilogue of a quantized dense layer.  The activations are the upstream's
// (recipe-infer/src/forward.rs:388-431; elementwise.hip, gapact.hip): leaky ReLU / PReLU with slope alpha,
// ELU with alpha, SELU with its two constants, tanh-form GELU.
__device__ __forceinline__ float dense_act(float z, int act, float alpha) {
    switch (act) {
    case QMM_DENSE_RELU: return fmaxf(z, 0.f);
    case QMM_DENSE_SIGMOID: return 1.f / (1.f + expf(-z));
    case QMM_DENSE_LEAKY_RELU:
    case QMM_DENSE_PRELU: return z > 0.f ? z : alpha * z;
    case QMM_DENSE_ELU: return z > 0.f ? z : alpha * (expf(z) - 1.f);
    case QMM_DENSE_SELU: return 1.0507009873554804934f * (z > 0.f ? z : 1.6732632423543772848f * (expf(z) - 1.f));
    case QMM_DENSE_TANH: return tanhf(z);
    case QMM_DENSE_SILU: return z / (1.f + expf(-z));
    case QMM_DENSE_GELU: return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
    }
    return z;
}
__global__ void f32_to_bf16_kernel(const float* __restrict__ x, __nv_bfloat16* __restrict__ out, long n) {
    const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = __float2bfloat16_rn(x[i]);
}
constexpr int QDENSE_GEMM_MIN_M = 64;  // rows from which a Q4_K dense layer takes the tensor-core GEMM
__global__ void dense_bias_act_kernel(float* __restrict__ y, const float* __restrict__ bias, long total, int n, int act, float alpha) {
    pdl_wait_prior_grids();
    const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < total) {
        float z = y[i];
        if (bias) z += bias[i % n];
        y[i] = dense_act(z, act, alpha);
    }
}

}  // namespace qmm

using namespace qmm;

extern "C" {

int launch_add_rmsnorm_q8_1(float* x, const float* add, const float* gamma, void* xq, float* out_f32, int rows, int cols, float eps,
                            void* stream) {
    if (!x || !xq) return QMM_ERR_NULL;
    if (rows <= 0 || cols <= 0 || cols % 32 != 0) return QMM_ERR_SHAPE;
    if (cols > NORM_MAX_PER_THREAD * 1024) return QMM_ERR_UNSUPPORTED;
    if (reinterpret_cast<uintptr_t>(xq) % 4 != 0) return QMM_ERR_ALIGN;
    PartPtrs parts = {};
    parts.p[0] = add;
    TpRecv none = {};
    return add_rmsnorm_launch(x, parts, add ? 1 : 0, (long)cols, gamma, static_cast<uint8_t*>(xq), cols, eps, none, out_f32, rows, false,
                              as_stream(stream));
}

int launch_rope_kv_append(float* qkv, void* kcache, void* vcache, int batch, int n_q_heads, int n_kv_heads, int head_dim, int pos,
                          int ctx_cap, float theta, void* stream) {
    if (!qkv || !kcache || !vcache) return QMM_ERR_NULL;
    if (batch <= 0 || n_q_heads <= 0 || n_kv_heads <= 0 || head_dim <= 0 || head_dim % 2 != 0 || pos < 0 || pos >= ctx_cap) return QMM_ERR_SHAPE;
    rope_kv_append_kernel<<<dim3(8, batch), 256, 0, as_stream(stream)>>>(qkv, static_cast<__half*>(kcache), static_cast<__half*>(vcache),
                                                                          n_q_heads, n_kv_heads, head_dim, pos, ctx_cap, theta);
    QMM_CUDA_TRY(cudaGetLastError());
    return QMM_OK;
}

int launch_glu_act_q8_1(const float* gate_up, void* xq, float* out_f32, int rows, int half, int act, void* stream) {
    if (!gate_up || !xq) return QMM_ERR_NULL;
    if (rows <= 0 || half <= 0 || half % 32 != 0) return QMM_ERR_SHAPE;
    if (act != 0 && act != 1) return QMM_ERR_UNSUPPORTED;
    if (reinterpret_cast<uintptr_t>(xq) % 4 != 0) return QMM_ERR_ALIGN;
    act_mul_q8_kernel<<<dim3((half / 32 + 3) / 4, rows), 128, 0, as_stream(stream)>>>(gate_up, static_cast<uint8_t*>(xq), half, act, out_f32);
    QMM_CUDA_TRY(cudaGetLastError());
    return QMM_OK;
}

int launch_embed_rows(int type, const void* table, const int* tokens, float* x, int batch, int hidden, int vocab, void* stream) {
    if (!table || !tokens || !x) return QMM_ERR_NULL;
    const long rb = qmm_row_bytes(type, hidden);
    if (type == QMM_TYPE_Q8_1) return QMM_ERR_TYPE;
    if (rb < 0) return (int)rb;
    if (batch <= 0 || vocab <= 0) return QMM_ERR_SHAPE;
    const dim3 grid((hidden + 255) / 256, batch);
    const uint8_t* t = static_cast<const uint8_t*>(table);
    cudaStream_t s = as_stream(stream);
    if (type == QMM_TYPE_Q6_K) embed_rows_kernel<QMM_TYPE_Q6_K><<<grid, 256, 0, s>>>(t, tokens, x, hidden, (int)rb, vocab, nullptr);
    else if (type == QMM_TYPE_Q4_K) embed_rows_kernel<QMM_TYPE_Q4_K><<<grid, 256, 0, s>>>(t, tokens, x, hidden, (int)rb, vocab, nullptr);
    else embed_rows_kernel<QMM_TYPE_Q8_0><<<grid, 256, 0, s>>>(t, tokens, x, hidden, (int)rb, vocab, nullptr);
    QMM_CUDA_TRY(cudaGetLastError());
    return QMM_OK;
}

long qmm_argmax_scratch_bytes(int batch) {
    if (batch <= 0) return QMM_ERR_SHAPE;
    return (long)batch * ARGMAX_ENTRY_PARTS * (long)sizeof(Candidate);
}

int launch_argmax_rows(const float* logits, void* scratch, int* out_index, float* out_value, int batch, int vocab, void* stream) {
    if (!logits || !scratch || !out_index) return QMM_ERR_NULL;
    if (batch <= 0 || vocab <= 0) return QMM_ERR_SHAPE;
    if (reinterpret_cast<uintptr_t>(scratch) % 8 != 0) return QMM_ERR_ALIGN;
    Candidate* cand = static_cast<Candidate*>(scratch);
    cudaStream_t s = as_stream(stream);
    argmax_partial_kernel<<<dim3(ARGMAX_ENTRY_PARTS, batch), 256, 0, s>>>(logits, cand, vocab);
    argmax_final_kernel<<<batch, 256, 0, s>>>(cand, ARGMAX_ENTRY_PARTS, out_index, 0, out_value);
    QMM_CUDA_TRY(cudaGetLastError());
    return QMM_OK;
}

long qmm_qdense_scratch_bytes(int type, int m, int k) {
    if (m <= 0 || k <= 0) return 0;
    const long q8 = (long)m * (k / 32) * Q8_1_BYTES, bf = (long)m * k * 2;
    return (type == QMM_TYPE_Q4_K && m >= QDENSE_GEMM_MIN_M && k % 256 == 0) ? (bf > q8 ? bf : q8) : q8;
}

int launch_qdense(int type, const void* w, const float* x, const float* bias, float* y, void* xq_scratch, int m, int n, int k, int act,
                  float alpha, void* stream) {
    if (!w || !x || !y || !xq_scratch) return QMM_ERR_NULL;
    if (act < QMM_DENSE_LINEAR || act > QMM_DENSE_GELU) return QMM_ERR_UNSUPPORTED;
    if (m <= 0 || n <= 0 || k <= 0) return QMM_ERR_SHAPE;
    cudaStream_t s = as_stream(stream);
    if (type == QMM_TYPE_Q4_K && m >= QDENSE_GEMM_MIN_M && k % 256 == 0 && reinterpret_cast<uintptr_t>(xq_scratch) % 16 == 0) {
        // many rows: x rounded to bf16, the prefill GEMM with its f32 accumulators as the output
        const long total = (long)m * k;
        f32_to_bf16_kernel<<<(unsigned)((total + 255) / 256), 256, 0, s>>>(x, static_cast<__nv_bfloat16*>(xq_scratch), total);
        QMM_CUDA_TRY(cudaGetLastError());
        if (int st = launch_qgemm_q4_k_bf16_f32acc(w, xq_scratch, y, m, n, k, stream)) return st;
    } else {
        if (int st = launch_quantize_q8_1(x, xq_scratch, m, k, stream)) return st;
        if (int st = launch_qmatvec(type, w, xq_scratch, y, m, n, k, stream)) return st;
    }
    if (bias || act != QMM_DENSE_LINEAR) {
        const long total = (long)m * n;
        dense_bias_act_kernel<<<(unsigned)((total + 255) / 256), 256, 0, s>>>(y, bias, total, n, act, alpha);
        QMM_CUDA_TRY(cudaGetLastError());
    }
    return QMM_OK;
}

int launch_scale_f32(float* x, float scalar, long n, void* stream) {
    if (!x) return QMM_ERR_NULL;
    if (n <= 0) return QMM_ERR_SHAPE;
    scale_f32_kernel<<<(unsigned)((n + 255) / 256), 256, 0, as_stream(stream)>>>(x, scalar, n);
    QMM_CUDA_TRY(cudaGetLastError());
    return QMM_OK;
}

}  // extern "C"
