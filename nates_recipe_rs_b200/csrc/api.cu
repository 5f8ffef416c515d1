// extern "C" surface of libqmm (declared in include/qmm.h) and the few pieces of
// host state shared by the launchers.
#include "qmm_common.cuh"
#ifdef QMM_TUNING
#include "qmm_tuning.h"
#endif

namespace qmm {

static thread_local int t_last_cuda_error = 0;
void set_last_cuda_error(cudaError_t e) { t_last_cuda_error = (int)e; }

int sm_count() {
    static int cached[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cached[dev] == 0) {
        int v = 0;
        if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) v = 148;
        cached[dev] = v;
    }
    return cached[dev];
}

static int g_overlap = 1;
bool overlap_enabled() { return g_overlap != 0; }

int qmatvec_launch(int type, const void* w, const void* xq, float* y, int m, int n, int k, cudaStream_t stream);
int qmatvec_launch_pitched(int type, const void* w, long row_pitch, const void* xq, float* y, long y_stride, int m, int n, int k, int cta_limit,
                           const TpPush* push, cudaStream_t stream);
int qblock_dots_launch(int type, const void* w, const void* xq, int32_t* out, int n, int k, cudaStream_t stream);
int quantize_q8_1_launch(const float* x, void* xq, int m, int k, cudaStream_t stream);
int quantize_weights_launch(int type, const float* w, void* out, long rows, int k, cudaStream_t stream);
int dequantize_f32_launch(int type, const void* w, float* out, long n_elems, cudaStream_t stream);
int dequantize_bf16_launch(int type, const void* w, void* out, long n_elems, cudaStream_t stream);
int qgemm_q4k_launch(const void* w, const void* x, void* y, float* yf, int m, int n, int k, cudaStream_t stream);
int gemm_bt_bf16_launch(const void* a, const void* b, void* y, float* yf, int m, int n, int k, cudaStream_t stream);
int matvec_tune(const char* key, int value);
int jobs_tune(const char* key, int value);
int qmatvec_jobs_launch(const qmm_matvec_job* jobs, int n_jobs, int m, cudaStream_t stream);
struct XBuild {  // qmatvec_jobs.cu
    const float* x_in;
    const float* x_add;
    const float* gamma;
    float* x_out;
    float eps;
    int act;
    int k;
};
int qmatvec_jobs_launch_ex(const qmm_matvec_job* jobs, int n_jobs, int m, const TpPush* push, const long* push_words, int x_mode,
                           const XBuild* xb, cudaStream_t stream);
constexpr int JOBS_X_NORM = 1, JOBS_X_GLU = 2;
void matvec_set_trace(unsigned long long* buf, int stride_words);

}  // namespace qmm

using namespace qmm;

extern "C" {

const char* qmm_status_string(int status) {
    switch (status) {
    case QMM_OK: return "ok";
    case QMM_ERR_NULL: return "null pointer";
    case QMM_ERR_SHAPE: return "bad shape (non-positive size, or k not a whole number of blocks)";
    case QMM_ERR_UNSUPPORTED: return "shape not supported by this kernel";
    case QMM_ERR_ALIGN: return "pointer not aligned as documented";
    case QMM_ERR_TYPE: return "unknown block type";
    case QMM_ERR_CUDA: return "CUDA runtime error (see qmm_last_cuda_error)";
    case QMM_ERR_SCRATCH: return "request exceeds the fixed scratch capacity";
    case QMM_ERR_IO: return "file could not be opened, read or written";
    case QMM_ERR_FORMAT: return "file format error (bad magic, truncated, or a tensor is missing or of another type)";
    }
    return "unknown status";
}

int qmm_last_cuda_error(void) { return t_last_cuda_error; }

int qmm_device_status(int* host_status) {
    if (!host_status) return QMM_ERR_NULL;
    QMM_CUDA_TRY(cudaDeviceSynchronize());
    int v = 0;
    QMM_CUDA_TRY(cudaMemcpyFromSymbol(&v, g_device_status, sizeof(int)));
    if (v != 0) {
        const int zero = 0;
        QMM_CUDA_TRY(cudaMemcpyToSymbol(g_device_status, &zero, sizeof(int)));
    }
    *host_status = v;
    return QMM_OK;
}

long qmm_row_bytes(int type, long k) {
    int be, bb;
    switch (type) {
    case QMM_TYPE_Q8_0: be = 32, bb = Q8_0_BYTES; break;
    case QMM_TYPE_Q8_1: be = 32, bb = Q8_1_BYTES; break;
    case QMM_TYPE_Q4_K: be = 256, bb = Q4_K_BYTES; break;
    case QMM_TYPE_Q6_K: be = 256, bb = Q6_K_BYTES; break;
    default: return QMM_ERR_TYPE;
    }
    if (k <= 0 || k % be != 0) return QMM_ERR_SHAPE;
    return k / be * bb;
}

int qmm_set_overlap(int on) {
    const int prev = g_overlap;
    g_overlap = on ? 1 : 0;
    return prev;
}

int qmm_tune(const char* key, int value) {
    const int st = matvec_tune(key, value);
    return st == QMM_ERR_UNSUPPORTED ? jobs_tune(key, value) : st;
}
#ifdef QMM_TUNING
int qmm_trace(void* buf, int stride_words) { matvec_set_trace(static_cast<unsigned long long*>(buf), stride_words); return QMM_OK; }
#endif

int launch_quantize_q8_1(const float* x, void* xq, int m, int k, void* stream) {
    return quantize_q8_1_launch(x, xq, m, k, as_stream(stream));
}
int launch_quantize_q8_0(const float* w, void* out, long rows, int k, void* stream) {
    return quantize_weights_launch(QMM_TYPE_Q8_0, w, out, rows, k, as_stream(stream));
}
int launch_quantize_q4_k(const float* w, void* out, long rows, int k, void* stream) {
    return quantize_weights_launch(QMM_TYPE_Q4_K, w, out, rows, k, as_stream(stream));
}
int launch_quantize_q6_k(const float* w, void* out, long rows, int k, void* stream) {
    return quantize_weights_launch(QMM_TYPE_Q6_K, w, out, rows, k, as_stream(stream));
}

int launch_dequantize_q8_0_f32(const void* w, float* out, long n, void* s) { return dequantize_f32_launch(QMM_TYPE_Q8_0, w, out, n, as_stream(s)); }
int launch_dequantize_q4_k_f32(const void* w, float* out, long n, void* s) { return dequantize_f32_launch(QMM_TYPE_Q4_K, w, out, n, as_stream(s)); }
int launch_dequantize_q6_k_f32(const void* w, float* out, long n, void* s) { return dequantize_f32_launch(QMM_TYPE_Q6_K, w, out, n, as_stream(s)); }
int launch_dequantize_q8_0_bf16(const void* w, void* out, long n, void* s) { return dequantize_bf16_launch(QMM_TYPE_Q8_0, w, out, n, as_stream(s)); }
int launch_dequantize_q4_k_bf16(const void* w, void* out, long n, void* s) { return dequantize_bf16_launch(QMM_TYPE_Q4_K, w, out, n, as_stream(s)); }
int launch_dequantize_q6_k_bf16(const void* w, void* out, long n, void* s) { return dequantize_bf16_launch(QMM_TYPE_Q6_K, w, out, n, as_stream(s)); }

int launch_qmatvec(int type, const void* w, const void* xq, float* y, int m, int n, int k, void* stream) {
    return qmatvec_launch(type, w, xq, y, m, n, k, as_stream(stream));
}
int launch_qmatvec_pitched(int type, const void* w, long row_pitch_bytes, const void* xq, float* y, int m, int n, int k, void* stream) {
    if (row_pitch_bytes < 0) return QMM_ERR_SHAPE;
    return qmatvec_launch_pitched(type, w, row_pitch_bytes, xq, y, n, m, n, k, 0, nullptr, as_stream(stream));
}
int launch_qmatvec_q8_0(const void* w, const void* xq, float* y, int m, int n, int k, void* s) { return qmatvec_launch(QMM_TYPE_Q8_0, w, xq, y, m, n, k, as_stream(s)); }
int launch_qmatvec_q4_k(const void* w, const void* xq, float* y, int m, int n, int k, void* s) { return qmatvec_launch(QMM_TYPE_Q4_K, w, xq, y, m, n, k, as_stream(s)); }
int launch_qmatvec_q6_k(const void* w, const void* xq, float* y, int m, int n, int k, void* s) { return qmatvec_launch(QMM_TYPE_Q6_K, w, xq, y, m, n, k, as_stream(s)); }

int launch_qmatvec_batch(const qmm_matvec_job* jobs, int n_jobs, int m, void* stream) {
    return qmatvec_jobs_launch(jobs, n_jobs, m, as_stream(stream));
}

int launch_norm_qmatvec_batch(const float* x_in, const float* x_add, const float* gamma, float* x_out, float eps, const qmm_matvec_job* jobs,
                              int n_jobs, int m, void* stream) {
    if (!x_in || !jobs) return QMM_ERR_NULL;
    if (n_jobs <= 0 || m <= 0) return QMM_ERR_SHAPE;
    if (x_out == x_in) return QMM_ERR_ALIGN;  // every CTA reads x_in while one of them writes x_out
    XBuild xb = {};
    xb.x_in = x_in, xb.x_add = x_add, xb.gamma = gamma, xb.x_out = x_out, xb.eps = eps, xb.k = jobs[0].k;
    return qmatvec_jobs_launch_ex(jobs, n_jobs, m, nullptr, nullptr, JOBS_X_NORM, &xb, as_stream(stream));
}
int launch_glu_qmatvec_batch(const float* gate_up, int act, const qmm_matvec_job* jobs, int n_jobs, int m, void* stream) {
    if (!gate_up || !jobs) return QMM_ERR_NULL;
    if (n_jobs <= 0 || m <= 0) return QMM_ERR_SHAPE;
    if (act != 0 && act != 1) return QMM_ERR_UNSUPPORTED;
    XBuild xb = {};
    xb.x_in = gate_up, xb.act = act, xb.k = jobs[0].k;
    return qmatvec_jobs_launch_ex(jobs, n_jobs, m, nullptr, nullptr, JOBS_X_GLU, &xb, as_stream(stream));
}

int launch_qgemm_q4_k_bf16(const void* w, const void* x, void* y, int m, int n, int k, void* stream) {
    if (!y) return QMM_ERR_NULL;
    return qgemm_q4k_launch(w, x, y, nullptr, m, n, k, as_stream(stream));
}
int launch_qgemm_q4_k_bf16_f32acc(const void* w, const void* x, float* yf, int m, int n, int k, void* stream) {
    if (!yf) return QMM_ERR_NULL;
    return qgemm_q4k_launch(w, x, nullptr, yf, m, n, k, as_stream(stream));
}

int launch_gemm_bt_bf16(const void* a, const void* b, void* out, int m, int n, int k, void* stream) {
    if (!out) return QMM_ERR_NULL;
    return gemm_bt_bf16_launch(a, b, out, nullptr, m, n, k, as_stream(stream));
}
int launch_gemm_bt_bf16_f32acc(const void* a, const void* b, float* out, int m, int n, int k, void* stream) {
    if (!out) return QMM_ERR_NULL;
    return gemm_bt_bf16_launch(a, b, nullptr, out, m, n, k, as_stream(stream));
}

int launch_qblock_dots(int type, const void* w, const void* xq, int32_t* out, int n, int k, void* stream) {
    return qblock_dots_launch(type, w, xq, out, n, k, as_stream(stream));
}

}  // extern "C"
