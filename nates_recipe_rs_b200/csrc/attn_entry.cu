// Stand-alone entry points for the decode attention (the engine calls the same kernels directly).
#include "qmm_formats.cuh"
#include <mutex>

namespace qmm {

static int attn_check(const float* qkv, const void* kc, const void* vc, const void* out_f32, const void* out_q8, int batch, int nqh, int nkv,
                      int hd, int len, int ctx_cap, int& splits, size_t& smem) {
    if (!qkv || !kc || !vc || (!out_f32 && !out_q8)) return QMM_ERR_NULL;
    if (batch <= 0 || nqh <= 0 || nkv <= 0 || hd <= 0 || len <= 0 || ctx_cap < len) return QMM_ERR_SHAPE;
    if (nqh % nkv || hd % 32 || hd > 256 || nqh / nkv > ATTN_MAX_GROUP) return QMM_ERR_UNSUPPORTED;
    if (reinterpret_cast<uintptr_t>(kc) % 16 || reinterpret_cast<uintptr_t>(vc) % 16 || reinterpret_cast<uintptr_t>(out_q8) % 4)
        return QMM_ERR_ALIGN;
    splits = (len + ATTN_CHUNK - 1) / ATTN_CHUNK;
    if (splits > ATTN_MAX_SPLITS) return QMM_ERR_UNSUPPORTED;
    const int group = nqh / nkv;
    smem = (size_t)ATTN_CHUNK * (2 * hd + 8) * sizeof(__half) + (size_t)group * (hd + ATTN_CHUNK + 2) * sizeof(float);
    return QMM_OK;
}

static int attn_run(const float* qkv, const void* kc, const void* vc, float* scratch, float* out_f32, void* out_q8, int batch, int nqh, int nkv,
                    int hd, int len, int ctx_cap, int splits, size_t smem, cudaStream_t s) {
    if (int st = attn_opt_in_smem(false, smem)) return st;
    if (attn_use_tc(batch, hd)) {
        // several sequences: scores and outputs on the f16 tensor cores (q and the probabilities rounded to f16)
        const size_t smem_tc = attn_tc_smem_bytes(hd);
        if (int st = attn_opt_in_smem(true, smem_tc)) return st;
        attn_decode_split_tc_kernel<<<dim3(nkv, batch, splits), ATTN_THREADS, smem_tc, s>>>(
            qkv, static_cast<const __half*>(kc), static_cast<const __half*>(vc), scratch, nqh, nkv, hd, len, ctx_cap, splits);
    } else {
        attn_decode_split_kernel<<<dim3(nkv, batch, splits), ATTN_THREADS, smem, s>>>(qkv, static_cast<const __half*>(kc),
                                                                                       static_cast<const __half*>(vc), scratch, nqh, nkv, hd,
                                                                                       len, ctx_cap, splits);
    }
    QMM_CUDA_TRY(cudaGetLastError());
    // the merge always produces Q8_1 blocks; a caller that only wants f32 gets them in a throw-away tail of the scratch
    uint8_t* q8 = static_cast<uint8_t*>(out_q8);
    if (!q8) q8 = reinterpret_cast<uint8_t*>(scratch + (size_t)batch * nqh * splits * (hd + 2));
    attn_combine_q8_kernel<<<dim3(nqh, batch), hd < 128 ? hd : 128, 0, s>>>(scratch, q8, out_f32, nqh, hd, splits);
    QMM_CUDA_TRY(cudaGetLastError());
    return QMM_OK;
}

static size_t attn_scratch_floats(int batch, int nqh, int hd, int splits) {
    // split results + room for a row of Q8_1 blocks per sequence (used when the caller passes no out_q8)
    return (size_t)batch * nqh * splits * (hd + 2) + ((size_t)batch * (nqh * hd / 32) * Q8_1_BYTES + 3) / 4;
}

// ---------------------------------------------------------------------------------------------
// Scratch that belongs to the library instead of the caller.  Some hosts of this code may not
// allocate device memory at the moment they need attention: a caller inside a frozen steady
// state (the upstream's AllocGuard panics on any allocation once a loop is frozen), a plugin
// that was handed fixed buffers by its host application, code running between the capture and
// the replay of a work graph.  For them one entry point works out of a fixed array that every
// GPU loading this library carries until the process exits.
constexpr size_t ATTN_STATIC_FLOATS = 1u << 20;  // 4 MiB per GPU
static __device__ __align__(256) float g_attn_static_scratch[ATTN_STATIC_FLOATS];

// `g_attn_static_scratch` is only a stand-in on the host side: it is not a device address and must
// never be handed to a kernel.  The device address is asked for once per device, with that device
// current, and remembered.
static int attn_static_scratch_ptr(float** out) {
    static float* cached[64] = {};
    static std::mutex guard;  // first calls from several host threads
    int dev = 0;
    QMM_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return QMM_ERR_UNSUPPORTED;
    std::lock_guard<std::mutex> lock(guard);
    if (!cached[dev]) {
        float* p = nullptr;
        QMM_CUDA_TRY(cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_attn_static_scratch));
        if (!p) return cuda_fail(cudaErrorInvalidSymbol);
        cached[dev] = p;
    }
    *out = cached[dev];
    return QMM_OK;
}

}  // namespace qmm

using namespace qmm;

extern "C" {

long qmm_attn_decode_scratch_bytes(int batch, int n_q_heads, int head_dim, int len) {
    if (batch <= 0 || n_q_heads <= 0 || head_dim <= 0 || len <= 0) return QMM_ERR_SHAPE;
    return (long)(attn_scratch_floats(batch, n_q_heads, head_dim, (len + ATTN_CHUNK - 1) / ATTN_CHUNK) * sizeof(float));
}

int launch_attn_decode(const float* qkv, const void* kcache, const void* vcache, float* scratch, float* out_f32, void* out_q8, int batch,
                       int n_q_heads, int n_kv_heads, int head_dim, int len, int ctx_cap, void* stream) {
    int splits = 0;
    size_t smem = 0;
    if (!scratch) return QMM_ERR_NULL;
    if (int st = attn_check(qkv, kcache, vcache, out_f32, out_q8, batch, n_q_heads, n_kv_heads, head_dim, len, ctx_cap, splits, smem)) return st;
    return attn_run(qkv, kcache, vcache, scratch, out_f32, out_q8, batch, n_q_heads, n_kv_heads, head_dim, len, ctx_cap, splits, smem,
                    as_stream(stream));
}

int launch_attn_decode_static(const float* qkv, const void* kcache, const void* vcache, float* out_f32, void* out_q8, int batch, int n_q_heads,
                              int n_kv_heads, int head_dim, int len, int ctx_cap, void* stream) {
    int splits = 0;
    size_t smem = 0;
    if (int st = attn_check(qkv, kcache, vcache, out_f32, out_q8, batch, n_q_heads, n_kv_heads, head_dim, len, ctx_cap, splits, smem)) return st;
    if (attn_scratch_floats(batch, n_q_heads, head_dim, splits) > ATTN_STATIC_FLOATS) return QMM_ERR_SCRATCH;
    float* scratch = nullptr;
    if (int st = attn_static_scratch_ptr(&scratch)) return st;
    return attn_run(qkv, kcache, vcache, scratch, out_f32, out_q8, batch, n_q_heads, n_kv_heads, head_dim, len, ctx_cap, splits, smem,
                    as_stream(stream));
}

}  // extern "C"
