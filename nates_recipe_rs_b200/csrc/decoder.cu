// Decode engine: the caller-side glue of the quantized path, in the role examples/gemma4.rs plays
// upstream (Arena::new: every activation buffer once, :231-271; layer(): the projection call sites,
// :638-742; lm_head + sampling, :758-783, 1021-1057), for a Llama/Gemma-style decoder with
// random-init GGUF-block weights.  One token per sequence per step; nothing is allocated after
// qmm_decoder_create.  Tensor parallel: Q/K/V/gate/up split by output rows, O/down by input
// columns; the partial outputs of a row-parallel projection are summed inside the next
// residual-add + RMSNorm + Q8_1 kernel, which reads the peers' partial buffers directly.
#include "qmm_formats.cuh"
#include "../../include/qmm_decoder.h"
#include <algorithm>
#include <string>
#include <vector>
#include <cstring>

namespace qmm {

int qmatvec_launch_strided(int type, const void* w, const void* xq, float* y, long y_stride, int m, int n, int k, cudaStream_t stream);
int qmatvec_launch_limited(int type, const void* w, const void* xq, float* y, long y_stride, int m, int n, int k, int cta_limit,
                           cudaStream_t stream);
int quantize_weights_launch(int type, const float* w, void* out, long rows, int k, cudaStream_t stream);
int qmatvec_launch_push(int type, const void* w, const void* xq, float* y, long y_stride, int m, int n, int k, int cta_limit,
                        const TpPush* push, cudaStream_t stream);
int gemm_bt_bf16_launch(const void* a, const void* b, void* y, float* yf, int m, int n, int k, cudaStream_t stream);
int dequantize_bf16_launch(int type, const void* w, void* out, long n_elems, cudaStream_t stream);
int attn_prefill_launch(const float* q, const void* k, const void* v, float* out, int t, int n_q_heads, int n_kv_heads, int head_dim, int prefix,
                        float kq_scale, long q_stride, long k_stride, long v_stride, long o_stride, cudaStream_t s, __nv_bfloat16* out_bf16, bool kv_f16, int t_kv, int q_pos0);
int qgemm_q4k_launch(const void* w, const void* x, void* y, float* yf, int m, int n, int k, cudaStream_t stream);
int qmatvec_launch_pitched(int type, const void* w, long row_pitch, const void* xq, float* y, long y_stride, int m, int n, int k, int cta_limit,
                           const TpPush* push, cudaStream_t stream);
int decoder_fusion();

constexpr int ARGMAX_PARTS = 256;

struct LayerWeights {
    float *attn_norm, *ffn_norm;
    uint8_t *wqk, *wv, *wo, *wgu, *wdown;
};
// Row pitch of a row-parallel shard: a tensor-parallel rank holds columns [r*K/tp, (r+1)*K/tp) of O and down as
// a matrix of its own; Q6_K rows of such a shard (210 bytes per 256 columns) need not be a multiple of 16 bytes
// long, which the tensor-core matvec's tensor copies require of every row start, so the shard's rows are padded
// to the next multiple of 48 bytes (a whole number of that kernel's 48-byte groups).  0 = rows back to back.
static long shard_pitch(int type, long k, int tp_size) {
    const long rb = type == QMM_TYPE_Q8_0 ? k / 32 * Q8_0_BYTES : (type == QMM_TYPE_Q4_K ? k / 256 * Q4_K_BYTES : k / 256 * Q6_K_BYTES);
    if (tp_size <= 1 || type != QMM_TYPE_Q6_K || rb % 48 == 0) return 0;
    return (rb + 47) / 48 * 48;
}

struct Decoder {
    qmm_decoder_config c;
    int dev;
    int nq, nkv;          // local heads
    int ffn_l, vocab_l;   // local ffn width and vocabulary slice
    int qk_rows, v_rows, qkv_cols;
    std::vector<LayerWeights> layers;
    float* final_norm = nullptr;
    uint8_t *head = nullptr, *embed = nullptr;  // embed == head when tp_size == 1
    __half *kcache = nullptr, *vcache = nullptr;
    // activations (allocated once)
    float *x = nullptr, *x_alt = nullptr, *x_home = nullptr, *qkv = nullptr, *gu = nullptr, *logits = nullptr, *attn_scratch = nullptr, *best_val = nullptr;
    uint8_t *xq_h = nullptr, *xq_attn = nullptr, *xq_ffn = nullptr;
    // projection outputs that the next residual + norm kernel adds: [0] after O, [1] after down.  With tensor
    // parallelism the matvec kernels store them into every rank's exchange area (comm) instead.
    float* part[2] = {nullptr, nullptr};
    TpComm* comm = nullptr;                    // tensor parallel only
    Candidate* argmax_cand = nullptr;          // argmax stage-one candidates: max_batch x ARGMAX_PARTS
    long o_pitch = 0, down_pitch = 0;          // row pitch of the O and down shards (0: rows back to back)
    int attn_splits = 1, attn_chunk = 0;
    std::vector<void*> allocs;
    // second stream for the V projection when its type differs from Q|K's (it then runs beside the Q|K
    // projection on its own share of the SMs instead of after it)
    cudaStream_t side = nullptr;
    cudaEvent_t fork = nullptr, join = nullptr;
    int sms = 0;
    long weight_bytes_per_token = 0;
    // buffers of the prompt path (prefill), allocated on first use for the longest prompt seen so far
    struct Prefill {
        int cap = 0;
        float *x = nullptr, *xn = nullptr, *qk = nullptr, *v = nullptr, *att = nullptr, *part = nullptr, *gu = nullptr, *act = nullptr;
        uint8_t *xq = nullptr, *q8 = nullptr;
        __nv_bfloat16* xb = nullptr;  // the bf16 form of a projection's input, written by the kernel that produces it
        __nv_bfloat16* wb = nullptr;  // a weight matrix decoded to bf16 (types without a fused GEMM)
        size_t wb_elems = 0;
    } pf;
};

static int type_row_bytes(int type, long k) {
    switch (type) {
    case QMM_TYPE_Q8_0: return (int)(k / 32 * Q8_0_BYTES);
    case QMM_TYPE_Q4_K: return (int)(k / 256 * Q4_K_BYTES);
    case QMM_TYPE_Q6_K: return (int)(k / 256 * Q6_K_BYTES);
    }
    return -1;
}

// rows x k slice of a (., k_full) matrix: element (r, c) = sigma * z(seed, (row0 + r) * k_full + col0 + c)
__global__ void fill_normal_2d_kernel(float* out, long rows, int k, uint64_t seed, float sigma, long row0, int col0, int k_full) {
    const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= rows * k) return;
    const long r = i / k;
    const int c = (int)(i - r * k);
    const uint64_t h1 = mix64(seed * 0xD1342543DE82EF95ull + (uint64_t)((row0 + r) * (long)k_full + col0 + c));
    const uint64_t h2 = mix64(h1);
    int s = 0;
#pragma unroll
    for (int q = 0; q < 4; ++q) s += (int)((h1 >> (16 * q)) & 0xFFFFu) + (int)((h2 >> (16 * q)) & 0xFFFFu);
    out[i] = __fmul_rn(__fmul_rn((float)(s - 262140), __fdiv_rn(1.0f, 53510.0f)), sigma);
}
__global__ void add_scalar_kernel(float* x, long n, float v) {
    const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) x[i] += v;
}
__global__ void f32_to_f16_kernel(const float* in, __half* out, long n) {
    const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = __float2half_rn(in[i]);
}

static inline int cuda_status(cudaError_t e) { return e == cudaSuccess ? QMM_OK : cuda_fail(e); }

template <typename T>
static int dev_alloc(Decoder* d, T** p, size_t bytes) {
    void* q = nullptr;
    QMM_CUDA_TRY(cudaMalloc(&q, bytes ? bytes : 16));
    d->allocs.push_back(q);
    *p = static_cast<T*>(q);
    return QMM_OK;
}

// Tensor ids for seeding and for qmm_decoder_get_tensor.
static uint64_t tensor_seed(const Decoder* d, int layer, int which) {
    return d->c.seed * 1000003ull + (uint64_t)(layer + 1) * 64ull + (uint64_t)which;
}

// Fills a packed (rows, k) matrix with quantized N(0, sigma) values.  Element (r, col) of the FULL
// (unsharded) matrix is fill_normal(seed, r * k_full + col); a shard takes rows [row0, row0+rows) and
// columns [col0, col0+k) of it, so every tensor-parallel layout holds the same model.
static int init_matrix(Decoder* d, uint8_t* dst, int type, long rows, int k, long row0, int col0, int k_full, uint64_t seed, float* tmp,
                       long tmp_elems, cudaStream_t s) {
    const long rows_per = tmp_elems / k;
    const int rb = type_row_bytes(type, k);
    for (long r = 0; r < rows; r += rows_per) {
        const long nr = rows - r < rows_per ? rows - r : rows_per;
        const long n = nr * k;
        fill_normal_2d_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(tmp, nr, k, seed, 0.02f, row0 + r, col0, k_full);
        QMM_CUDA_TRY(cudaGetLastError());
        if (int st = quantize_weights_launch(type, tmp, dst + (size_t)r * rb, nr, k, s)) return st;
    }
    return QMM_OK;
}

static int init_gamma(Decoder* d, float* g, int n, uint64_t seed, cudaStream_t s) {
    fill_normal_kernel<<<(n + 255) / 256, 256, 0, s>>>(g, n, seed, 0.1f, 0);
    add_scalar_kernel<<<(n + 255) / 256, 256, 0, s>>>(g, n, 1.0f);
    QMM_CUDA_TRY(cudaGetLastError());
    return QMM_OK;
}

// Where a decoder's weights come from: a seeded closed-form model quantized on the device, or a GGUF file.
// matrix(): the packed (rows, k) shard made of rows [row0, row0 + rows) and columns [col0, col0 + k) of the full
// (., k_full) tensor `which` of `layer`; vector(): an f32 norm gain of n values.
struct WeightSource {
    virtual ~WeightSource() {}
    virtual int matrix(Decoder* d, uint8_t* dst, int type, int layer, int which, long rows, int k, long row0, int col0, int k_full,
                       cudaStream_t s) = 0;
    virtual int vector(Decoder* d, float* dst, int layer, int which, int n, cudaStream_t s) = 0;
};

struct SeededSource : WeightSource {
    float* tmp = nullptr;  // f32 staging on the device, owned by the decoder's allocation list until create() frees it
    long tmp_elems = 0;
    int matrix(Decoder* d, uint8_t* dst, int type, int layer, int which, long rows, int k, long row0, int col0, int k_full,
               cudaStream_t s) override {
        // the head and the embedding of a tied model are the same tensor
        const int seed_which = which == QMM_T_EMBED ? QMM_T_HEAD : which;
        return init_matrix(d, dst, type, rows, k, row0, col0, k_full, tensor_seed(d, layer, seed_which), tmp, tmp_elems, s);
    }
    int vector(Decoder* d, float* dst, int layer, int which, int n, cudaStream_t s) override {
        return init_gamma(d, dst, n, tensor_seed(d, layer, which), s);
    }
};

int gguf_upload_rows(GgufFile* f, long index, uint64_t row0, uint64_t rows, uint64_t col_off, uint64_t width, void* device_dst,
                     cudaStream_t stream);

// GGUF tensor names of a Llama/Gemma-style decoder (the naming convention of the format's reference tools)
static std::string gguf_tensor_name(int layer, int which) {
    const char* base = nullptr;
    switch (which) {
    case QMM_T_ATTN_NORM: base = "attn_norm"; break;
    case QMM_T_WQ: base = "attn_q"; break;
    case QMM_T_WK: base = "attn_k"; break;
    case QMM_T_WV: base = "attn_v"; break;
    case QMM_T_WO: base = "attn_output"; break;
    case QMM_T_FFN_NORM: base = "ffn_norm"; break;
    case QMM_T_WGATE: base = "ffn_gate"; break;
    case QMM_T_WUP: base = "ffn_up"; break;
    case QMM_T_WDOWN: base = "ffn_down"; break;
    case QMM_T_FINAL_NORM: return "output_norm.weight";
    case QMM_T_HEAD: return "output.weight";
    case QMM_T_EMBED: return "token_embd.weight";
    }
    return "blk." + std::to_string(layer) + "." + (base ? base : "?") + ".weight";
}

struct GgufSource : WeightSource {
    GgufFile* f = nullptr;
    long find(int layer, int which) const {
        auto it = f->by_name.find(gguf_tensor_name(layer, which));
        if (it == f->by_name.end() && which == QMM_T_HEAD) it = f->by_name.find(gguf_tensor_name(layer, QMM_T_EMBED));  // tied
        return it == f->by_name.end() ? -1 : it->second;
    }
    int matrix(Decoder*, uint8_t* dst, int type, int layer, int which, long rows, int k, long row0, int col0, int k_full,
               cudaStream_t s) override {
        const long idx = find(layer, which);
        if (idx < 0) return QMM_ERR_FORMAT;
        const GgufTensor& t = f->tensors[idx];
        if ((int)t.type != type || t.n_dims != 2 || (long)t.dims[0] != k_full || (long)t.dims[1] < row0 + rows) return QMM_ERR_FORMAT;
        const int be = type == QMM_TYPE_Q8_0 ? 32 : 256;
        if (col0 % be != 0 || k % be != 0) return QMM_ERR_SHAPE;
        const uint64_t bb = (uint64_t)type_row_bytes(type, be);
        return gguf_upload_rows(f, idx, (uint64_t)row0, (uint64_t)rows, (uint64_t)(col0 / be) * bb, (uint64_t)(k / be) * bb, dst, s);
    }
    int vector(Decoder*, float* dst, int layer, int which, int n, cudaStream_t s) override {
        auto it = f->by_name.find(gguf_tensor_name(layer, which));
        if (it == f->by_name.end()) return QMM_ERR_FORMAT;
        const GgufTensor& t = f->tensors[it->second];
        if (t.type != 0 || (long)t.dims[0] != n || t.bytes != (uint64_t)n * 4) return QMM_ERR_FORMAT;
        return gguf_upload_rows(f, it->second, 0, 1, 0, (uint64_t)n * 4, dst, s);
    }
};

static void prefill_free(Decoder* d);
static void destroy(Decoder* d) {
    if (!d) return;
    prefill_free(d);
    tp_comm_destroy(d->comm);
    for (void* p : d->allocs) cudaFree(p);
    if (d->fork) cudaEventDestroy(d->fork);
    if (d->join) cudaEventDestroy(d->join);
    if (d->side) cudaStreamDestroy(d->side);
    delete d;
}

// A row-parallel shard (hidden rows, k columns out of k_full): rows back to back, or `pitch` bytes apart
// (filled densely into a staging allocation first, then spread; the padding is zeroed).
static int fill_row_parallel(Decoder* d, WeightSource* src, uint8_t** dst, int type, int layer, int which, int k, int col0, int k_full, long pitch,
                             cudaStream_t s) {
    const int H = d->c.hidden;
    const size_t rb = (size_t)type_row_bytes(type, k);
    if (!pitch) {
        if (int st = dev_alloc(d, dst, (size_t)H * rb)) return st;
        return src->matrix(d, *dst, type, layer, which, H, k, 0, col0, k_full, s);
    }
    if (int st = dev_alloc(d, dst, (size_t)H * pitch)) return st;
    void* dense = nullptr;
    QMM_CUDA_TRY(cudaMalloc(&dense, (size_t)H * rb));
    int st = src->matrix(d, static_cast<uint8_t*>(dense), type, layer, which, H, k, 0, col0, k_full, s);
    cudaError_t e = cudaSuccess;
    if (!st) e = cudaMemsetAsync(*dst, 0, (size_t)H * pitch, s);
    if (!st && e == cudaSuccess) e = cudaMemcpy2DAsync(*dst, (size_t)pitch, dense, rb, rb, (size_t)H, cudaMemcpyDeviceToDevice, s);
    if (!st && e == cudaSuccess) e = cudaStreamSynchronize(s);
    cudaFree(dense);
    if (!st && e != cudaSuccess) st = cuda_fail(e);
    return st;
}

static int create(const qmm_decoder_config* cfg, WeightSource* src, Decoder** out) {
    const qmm_decoder_config& c = *cfg;
    if (c.n_layers <= 0 || c.hidden <= 0 || c.head_dim <= 0 || c.n_q_heads <= 0 || c.n_kv_heads <= 0 || c.ffn <= 0 || c.vocab <= 0 ||
        c.ctx_len <= 0 || c.max_batch <= 0 || c.tp_size <= 0 || c.tp_rank < 0 || c.tp_rank >= c.tp_size)
        return QMM_ERR_SHAPE;
    if (c.hidden % 256 || c.head_dim % 32 || c.head_dim > 256 || (c.n_q_heads * c.head_dim) % (256 * c.tp_size) || c.ffn % (256 * c.tp_size) ||
        c.n_q_heads % c.n_kv_heads || c.n_kv_heads % c.tp_size || c.vocab % c.tp_size || c.hidden > NORM_MAX_PER_THREAD * 1024 ||
        c.n_q_heads / c.n_kv_heads > ATTN_MAX_GROUP || c.tp_size > QMM_DECODER_MAX_TP)
        return QMM_ERR_UNSUPPORTED;
    Decoder* d = new Decoder();
    d->c = c;
    cudaGetDevice(&d->dev);
    d->nq = c.n_q_heads / c.tp_size;
    d->nkv = c.n_kv_heads / c.tp_size;
    d->ffn_l = c.ffn / c.tp_size;
    d->vocab_l = c.vocab / c.tp_size;
    d->qk_rows = (d->nq + d->nkv) * c.head_dim;
    d->v_rows = d->nkv * c.head_dim;
    d->qkv_cols = (d->nq + 2 * d->nkv) * c.head_dim;
    const int H = c.hidden, B = c.max_batch, hd = c.head_dim;
    const int ao = d->nq * hd;  // local attention output width = K of the O projection shard
    cudaStream_t s = nullptr;
    int st = QMM_OK;
#define TRY(e)                \
    do {                      \
        if ((st = (e)) != 0) { \
            destroy(d);       \
            return st;        \
        }                     \
    } while (0)
    d->sms = sm_count();
    if (cudaStreamCreateWithFlags(&d->side, cudaStreamNonBlocking) != cudaSuccess ||
        cudaEventCreateWithFlags(&d->fork, cudaEventDisableTiming) != cudaSuccess ||
        cudaEventCreateWithFlags(&d->join, cudaEventDisableTiming) != cudaSuccess) {
        destroy(d);
        return cuda_fail(cudaGetLastError());
    }
    float* tmp = nullptr;
    if (SeededSource* seeded = dynamic_cast<SeededSource*>(src)) {
        seeded->tmp_elems = 32l << 20;  // 128 MB of f32 staging for initialisation
        TRY(dev_alloc(d, &tmp, seeded->tmp_elems * sizeof(float)));
        seeded->tmp = tmp;
    }
    const int r = c.tp_rank;
    d->o_pitch = shard_pitch(c.type_attn_o, ao, c.tp_size);
    d->down_pitch = shard_pitch(c.type_ffn_down, d->ffn_l, c.tp_size);
    d->layers.resize(c.n_layers);
    long per_token = 0;
    for (int l = 0; l < c.n_layers; ++l) {
        LayerWeights& L = d->layers[l];
        TRY(dev_alloc(d, &L.attn_norm, H * sizeof(float)));
        TRY(dev_alloc(d, &L.ffn_norm, H * sizeof(float)));
        TRY(src->vector(d, L.attn_norm, l, QMM_T_ATTN_NORM, H, s));
        TRY(src->vector(d, L.ffn_norm, l, QMM_T_FFN_NORM, H, s));
        // [q heads | k heads] of this rank: rows of the full Wq then rows of the full Wk
        // (with V right behind them when it has the same type: one projection launch instead of two)
        const size_t qk_b = (size_t)d->qk_rows * type_row_bytes(c.type_attn_qk, H);
        const size_t v_b = (size_t)d->v_rows * type_row_bytes(c.type_attn_v, H);
        const bool qkv_fused = c.type_attn_v == c.type_attn_qk;
        TRY(dev_alloc(d, &L.wqk, qk_b + (qkv_fused ? v_b : 0)));
        TRY(src->matrix(d, L.wqk, c.type_attn_qk, l, QMM_T_WQ, (long)d->nq * hd, H, (long)r * d->nq * hd, 0, H, s));
        TRY(src->matrix(d, L.wqk + (size_t)d->nq * hd * type_row_bytes(c.type_attn_qk, H), c.type_attn_qk, l, QMM_T_WK, (long)d->nkv * hd, H,
                        (long)r * d->nkv * hd, 0, H, s));
        if (qkv_fused) {
            L.wv = L.wqk + qk_b;
        } else {
            TRY(dev_alloc(d, &L.wv, v_b));
        }
        TRY(src->matrix(d, L.wv, c.type_attn_v, l, QMM_T_WV, d->v_rows, H, (long)r * d->v_rows, 0, H, s));
        const size_t o_b = (size_t)H * type_row_bytes(c.type_attn_o, ao);
        TRY(fill_row_parallel(d, src, &L.wo, c.type_attn_o, l, QMM_T_WO, ao, r * ao, c.n_q_heads * hd, d->o_pitch, s));
        const size_t gu_b = (size_t)2 * d->ffn_l * type_row_bytes(c.type_ffn_gate_up, H);
        TRY(dev_alloc(d, &L.wgu, gu_b));
        TRY(src->matrix(d, L.wgu, c.type_ffn_gate_up, l, QMM_T_WGATE, d->ffn_l, H, (long)r * d->ffn_l, 0, H, s));
        TRY(src->matrix(d, L.wgu + (size_t)d->ffn_l * type_row_bytes(c.type_ffn_gate_up, H), c.type_ffn_gate_up, l, QMM_T_WUP, d->ffn_l, H,
                        (long)r * d->ffn_l, 0, H, s));
        const size_t dn_b = (size_t)H * type_row_bytes(c.type_ffn_down, d->ffn_l);
        TRY(fill_row_parallel(d, src, &L.wdown, c.type_ffn_down, l, QMM_T_WDOWN, d->ffn_l, r * d->ffn_l, c.ffn, d->down_pitch, s));
        per_token += (long)(qk_b + v_b + o_b + gu_b + dn_b);
    }
    TRY(dev_alloc(d, &d->final_norm, H * sizeof(float)));
    TRY(src->vector(d, d->final_norm, -1, QMM_T_FINAL_NORM, H, s));
    const size_t head_b = (size_t)d->vocab_l * type_row_bytes(c.type_head, H);
    TRY(dev_alloc(d, &d->head, head_b));
    TRY(src->matrix(d, d->head, c.type_head, -1, QMM_T_HEAD, d->vocab_l, H, (long)r * d->vocab_l, 0, H, s));
    per_token += (long)head_b;
    GgufSource* from_file = dynamic_cast<GgufSource*>(src);
    const bool tied = !from_file || from_file->f->by_name.find("output.weight") == from_file->f->by_name.end();
    if (c.tp_size == 1 && tied) {
        d->embed = d->head;  // tied embedding
    } else {                 // every rank needs every row of the embedding
        TRY(dev_alloc(d, &d->embed, (size_t)c.vocab * type_row_bytes(c.type_head, H)));
        TRY(src->matrix(d, d->embed, c.type_head, -1, QMM_T_EMBED, c.vocab, H, 0, 0, H, s));
    }
    d->weight_bytes_per_token = per_token;

    const size_t cache_elems = (size_t)c.n_layers * B * c.ctx_len * d->nkv * hd;
    TRY(dev_alloc(d, &d->kcache, cache_elems * sizeof(__half)));
    TRY(dev_alloc(d, &d->vcache, cache_elems * sizeof(__half)));
    TRY(cuda_status(cudaMemsetAsync(d->kcache, 0, cache_elems * sizeof(__half), s)));
    TRY(cuda_status(cudaMemsetAsync(d->vcache, 0, cache_elems * sizeof(__half), s)));

    TRY(dev_alloc(d, &d->x, (size_t)B * H * sizeof(float)));
    TRY(dev_alloc(d, &d->x_alt, (size_t)B * H * sizeof(float)));
    d->x_home = d->x;
    TRY(dev_alloc(d, &d->qkv, (size_t)B * d->qkv_cols * sizeof(float)));
    TRY(dev_alloc(d, &d->gu, (size_t)B * 2 * d->ffn_l * sizeof(float)));
    TRY(dev_alloc(d, &d->logits, (size_t)B * d->vocab_l * sizeof(float)));
    TRY(dev_alloc(d, &d->best_val, (size_t)B * sizeof(float)));
    TRY(dev_alloc(d, &d->xq_h, (size_t)B * (H / 32) * Q8_1_BYTES));
    TRY(dev_alloc(d, &d->xq_attn, (size_t)B * (ao / 32) * Q8_1_BYTES));
    TRY(dev_alloc(d, &d->xq_ffn, (size_t)B * (d->ffn_l / 32) * Q8_1_BYTES));
    // context splits of ATTN_CHUNK positions
    d->attn_chunk = ATTN_CHUNK;
    d->attn_splits = (c.ctx_len + ATTN_CHUNK - 1) / ATTN_CHUNK;
    if (d->attn_splits > ATTN_MAX_SPLITS) {
        destroy(d);
        return QMM_ERR_UNSUPPORTED;
    }
    TRY(dev_alloc(d, &d->attn_scratch, (size_t)B * d->nq * d->attn_splits * (hd + 2) * sizeof(float)));

    TRY(dev_alloc(d, &d->part[0], (size_t)B * H * sizeof(float)));
    TRY(dev_alloc(d, &d->part[1], (size_t)B * H * sizeof(float)));
    TRY(dev_alloc(d, &d->argmax_cand, (size_t)B * ARGMAX_PARTS * sizeof(Candidate)));
    if (c.tp_size > 1) {
        // one exchange carries a (batch, hidden) partial output, or two words per sequence for the token pick
        const long cap = (long)B * H > 2l * B ? (long)B * H : 2l * B;
        TRY(tp_comm_create(c.tp_rank, c.tp_size, cap, &d->comm));
    }
    TRY(cuda_status(cudaStreamSynchronize(s)));
    if (tmp) {  // the staging buffer of the initialisation is not needed again
        d->allocs.erase(std::find(d->allocs.begin(), d->allocs.end(), static_cast<void*>(tmp)));
        TRY(cuda_status(cudaFree(tmp)));
    }
#undef TRY
    *out = d;
    return QMM_OK;
}


template <typename... KArgs, typename... Args>
static int launch_pdl(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = overlap_enabled() ? 1 : 0;
    QMM_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...));
    return QMM_OK;
}

// residual add of the projection output `which` (or none: -1), RMSNorm with gamma, Q8_1 into xq_h
static int add_norm(Decoder* d, int which, const float* gamma, int batch, cudaStream_t s) {
    PartPtrs parts = {};
    TpRecv rcv = {};
    int n_parts = 0;
    if (which >= 0) {
        if (d->comm) {
            rcv = tp_comm_recv(d->comm);
        } else {
            n_parts = 1;
            parts.p[0] = d->part[which];
        }
    }
    return add_rmsnorm_launch(d->x, parts, n_parts, (long)d->c.hidden, gamma, d->xq_h, d->c.hidden, d->c.rms_eps, rcv, nullptr, batch, true, s);
}

// row-parallel projection (O, down): the output goes to part[which], or with tensor parallelism into every
// rank's exchange area, where the next add_norm finds the partial outputs of all ranks
static int row_parallel(Decoder* d, int type, const uint8_t* w, const uint8_t* xq, int which, int batch, int k, cudaStream_t s) {
    const int H = d->c.hidden;
    const long pitch = which == 0 ? d->o_pitch : d->down_pitch;
    if (!d->comm) return qmatvec_launch_pitched(type, w, pitch, xq, d->part[which], H, batch, H, k, 0, nullptr, s);
    const TpPush push = tp_comm_push(d->comm, 0);
    return qmatvec_launch_pitched(type, w, pitch, xq, d->part[which], H, batch, H, k, 0, &push, s);
}

// Small batches on one GPU: the residual add + norm + quantization before a block's projections, and the
// gated activation before the down projection, are built inside the job-list matvec launch that needs them
// (JOBS_X_NORM / JOBS_X_GLU) instead of in launches of their own.  The residual alternates between two buffers:
// every CTA reads the old one while CTA 0 writes the new one.  QMM_ERR_UNSUPPORTED: the caller takes the
// separate kernels.
static qmm_matvec_job make_job(int type, const uint8_t* w, float* y, int n, int k, long y_stride) {
    qmm_matvec_job q = {};
    q.type = type, q.n = n, q.k = k, q.w = w, q.y = y, q.y_stride = y_stride;
    return q;
}
static int norm_proj(Decoder* d, int which, const float* gamma, const qmm_matvec_job* jobs, int n_jobs, int batch, cudaStream_t s) {
    XBuild xb = {};
    xb.x_in = d->x, xb.gamma = gamma, xb.eps = d->c.rms_eps, xb.k = d->c.hidden;
    if (which >= 0) xb.x_add = d->part[which], xb.x_out = d->x_alt;
    const int st = qmatvec_jobs_launch_ex(jobs, n_jobs, batch, nullptr, nullptr, JOBS_X_NORM, &xb, s);
    if (st == QMM_OK && which >= 0) std::swap(d->x, d->x_alt);
    return st;
}
static int glu_proj(Decoder* d, const qmm_matvec_job* job, int batch, cudaStream_t s) {
    XBuild xb = {};
    xb.x_in = d->gu, xb.act = d->c.act, xb.k = d->ffn_l;
    return qmatvec_jobs_launch_ex(job, 1, batch, nullptr, nullptr, JOBS_X_GLU, &xb, s);
}

static int step(Decoder* d, const int* tokens, int batch, int pos, int* next_tokens, float* logits_out, float* best_out, cudaStream_t s) {
    const qmm_decoder_config& c = d->c;
    if (!tokens || !next_tokens) return QMM_ERR_NULL;
    if (batch <= 0 || batch > c.max_batch || pos < 0 || pos >= c.ctx_len) return QMM_ERR_SHAPE;
    const int H = c.hidden, hd = c.head_dim, ao = d->nq * hd;
    int st;
#define TRY(e) \
    do {       \
        if ((st = (e)) != 0) return st; \
    } while (0)
    const int fuse_level = batch <= 2 ? decoder_fusion() : 0;
    const bool fuse = !d->comm && fuse_level >= 2;       // norms inside the matvec launches
    const bool fuse_glu = !d->comm && fuse_level >= 3;   // gated activation inside the down launch
    const bool qkv_list = fuse_level >= 1;               // Q|K and V of different types as one job list
    if (d->x_home && d->x != d->x_home) std::swap(d->x, d->x_alt);  // every step starts in the same buffer
    {   // embedding
        const int rb = type_row_bytes(c.type_head, H);
        const dim3 grid((H + 255) / 256, batch);
        if (c.type_head == QMM_TYPE_Q6_K) TRY(launch_pdl(embed_rows_kernel<QMM_TYPE_Q6_K>, grid, dim3(256), 0, s, d->embed, tokens, d->x, H, rb, c.vocab, (unsigned*)nullptr));
        else if (c.type_head == QMM_TYPE_Q4_K) TRY(launch_pdl(embed_rows_kernel<QMM_TYPE_Q4_K>, grid, dim3(256), 0, s, d->embed, tokens, d->x, H, rb, c.vocab, (unsigned*)nullptr));
        else TRY(launch_pdl(embed_rows_kernel<QMM_TYPE_Q8_0>, grid, dim3(256), 0, s, d->embed, tokens, d->x, H, rb, c.vocab, (unsigned*)nullptr));
    }
    const size_t cache_layer = (size_t)c.max_batch * c.ctx_len * d->nkv * hd;
    const int len = pos + 1;
    const int splits = (len + d->attn_chunk - 1) / d->attn_chunk;
    const int group = d->nq / d->nkv;
    const size_t attn_smem = (size_t)ATTN_CHUNK * (2 * hd + 8) * sizeof(__half) + (size_t)group * (hd + ATTN_CHUNK + 2) * sizeof(float);
    for (int l = 0; l < c.n_layers; ++l) {
        const LayerWeights& L = d->layers[l];
        bool qkv_done = false;
        if (fuse) {  // norm + Q|K (+ V) in one launch
            qmm_matvec_job jobs[2];
            int nj = 1;
            if (c.type_attn_v == c.type_attn_qk) {
                jobs[0] = make_job(c.type_attn_qk, L.wqk, d->qkv, d->qk_rows + d->v_rows, H, d->qkv_cols);
            } else {
                jobs[0] = make_job(c.type_attn_qk, L.wqk, d->qkv, d->qk_rows, H, d->qkv_cols);
                jobs[1] = make_job(c.type_attn_v, L.wv, d->qkv + d->qk_rows, d->v_rows, H, d->qkv_cols);
                nj = 2;
            }
            st = norm_proj(d, l == 0 ? -1 : 1, L.attn_norm, jobs, nj, batch, s);
            if (st != QMM_OK && st != QMM_ERR_UNSUPPORTED) return st;
            qkv_done = st == QMM_OK;
        }
        if (!qkv_done) TRY(add_norm(d, l == 0 ? -1 : 1, L.attn_norm, batch, s));
        if (qkv_done) {
        } else if (c.type_attn_v == c.type_attn_qk) {  // V's rows follow K's in memory: one launch
            TRY(qmatvec_launch_strided(c.type_attn_qk, L.wqk, d->xq_h, d->qkv, d->qkv_cols, batch, d->qk_rows + d->v_rows, H, s));
        } else if (qkv_list && [&]() {
                       qmm_matvec_job jobs[2] = {make_job(c.type_attn_qk, L.wqk, d->qkv, d->qk_rows, H, d->qkv_cols),
                                                 make_job(c.type_attn_v, L.wv, d->qkv + d->qk_rows, d->v_rows, H, d->qkv_cols)};
                       jobs[0].xq = jobs[1].xq = d->xq_h;
                       st = qmatvec_jobs_launch_ex(jobs, 2, batch, nullptr, nullptr, 0, nullptr, s);
                       return st != QMM_ERR_UNSUPPORTED;
                   }()) {
            if (st) return st;  // one launch walked both matrices
        } else {
            // two kernels side by side: the SMs are shared in proportion to the weight bytes
            const double qk_b = (double)d->qk_rows * type_row_bytes(c.type_attn_qk, H), v_b = (double)d->v_rows * type_row_bytes(c.type_attn_v, H);
            int v_ctas = (int)(d->sms * v_b / (qk_b + v_b) + 0.5);
            if (v_ctas < 1) v_ctas = 1;
            if (v_ctas > d->sms - 1) v_ctas = d->sms - 1;
            QMM_CUDA_TRY(cudaEventRecord(d->fork, s));  // after the norm that produced the activations
            QMM_CUDA_TRY(cudaStreamWaitEvent(d->side, d->fork, 0));
            TRY(qmatvec_launch_limited(c.type_attn_qk, L.wqk, d->xq_h, d->qkv, d->qkv_cols, batch, d->qk_rows, H, d->sms - v_ctas, s));
            TRY(qmatvec_launch_limited(c.type_attn_v, L.wv, d->xq_h, d->qkv + d->qk_rows, d->qkv_cols, batch, d->v_rows, H, v_ctas, d->side));
            QMM_CUDA_TRY(cudaEventRecord(d->join, d->side));
            QMM_CUDA_TRY(cudaStreamWaitEvent(s, d->join, 0));
        }
        __half* kc = d->kcache + (size_t)l * cache_layer;
        __half* vc = d->vcache + (size_t)l * cache_layer;
        TRY(launch_pdl(rope_kv_append_kernel, dim3(8, batch), dim3(256), 0, s, d->qkv, kc, vc, d->nq, d->nkv, hd, pos, c.ctx_len, c.rope_theta));
        if (attn_use_tc(batch, hd)) {
            TRY(launch_pdl(attn_decode_split_tc_kernel, dim3(d->nkv, batch, splits), dim3(ATTN_THREADS), attn_tc_smem_bytes(hd), s,
                           (const float*)d->qkv, (const __half*)kc, (const __half*)vc, d->attn_scratch, d->nq, d->nkv, hd, len, c.ctx_len, splits));
        } else {
            TRY(launch_pdl(attn_decode_split_kernel, dim3(d->nkv, batch, splits), dim3(ATTN_THREADS), attn_smem, s, (const float*)d->qkv,
                           (const __half*)kc, (const __half*)vc, d->attn_scratch, d->nq, d->nkv, hd, len, c.ctx_len, splits));
        }
        TRY(launch_pdl(attn_combine_q8_kernel, dim3(d->nq, batch), dim3(hd < 128 ? hd : 128), 0, s, (const float*)d->attn_scratch, d->xq_attn,
                       (float*)nullptr, d->nq, hd, splits));
        TRY(row_parallel(d, c.type_attn_o, L.wo, d->xq_attn, 0, batch, ao, s));
        st = QMM_ERR_UNSUPPORTED;
        if (fuse) {  // norm + gate|up in one launch
            const qmm_matvec_job gu = make_job(c.type_ffn_gate_up, L.wgu, d->gu, 2 * d->ffn_l, H, 2 * d->ffn_l);
            st = norm_proj(d, 0, L.ffn_norm, &gu, 1, batch, s);
            if (st != QMM_OK && st != QMM_ERR_UNSUPPORTED) return st;
        }
        if (st != QMM_OK) {
            TRY(add_norm(d, 0, L.ffn_norm, batch, s));
            TRY(qmatvec_launch_strided(c.type_ffn_gate_up, L.wgu, d->xq_h, d->gu, 2 * d->ffn_l, batch, 2 * d->ffn_l, H, s));
        }
        st = QMM_ERR_UNSUPPORTED;
        if (fuse_glu) {  // gated activation + down in one launch
            const qmm_matvec_job dn = make_job(c.type_ffn_down, L.wdown, d->part[1], H, d->ffn_l, H);
            st = glu_proj(d, &dn, batch, s);
            if (st != QMM_OK && st != QMM_ERR_UNSUPPORTED) return st;
        }
        if (st != QMM_OK) {
            TRY(launch_pdl(act_mul_q8_kernel, dim3((d->ffn_l / 32 + 3) / 4, batch), dim3(128), 0, s, (const float*)d->gu, d->xq_ffn, d->ffn_l, c.act, (float*)nullptr));
            TRY(row_parallel(d, c.type_ffn_down, L.wdown, d->xq_ffn, 1, batch, d->ffn_l, s));
        }
    }
    float* lg = logits_out ? logits_out : d->logits;
    st = QMM_ERR_UNSUPPORTED;
    if (fuse) {  // final norm + head in one launch
        const qmm_matvec_job hj = make_job(c.type_head, d->head, lg, d->vocab_l, H, d->vocab_l);
        st = norm_proj(d, 1, d->final_norm, &hj, 1, batch, s);
        if (st != QMM_OK && st != QMM_ERR_UNSUPPORTED) return st;
    }
    if (st != QMM_OK) {
        TRY(add_norm(d, 1, d->final_norm, batch, s));
        TRY(qmatvec_launch_strided(c.type_head, d->head, d->xq_h, lg, d->vocab_l, batch, d->vocab_l, H, s));
    }
    float* bv = best_out ? best_out : d->best_val;
    TRY(launch_pdl(argmax_partial_kernel, dim3(ARGMAX_PARTS, batch), dim3(256), 0, s, (const float*)lg, d->argmax_cand, d->vocab_l));
    TRY(launch_pdl(argmax_final_kernel, dim3(batch), dim3(256), 0, s, (const Candidate*)d->argmax_cand, ARGMAX_PARTS, next_tokens,
                   c.tp_rank * d->vocab_l, bv));
    if (d->comm) {
        TRY(launch_pdl(tp_pick_token_kernel, dim3(1), dim3(batch < 32 ? 32 : ((batch + 31) & ~31)), 0, s, (const float*)bv, next_tokens,
                       tp_comm_push(d->comm, 0), tp_comm_recv(d->comm), batch));
    }
#undef TRY
    return QMM_OK;
}

// ---- the prompt path: all positions of a prompt through every layer at once, as the upstream's layer function does
// (examples/gemma4.rs:638-742: every projection is one gpu_gemm_bt_f64_into over the t rows, the attention one
// gpu_gqa_attn_into).  Projections: launch_qdense without bias or activation, i.e. the tcgen05 GEMM on bf16(x) for
// Q4_K weights from 64 rows on and the Q8_1 matvec otherwise; attention: the sequence kernel, causal; the small
// operators are the decode path's kernels with one row per position.  Fills the KV cache of sequence `seq` for
// positions 0..t-1 and returns the greedy token after the last position.  One GPU only.
static void prefill_free(Decoder* d) {
    Decoder::Prefill& f = d->pf;
    void* ptrs[] = {f.x, f.xn, f.qk, f.v, f.att, f.part, f.gu, f.act, f.xq, f.q8, f.wb, f.xb};
    for (void* p : ptrs)
        if (p) cudaFree(p);
    f = Decoder::Prefill{};
}
static int prefill_reserve(Decoder* d, int t) {
    Decoder::Prefill& f = d->pf;
    if (t <= f.cap) return QMM_OK;
    prefill_free(d);
    const qmm_decoder_config& c = d->c;
    const size_t H = c.hidden, T = (size_t)t, ao = (size_t)d->nq * c.head_dim, ffn = d->ffn_l;
    const size_t kmax = std::max(std::max(H, ao), ffn);
    const size_t dense_scratch = std::max(T * kmax * 2, T * (kmax / 32) * Q8_1_BYTES);  // bf16 or Q8_1 form of a projection's input
    struct { void** p; size_t bytes; } want[] = {
        {(void**)&f.x, T * H * 4},      {(void**)&f.xn, T * H * 4},        {(void**)&f.qk, T * (size_t)d->qkv_cols * 4}, {(void**)&f.v, T * (size_t)d->v_rows * 4},
        {(void**)&f.att, T * ao * 4},   {(void**)&f.part, T * H * 4},      {(void**)&f.gu, T * 2 * ffn * 4},             {(void**)&f.act, T * ffn * 4},
        {(void**)&f.xq, dense_scratch}, {(void**)&f.q8, T * (kmax / 32) * Q8_1_BYTES}, {(void**)&f.xb, T * kmax * 2}};
    for (auto& w : want)
        if (cudaMalloc(w.p, w.bytes) != cudaSuccess) {
            prefill_free(d);
            return cuda_fail(cudaErrorMemoryAllocation);
        }
    // the largest matrix of a type without a fused GEMM, decoded to bf16 one at a time
    size_t wb = 0;
    auto note = [&](int type, size_t n, size_t k) {
        if (type != QMM_TYPE_Q4_K) wb = std::max(wb, n * k);
    };
    note(c.type_attn_qk, (size_t)d->qk_rows + (c.type_attn_v == c.type_attn_qk ? d->v_rows : 0), H);
    note(c.type_attn_v, d->v_rows, H);
    note(c.type_attn_o, H, ao);
    note(c.type_ffn_gate_up, 2 * ffn, H);
    note(c.type_ffn_down, H, ffn);
    if (wb && cudaMalloc((void**)&f.wb, wb * 2) != cudaSuccess) {
        prefill_free(d);
        return cuda_fail(cudaErrorMemoryAllocation);
    }
    f.wb_elems = wb;
    f.cap = t;
    return QMM_OK;
}

// One projection of the prompt path: y(t, n) = x(t, k) . w(n, k)^T.  From 64 rows on the input is read as bf16 from
// f.xb (written by the kernel that produced x; `x` itself may then be stale): Q4_K through the fused tcgen05 GEMM, other
// types decoded to bf16 (bit-identical to launch_dequantize_*_bf16) and multiplied by the same kernel with TMA-fed
// weight tiles.  Fewer rows: launch_qdense on the f32 input (the Q8_1 matvec).
static int prefill_dense(Decoder* d, int type, const uint8_t* w, const float* x, float* y, int t, int n, int k, cudaStream_t s) {
    Decoder::Prefill& f = d->pf;
    const bool gemm = t >= 64 && k % 256 == 0;   // then f.xb holds bf16(x), written by the kernel that produced x
    if (gemm && type == QMM_TYPE_Q4_K) return qgemm_q4k_launch(w, f.xb, nullptr, y, t, n, k, s);
    if (!gemm || (size_t)n * k > f.wb_elems) return launch_qdense(type, w, x, nullptr, y, f.xq, t, n, k, QMM_DENSE_LINEAR, 0.f, s);
    if (int st = dequantize_bf16_launch(type, w, f.wb, (long)n * k, s)) return st;
    return gemm_bt_bf16_launch(f.xb, f.wb, nullptr, y, t, n, k, s);
}

// pos0: the position of tokens[0]; the cache of sequence `seq` already holds positions 0 .. pos0-1
static int prefill(Decoder* d, const int* tokens, int t, int seq, int pos0, int* next_token, float* logits_out, cudaStream_t s) {
    const qmm_decoder_config& c = d->c;
    if (!tokens || !next_token) return QMM_ERR_NULL;
    if (d->comm || c.tp_size != 1) return QMM_ERR_UNSUPPORTED;
    if (t <= 0 || pos0 < 0 || (long)pos0 + t > c.ctx_len || seq < 0 || seq >= c.max_batch) return QMM_ERR_SHAPE;
    int st;
#define TRY(e) \
    do {       \
        if ((st = (e)) != 0) return st; \
    } while (0)
    if (c.head_dim / 2 > 256 || (d->nkv * c.head_dim) % 4 || d->qk_rows % 4 || d->v_rows % 4) return QMM_ERR_UNSUPPORTED;  // rope_seq_append_kernel
    TRY(prefill_reserve(d, t));
    Decoder::Prefill& f = d->pf;
    const int H = c.hidden, hd = c.head_dim, nq = d->nq, nkv = d->nkv, ao = nq * hd, ffn = d->ffn_l;
    const bool v_fused = c.type_attn_v == c.type_attn_qk;  // V's rows follow K's in the same matrix
    const long qk_stride = v_fused ? d->qkv_cols : d->qk_rows;
    const float* vbuf = v_fused ? f.qk + d->qk_rows : f.v;
    const long v_stride = v_fused ? d->qkv_cols : d->v_rows;
    const TpRecv none = {};
    // From 64 positions on every projection is a GEMM on a bf16 input: the kernels that produce those inputs write bf16 (f.xb)
    // and skip the f32 copy.
    float* const xn_f32 = (t >= 64 && H % 256 == 0) ? nullptr : f.xn;
    const bool seq_norm = !xn_f32 && add_rmsnorm_bf16_fits(H, (long)H);  // then neither the f32 nor the Q8_1 form of the norm is read
    {   // embedding
        const int rb = type_row_bytes(c.type_head, H);
        const dim3 grid((H + 255) / 256, t);
        if (c.type_head == QMM_TYPE_Q6_K) embed_rows_kernel<QMM_TYPE_Q6_K><<<grid, 256, 0, s>>>(d->embed, tokens, f.x, H, rb, c.vocab, (unsigned*)nullptr);
        else if (c.type_head == QMM_TYPE_Q4_K) embed_rows_kernel<QMM_TYPE_Q4_K><<<grid, 256, 0, s>>>(d->embed, tokens, f.x, H, rb, c.vocab, (unsigned*)nullptr);
        else embed_rows_kernel<QMM_TYPE_Q8_0><<<grid, 256, 0, s>>>(d->embed, tokens, f.x, H, rb, c.vocab, (unsigned*)nullptr);
        QMM_CUDA_TRY(cudaGetLastError());
    }
    const size_t cache_layer = (size_t)c.max_batch * c.ctx_len * nkv * hd;
    PartPtrs parts = {};
    parts.p[0] = f.part;
    for (int l = 0; l < c.n_layers; ++l) {
        const LayerWeights& L = d->layers[l];
        // x += down output of the previous layer; xn = RMSNorm(x) * gamma
        if (seq_norm) TRY(add_rmsnorm_bf16_launch(f.x, l > 0 ? f.part : nullptr, (long)H, L.attn_norm, H, c.rms_eps, f.xb, t, s));
        else TRY(add_rmsnorm_launch(f.x, parts, l > 0 ? 1 : 0, (long)H, L.attn_norm, f.q8, H, c.rms_eps, none, xn_f32, t, false, s, f.xb));
        TRY(prefill_dense(d, c.type_attn_qk, L.wqk, f.xn, f.qk, t, v_fused ? d->qk_rows + d->v_rows : d->qk_rows, H, s));
        if (!v_fused) TRY(prefill_dense(d, c.type_attn_v, L.wv, f.xn, f.v, t, d->v_rows, H, s));
        rope_seq_append_kernel<<<t, 256, 0, s>>>(f.qk, qk_stride, vbuf, v_stride, d->kcache + (size_t)l * cache_layer,
                                                            d->vcache + (size_t)l * cache_layer, nq, nkv, hd, pos0, seq, c.ctx_len, c.rope_theta);
        QMM_CUDA_TRY(cudaGetLastError());
        // (from 64 positions on the O projection is a GEMM and reads the attention's output as bf16)
        {   // keys and values: the f16 rows that the kernel above has just appended to the cache (row = position)
            const size_t seq_off = (size_t)l * cache_layer + (size_t)seq * c.ctx_len * nkv * hd;
            // (head_dim is a multiple of 32: 16-byte rows; causal throughout: prefix = the sequence's length so far)
            TRY(attn_prefill_launch(f.qk, d->kcache + seq_off, d->vcache + seq_off, f.att, t, nq, nkv, hd, pos0 + t, rsqrtf((float)hd), qk_stride,
                                    (long)nkv * hd, (long)nkv * hd, ao, s, (t >= 64 && ao % 256 == 0) ? f.xb : nullptr, true, pos0 + t, pos0));
        }
        TRY(prefill_dense(d, c.type_attn_o, L.wo, f.att, f.part, t, H, ao, s));
        if (seq_norm) TRY(add_rmsnorm_bf16_launch(f.x, f.part, (long)H, L.ffn_norm, H, c.rms_eps, f.xb, t, s));
        else TRY(add_rmsnorm_launch(f.x, parts, 1, (long)H, L.ffn_norm, f.q8, H, c.rms_eps, none, xn_f32, t, false, s, f.xb));
        TRY(prefill_dense(d, c.type_ffn_gate_up, L.wgu, f.xn, f.gu, t, 2 * ffn, H, s));
        {
            const long quads = (long)t * (ffn / 4);
            const bool gemm = t >= 64 && ffn % 256 == 0;  // then the down projection reads bf16
            act_mul_f32_kernel<<<(unsigned)((quads + 255) / 256), 256, 0, s>>>((const float*)f.gu, gemm ? nullptr : f.act, gemm ? f.xb : nullptr, ffn,
                                                                             c.act, quads);
            QMM_CUDA_TRY(cudaGetLastError());
        }
        TRY(prefill_dense(d, c.type_ffn_down, L.wdown, f.act, f.part, t, H, ffn, s));
    }
    // the last position only: residual, final norm, head, greedy token
    PartPtrs last = {};
    last.p[0] = f.part + (size_t)(t - 1) * H;
    TRY(add_rmsnorm_launch(f.x + (size_t)(t - 1) * H, last, 1, (long)H, d->final_norm, d->xq_h, H, c.rms_eps, none, nullptr, 1, false, s));
    float* lg = logits_out ? logits_out : d->logits;
    TRY(qmatvec_launch_strided(c.type_head, d->head, d->xq_h, lg, d->vocab_l, 1, d->vocab_l, H, s));
    TRY(launch_pdl(argmax_partial_kernel, dim3(ARGMAX_PARTS, 1), dim3(256), 0, s, (const float*)lg, d->argmax_cand, d->vocab_l));
    TRY(launch_pdl(argmax_final_kernel, dim3(1), dim3(256), 0, s, (const Candidate*)d->argmax_cand, ARGMAX_PARTS, next_token, 0, d->best_val));
#undef TRY
    return QMM_OK;
}

}  // namespace qmm

using namespace qmm;

extern "C" {

static int finish_create(const qmm_decoder_config* cfg, WeightSource* src, void** handle);

int qmm_decoder_create(const qmm_decoder_config* cfg, void** handle) {
    if (!cfg || !handle) return QMM_ERR_NULL;
    SeededSource src;
    return finish_create(cfg, &src, handle);
}

// Reads the hyper-parameters of a Llama/Gemma-style decoder from the metadata of a GGUF file ("<arch>." keys of
// the format's naming convention) and the block types from its tensors, then builds this rank's shard of it.
int qmm_decoder_create_from_gguf(const char* path, int max_batch, int ctx_len, int tp_rank, int tp_size, void** handle) {
    if (!path || !handle) return QMM_ERR_NULL;
    void* fv = nullptr;
    if (int st = qmm_gguf_open(path, &fv)) return st;
    GgufFile* f = static_cast<GgufFile*>(fv);
    auto u = [&](const std::string& key, unsigned long long dflt) {
        auto it = f->meta.find(key);
        return it == f->meta.end() ? dflt : (unsigned long long)it->second.u;
    };
    auto fl = [&](const std::string& key, double dflt) {
        auto it = f->meta.find(key);
        return it == f->meta.end() ? dflt : it->second.f;
    };
    auto type_of = [&](int layer, int which) -> int {
        auto it = f->by_name.find(gguf_tensor_name(layer, which));
        return it == f->by_name.end() ? -1 : (int)f->tensors[it->second].type;
    };
    std::string arch = "llama";
    if (f->meta.count("general.architecture")) arch = f->meta["general.architecture"].s;
    qmm_decoder_config c = {};
    c.n_layers = (int)u(arch + ".block_count", 0);
    c.hidden = (int)u(arch + ".embedding_length", 0);
    c.ffn = (int)u(arch + ".feed_forward_length", 0);
    c.n_q_heads = (int)u(arch + ".attention.head_count", 0);
    c.n_kv_heads = (int)u(arch + ".attention.head_count_kv", c.n_q_heads);
    c.head_dim = (int)u(arch + ".attention.key_length", c.n_q_heads ? c.hidden / c.n_q_heads : 0);
    c.ctx_len = ctx_len > 0 ? ctx_len : (int)u(arch + ".context_length", 0);
    c.rope_theta = (float)fl(arch + ".rope.freq_base", 10000.0);
    c.rms_eps = (float)fl(arch + ".attention.layer_norm_rms_epsilon", 1e-6);
    // gated GELU for the Gemma family, SiLU otherwise; "qmm.activation" (0 / 1) overrides
    c.act = (int)u("qmm.activation", arch.find("gemma") != std::string::npos ? QMM_ACT_GELU_TANH : QMM_ACT_SILU);
    c.max_batch = max_batch;
    c.tp_rank = tp_rank, c.tp_size = tp_size;
    c.type_attn_qk = type_of(0, QMM_T_WQ), c.type_attn_v = type_of(0, QMM_T_WV), c.type_attn_o = type_of(0, QMM_T_WO);
    c.type_ffn_gate_up = type_of(0, QMM_T_WGATE), c.type_ffn_down = type_of(0, QMM_T_WDOWN);
    const int t_embd = type_of(-1, QMM_T_EMBED), t_out = type_of(-1, QMM_T_HEAD);
    c.type_head = t_out >= 0 ? t_out : t_embd;
    int st = QMM_OK;
    if (t_embd < 0 || c.type_attn_qk < 0 || c.type_attn_v < 0 || c.type_attn_o < 0 || c.type_ffn_gate_up < 0 || c.type_ffn_down < 0) st = QMM_ERR_FORMAT;
    else if (t_embd != c.type_head) st = QMM_ERR_UNSUPPORTED;  // the engine decodes embedding rows with the head's block type
    else if (type_of(0, QMM_T_WK) != c.type_attn_qk || type_of(0, QMM_T_WUP) != c.type_ffn_gate_up) st = QMM_ERR_UNSUPPORTED;
    if (!st) {
        // one block type per role across the layers (the engine keeps one kernel choice per role)
        for (int l = 1; l < c.n_layers && !st; ++l)
            if (type_of(l, QMM_T_WQ) != c.type_attn_qk || type_of(l, QMM_T_WK) != c.type_attn_qk || type_of(l, QMM_T_WV) != c.type_attn_v ||
                type_of(l, QMM_T_WO) != c.type_attn_o || type_of(l, QMM_T_WGATE) != c.type_ffn_gate_up ||
                type_of(l, QMM_T_WUP) != c.type_ffn_gate_up || type_of(l, QMM_T_WDOWN) != c.type_ffn_down)
                st = QMM_ERR_UNSUPPORTED;
        auto it = f->by_name.find("token_embd.weight");
        c.vocab = (int)f->tensors[it->second].dims[1];
    }
    if (!st) {
        GgufSource src;
        src.f = f;
        st = finish_create(&c, &src, handle);
    }
    qmm_gguf_close(f);
    return st;
}

// Writes the model of a single-GPU decoder as a GGUF file (synthetic models for tests and examples).
int qmm_decoder_export_gguf(void* handle, const char* path, const char* architecture) {
    if (!handle || !path) return QMM_ERR_NULL;
    Decoder* d = static_cast<Decoder*>(handle);
    const qmm_decoder_config& c = d->c;
    if (c.tp_size != 1) return QMM_ERR_UNSUPPORTED;
    const std::string arch = architecture ? architecture : "llama";
    void* w = nullptr;
    if (int st = qmm_gguf_writer_create(path, &w)) return st;
    qmm_gguf_writer_meta_str(w, "general.architecture", arch.c_str());
    qmm_gguf_writer_meta_u32(w, (arch + ".block_count").c_str(), c.n_layers);
    qmm_gguf_writer_meta_u32(w, (arch + ".embedding_length").c_str(), c.hidden);
    qmm_gguf_writer_meta_u32(w, (arch + ".feed_forward_length").c_str(), c.ffn);
    qmm_gguf_writer_meta_u32(w, (arch + ".attention.head_count").c_str(), c.n_q_heads);
    qmm_gguf_writer_meta_u32(w, (arch + ".attention.head_count_kv").c_str(), c.n_kv_heads);
    qmm_gguf_writer_meta_u32(w, (arch + ".attention.key_length").c_str(), c.head_dim);
    qmm_gguf_writer_meta_u32(w, (arch + ".context_length").c_str(), c.ctx_len);
    qmm_gguf_writer_meta_f32(w, (arch + ".rope.freq_base").c_str(), c.rope_theta);
    qmm_gguf_writer_meta_f32(w, (arch + ".attention.layer_norm_rms_epsilon").c_str(), c.rms_eps);
    qmm_gguf_writer_meta_u32(w, "qmm.activation", c.act);
    const int H = c.hidden, hd = c.head_dim;
    std::vector<uint8_t> host;
    int st = cudaDeviceSynchronize() == cudaSuccess ? QMM_OK : QMM_ERR_CUDA;
    auto add = [&](int layer, int which, int type, const void* dev, long rows, long k) {
        if (st) return;
        const long bytes = type == 0 ? rows * k * 4 : rows * (long)type_row_bytes(type, k);
        host.resize((size_t)bytes);
        if (cudaMemcpy(host.data(), dev, (size_t)bytes, cudaMemcpyDeviceToHost) != cudaSuccess) {
            st = QMM_ERR_CUDA;
            return;
        }
        const long dims[2] = {k, rows};
        st = qmm_gguf_writer_add_tensor(w, gguf_tensor_name(layer, which).c_str(), type, rows > 1 || type != 0 ? 2 : 1, dims, host.data(), bytes);
    };
    add(-1, QMM_T_EMBED, c.type_head, d->embed, c.vocab, H);
    for (int l = 0; l < c.n_layers; ++l) {
        const LayerWeights& L = d->layers[l];
        const size_t rbqk = type_row_bytes(c.type_attn_qk, H), rbgu = type_row_bytes(c.type_ffn_gate_up, H);
        add(l, QMM_T_ATTN_NORM, 0, L.attn_norm, 1, H);
        add(l, QMM_T_WQ, c.type_attn_qk, L.wqk, (long)c.n_q_heads * hd, H);
        add(l, QMM_T_WK, c.type_attn_qk, L.wqk + (size_t)c.n_q_heads * hd * rbqk, (long)c.n_kv_heads * hd, H);
        add(l, QMM_T_WV, c.type_attn_v, L.wv, (long)c.n_kv_heads * hd, H);
        add(l, QMM_T_WO, c.type_attn_o, L.wo, H, (long)c.n_q_heads * hd);
        add(l, QMM_T_FFN_NORM, 0, L.ffn_norm, 1, H);
        add(l, QMM_T_WGATE, c.type_ffn_gate_up, L.wgu, c.ffn, H);
        add(l, QMM_T_WUP, c.type_ffn_gate_up, L.wgu + (size_t)c.ffn * rbgu, c.ffn, H);
        add(l, QMM_T_WDOWN, c.type_ffn_down, L.wdown, H, c.ffn);
    }
    add(-1, QMM_T_FINAL_NORM, 0, d->final_norm, 1, H);
    if (d->embed != d->head) add(-1, QMM_T_HEAD, c.type_head, d->head, c.vocab, H);
    const int fin = qmm_gguf_writer_finish(w);
    return st ? st : fin;
}

static int finish_create(const qmm_decoder_config* cfg, WeightSource* src, void** handle) {
    Decoder* d = nullptr;
    const int st = create(cfg, src, &d);
    if (st) return st;
    // attention kernel: opt in to the shared memory its largest context split needs
    const int group = d->nq / d->nkv;
    const size_t attn_smem = (size_t)ATTN_CHUNK * (2 * cfg->head_dim + 8) * sizeof(__half) +
                             (size_t)group * (cfg->head_dim + ATTN_CHUNK + 2) * sizeof(float);
    if (attn_smem > 200 * 1024) {
        destroy(d);
        return QMM_ERR_UNSUPPORTED;
    }
    if (attn_opt_in_smem(true, attn_tc_smem_bytes(cfg->head_dim)) != QMM_OK || attn_opt_in_smem(false, attn_smem) != QMM_OK) {
        destroy(d);
        return QMM_ERR_CUDA;
    }
    *handle = d;
    return QMM_OK;
}

int qmm_decoder_destroy(void* handle) {
    if (!handle) return QMM_ERR_NULL;
    cudaDeviceSynchronize();
    destroy(static_cast<Decoder*>(handle));
    return QMM_OK;
}

long qmm_decoder_weight_bytes(void* handle) { return handle ? static_cast<Decoder*>(handle)->weight_bytes_per_token : QMM_ERR_NULL; }

int qmm_decoder_get_tensor(void* handle, int layer, int which, void** ptr, long* bytes) {
    if (!handle || !ptr || !bytes) return QMM_ERR_NULL;
    Decoder* d = static_cast<Decoder*>(handle);
    const qmm_decoder_config& c = d->c;
    const int H = c.hidden, ao = d->nq * c.head_dim;
    if (layer >= c.n_layers) return QMM_ERR_SHAPE;
    if (layer >= 0) {
        const LayerWeights& L = d->layers[layer];
        switch (which) {
        case QMM_T_ATTN_NORM: *ptr = L.attn_norm, *bytes = H * 4l; return QMM_OK;
        case QMM_T_FFN_NORM: *ptr = L.ffn_norm, *bytes = H * 4l; return QMM_OK;
        case QMM_T_WQ: *ptr = L.wqk, *bytes = (long)d->qk_rows * type_row_bytes(c.type_attn_qk, H); return QMM_OK;
        case QMM_T_WV: *ptr = L.wv, *bytes = (long)d->v_rows * type_row_bytes(c.type_attn_v, H); return QMM_OK;
        case QMM_T_WO: *ptr = L.wo, *bytes = (long)H * type_row_bytes(c.type_attn_o, ao); return QMM_OK;
        case QMM_T_WGATE: *ptr = L.wgu, *bytes = 2l * d->ffn_l * type_row_bytes(c.type_ffn_gate_up, H); return QMM_OK;
        case QMM_T_WDOWN: *ptr = L.wdown, *bytes = (long)H * type_row_bytes(c.type_ffn_down, d->ffn_l); return QMM_OK;
        }
        return QMM_ERR_TYPE;
    }
    switch (which) {
    case QMM_T_FINAL_NORM: *ptr = d->final_norm, *bytes = H * 4l; return QMM_OK;
    case QMM_T_HEAD: *ptr = d->head, *bytes = (long)d->vocab_l * type_row_bytes(c.type_head, H); return QMM_OK;
    case QMM_T_EMBED: *ptr = d->embed, *bytes = (long)c.vocab * type_row_bytes(c.type_head, H); return QMM_OK;
    }
    return QMM_ERR_TYPE;
}

int qmm_decoder_read_tensor(void* handle, int layer, int which, void* host_dst, long capacity) {
    void* p = nullptr;
    long n = 0;
    if (!host_dst) return QMM_ERR_NULL;
    if (int st = qmm_decoder_get_tensor(handle, layer, which, &p, &n)) return st;
    if (n > capacity) return QMM_ERR_SHAPE;
    QMM_CUDA_TRY(cudaDeviceSynchronize());
    Decoder* d = static_cast<Decoder*>(handle);
    const long pitch = layer >= 0 ? (which == QMM_T_WO ? d->o_pitch : (which == QMM_T_WDOWN ? d->down_pitch : 0)) : 0;
    if (pitch) {  // the rows lie `pitch` bytes apart on the device: the copy packs them
        const size_t rb = (size_t)n / d->c.hidden;
        QMM_CUDA_TRY(cudaMemcpy2D(host_dst, rb, p, (size_t)pitch, rb, (size_t)d->c.hidden, cudaMemcpyDeviceToHost));
        return QMM_OK;
    }
    QMM_CUDA_TRY(cudaMemcpy(host_dst, p, (size_t)n, cudaMemcpyDeviceToHost));
    return QMM_OK;
}

int qmm_decoder_fill_cache(void* handle, unsigned long long seed, void* stream) {
    if (!handle) return QMM_ERR_NULL;
    Decoder* d = static_cast<Decoder*>(handle);
    cudaStream_t s = as_stream(stream);
    const size_t total = (size_t)d->c.n_layers * d->c.max_batch * d->c.ctx_len * d->nkv * d->c.head_dim;
    const size_t chunk = 16u << 20;
    float* tmp = nullptr;
    QMM_CUDA_TRY(cudaMalloc(&tmp, chunk * sizeof(float)));
    int rc = QMM_OK;
    for (int which = 0; which < 2 && rc == QMM_OK; ++which) {
        __half* dst = which ? d->vcache : d->kcache;
        for (size_t off = 0; off < total; off += chunk) {
            const long n = (long)(total - off < chunk ? total - off : chunk);
            fill_normal_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(tmp, n, seed + which, 1.0f, (long)off);
            f32_to_f16_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(tmp, dst + off, n);
            if (cudaGetLastError() != cudaSuccess) {
                rc = cuda_fail(cudaErrorLaunchFailure);
                break;
            }
        }
    }
    cudaStreamSynchronize(s);
    cudaFree(tmp);
    return rc;
}

int qmm_decoder_ipc_export(void* handle, void* out_handle_64_bytes) {
    if (!handle || !out_handle_64_bytes) return QMM_ERR_NULL;
    Decoder* d = static_cast<Decoder*>(handle);
    if (!d->comm) return QMM_ERR_UNSUPPORTED;  // single GPU: nothing to exchange
    return tp_comm_export(d->comm, out_handle_64_bytes);
}

int qmm_decoder_ipc_import(void* handle, int peer_rank, const void* handle_64_bytes) {
    if (!handle || !handle_64_bytes) return QMM_ERR_NULL;
    Decoder* d = static_cast<Decoder*>(handle);
    if (!d->comm) return QMM_ERR_UNSUPPORTED;
    return tp_comm_import(d->comm, peer_rank, handle_64_bytes);
}

int qmm_decoder_tp_ready(void* handle) {
    if (!handle) return QMM_ERR_NULL;
    Decoder* d = static_cast<Decoder*>(handle);
    return d->comm ? tp_comm_ready(d->comm) : QMM_OK;
}

int qmm_decoder_prefill(void* handle, const int* tokens, int n_tokens, int seq, int* next_token, float* logits_out, void* stream) {
    if (!handle) return QMM_ERR_NULL;
    Decoder* d = static_cast<Decoder*>(handle);
    return prefill(d, tokens, n_tokens, seq, 0, next_token, logits_out, static_cast<cudaStream_t>(stream));
}

int qmm_decoder_prefill_at(void* handle, const int* tokens, int n_tokens, int seq, int pos0, int* next_token, float* logits_out, void* stream) {
    if (!handle) return QMM_ERR_NULL;
    Decoder* d = static_cast<Decoder*>(handle);
    return prefill(d, tokens, n_tokens, seq, pos0, next_token, logits_out, static_cast<cudaStream_t>(stream));
}

int qmm_decoder_step(void* handle, const int* tokens, int batch, int pos, int* next_tokens, float* logits, float* best, void* stream) {
    if (!handle) return QMM_ERR_NULL;
    return step(static_cast<Decoder*>(handle), tokens, batch, pos, next_tokens, logits, best, as_stream(stream));
}

}  // extern "C"
