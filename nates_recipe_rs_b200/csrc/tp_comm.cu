// Tensor-parallel exchange object and the row-parallel projections that use it.
//
// The upstream runs on one GPU (its layer() issues every projection on the null stream of one device:
// examples/gemma4.rs:653-679); partitioning a layer over the GPUs of a box splits O and down by input
// columns, and their partial outputs have to be summed over the ranks.  A TpComm is one rank's end of
// that sum: an exchange area every peer has mapped, into which the matvec kernels of all ranks store
// their outputs directly (qmm_common.cuh: TpPush / TpRecv, one 64-bit word {value, sequence number} per
// output), and a small kernel that adds the ranks' words in rank order - the same order on every
// rank, so all ranks hold bit-identical sums.  No collective library is involved and no rank ever reads
// remote memory; the only traffic is the posted stores of the producing kernel.
#include "qmm_formats.cuh"
#include <cstring>
#include <vector>

namespace qmm {

int qmatvec_launch_push(int type, const void* w, const void* xq, float* y, long y_stride, int m, int n, int k, int cta_limit,
                        const TpPush* push, cudaStream_t stream);
int qmatvec_jobs_launch_push(const qmm_matvec_job* jobs, int n_jobs, int m, const TpPush* push, const long* push_words, cudaStream_t stream);

struct TpComm {
    int rank = 0, tp = 1, dev = 0;
    long cap = 0;                                   // words per source rank and buffer
    unsigned long long* local = nullptr;            // [2][tp][cap] words, then the counter and ticket words
    unsigned* counter = nullptr;
    unsigned* ticket = nullptr;
    unsigned long long* peer[QMM_TP_MAX] = {};      // the ranks' areas as mapped here (own entry = local)
    bool ready = false;
};

TpPush tp_comm_push(const TpComm* c, long word0) {
    TpPush s = {};
    for (int r = 0; r < c->tp; ++r) s.dst[r] = c->peer[r] + (long)c->rank * c->cap;
    s.counter = c->counter;
    s.buf_words = (long)c->tp * c->cap;
    s.word0 = word0;
    s.tp = c->tp;
    return s;
}
TpRecv tp_comm_recv(const TpComm* c) {
    TpRecv r = {};
    r.base = c->local;
    r.counter = c->counter;
    r.ticket = c->ticket;
    r.buf_words = (long)c->tp * c->cap;
    r.src_words = c->cap;
    r.tp = c->tp;
    return r;
}

int tp_comm_create(int rank, int world, long capacity_words, TpComm** out) {
    if (!out) return QMM_ERR_NULL;
    if (world < 1 || world > QMM_TP_MAX || rank < 0 || rank >= world || capacity_words <= 0) return QMM_ERR_SHAPE;
    TpComm* c = new TpComm();
    c->rank = rank, c->tp = world;
    c->cap = (capacity_words + 31) & ~31l;
    cudaGetDevice(&c->dev);
    const size_t words = (size_t)2 * world * c->cap;
    void* p = nullptr;
    cudaError_t e = cudaMalloc(&p, words * 8 + 256);
    if (e == cudaSuccess) e = cudaMemset(p, 0, words * 8 + 256);
    if (e != cudaSuccess) {
        if (p) cudaFree(p);
        delete c;
        return cuda_fail(e);
    }
    c->local = static_cast<unsigned long long*>(p);
    c->counter = reinterpret_cast<unsigned*>(c->local + words);
    c->ticket = c->counter + 1;
    c->peer[rank] = c->local;
    c->ready = world == 1;
    *out = c;
    return QMM_OK;
}

void tp_comm_destroy(TpComm* c) {
    if (!c) return;
    for (int r = 0; r < c->tp; ++r)
        if (c->peer[r] && c->peer[r] != c->local) cudaIpcCloseMemHandle(c->peer[r]);
    if (c->local) cudaFree(c->local);
    delete c;
}

int tp_comm_export(TpComm* c, void* out64) {
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    cudaIpcMemHandle_t h;
    QMM_CUDA_TRY(cudaIpcGetMemHandle(&h, c->local));
    std::memcpy(out64, &h, 64);
    return QMM_OK;
}

int tp_comm_import(TpComm* c, int peer_rank, const void* handle64) {
    if (peer_rank < 0 || peer_rank >= c->tp) return QMM_ERR_SHAPE;
    if (peer_rank == c->rank) return QMM_OK;
    cudaIpcMemHandle_t h;
    std::memcpy(&h, handle64, 64);
    void* p = nullptr;
    QMM_CUDA_TRY(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
    c->peer[peer_rank] = static_cast<unsigned long long*>(p);
    return QMM_OK;
}

int tp_comm_ready(TpComm* c) {
    for (int r = 0; r < c->tp; ++r)
        if (!c->peer[r]) return QMM_ERR_NULL;  // a peer has not been imported
    c->ready = true;
    return QMM_OK;
}

// ---- the sum: y = sum over source ranks of the words of the current exchange, segment by segment ----
constexpr int TP_SUM_MAX_SEGS = 72;
struct TpSumSegs {
    float* y[TP_SUM_MAX_SEGS];
    long word[TP_SUM_MAX_SEGS];
    int start[TP_SUM_MAX_SEGS + 1];  // first flat element of each segment; start[n] = total
    int n;
};

__global__ void __launch_bounds__(256) tp_sum_kernel(const TpRecv rcv, const __grid_constant__ TpSumSegs segs) {
    __shared__ int give_up;
    pdl_release_dependents();
    if (threadIdx.x == 0) give_up = 0;
    __syncthreads();
    pdl_wait_prior_grids();  // this rank's own words are stored by the preceding kernel
    const unsigned seq = tp_next_seq(rcv.counter);
    const int total = segs.start[segs.n];
    for (int g = blockIdx.x * blockDim.x + threadIdx.x; g < total; g += gridDim.x * blockDim.x) {
        int s = 0;
        while (g >= segs.start[s + 1]) ++s;
        const int i = g - segs.start[s];
        float acc = 0.f;
        bool ok = true;
        for (int r = 0; r < rcv.tp && ok; ++r) {  // fixed order: every rank computes the same sum
            float v;
            ok = tp_poll_word(rcv, seq, r, segs.word[s] + i, v, &give_up);
            acc += v;
        }
        if (ok) segs.y[s][i] = acc;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        if (give_up) atomicExch(&g_device_status, DEV_TIMEOUT_PEER);
        tp_consumer_done(rcv, seq, gridDim.x);
    }
}

static int tp_sum_launch(const TpComm* c, const TpSumSegs& segs, cudaStream_t stream) {
    const int total = segs.start[segs.n];
    int grid = (total + 255) / 256;
    if (grid > 4 * sm_count()) grid = 4 * sm_count();
    if (grid < 1) grid = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(256);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = overlap_enabled() ? 1 : 0;
    QMM_CUDA_TRY(cudaLaunchKernelEx(&cfg, tp_sum_kernel, tp_comm_recv(c), segs));
    return QMM_OK;
}

}  // namespace qmm

using namespace qmm;

extern "C" {

int qmm_tp_comm_create(int rank, int world, long capacity_floats, void** comm) {
    TpComm* c = nullptr;
    if (!comm) return QMM_ERR_NULL;
    if (int st = tp_comm_create(rank, world, capacity_floats, &c)) return st;
    *comm = c;
    return QMM_OK;
}
int qmm_tp_comm_destroy(void* comm) {
    if (!comm) return QMM_ERR_NULL;
    cudaDeviceSynchronize();
    tp_comm_destroy(static_cast<TpComm*>(comm));
    return QMM_OK;
}
int qmm_tp_comm_export(void* comm, void* out_handle_64_bytes) {
    if (!comm || !out_handle_64_bytes) return QMM_ERR_NULL;
    return tp_comm_export(static_cast<TpComm*>(comm), out_handle_64_bytes);
}
int qmm_tp_comm_import(void* comm, int peer_rank, const void* handle_64_bytes) {
    if (!comm || !handle_64_bytes) return QMM_ERR_NULL;
    return tp_comm_import(static_cast<TpComm*>(comm), peer_rank, handle_64_bytes);
}
int qmm_tp_comm_ready(void* comm) {
    if (!comm) return QMM_ERR_NULL;
    return tp_comm_ready(static_cast<TpComm*>(comm));
}

int launch_qmatvec_tp(void* comm, int type, const void* w, const void* xq, float* y, int m, int n, int k, void* stream) {
    if (!comm) return QMM_ERR_NULL;
    TpComm* c = static_cast<TpComm*>(comm);
    if (!c->ready) return QMM_ERR_NULL;
    if (m <= 0 || n <= 0) return QMM_ERR_SHAPE;
    if ((long)m * n > c->cap) return QMM_ERR_SCRATCH;
    if (m > TP_SUM_MAX_SEGS) return QMM_ERR_UNSUPPORTED;
    const TpPush push = tp_comm_push(c, 0);
    if (int st = qmatvec_launch_push(type, w, xq, y, n, m, n, k, 0, &push, as_stream(stream))) return st;
    TpSumSegs segs = {};
    segs.n = 1;
    segs.y[0] = y, segs.word[0] = 0, segs.start[0] = 0, segs.start[1] = m * n;  // (m, n) contiguous in y and in the slots
    return tp_sum_launch(c, segs, as_stream(stream));
}

int launch_qmatvec_batch_tp(void* comm, const qmm_matvec_job* jobs, int n_jobs, int m, void* stream) {
    if (!comm || !jobs) return QMM_ERR_NULL;
    TpComm* c = static_cast<TpComm*>(comm);
    if (!c->ready) return QMM_ERR_NULL;
    if (n_jobs <= 0 || m <= 0) return QMM_ERR_SHAPE;
    std::vector<long> words(n_jobs, -1);
    TpSumSegs segs = {};
    long next = 0;
    for (int i = 0; i < n_jobs; ++i) {
        if (!jobs[i].tp_sum) continue;
        if (jobs[i].n <= 0) return QMM_ERR_SHAPE;
        const long ys = jobs[i].y_stride ? jobs[i].y_stride : jobs[i].n;
        words[i] = next;
        for (int mi = 0; mi < m; ++mi) {  // one segment per activation row: contiguous in y and in the slots
            if (segs.n >= TP_SUM_MAX_SEGS) return QMM_ERR_UNSUPPORTED;
            segs.y[segs.n] = jobs[i].y + (size_t)mi * ys;
            segs.word[segs.n] = next + (long)mi * ys;
            segs.start[segs.n + 1] = segs.start[segs.n] + jobs[i].n;
            ++segs.n;
        }
        next += (long)(m - 1) * ys + jobs[i].n;
        next = (next + 31) & ~31l;
    }
    if (next > c->cap) return QMM_ERR_SCRATCH;
    const TpPush push = tp_comm_push(c, 0);
    cudaStream_t s = as_stream(stream);
    int st = qmatvec_jobs_launch_push(jobs, n_jobs, m, segs.n ? &push : nullptr, segs.n ? words.data() : nullptr, s);
    if (st == QMM_ERR_UNSUPPORTED && segs.n) {
        // outside the persistent kernel (more than two activation rows, ...): one launch per job
        for (int i = 0; i < n_jobs; ++i) {
            const qmm_matvec_job& q = jobs[i];
            if (q.select) return QMM_ERR_UNSUPPORTED;
            TpPush pj = push;
            pj.word0 = words[i];
            st = qmatvec_launch_push(q.type, q.w, q.xq, q.y, q.y_stride ? q.y_stride : q.n, m, q.n, q.k, 0, words[i] >= 0 ? &pj : nullptr, s);
            if (st) return st;
        }
    }
    if (st) return st;
    return segs.n ? tp_sum_launch(c, segs, s) : QMM_OK;
}

}  // extern "C"
