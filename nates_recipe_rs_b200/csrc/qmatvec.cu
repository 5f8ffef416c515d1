// Fused dequant-matvec for decode:  y(m,n) = xq(m,k) . w(n,k)^T
// w: Q8_0 / Q4_K / Q6_K packed rows (GGUF bytes), xq: Q8_1 activations.
//
// Replaces the upstream pair widen_bf16_f64 + gemm_bt_f64
// (gpu-core/src/kernels/f64_infer.hip:12-23, gpu-core/src/kernels/gemm_f64.hip:14-54),
// which stages one weight row per block in shared memory and re-reads the
// activations from cache for every row.  The structure here is the opposite:
//
//   * one persistent CTA per SM owns a contiguous range of weight rows, i.e. a
//     contiguous byte range of w, and streams it through a ring of shared-memory
//     stages with 1-D bulk async copies (cp.async.bulk + mbarrier), issued by a
//     dedicated producer warp, so ~100 KB per SM is in flight without any thread
//     holding a load;
//   * the activations never touch shared memory: the K axis is split over KW
//     warps x 32 lanes x P passes, each lane keeps the Q8_1 words of its own
//     slices in registers for the whole kernel and meets every row there;
//   * rows are dealt to the row-group warps in batches of RB consecutive rows,
//     round-robin over the whole CTA range, so the stage size is independent of
//     the warp count; the RB x M partial sums of a batch are reduced across the
//     warp together (warp_multi_sum);
//   * a row's KW partial sums are combined in a fixed order by the producer warp
//     (no atomics: reruns are bit-identical, the upstream's determinism rule,
//     gpu-core/src/kernels/gemm_f64.hip:12);
//   * with programmatic dependent launch the next kernel's weight stream starts
//     while this one drains; only activations and outputs wait for the
//     predecessor.
#include "qmm_formats.cuh"
#include <string>

namespace qmm {

struct MatvecParams {
    const uint8_t* w;
    const uint8_t* xq;
    float* y;
    long y_stride;    // floats between output rows (>= n)
    int m;            // activation rows in this launch (<= M of the instantiation)
    int n, k;
    int row_bytes;    // packed bytes of one weight row
    int xq_row_bytes;
    int units;        // k / UNIT_ELEMS
    int kw;           // warps along K
    int rg;           // row groups (warps along rows)
    int rows_stage;   // rows per stage, a multiple of RB
    int nst;          // stages in the ring
    int slot_bytes;   // bytes per ring slot (128-aligned, >= rows_stage*row_bytes + 32)
    int pstage;       // floats per partial-sum stage: rows_stage * kw * M
    int partial_off;  // byte offset of the partial-sum area in dynamic shared memory
    int ring_off;     // byte offset of the ring
    int rows_q, rows_r;  // n / grid and n % grid
    int probe;        // 0 = normal; 1 = stream only: every wait and arrival happens, the arithmetic is skipped
    unsigned long long* trace;  // optional (tuning aid): 4 global-timer stamps per CTA
    TpPush push;      // tensor parallel: the outputs go to every rank's exchange area instead of y
};

constexpr int MAX_STAGES = 8;
constexpr int MAX_CONSUMER_WARPS = 24;

struct __align__(16) MatvecSmemHeader {
    uint64_t full[MAX_STAGES];
    uint64_t empty[MAX_STAGES];
    int abort_flag;
};

// Sums V per-lane values across the warp at once: each round halves the number of
// live values while doubling the lanes that share one, so V values cost
// (V-1) + log2(32/V) shuffles instead of 5V.  On return v[0] of lane L holds the
// warp total of value number L / (32/V).  The order of additions is fixed.
template <int V>
__device__ __forceinline__ void warp_multi_sum(float (&v)[V], int lane) {
    int off = 16;
#pragma unroll
    for (int width = V; width > 1; width >>= 1, off >>= 1) {
        const bool up = (lane & off) != 0;
#pragma unroll
        for (int i = 0; i < width / 2; ++i) {
            const float send = up ? v[i] : v[i + width / 2];
            const float keep = up ? v[i + width / 2] : v[i];
            v[i] = keep + __shfl_xor_sync(0xffffffffu, send, off);
        }
    }
#pragma unroll
    for (; off > 0; off >>= 1) v[0] += __shfl_xor_sync(0xffffffffu, v[0], off);
}

// Partial sums live in shared memory as [stage % (2*nst)][row][kw][M]; the producer
// warp adds the kw entries of a row in a fixed order.  Depth 2*nst because the
// producer refills a ring slot before it folds the stage that just left it.
template <int TYPE, int UW, int P, int M, int RB>
__global__ void __launch_bounds__((MAX_CONSUMER_WARPS + 1) * 32, 1) qmatvec_kernel(const MatvecParams p) {
    using F = Fmt<TYPE, UW>;
    constexpr int V = M * RB;
    extern __shared__ __align__(128) uint8_t smem[];
    MatvecSmemHeader* hdr = reinterpret_cast<MatvecSmemHeader*>(smem);
    float* partial = reinterpret_cast<float*>(smem + p.partial_off);
    uint8_t* ring = smem + p.ring_off;
    volatile int* cta_abort = &hdr->abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_consumers = p.kw * p.rg;

    // contiguous row range of this CTA
    // (n / grid rows each, the first n % grid CTAs one more: no division on the device)
    const int bx = (int)blockIdx.x;
    const long row_begin = (long)bx * p.rows_q + min(bx, p.rows_r);
    const int n_rows = p.rows_q + (bx < p.rows_r ? 1 : 0);
    const int n_it = (n_rows + p.rows_stage - 1) / p.rows_stage;
    const uintptr_t w_begin = reinterpret_cast<uintptr_t>(p.w) + (size_t)row_begin * p.row_bytes;
    const uint32_t stage_bytes = (uint32_t)p.rows_stage * p.row_bytes;

    if (threadIdx.x == 0) {
        for (int s = 0; s < p.nst; ++s) {
            mbar_init(smem_u32(&hdr->full[s]), 1);
            mbar_init(smem_u32(&hdr->empty[s]), n_consumers);
        }
        hdr->abort_flag = 0;
        mbar_fence_init();
    }
    __syncthreads();
    pdl_release_dependents();
    if (p.trace && threadIdx.x == 0) p.trace[blockIdx.x * 4 + 0] = globaltimer_ns();

    if (warp == n_consumers) {
        // ------------------------------------------------------------ producer
        auto issue = [&](int it) {
            const int slot = it % p.nst;
            const int nr = min(p.rows_stage, n_rows - it * p.rows_stage);
            const uintptr_t g = w_begin + (size_t)it * stage_bytes;
            const uint32_t head = (uint32_t)(g & 15);
            const uint32_t bytes = (head + (uint32_t)nr * p.row_bytes + 15u) & ~15u;
            const uint32_t bar = smem_u32(&hdr->full[slot]);
            mbar_arrive_expect_tx(bar, bytes);
            bulk_g2s(smem_u32(ring + (size_t)slot * p.slot_bytes), reinterpret_cast<const void*>(g - head), bytes, bar);
        };
        int issued = 0;
        if (lane == 0)
            for (; issued < n_it && issued < p.nst; ++issued) issue(issued);
        pdl_wait_prior_grids();  // y may still be read by the preceding kernel
        const unsigned seq = p.push.tp > 0 ? tp_next_seq(p.push.counter) : 0u;
        bool ok = true;
        // ring slot, its phase and the partial-sum slot of stage `it`, kept incrementally (no divisions)
        int slot = 0, pslot = 0;
        uint32_t phase = 0;
        for (int it = 0; it < n_it; ++it) {
            ok = mbar_wait_bounded(smem_u32(&hdr->empty[slot]), phase, cta_abort);
            if (!ok) {
                if (lane == 0 && !*cta_abort) {
                    atomicExch(&g_device_status, DEV_TIMEOUT_EMPTY);
                    *cta_abort = 1;
                }
                break;
            }
            if (lane == 0 && it + p.nst < n_it) {
                issue(it + p.nst);
                issued = it + p.nst + 1;
            }
            const int nr = min(p.rows_stage, n_rows - it * p.rows_stage);
            const float* ps = partial + (size_t)pslot * p.pstage;
            const long yrow = row_begin + (long)it * p.rows_stage;
            for (int idx = lane; idx < nr * M; idx += 32) {  // idx = r*M + mi
                const int r = idx / M, mi = idx - r * M;
                const float* src = ps + (size_t)r * p.kw * M + mi;
                float acc = 0.f;
                for (int q = 0; q < p.kw; ++q) acc += src[q * M];
                if (mi < p.m) tp_store_out(p.push, seq, p.y, p.y_stride, mi, yrow + r, acc);
            }
            if (++slot == p.nst) slot = 0, phase ^= 1;
            if (++pslot == 2 * p.nst) pslot = 0;
        }
        issued = __shfl_sync(0xffffffffu, issued, 0);
        if (p.trace && lane == 0) p.trace[blockIdx.x * 4 + 3] = globaltimer_ns();
        if (!ok && lane == 0) {
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
        return;
    }

    // ---------------------------------------------------------------- consumers
    const int kwi = warp % p.kw, rgi = warp / p.kw;
    typename F::XRegs x[M][P];
    int unit[P];
    uint32_t unit_off[P];  // byte offset of the unit's block within a row
    pdl_wait_prior_grids();  // activations come from the preceding kernel
    if (p.trace && threadIdx.x == 0) p.trace[blockIdx.x * 4 + 1] = globaltimer_ns();
#pragma unroll
    for (int pp = 0; pp < P; ++pp) {
        const int u = (pp * p.kw + kwi) * 32 + lane;
        // lanes past the end of the row re-read unit 0 against zero activations
        unit[pp] = u < p.units ? u : 0;
        unit_off[pp] = F::unit_offset(unit[pp]);
#pragma unroll
        for (int mi = 0; mi < M; ++mi) {
            if (u < p.units && mi < p.m)
                F::load_x(p.xq + (size_t)mi * p.xq_row_bytes, u, x[mi][pp]);
            else
                F::zero_x(x[mi][pp]);
        }
    }
    // after warp_multi_sum lane L owns value number L / (32/V) = (row j of the batch, activation row mi)
    constexpr int LANES_PER_VALUE = 32 / V;
    const int my_val = lane / LANES_PER_VALUE, my_j = my_val / M, my_mi = my_val - my_j * M;
    const bool writer = (lane % LANES_PER_VALUE) == 0;
    const uint32_t w_begin_lo = (uint32_t)(w_begin & 15);
    const uint32_t ring_s = smem_u32(ring);
    const uint32_t my_ps = ((uint32_t)my_j * p.kw + kwi) * M + my_mi;
    const uint32_t batch_bytes = (uint32_t)RB * p.row_bytes;
    const uint32_t batch_ps = (uint32_t)RB * p.kw * M;
    const int bps = p.rows_stage / RB;  // batches per full stage
    // batches are numbered over the CTA's whole row range; batch g belongs to row group g % rg
    int next_b = rgi;                   // this warp's next batch, relative to the current stage

    // ring slot, its phase and the partial-sum slot of stage `it`, kept incrementally (no divisions)
    int slot = 0, pslot = 0;
    uint32_t phase = 0;
    uint32_t head = w_begin_lo;  // low four address bits of the stage's first byte
    for (int it = 0; it < n_it; ++it) {
        const int nr = min(p.rows_stage, n_rows - it * p.rows_stage);
        const int nb = (nr + RB - 1) / RB;
        // Every warp waits for every stage's data, with or without work in it.  The copy of this use of the
        // slot is only issued after all warps released the previous use, so once the data is seen this
        // warp's arrival below lands in the right phase, the parity test cannot be a phase off, and no
        // copy can still be in flight when the CTA exits.
        if (!mbar_wait_bounded(smem_u32(&hdr->full[slot]), phase, cta_abort)) {
            if (lane == 0 && !*cta_abort) {
                atomicExch(&g_device_status, DEV_TIMEOUT_FULL);
                *cta_abort = 1;
            }
            return;
        }
        if (next_b < nb) {
            if (p.trace && threadIdx.x == 0 && it == 0) p.trace[blockIdx.x * 4 + 2] = globaltimer_ns();
            const uint32_t base = ring_s + (uint32_t)slot * p.slot_bytes + head;
            float* ps = partial + (uint32_t)pslot * p.pstage + my_ps;
            // Whole batches only: rows past nr (last stage of the CTA) hold stale bytes of an
            // earlier stage; their sums land in partial entries that nobody reads.
            if (p.probe == 0) {
                for (; next_b < nb; next_b += p.rg) {
                    const uint32_t row0 = base + (uint32_t)next_b * batch_bytes;
                    float acc[V];
#pragma unroll
                    for (int v = 0; v < V; ++v) acc[v] = 0.f;
#pragma unroll
                    for (int j = 0; j < RB; ++j) {
                        const uint32_t row = row0 + (uint32_t)j * p.row_bytes;
#pragma unroll
                        for (int pp = 0; pp < P; ++pp) {
                            typename F::WRegs wr;
                            F::load_w_s(row, unit_off[pp], unit[pp], wr);
#pragma unroll
                            for (int mi = 0; mi < M; ++mi) acc[j * M + mi] += F::dot(wr, unit[pp], x[mi][pp], nullptr);
                        }
                    }
                    warp_multi_sum<V>(acc, lane);
                    if (writer) ps[(uint32_t)next_b * batch_ps] = acc[0];
                }
            } else {
                next_b += ((nb - next_b + p.rg - 1) / p.rg) * p.rg;
            }
        }
        next_b -= bps;  // renumber relative to the next stage (only the last stage is short)
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&hdr->empty[slot]));
        if (++slot == p.nst) slot = 0, phase ^= 1;
        if (++pslot == 2 * p.nst) pslot = 0;
        head = (head + stage_bytes) & 15u;
    }
}

// ------------------------------------------------------------------- host side

static int type_geometry(int type, int& block_elems, int& block_bytes, int& unit_elems, int& w_align) {
    switch (type) {
    case QMM_TYPE_Q8_0: block_elems = 32, block_bytes = Q8_0_BYTES, unit_elems = 32, w_align = 2; return QMM_OK;
    case QMM_TYPE_Q4_K: block_elems = 256, block_bytes = Q4_K_BYTES, unit_elems = 64, w_align = 16; return QMM_OK;
    case QMM_TYPE_Q6_K: block_elems = 256, block_bytes = Q6_K_BYTES, unit_elems = 64, w_align = 2; return QMM_OK;
    }
    return QMM_ERR_TYPE;
}

constexpr int STAGE_MAX_BYTES = 48 * 1024;  // one packed row must fit this
// tunables (qmm_tune): preferred bytes per stage, ring bytes per CTA, consumer warps per CTA,
// Q4_K unit width (0 = automatic), upper bound on rows per batch
static int g_stage_target = 48 * 1024;
static int g_ring_budget = 150 * 1024;
static int g_consumer_warps = 16;
static bool g_consumer_warps_set = false;  // set through qmm_tune: used as given
static int g_q4k_unit = 0;
static int g_rb_max = 4;
static int g_probe = 0;
static int g_ctas_per_sm = 1;  // persistent CTAs per SM (2 needs a ring and a warp count that fit twice)
static unsigned long long* g_trace = nullptr;
static int g_trace_stride = 0, g_trace_count = 0;
// tuning aid: the next launches write 4 time stamps per CTA at trace + launch_index * stride
void matvec_set_trace(unsigned long long* buf, int stride_words) { g_trace = buf; g_trace_stride = stride_words; g_trace_count = 0; }
void gemm_set_probe(int v);
int gemm_set_mb(int v);
int gemm_set_ksplit(int v);
int mma_set_min_m(int v);
int attn_set_tc_min_batch(int v);
int mma_min_m();
int mma_acc_set(const char* key, int v);
int mma_group_rows();
int qmatvec_mma_launch(int type, const void* w, long row_pitch, const void* xq, float* y, long y_stride, int m, int n, int k, int cta_limit,
                       unsigned long long* trace, const TpPush* push, cudaStream_t stream);
int umv_set_min_m(int v);
int umv_set_ksplit(int v);
int umv_min_m();
int umv_min_k();
int umv_set_min_k(int v);
int qmatvec_umma_launch(const void* w, const void* xq, float* y, long y_stride, int m, int n, int k, const TpPush* push, cudaStream_t stream);
int matvec_tune(const char* key, int value) {
    const std::string k(key ? key : "");
#ifdef QMM_TUNING  // wrong results by design: development builds only
    if (k == "gemm_probe" && value >= 0 && value <= 2) return gemm_set_probe(value), QMM_OK;
    if (k == "probe" && value >= 0 && value <= 1) return g_probe = value, QMM_OK;
#endif
    if (k == "stage_bytes" && value >= 1024 && value <= STAGE_MAX_BYTES) return g_stage_target = value, QMM_OK;
    if (k == "ring_bytes" && value >= 8 * 1024 && value <= 190 * 1024) return g_ring_budget = value, QMM_OK;
    if (k == "consumer_warps" && value >= 1 && value <= MAX_CONSUMER_WARPS) return g_consumer_warps = value, g_consumer_warps_set = true, QMM_OK;
    if (k == "q4k_unit" && (value == 0 || value == 1 || value == 2 || value == 4)) return g_q4k_unit = value, QMM_OK;
    if (k == "rb_max" && (value == 1 || value == 2 || value == 4)) return g_rb_max = value, QMM_OK;
    if (k == "ctas_per_sm" && value >= 1 && value <= 2) return g_ctas_per_sm = value, QMM_OK;
    if (k == "mma_min_m") return mma_set_min_m(value);
    if (k == "umma_min_m") return umv_set_min_m(value);
    if (k == "umma_ksplit") return umv_set_ksplit(value);
    if (k == "umma_min_k") return umv_set_min_k(value);
    if (k.rfind("mma_acc", 0) == 0) return mma_acc_set(key, value);
    if (k == "gemm_mb") return gemm_set_mb(value);
    if (k == "gemm_ksplit") return gemm_set_ksplit(value);
    if (k == "attn_tc_min_batch") return attn_set_tc_min_batch(value);
    return QMM_ERR_UNSUPPORTED;
}

template <int TYPE, int UW, int P, int M, int RB>
static int launch_inst(const MatvecParams& p, int grid, int threads, size_t smem, cudaStream_t stream) {
    auto kern = qmatvec_kernel<TYPE, UW, P, M, RB>;
    static size_t configured[64] = {};  // per instantiation and device; racing writers store the same facts
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

// Instantiated (activation-row tile M, rows per batch RB) pairs: M=1: RB 4, 2, 1; M=2: RB 2, 1; M=4: RB 1.
template <int TYPE, int UW, int P>
static int launch_m(const MatvecParams& p, int grid, int threads, size_t smem, int mtile, int rb, cudaStream_t stream) {
    if (mtile == 1 && rb == 4) return launch_inst<TYPE, UW, P, 1, 4>(p, grid, threads, smem, stream);
    if (mtile == 1 && rb == 2) return launch_inst<TYPE, UW, P, 1, 2>(p, grid, threads, smem, stream);
    if (mtile == 1) return launch_inst<TYPE, UW, P, 1, 1>(p, grid, threads, smem, stream);
    if (mtile == 2 && rb == 2) return launch_inst<TYPE, UW, P, 2, 2>(p, grid, threads, smem, stream);
    if (mtile == 2) return launch_inst<TYPE, UW, P, 2, 1>(p, grid, threads, smem, stream);
    return launch_inst<TYPE, UW, P, 4, 1>(p, grid, threads, smem, stream);
}

template <int TYPE, int UW>
static int launch_p(const MatvecParams& p, int passes, int grid, int threads, size_t smem, int mtile, int rb, cudaStream_t stream) {
    if constexpr (UW == 1) {
        if (passes == 2) return launch_m<TYPE, UW, 2>(p, grid, threads, smem, mtile, rb, stream);
        if (passes == 4) return launch_m<TYPE, UW, 4>(p, grid, threads, smem, mtile, rb, stream);
    }
    return launch_m<TYPE, UW, 1>(p, grid, threads, smem, mtile, rb, stream);
}

int qmatvec_launch_strided(int type, const void* w, const void* xq, float* y, long y_stride, int m, int n, int k, cudaStream_t stream);
int qmatvec_launch_limited(int type, const void* w, const void* xq, float* y, long y_stride, int m, int n, int k, int cta_limit,
                           cudaStream_t stream);
int qmatvec_launch_push(int type, const void* w, const void* xq, float* y, long y_stride, int m, int n, int k, int cta_limit,
                        const TpPush* push, cudaStream_t stream);
int qmatvec_launch_pitched(int type, const void* w, long row_pitch, const void* xq, float* y, long y_stride, int m, int n, int k, int cta_limit,
                           const TpPush* push, cudaStream_t stream);
int qmatvec_launch(int type, const void* w, const void* xq, float* y, int m, int n, int k, cudaStream_t stream) {
    return qmatvec_launch_strided(type, w, xq, y, n, m, n, k, stream);
}

// y_stride: floats between consecutive output rows (lets several projections write slices of one row)
int qmatvec_launch_strided(int type, const void* w, const void* xq, float* y, long y_stride, int m, int n, int k, cudaStream_t stream) {
    return qmatvec_launch_limited(type, w, xq, y, y_stride, m, n, k, 0, stream);
}

// cta_limit > 0: use at most that many CTAs (SMs), so that two independent projections launched on
// two streams share the GPU side by side instead of one after the other
int qmatvec_launch_limited(int type, const void* w, const void* xq, float* y, long y_stride, int m, int n, int k, int cta_limit,
                           cudaStream_t stream) {
    return qmatvec_launch_push(type, w, xq, y, y_stride, m, n, k, cta_limit, nullptr, stream);
}

// push != nullptr (tensor parallel): output (mi, row) goes to slot push->word0 + mi * y_stride + row of every
// rank's exchange area instead of y (y must still be a valid pointer; it is not written)
int qmatvec_launch_push(int type, const void* w, const void* xq, float* y, long y_stride, int m, int n, int k, int cta_limit,
                        const TpPush* push, cudaStream_t stream) {
    return qmatvec_launch_pitched(type, w, 0, xq, y, y_stride, m, n, k, cta_limit, push, stream);
}

// row_pitch: bytes from one weight row to the next (0 = the packed row bytes: rows back to back).  A pitch
// lets a loader pad rows so that each starts on a 16-byte boundary (Q6_K rows of 210 * k/256 bytes do not
// in general), which the tensor-core kernel's tensor copies need; the padding is streamed and ignored.
int qmatvec_launch_pitched(int type, const void* w, long row_pitch, const void* xq, float* y, long y_stride, int m, int n, int k, int cta_limit,
                           const TpPush* push, cudaStream_t stream) {
    if (!w || !xq || !y) return QMM_ERR_NULL;
    if (y_stride < n) return QMM_ERR_SHAPE;
    int block_elems, block_bytes, unit_elems, w_align;
    if (int st = type_geometry(type, block_elems, block_bytes, unit_elems, w_align)) return st;
    if (m <= 0 || n <= 0 || k <= 0 || k % block_elems != 0) return QMM_ERR_SHAPE;
    if (reinterpret_cast<uintptr_t>(w) % w_align != 0 || reinterpret_cast<uintptr_t>(xq) % 4 != 0 ||
        reinterpret_cast<uintptr_t>(y) % 4 != 0)
        return QMM_ERR_ALIGN;

    MatvecParams p = {};
    p.w = static_cast<const uint8_t*>(w);
    p.n = n;
    p.k = k;
    p.row_bytes = k / block_elems * block_bytes;
    if (row_pitch) {
        if (row_pitch < p.row_bytes || row_pitch % 2 != 0 || row_pitch > STAGE_MAX_BYTES) return QMM_ERR_SHAPE;
        p.row_bytes = (int)row_pitch;  // all addressing goes by the pitch; the units of a row come from k
    }
    p.xq_row_bytes = k / QK8 * Q8_1_BYTES;
    p.probe = g_probe;
    p.trace = g_trace ? g_trace + (size_t)(g_trace_count++) * g_trace_stride : nullptr;
    if (p.row_bytes > STAGE_MAX_BYTES) return QMM_ERR_UNSUPPORTED;
    int sms = sm_count() * g_ctas_per_sm;
    if (cta_limit > 0 && cta_limit < sms) sms = cta_limit;
    // Small matrices are all fixed cost per warp (activation loads, set-up): fewer warps per CTA measured
    // 5-12 % faster when a CTA's share of the weights is below ~100 KB (sweeps over the decode shapes).
    int nw = g_consumer_warps;
    if (!g_consumer_warps_set) {
        const long cta_bytes = (long)n * p.row_bytes / sms;
        nw = cta_bytes <= 32 * 1024 ? 8 : (cta_bytes <= 96 * 1024 ? 12 : 16);
    }
    const int rows_per_cta = (n + sms - 1) / sms;
    p.partial_off = (int)((sizeof(MatvecSmemHeader) + 127) & ~size_t(127));
    constexpr size_t SMEM_LIMIT = 200 * 1024;

    // From mma_min_m activation rows on, groups of up to 16 rows go to the tensor-core kernel where it
    // supports the shape; what is left (fewer rows, other types and shapes) takes the dp4a kernel below.
    int m_done = 0;
    // Q4_K rows back to back, from umma_min_m activation rows on: groups of up to 32 rows through the tcgen05 integer kernel.
    // Not for short rows (the column shards of a tensor-parallel O or down projection): its launch has about 6 us of fixed
    // cost, and below 16 super-blocks per row, or for a matrix under 32 M weights (few tiles, K split over clusters), the
    // mma.sync kernel measured as fast or faster (70B batch 32 on 8 GPUs: 2232 against 2118 tok/s).  It takes no CTA
    // limit: a tile of 128 rows per CTA is its grid.
    if (type == QMM_TYPE_Q4_K && !g_probe && umv_min_m() > 0 && k >= umv_min_k() && (long)n * k >= 2l * umv_min_k() * umv_min_k() && (row_pitch == 0 || row_pitch == (long)k / block_elems * block_bytes)) {
        while (m - m_done >= umv_min_m()) {
            const int mg = m - m_done < 32 ? m - m_done : 32;
            TpPush sub = {};
            if (push) sub = *push, sub.word0 += (long)m_done * y_stride;
            const int st = qmatvec_umma_launch(w, static_cast<const uint8_t*>(xq) + (size_t)m_done * p.xq_row_bytes, y + (size_t)m_done * y_stride, y_stride,
                                               mg, n, k, push ? &sub : nullptr, stream);
            if (st == QMM_ERR_UNSUPPORTED) break;
            if (st) return st;
            m_done += mg;
        }
    }
    if (mma_min_m() > 0 && !g_probe) {
        while (m - m_done >= mma_min_m()) {
            const int mg = m - m_done < mma_group_rows() ? m - m_done : mma_group_rows();
            TpPush sub = {};
            if (push) sub = *push, sub.word0 += (long)m_done * y_stride;
            const int st = qmatvec_mma_launch(type, w, row_pitch, static_cast<const uint8_t*>(xq) + (size_t)m_done * p.xq_row_bytes,
                                              y + (size_t)m_done * y_stride, y_stride, mg, n, k, cta_limit, p.trace, push ? &sub : nullptr, stream);
            if (st == QMM_ERR_UNSUPPORTED) break;
            if (st) return st;
            m_done += mg;
        }
    }

    for (int m0 = m_done; m0 < m; m0 += 4) {
        const int left = m - m0;
        const int mt = left >= 3 ? 4 : left;  // register tile of 1, 2 or 4 activation rows
        p.m = left < mt ? left : mt;
        p.xq = static_cast<const uint8_t*>(xq) + (size_t)m0 * p.xq_row_bytes;
        p.y = y + (size_t)m0 * y_stride;
        p.y_stride = y_stride;
        p.push = TpPush{};
        if (push) p.push = *push, p.push.word0 += (long)m0 * y_stride;

        // Q4_K unit width: one 32-byte group per lane measured fastest on every decode shape (wider units
        // decode the packed scales less often but cost registers and occupancy); "q4k_unit" overrides.
        int uw = 1;
        if (type == QMM_TYPE_Q4_K && g_q4k_unit) {
            uw = g_q4k_unit;
            while (uw > 1 && (uw * mt > 4 || k % (64 * uw) != 0)) uw /= 2;
        }
        p.units = k / (unit_elems * uw);
        // K split: the fewest passes that keep the K axis within the consumer warps (passes > 1 only for UW = 1)
        int passes = 1;
        while (passes <= 4 && (p.units + 32 * passes - 1) / (32 * passes) > nw) passes *= 2;
        if (passes > 4 || (passes > 1 && uw > 1)) return QMM_ERR_UNSUPPORTED;
        p.kw = (p.units + 32 * passes - 1) / (32 * passes);
        p.rg = nw / p.kw;

        // rows per batch: as many as instantiated for this M, not beyond what keeps every row group busy
        int rb = mt == 1 ? 4 : (mt == 2 ? 2 : 1);
        if (rb > g_rb_max) rb = g_rb_max;
        while (rb > 1 && (p.rg * rb > rows_per_cta * 2 || rb * p.row_bytes > STAGE_MAX_BYTES)) rb /= 2;
        // rows per stage: whole batches, near the target size, at most a CTA's share
        int batches = g_stage_target / (rb * p.row_bytes);
        if (batches < 1) batches = 1;
        while (batches > 1 && (batches - 1) * rb >= rows_per_cta) --batches;
        p.rows_stage = rb * batches;
        p.slot_bytes = (p.rows_stage * p.row_bytes + 32 + 127) & ~127;
        const int threads = (p.kw * p.rg + 1) * 32;
        int grid = (n + p.rows_stage - 1) / p.rows_stage;
        if (grid > sms) grid = sms;
        p.rows_q = n / grid, p.rows_r = n % grid;
        p.pstage = p.rows_stage * p.kw * mt;
        // stages: as many as the ring budget allows, fewer if the partial sums (two per stage) crowd them out
        const size_t per_stage = (size_t)p.slot_bytes + 2 * (size_t)p.pstage * sizeof(float);
        p.nst = g_ring_budget / p.slot_bytes;
        const int fit = (int)((SMEM_LIMIT - p.partial_off - 256) / per_stage);
        if (p.nst > fit) p.nst = fit;
        if (p.nst > MAX_STAGES) p.nst = MAX_STAGES;
        if (p.nst < 2) {
            if (fit < 2) return QMM_ERR_UNSUPPORTED;
            p.nst = 2;
        }
        const size_t partial_bytes = (size_t)2 * p.nst * p.pstage * sizeof(float);
        p.ring_off = (int)((p.partial_off + partial_bytes + 127) & ~size_t(127));
        const size_t smem = (size_t)p.ring_off + (size_t)p.nst * p.slot_bytes;
        if (smem > SMEM_LIMIT) return QMM_ERR_UNSUPPORTED;
        int st;
        if (type == QMM_TYPE_Q8_0) st = launch_p<QMM_TYPE_Q8_0, 1>(p, passes, grid, threads, smem, mt, rb, stream);
        else if (type == QMM_TYPE_Q6_K) st = launch_p<QMM_TYPE_Q6_K, 1>(p, passes, grid, threads, smem, mt, rb, stream);
        else if (uw == 4) st = launch_p<QMM_TYPE_Q4_K, 4>(p, passes, grid, threads, smem, mt, rb, stream);
        else if (uw == 2) st = launch_p<QMM_TYPE_Q4_K, 2>(p, passes, grid, threads, smem, mt, rb, stream);
        else st = launch_p<QMM_TYPE_Q4_K, 1>(p, passes, grid, threads, smem, mt, rb, stream);
        if (st) return st;
    }
    return QMM_OK;
}

// ------------------------------------------- per-block integer sums (parity)
template <int TYPE>
__global__ void qblock_dots_kernel(const uint8_t* w, const uint8_t* xq, int32_t* out, int n, int units, int row_bytes) {
    using F = Fmt<TYPE, 1>;
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long)n * units) return;
    const int r = (int)(idx / units), u = (int)(idx - (long)r * units);
    typename F::XRegs x;
    F::load_x(xq, u, x);
    typename F::WRegs wr;
    F::load_w(w + (size_t)r * row_bytes, u, wr);
    int sums[4];
    (void)F::dot(wr, u, x, sums);
    int32_t* o = out + ((size_t)r * units + u) * F::SUMS_PER_UNIT;
    if (TYPE == QMM_TYPE_Q6_K) {
        // unit u = (block, half h, l0): run t is scale group 8h + 2t + (u&1) of the block
        int32_t* ob = out + ((size_t)r * units + (u & ~3)) * 4;
        const int h = (u >> 1) & 1;
        for (int t = 0; t < 4; ++t) ob[8 * h + 2 * t + (u & 1)] = sums[t];
    } else {
        for (int t = 0; t < F::SUMS_PER_UNIT; ++t) o[t] = sums[t];
    }
}

int qblock_dots_launch(int type, const void* w, const void* xq, int32_t* out, int n, int k, cudaStream_t stream) {
    if (!w || !xq || !out) return QMM_ERR_NULL;
    int block_elems, block_bytes, unit_elems, w_align;
    if (int st = type_geometry(type, block_elems, block_bytes, unit_elems, w_align)) return st;
    if (n <= 0 || k <= 0 || k % block_elems != 0) return QMM_ERR_SHAPE;
    if (reinterpret_cast<uintptr_t>(w) % w_align != 0 || reinterpret_cast<uintptr_t>(xq) % 4 != 0) return QMM_ERR_ALIGN;
    const int units = k / unit_elems, row_bytes = k / block_elems * block_bytes;
    const long total = (long)n * units;
    const int threads = 128;
    const unsigned grid = (unsigned)((total + threads - 1) / threads);
    const uint8_t* wb = static_cast<const uint8_t*>(w);
    const uint8_t* xb = static_cast<const uint8_t*>(xq);
    switch (type) {
    case QMM_TYPE_Q8_0: qblock_dots_kernel<QMM_TYPE_Q8_0><<<grid, threads, 0, stream>>>(wb, xb, out, n, units, row_bytes); break;
    case QMM_TYPE_Q4_K: qblock_dots_kernel<QMM_TYPE_Q4_K><<<grid, threads, 0, stream>>>(wb, xb, out, n, units, row_bytes); break;
    default: qblock_dots_kernel<QMM_TYPE_Q6_K><<<grid, threads, 0, stream>>>(wb, xb, out, n, units, row_bytes); break;
    }
    QMM_CUDA_TRY(cudaGetLastError());
    return QMM_OK;
}

}  // namespace qmm
