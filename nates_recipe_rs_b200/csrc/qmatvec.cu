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
//   * each lane unpacks its slice of a row with a handful of logic ops and
//     accumulates with dp4a; a row's KW partial sums are combined in a fixed
//     order by the producer warp, which is idle between copies (no atomics:
//     reruns are bit-identical, the upstream's determinism rule,
//     gpu-core/src/kernels/gemm_f64.hip:12);
//   * with programmatic dependent launch the next kernel's weight stream starts
//     while this one drains; only activations and outputs wait for the
//     predecessor.
#include "qmm_formats.cuh"

namespace qmm {

struct MatvecParams {
    const uint8_t* w;
    const uint8_t* xq;
    float* y;
    int m;           // activation rows in this launch (<= M of the instantiation)
    int n, k;
    int row_bytes;   // packed bytes of one weight row
    int xq_row_bytes;
    int units;       // k / UNIT_ELEMS
    int kw;          // warps along K
    int rg;          // row groups (warps along rows)
    int rows_stage;  // rows per stage
    int nst;         // stages in the ring
    int slot_bytes;  // bytes per ring slot (128-aligned, >= rows_stage*row_bytes + 32)
    int partial_off; // byte offset of the partial-sum area in dynamic shared memory
    int ring_off;    // byte offset of the ring
};

constexpr int MAX_STAGES = 8;
constexpr int MAX_CONSUMER_WARPS = 16;

struct __align__(16) MatvecSmemHeader {
    uint64_t full[MAX_STAGES];
    uint64_t empty[MAX_STAGES];
    int abort_flag;
};

template <int TYPE, int P, int M>
__global__ void __launch_bounds__((MAX_CONSUMER_WARPS + 1) * 32, 1) qmatvec_kernel(const MatvecParams p) {
    using F = Fmt<TYPE>;
    extern __shared__ __align__(128) uint8_t smem[];
    MatvecSmemHeader* hdr = reinterpret_cast<MatvecSmemHeader*>(smem);
    float* partial = reinterpret_cast<float*>(smem + p.partial_off);
    uint8_t* ring = smem + p.ring_off;
    volatile int* cta_abort = &hdr->abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_consumers = p.kw * p.rg;

    // contiguous row range of this CTA
    const long row_begin = (long)blockIdx.x * p.n / gridDim.x;
    const long row_end = (long)(blockIdx.x + 1) * p.n / gridDim.x;
    const int n_rows = (int)(row_end - row_begin);
    const int n_it = (n_rows + p.rows_stage - 1) / p.rows_stage;

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

    if (warp == n_consumers) {
        // ------------------------------------------------------------ producer
        auto issue = [&](int it) {
            const int slot = it % p.nst;
            const long r0 = row_begin + (long)it * p.rows_stage;
            const int nr = min(p.rows_stage, (int)(row_end - r0));
            const uintptr_t g = reinterpret_cast<uintptr_t>(p.w) + (size_t)r0 * p.row_bytes;
            const uint32_t head = (uint32_t)(g & 15);
            const uint32_t bytes = (head + (uint32_t)nr * p.row_bytes + 15u) & ~15u;
            const uint32_t bar = smem_u32(&hdr->full[slot]);
            mbar_arrive_expect_tx(bar, bytes);
            bulk_g2s(smem_u32(ring + (size_t)slot * p.slot_bytes), reinterpret_cast<const void*>(g - head), bytes, bar);
        };
        int issued = 0;
        if (lane == 0)
            for (; issued < n_it && issued < p.nst; ++issued) issue(issued);
        issued = __shfl_sync(0xffffffffu, issued, 0);
        pdl_wait_prior_grids();  // y may still be read by the preceding kernel
        bool ok = true;
        for (int it = 0; it < n_it; ++it) {
            const int slot = it % p.nst;
            ok = mbar_wait_bounded(smem_u32(&hdr->empty[slot]), (it / p.nst) & 1, cta_abort);
            if (!ok) {
                if (lane == 0 && !*cta_abort) {
                    atomicExch(&g_device_status, DEV_TIMEOUT_EMPTY);
                    *cta_abort = 1;
                }
                break;
            }
            const long r0 = row_begin + (long)it * p.rows_stage;
            const int nr = min(p.rows_stage, (int)(row_end - r0));
            const float* ps = partial + (size_t)slot * p.rows_stage * p.kw * M;
            for (int idx = lane; idx < nr * M; idx += 32) {
                const int r = idx / M, mi = idx - r * M;
                float acc = 0.f;
                for (int q = 0; q < p.kw; ++q) acc += ps[(r * p.kw + q) * M + mi];
                if (mi < p.m) p.y[(size_t)mi * p.n + r0 + r] = acc;
            }
            __syncwarp();
            if (lane == 0 && it + p.nst < n_it) {
                issue(it + p.nst);
                issued = it + p.nst + 1;
            }
        }
        if (!ok && lane == 0) {
            // wait (bounded) for copies still in flight before the CTA's shared memory is released
            issued = max(issued, min(n_it, p.nst));
            for (int it = max(0, issued - p.nst); it < issued; ++it) {
                const uint64_t t0 = globaltimer_ns();
                while (!mbar_try_wait(smem_u32(&hdr->full[it % p.nst]), (it / p.nst) & 1)) {
                    if (globaltimer_ns() - t0 > WAIT_LIMIT_NS) {
                        atomicExch(&g_device_status, DEV_TIMEOUT_DRAIN);
                        break;
                    }
                }
            }
        }
        return;
    }
    if (warp > n_consumers) return;

    // ---------------------------------------------------------------- consumers
    const int kwi = warp % p.kw, rgi = warp / p.kw;
    XRegs x[M][P];
    int unit[P];
    pdl_wait_prior_grids();  // activations come from the preceding kernel
#pragma unroll
    for (int pp = 0; pp < P; ++pp) {
        unit[pp] = (pp * p.kw + kwi) * 32 + lane;
#pragma unroll
        for (int mi = 0; mi < M; ++mi) {
            if (unit[pp] < p.units && mi < p.m)
                F::load_x(p.xq + (size_t)mi * p.xq_row_bytes, unit[pp], x[mi][pp]);
            else
                F::zero_x(x[mi][pp]);
        }
    }

    for (int it = 0; it < n_it; ++it) {
        const int slot = it % p.nst;
        if (!mbar_wait_bounded(smem_u32(&hdr->full[slot]), (it / p.nst) & 1, cta_abort)) {
            if (lane == 0 && !*cta_abort) {
                atomicExch(&g_device_status, DEV_TIMEOUT_FULL);
                *cta_abort = 1;
            }
            return;
        }
        const long r0 = row_begin + (long)it * p.rows_stage;
        const int nr = min(p.rows_stage, (int)(row_end - r0));
        const uint32_t head = (uint32_t)((reinterpret_cast<uintptr_t>(p.w) + (size_t)r0 * p.row_bytes) & 15);
        const uint8_t* base = ring + (size_t)slot * p.slot_bytes + head;
        float* ps = partial + (size_t)slot * p.rows_stage * p.kw * M;
        for (int r = rgi; r < nr; r += p.rg) {
            const uint8_t* row = base + (size_t)r * p.row_bytes;
            float acc[M];
#pragma unroll
            for (int mi = 0; mi < M; ++mi) acc[mi] = 0.f;
#pragma unroll
            for (int pp = 0; pp < P; ++pp) {
                if (unit[pp] < p.units) {
                    typename F::WRegs wr;
                    F::load_w(row, unit[pp], wr);
#pragma unroll
                    for (int mi = 0; mi < M; ++mi) acc[mi] += F::dot(wr, unit[pp], x[mi][pp], nullptr);
                }
            }
#pragma unroll
            for (int mi = 0; mi < M; ++mi) {
                const float v = warp_sum(acc[mi]);
                if (lane == 0) ps[(r * p.kw + kwi) * M + mi] = v;
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&hdr->empty[slot]));
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

constexpr int STAGE_TARGET_BYTES = 18 * 1024;  // preferred bytes per stage
constexpr int STAGE_MAX_BYTES = 48 * 1024;     // one packed row must fit this
constexpr int RING_BUDGET_BYTES = 100 * 1024;  // ring size that still lets two CTAs share an SM

template <int TYPE, int P, int M>
static int launch_inst(const MatvecParams& p, int grid, int threads, size_t smem, cudaStream_t stream) {
    auto kern = qmatvec_kernel<TYPE, P, M>;
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

template <int TYPE, int P>
static int launch_m(const MatvecParams& p, int grid, int threads, size_t smem, int mtile, cudaStream_t stream) {
    switch (mtile) {
    case 1: return launch_inst<TYPE, P, 1>(p, grid, threads, smem, stream);
    case 2: return launch_inst<TYPE, P, 2>(p, grid, threads, smem, stream);
    default: return launch_inst<TYPE, P, 4>(p, grid, threads, smem, stream);
    }
}

template <int TYPE>
static int launch_p(const MatvecParams& p, int passes, int grid, int threads, size_t smem, int mtile, cudaStream_t stream) {
    switch (passes) {
    case 1: return launch_m<TYPE, 1>(p, grid, threads, smem, mtile, stream);
    case 2: return launch_m<TYPE, 2>(p, grid, threads, smem, mtile, stream);
    default: return launch_m<TYPE, 4>(p, grid, threads, smem, mtile, stream);
    }
}

int qmatvec_launch(int type, const void* w, const void* xq, float* y, int m, int n, int k, cudaStream_t stream) {
    if (!w || !xq || !y) return QMM_ERR_NULL;
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
    p.xq_row_bytes = k / QK8 * Q8_1_BYTES;
    p.units = k / unit_elems;
    if (p.row_bytes > STAGE_MAX_BYTES) return QMM_ERR_UNSUPPORTED;

    // K split: the fewest passes that keep the K axis within MAX_CONSUMER_WARPS warps
    int passes = 1;
    while (passes <= 4 && (p.units + 32 * passes - 1) / (32 * passes) > MAX_CONSUMER_WARPS) passes *= 2;
    if (passes > 4) return QMM_ERR_UNSUPPORTED;
    p.kw = (p.units + 32 * passes - 1) / (32 * passes);
    p.rg = MAX_CONSUMER_WARPS / p.kw;
    const int sms = sm_count();
    // rows per stage: a multiple of the row groups, near the target size, never more than a CTA's share
    const int rows_per_cta = (n + sms - 1) / sms;
    int per_group = STAGE_TARGET_BYTES / (p.rg * p.row_bytes);
    if (per_group < 1) per_group = 1;
    p.rows_stage = p.rg * per_group;
    while (p.rows_stage > p.rg && p.rows_stage - p.rg >= rows_per_cta) p.rows_stage -= p.rg;
    while (p.rows_stage > 1 && p.rows_stage * p.row_bytes > STAGE_MAX_BYTES) --p.rows_stage;
    p.slot_bytes = (p.rows_stage * p.row_bytes + 32 + 127) & ~127;
    p.nst = RING_BUDGET_BYTES / p.slot_bytes;
    if (p.nst < 2) p.nst = 2;
    if (p.nst > MAX_STAGES) p.nst = MAX_STAGES;
    const int threads = (p.kw * p.rg + 1) * 32;
    int grid = (n + p.rows_stage - 1) / p.rows_stage;
    if (grid > sms) grid = sms;

    for (int m0 = 0; m0 < m; m0 += 4) {
        const int left = m - m0;
        const int mt = left >= 3 ? 4 : left;  // register tile of 1, 2 or 4 activation rows
        p.m = left < mt ? left : mt;
        p.xq = static_cast<const uint8_t*>(xq) + (size_t)m0 * p.xq_row_bytes;
        p.y = y + (size_t)m0 * n;
        p.partial_off = (int)((sizeof(MatvecSmemHeader) + 127) & ~size_t(127));
        const size_t partial_bytes = (size_t)p.nst * p.rows_stage * p.kw * mt * sizeof(float);
        p.ring_off = (int)((p.partial_off + partial_bytes + 127) & ~size_t(127));
        const size_t smem = (size_t)p.ring_off + (size_t)p.nst * p.slot_bytes;
        if (smem > 200 * 1024) return QMM_ERR_UNSUPPORTED;
        int st;
        switch (type) {
        case QMM_TYPE_Q8_0: st = launch_p<QMM_TYPE_Q8_0>(p, passes, grid, threads, smem, mt, stream); break;
        case QMM_TYPE_Q4_K: st = launch_p<QMM_TYPE_Q4_K>(p, passes, grid, threads, smem, mt, stream); break;
        default: st = launch_p<QMM_TYPE_Q6_K>(p, passes, grid, threads, smem, mt, stream); break;
        }
        if (st) return st;
    }
    return QMM_OK;
}

// ------------------------------------------- per-block integer sums (parity)
template <int TYPE>
__global__ void qblock_dots_kernel(const uint8_t* w, const uint8_t* xq, int32_t* out, int n, int units, int row_bytes) {
    using F = Fmt<TYPE>;
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long)n * units) return;
    const int r = (int)(idx / units), u = (int)(idx - (long)r * units);
    XRegs x;
    F::zero_x(x);
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
