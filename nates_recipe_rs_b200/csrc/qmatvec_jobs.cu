// Job-list decode matvec: ONE launch walks a list of independent projections
//     y_j(m, n_j) = xq_j(m, k_j) . w_j(n_j, k_j)^T        j = 0 .. n_jobs-1
// with persistent CTAs that never leave the SM between matrices.  The upstream issues such
// projections one launch after the other on the same input (q, k, v: examples/gemma4.rs:653-667;
// gate and up: :675-678; the chosen experts' gate_up and down: :726-742); each launch of the
// single-matrix kernel (qmatvec.cu) pays ~2.5 us in which the weight stream stands still (CTA
// start, barrier set-up, first copies in flight, activation loads, tail), which at 33 MB per matrix
// is a third of the time.  Here
//   * the producer warp keeps the ring of bulk copies (cp.async.bulk + mbarrier) full ACROSS job
//     boundaries: while the consumer warps finish job j it is already streaming job j+1;
//   * the Q8_1 activations of the next job are fetched into shared memory by a bulk copy as soon as
//     every warp has taken the current job's activations into registers, so a job starts with a few
//     shared-memory loads instead of a round trip to L2;
//   * the share of rows a CTA owns is rotated from job to job so that the one-row imbalance of
//     n % grid does not pile up on the same CTAs;
//   * a job may select its matrix on the device (w + select[0] * stride): the experts a router
//     picked are streamed without the host ever seeing the choice.
// Everything else is the single-matrix kernel's arithmetic (same Fmt<>::dot, same fixed-order
// fold of the K-split partial sums by the producer warp: reruns are bit identical).
// Restrictions (the launcher falls back to one launch per job otherwise): m <= 2, every
// job's K fits the consumer warps in one pass, xq 16-byte aligned.
#include "qmm_formats.cuh"
#include <string>

namespace qmm {

constexpr int JOBS_MAX = 36;           // jobs per launch (the descriptor array travels as kernel parameter)
constexpr int JOBS_MAX_STAGES = 8;
constexpr int JOBS_MAX_WARPS = 24;     // consumer warps

struct JobDesc {
    const uint8_t* w;
    const uint8_t* xq;
    float* y;
    const int* sel;       // optional: the matrix is w + sel[0] * sel_stride
    long sel_stride;
    int y_stride;         // floats between the output rows of two activation rows
    int n, k, type;
    int row_bytes, xq_row_bytes, units;
    int rows_stage;       // weight rows per ring stage (a multiple of rb)
    int kw, rg, rb;       // warps along K, row groups, rows reduced together
    int rows_q, rows_r;   // n / grid, n % grid
    int rot;              // rotation of the CTA -> row-range assignment (0 <= rot < grid)
    long push_word;       // tensor parallel: slot index of this job's y[0][0] in the exchange areas, or -1: plain stores to y
};

// How the activations of a list are made when the kernel builds them itself (all jobs then share them):
//   JOBS_X_NORM  xq = Q8_1( rmsnorm(x_in + x_add) * gamma ), the sum also written to x_out by CTA 0: the residual
//                update, the norm and the quantization that precede the projections of a block, without a launch
//                of their own (each CTA repeats them for the one row it needs: 2 x hidden floats out of L2)
//   JOBS_X_GLU   xq = Q8_1( act(gate) * up ) from the fused [gate | up] output of the preceding projection
// (XBuild and the mode constants are declared in api.cu, the first file of the translation unit:
//   x_in   NORM: residual (m, k); GLU: gate_up (m, 2k)      x_add  NORM: output of the preceding projection to add, or NULL
//   gamma  NORM: gains, or NULL                              x_out  NORM: where the updated residual goes (not x_in), or NULL)
constexpr int JOBS_X_GLOBAL = 0;

struct JobList {
    JobDesc job[JOBS_MAX];
    int n_jobs, m;
    int nst, slot_bytes, pstage_max;
    int x_off, partial_off, ring_off;
    int n_consumers, any_sel;
    int x_mode;           // JOBS_X_*
    TpPush push;          // used by the jobs with push_word >= 0
    XBuild xb;
};
static_assert(sizeof(JobList) <= 4096, "the job list travels as a kernel parameter");

struct __align__(16) JobsSmemHeader {
    uint64_t full[JOBS_MAX_STAGES];
    uint64_t empty[JOBS_MAX_STAGES];
    uint64_t xfull;
    int abort_flag;
    float red[JOBS_MAX_WARPS];  // sum-of-squares partials of the activation builder
};

// rows of job J owned by CTA bx
__device__ __forceinline__ void job_cta_rows(const JobDesc& J, int bx, int grid, long& row_begin, int& n_rows) {
    int b = bx + J.rot;
    if (b >= grid) b -= grid;
    row_begin = (long)b * J.rows_q + min(b, J.rows_r);
    n_rows = J.rows_q + (b < J.rows_r ? 1 : 0);
}

// position of a CTA in its flattened list of stages
struct JobCursor {
    int j, it, n_it, n_rows;
    long row_begin;
    uintptr_t w_begin;
};

template <int V>
__device__ __forceinline__ void jobs_warp_multi_sum(float (&v)[V], int lane) {
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

// What a consumer warp carries from job to job, and the per-job values it needs, all by value: a
// reference into the parameter block would have to be re-read after every shared-memory store.
struct ConsumerState {
    int slot, pslot;
    uint32_t phase;
    int ok;
};
struct JobArgs {
    int kw, rg, units, row_bytes, xq_row_bytes, rows_stage, n_rows;
    int m, nst, slot_bytes, pstage_max;
    uint32_t w_lo, x_parity;
    int x_wait;   // 0: the activations were built by the kernel itself and are in place
};

// All stages of one job for one consumer warp.  st.ok = 0 after a timeout (the CTA unwinds).
template <int TYPE, int M, int RB>
__device__ __noinline__ ConsumerState consume_job(const JobArgs a, JobsSmemHeader* hdr, uint32_t ring_s, float* partial, const uint8_t* xs,
                                                  int warp, int lane, ConsumerState st, volatile int* cta_abort) {
    using F = Fmt<TYPE, 1>;
    constexpr int V = M * RB;
    const int kw = a.kw, rg = a.rg;
    const bool active = warp < kw * rg;
    const int rgi = active ? warp / kw : rg;
    const int kwi = active ? warp - rgi * kw : 0;
    const int u_raw = kwi * 32 + lane;
    const bool have = active && u_raw < a.units;
    const int unit = have ? u_raw : 0;  // lanes past the end of the row re-read unit 0 against zero activations
    const uint32_t unit_off = F::unit_offset(unit);
    typename F::XRegs x[M];
    // Every warp waits for every job's activations, also one without a share in this job: a warp that
    // skipped a phase of this barrier could not tell the next phase from the one before it.
    if (a.x_wait && !mbar_wait_bounded(smem_u32(&hdr->xfull), a.x_parity, cta_abort)) {
        if (lane == 0 && !*cta_abort) {
            atomicExch(&g_device_status, DEV_TIMEOUT_FULL);
            *cta_abort = 1;
        }
        st.ok = 0;
        return st;
    }
#pragma unroll
    for (int mi = 0; mi < M; ++mi) {
        if (have && mi < a.m)
            F::load_x(xs + (size_t)mi * a.xq_row_bytes, unit, x[mi]);
        else
            F::zero_x(x[mi]);
    }
    constexpr int LANES_PER_VALUE = 32 / V;
    const int my_val = lane / LANES_PER_VALUE, my_j = my_val / M, my_mi = my_val - my_j * M;
    const bool writer = (lane % LANES_PER_VALUE) == 0;
    const uint32_t my_ps = ((uint32_t)my_j * kw + kwi) * M + my_mi;
    const uint32_t row_bytes = (uint32_t)a.row_bytes;
    const uint32_t batch_bytes = (uint32_t)RB * row_bytes;
    const uint32_t batch_ps = (uint32_t)RB * kw * M;
    const uint32_t stage_bytes = (uint32_t)a.rows_stage * row_bytes;
    const int rows_stage = a.rows_stage, n_rows = a.n_rows, nst = a.nst;
    const uint32_t slot_bytes = (uint32_t)a.slot_bytes, pstage_max = (uint32_t)a.pstage_max;
    const int bps = rows_stage / RB;
    int next_b = active ? rgi : 0x3fffffff;  // this warp's next batch, relative to the current stage
    uint32_t head = a.w_lo;                   // low four address bits of the stage's first byte
    const uint32_t full0 = smem_u32(&hdr->full[0]), empty0 = smem_u32(&hdr->empty[0]);
    for (int r_lo = 0; r_lo < n_rows; r_lo += rows_stage) {
        const int nr = min(rows_stage, n_rows - r_lo);
        const int nb = (nr + RB - 1) / RB;
        // Every warp waits for every stage's data, with or without work in it.  The copy of this use of the
        // slot is only issued after all warps released the previous use, so once the data is seen this
        // warp's arrival below lands in the right phase and the parity test cannot be a phase off.
        if (!mbar_wait_bounded(full0 + 8u * st.slot, st.phase, cta_abort)) {
            if (lane == 0 && !*cta_abort) {
                atomicExch(&g_device_status, DEV_TIMEOUT_FULL);
                *cta_abort = 1;
            }
            st.ok = 0;
            return st;
        }
        if (next_b < nb) {
            const uint32_t base = ring_s + (uint32_t)st.slot * slot_bytes + head;
            float* ps = partial + (uint32_t)st.pslot * pstage_max + my_ps;
            // Whole batches only: rows past nr (last stage of the job) hold stale bytes of an earlier stage;
            // their sums land in partial entries that nobody reads.
            for (; next_b < nb; next_b += rg) {
                const uint32_t row0 = base + (uint32_t)next_b * batch_bytes;
                float acc[V];
#pragma unroll
                for (int v = 0; v < V; ++v) acc[v] = 0.f;
#pragma unroll
                for (int j = 0; j < RB; ++j) {
                    typename F::WRegs wr;
                    F::load_w_s(row0 + (uint32_t)j * row_bytes, unit_off, unit, wr);
#pragma unroll
                    for (int mi = 0; mi < M; ++mi) acc[j * M + mi] += F::dot(wr, unit, x[mi], nullptr);
                }
                jobs_warp_multi_sum<V>(acc, lane);
                if (writer) ps[(uint32_t)next_b * batch_ps] = acc[0];
            }
        }
        next_b -= bps;  // renumber relative to the next stage (warps without a share stay far above any nb)
        __syncwarp();
        if (lane == 0) mbar_arrive(empty0 + 8u * st.slot);
        if (++st.slot == nst) st.slot = 0, st.phase ^= 1;
        if (++st.pslot == 2 * nst) st.pslot = 0;
        head = (head + stage_bytes) & 15u;
    }
    return st;
}

template <int TYPE, int M>
__device__ __forceinline__ ConsumerState consume_job_rb(int rb, const JobArgs& a, JobsSmemHeader* hdr, uint32_t ring_s, float* partial,
                                                        const uint8_t* xs, int warp, int lane, ConsumerState st, volatile int* cta_abort) {
    if constexpr (M == 1) {
        if (rb == 4) return consume_job<TYPE, M, 4>(a, hdr, ring_s, partial, xs, warp, lane, st, cta_abort);
    }
    if (rb == 2) return consume_job<TYPE, M, 2>(a, hdr, ring_s, partial, xs, warp, lane, st, cta_abort);
    return consume_job<TYPE, M, 1>(a, hdr, ring_s, partial, xs, warp, lane, st, cta_abort);
}

__device__ __forceinline__ void consumers_sync(int n_threads) { asm volatile("bar.sync 1, %0;" ::"r"(n_threads) : "memory"); }

// One Q8_1 block into shared memory from the 32 values held one per lane (the arithmetic of quantize_q8_kernel).
__device__ __forceinline__ void warp_q8_1_to_smem(float v, uint8_t* blk, int lane) {
    float amax = fabsf(v);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const uint16_t dh = __half_as_ushort(__float2half_rn(fminf(__fdiv_rn(amax, 127.0f), 65504.0f)));
    const float df = f16_bits_to_f32(dh);
    int q = (df > 0.0f) ? (int)roundf(__fdiv_rn(v, df)) : 0;
    q = q < -127 ? -127 : (q > 127 ? 127 : q);
    blk[4 + lane] = (uint8_t)(int8_t)q;
    int sum = q;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    if (lane == 0) {
        *reinterpret_cast<uint16_t*>(blk) = dh;
        *reinterpret_cast<uint16_t*>(blk + 2) = __half_as_ushort(__float2half_rn(__fmul_rn(df, (float)sum)));
    }
}

// The consumer warps of a CTA build the activations of the whole list in the staging area (see XBuild).
// A warp owns whole blocks of 32 consecutive elements (block w, w + n_warps, ...); all of a lane's loads are
// issued before the first use, so the builder costs one round trip to L2, not one per element.
constexpr int XB_MAX_BLOCKS = 20;  // blocks per warp the norm builder keeps in registers (K <= 20 * 32 * warps)
constexpr int XB_GLU_CHUNK = 8;
__device__ __noinline__ void build_activations(const XBuild xb, int mode, int m, uint8_t* xs, float* red, int warp, int lane, int n_warps,
                                               bool writes_residual) {
    const int k = xb.k, n_thr = n_warps * 32, n_blk = k / 32;
    const int xq_row_bytes = n_blk * Q8_1_BYTES;
    for (int mi = 0; mi < m; ++mi) {
        uint8_t* xrow = xs + (size_t)mi * xq_row_bytes;
        if (mode == JOBS_X_NORM) {
            const float* xi = xb.x_in + (size_t)mi * k;
            const float* xa = xb.x_add ? xb.x_add + (size_t)mi * k : nullptr;
            float v[XB_MAX_BLOCKS], a[XB_MAX_BLOCKS], g[XB_MAX_BLOCKS];
#pragma unroll
            for (int j = 0; j < XB_MAX_BLOCKS; ++j) {
                const int blk = warp + j * n_warps;
                const int e = blk * 32 + lane;
                const bool in = blk < n_blk;
                v[j] = in ? xi[e] : 0.f;
                a[j] = (in && xa) ? xa[e] : 0.f;
                g[j] = (in && xb.gamma) ? xb.gamma[e] : 1.f;
            }
            float ss = 0.f;
#pragma unroll
            for (int j = 0; j < XB_MAX_BLOCKS; ++j) {
                v[j] += a[j];
                ss += v[j] * v[j];
            }
            ss = warp_sum(ss);
            consumers_sync(n_thr);  // red[] of the previous row has been read
            if (lane == 0) red[warp] = ss;
            consumers_sync(n_thr);
            float tot = 0.f;
            for (int w = 0; w < n_warps; ++w) tot += red[w];  // fixed order
            const float inv = rsqrtf(tot / (float)k + xb.eps);
#pragma unroll
            for (int j = 0; j < XB_MAX_BLOCKS; ++j) {
                const int blk = warp + j * n_warps;
                if (blk < n_blk) {
                    if (writes_residual && xb.x_out) xb.x_out[(size_t)mi * k + blk * 32 + lane] = v[j];
                    warp_q8_1_to_smem(v[j] * inv * g[j], xrow + (size_t)blk * Q8_1_BYTES, lane);
                }
            }
        } else {
            const float* gu = xb.x_in + (size_t)mi * 2 * k;
            for (int b0 = warp; b0 < n_blk; b0 += n_warps * XB_GLU_CHUNK) {
                float gg[XB_GLU_CHUNK], uu[XB_GLU_CHUNK];
#pragma unroll
                for (int j = 0; j < XB_GLU_CHUNK; ++j) {
                    const int blk = b0 + j * n_warps;
                    gg[j] = blk < n_blk ? gu[blk * 32 + lane] : 0.f;
                    uu[j] = blk < n_blk ? gu[k + blk * 32 + lane] : 0.f;
                }
#pragma unroll
                for (int j = 0; j < XB_GLU_CHUNK; ++j) {
                    const int blk = b0 + j * n_warps;
                    if (blk < n_blk) {
                        const float gv = gg[j];
                        const float av = xb.act == 0 ? 0.5f * gv * (1.0f + tanhf(0.7978845608028654f * (gv + 0.044715f * gv * gv * gv)))
                                                      : gv / (1.0f + __expf(-gv));
                        warp_q8_1_to_smem(av * uu[j], xrow + (size_t)blk * Q8_1_BYTES, lane);
                    }
                }
            }
        }
    }
    consumers_sync(n_thr);  // every block of the staging area is written
}

template <int M>
__global__ void __launch_bounds__((JOBS_MAX_WARPS + 1) * 32, 1) qmatvec_jobs_kernel(const __grid_constant__ JobList L) {
    extern __shared__ __align__(128) uint8_t smem[];
    JobsSmemHeader* hdr = reinterpret_cast<JobsSmemHeader*>(smem);
    uint8_t* xs = smem + L.x_off;
    float* partial = reinterpret_cast<float*>(smem + L.partial_off);
    uint8_t* ring = smem + L.ring_off;
    volatile int* cta_abort = &hdr->abort_flag;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int bx = (int)blockIdx.x, grid = (int)gridDim.x;

    if (threadIdx.x == 0) {
        for (int s = 0; s < L.nst; ++s) {
            mbar_init(smem_u32(&hdr->full[s]), 1);
            mbar_init(smem_u32(&hdr->empty[s]), L.n_consumers);
        }
        mbar_init(smem_u32(&hdr->xfull), 1);
        hdr->abort_flag = 0;
        mbar_fence_init();
    }
    __syncthreads();
    pdl_release_dependents();

    if (warp == L.n_consumers) {
        // ------------------------------------------------------------ producer
        // (all lanes keep the cursors; lane 0 issues the copies, the warp folds together)
        auto enter_job = [&](JobCursor& c) {  // skips jobs in which this CTA owns no row
            while (c.j < L.n_jobs) {
                const JobDesc& J = L.job[c.j];
                job_cta_rows(J, bx, grid, c.row_begin, c.n_rows);
                if (c.n_rows > 0) {
                    uintptr_t wb = reinterpret_cast<uintptr_t>(J.w);
                    if (J.sel) wb += (size_t)((long)__ldg(J.sel) * J.sel_stride);
                    c.w_begin = wb + (size_t)c.row_begin * J.row_bytes;
                    c.n_it = (c.n_rows + J.rows_stage - 1) / J.rows_stage;
                    c.it = 0;
                    return;
                }
                ++c.j;
            }
        };
        auto advance = [&](JobCursor& c) {
            if (++c.it >= c.n_it) {
                ++c.j;
                enter_job(c);
            }
        };
        auto issue = [&](const JobCursor& c, int slot) {
            const JobDesc& J = L.job[c.j];
            const int nr = min(J.rows_stage, c.n_rows - c.it * J.rows_stage);
            const uintptr_t g = c.w_begin + (size_t)c.it * J.rows_stage * J.row_bytes;
            const uint32_t head = (uint32_t)(g & 15);
            const uint32_t bytes = (head + (uint32_t)nr * J.row_bytes + 15u) & ~15u;
            const uint32_t bar = smem_u32(&hdr->full[slot]);
            mbar_arrive_expect_tx(bar, bytes);
            bulk_g2s(smem_u32(ring + (size_t)slot * L.slot_bytes), reinterpret_cast<const void*>(g - head), bytes, bar);
        };
        auto issue_x = [&](int j) {
            const JobDesc& J = L.job[j];
            const uint32_t bytes = (uint32_t)L.m * J.xq_row_bytes;
            const uint32_t bar = smem_u32(&hdr->xfull);
            mbar_arrive_expect_tx(bar, bytes);
            bulk_g2s(smem_u32(xs), J.xq, bytes, bar);
        };
        if (L.any_sel) pdl_wait_prior_grids();  // a selector comes from the preceding kernel
        JobCursor is = {}, fo = {};
        enter_job(is);
        fo = is;
        int issued = 0;  // stages issued so far
        for (; issued < L.nst && is.j < L.n_jobs; ++issued) {
            if (lane == 0) issue(is, issued);
            advance(is);
        }
        if (!L.any_sel) pdl_wait_prior_grids();  // activations come from the preceding kernel, y may still be read by it
        const unsigned push_seq = L.push.tp > 0 ? tp_next_seq(L.push.counter) : 0u;
        int x_issued = 0;  // activation copies issued
        const bool copies_x = L.x_mode == JOBS_X_GLOBAL;
        if (copies_x && fo.j < L.n_jobs) {
            if (lane == 0) issue_x(fo.j);
            x_issued = 1;
        }
        bool ok = true;
        int slot = 0, pslot = 0;
        uint32_t phase = 0;
        while (fo.j < L.n_jobs) {
            ok = mbar_wait_bounded(smem_u32(&hdr->empty[slot]), phase, cta_abort);
            if (!ok) {
                if (lane == 0 && !*cta_abort) {
                    atomicExch(&g_device_status, DEV_TIMEOUT_EMPTY);
                    *cta_abort = 1;
                }
                break;
            }
            const JobDesc& J = L.job[fo.j];
            if (copies_x && fo.it == 0) {
                // every warp holds this job's activations in registers: the staging area is free for the next job's
                JobCursor nx = fo;
                nx.it = nx.n_it;  // step to the next job in which this CTA owns rows
                advance(nx);
                if (nx.j < L.n_jobs) {
                    if (lane == 0) issue_x(nx.j);
                    ++x_issued;
                }
            }
            if (is.j < L.n_jobs) {
                if (lane == 0) issue(is, slot);
                advance(is);
                ++issued;
            }
            // fold the K-split partial sums of this stage in a fixed order
            const int nr = min(J.rows_stage, fo.n_rows - fo.it * J.rows_stage);
            const float* ps = partial + (size_t)pslot * L.pstage_max;
            const long yrow = fo.row_begin + (long)fo.it * J.rows_stage;
            const int kwj = J.kw, ysj = J.y_stride, mj = L.m;
            float* const yj = J.y;
            const long pw = J.push_word;
            for (int idx = lane; idx < nr * M; idx += 32) {  // idx = r*M + mi
                const int r = idx / M, mi = idx - r * M;
                const float* src = ps + (size_t)r * kwj * M + mi;
                float acc = 0.f;
                for (int q = 0; q < kwj; ++q) acc += src[q * M];
                if (mi < mj) {
                    if (pw >= 0)
                        tp_push_word(L.push, push_seq, pw + (long)mi * ysj + yrow + r, acc);
                    else
                        yj[(size_t)mi * ysj + yrow + r] = acc;
                }
            }
            advance(fo);
            if (++slot == L.nst) slot = 0, phase ^= 1;
            if (++pslot == 2 * L.nst) pslot = 0;
        }
        if (!ok && lane == 0) {
            // wait (bounded) for copies still in flight before the CTA's shared memory is released
            const int first = issued > L.nst ? issued - L.nst : 0;
            for (int s = first; s < issued; ++s) {
                const long long t0 = clock64();
                while (!mbar_try_wait(smem_u32(&hdr->full[s % L.nst]), (s / L.nst) & 1)) {
                    if (clock64() - t0 > WAIT_LIMIT_CYCLES) {
                        atomicExch(&g_device_status, DEV_TIMEOUT_DRAIN);
                        break;
                    }
                }
            }
            if (x_issued > 0) {
                const long long t0 = clock64();
                while (!mbar_try_wait(smem_u32(&hdr->xfull), (x_issued - 1) & 1)) {
                    if (clock64() - t0 > WAIT_LIMIT_CYCLES) {
                        atomicExch(&g_device_status, DEV_TIMEOUT_DRAIN);
                        break;
                    }
                }
            }
        }
        return;
    }
    if (warp > L.n_consumers) return;

    // ---------------------------------------------------------------- consumers
    const uint32_t ring_s = smem_u32(ring);
    ConsumerState st = {0, 0, 0u, 1};
    uint32_t x_parity = 0;
    if (L.x_mode != JOBS_X_GLOBAL) {
        pdl_wait_prior_grids();  // the inputs of the builder come from the preceding kernel
        build_activations(L.xb, L.x_mode, L.m, xs, hdr->red, warp, lane, L.n_consumers, bx == 0);
    }
    for (int j = 0; j < L.n_jobs; ++j) {
        const JobDesc& J = L.job[j];
        long row_begin;
        int n_rows;
        job_cta_rows(J, bx, grid, row_begin, n_rows);
        if (n_rows <= 0) continue;
        JobArgs a;
        a.kw = J.kw, a.rg = J.rg, a.units = J.units, a.row_bytes = J.row_bytes, a.xq_row_bytes = J.xq_row_bytes;
        a.rows_stage = J.rows_stage, a.n_rows = n_rows;
        a.m = L.m, a.nst = L.nst, a.slot_bytes = L.slot_bytes, a.pstage_max = L.pstage_max;
        // low address bits of this CTA's first row (a selector moves the matrix by a multiple of 16 bytes)
        a.w_lo = (uint32_t)((reinterpret_cast<uintptr_t>(J.w) + (size_t)row_begin * J.row_bytes) & 15);
        a.x_parity = x_parity;
        a.x_wait = L.x_mode == JOBS_X_GLOBAL;
        const int type = J.type, rb = J.rb;
        if (type == QMM_TYPE_Q4_K)
            st = consume_job_rb<QMM_TYPE_Q4_K, M>(rb, a, hdr, ring_s, partial, xs, warp, lane, st, cta_abort);
        else if (type == QMM_TYPE_Q6_K)
            st = consume_job_rb<QMM_TYPE_Q6_K, M>(rb, a, hdr, ring_s, partial, xs, warp, lane, st, cta_abort);
        else
            st = consume_job_rb<QMM_TYPE_Q8_0, M>(rb, a, hdr, ring_s, partial, xs, warp, lane, st, cta_abort);
        if (!st.ok) return;
        x_parity ^= 1;
    }
}

// ------------------------------------------------------------------- host side
int qmatvec_launch_strided(int type, const void* w, const void* xq, float* y, long y_stride, int m, int n, int k, cudaStream_t stream);

static int g_jobs_warps = 14;
static int g_jobs_ring = 150 * 1024;
static int g_jobs_stage = 48 * 1024;
static int g_jobs_rotate = 1;
// decode engine at batch <= 2 on one GPU (default 0: every operator its own launch): 1 = Q|K and V as one job list; 2 = also the norms built inside the matvec
// launches; 3 = also the gated activation (all three measured slower than the separate launches: 2 and 3 repeat the small operator in every CTA;
// kept for experiments)
static int g_decoder_fuse = 0;
int decoder_fusion() { return g_decoder_fuse; }
int jobs_tune(const char* key, int value) {
    const std::string k(key ? key : "");
    if (k == "jobs_warps" && value >= 1 && value <= JOBS_MAX_WARPS) return g_jobs_warps = value, QMM_OK;
    if (k == "jobs_ring_bytes" && value >= 8 * 1024 && value <= 190 * 1024) return g_jobs_ring = value, QMM_OK;
    if (k == "jobs_stage_bytes" && value >= 1024 && value <= 48 * 1024) return g_jobs_stage = value, QMM_OK;
    if (k == "jobs_rotate" && (value == 0 || value == 1)) return g_jobs_rotate = value, QMM_OK;
    if (k == "decoder_fuse" && value >= 0 && value <= 3) return g_decoder_fuse = value, QMM_OK;
    return QMM_ERR_UNSUPPORTED;
}

template <int M>
static int jobs_launch_inst(const JobList& L, int grid, size_t smem, cudaStream_t stream) {
    auto kern = qmatvec_jobs_kernel<M>;
    static size_t configured[64] = {};  // per instantiation and device; racing writers store the same facts
    int dev = 0;
    QMM_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || smem > configured[dev]) {
        QMM_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        if (dev >= 0 && dev < 64) configured[dev] = smem;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3((L.n_consumers + 1) * 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = overlap_enabled() ? 1 : 0;
    QMM_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, L));
    return QMM_OK;
}

static int job_geometry(int type, int& block_elems, int& block_bytes, int& w_align) {
    switch (type) {
    case QMM_TYPE_Q8_0: block_elems = 32, block_bytes = Q8_0_BYTES, w_align = 2; return QMM_OK;
    case QMM_TYPE_Q4_K: block_elems = 256, block_bytes = Q4_K_BYTES, w_align = 16; return QMM_OK;
    case QMM_TYPE_Q6_K: block_elems = 256, block_bytes = Q6_K_BYTES, w_align = 2; return QMM_OK;
    }
    return QMM_ERR_TYPE;
}

// Validates the jobs, then launches them in groups of up to JOBS_MAX.  Shapes the persistent kernel does
// not take (see the head of this file) run as one single-matrix launch per job instead; a job with a
// device-side selector has no such fallback and is rejected with QMM_ERR_UNSUPPORTED.
int qmatvec_jobs_launch_ex(const qmm_matvec_job* jobs, int n_jobs, int m, const TpPush* push, const long* push_words, int x_mode,
                           const XBuild* xb, cudaStream_t stream);
int qmatvec_jobs_launch_push(const qmm_matvec_job* jobs, int n_jobs, int m, const TpPush* push, const long* push_words, cudaStream_t stream) {
    return qmatvec_jobs_launch_ex(jobs, n_jobs, m, push, push_words, JOBS_X_GLOBAL, nullptr, stream);
}
int qmatvec_jobs_launch(const qmm_matvec_job* jobs, int n_jobs, int m, cudaStream_t stream) {
    return qmatvec_jobs_launch_ex(jobs, n_jobs, m, nullptr, nullptr, JOBS_X_GLOBAL, nullptr, stream);
}

// push / push_words (tensor parallel, both or neither): job i with push_words[i] >= 0 sends its outputs to slot
// push_words[i] + mi * y_stride + row of every rank's exchange area instead of storing them to its y.  Such a
// list has no per-job fallback: QMM_ERR_UNSUPPORTED when it does not fit the persistent kernel.
// x_mode != JOBS_X_GLOBAL: the kernel builds the activations itself (xb; every job must have K = xb->k, the
// jobs' xq pointers are not used); such a list has no fallback either and must fit one launch.
int qmatvec_jobs_launch_ex(const qmm_matvec_job* jobs, int n_jobs, int m, const TpPush* push, const long* push_words, int x_mode,
                           const XBuild* xb, cudaStream_t stream) {
    if (!jobs) return QMM_ERR_NULL;
    const bool builds = x_mode != JOBS_X_GLOBAL;
    if (builds && (!xb || !xb->x_in)) return QMM_ERR_NULL;
    if (builds && (n_jobs > JOBS_MAX || xb->k % 32 != 0)) return QMM_ERR_UNSUPPORTED;
    if (x_mode == JOBS_X_NORM && xb->k > XB_MAX_BLOCKS * 32 * g_jobs_warps) return QMM_ERR_UNSUPPORTED;
    if (n_jobs <= 0 || m <= 0) return QMM_ERR_SHAPE;
    const int sms = sm_count();
    const int nw = g_jobs_warps;
    bool fits = m <= 2;
    bool any_sel = false;
    for (int i = 0; i < n_jobs; ++i) {
        const qmm_matvec_job& q = jobs[i];
        if (!q.w || (!q.xq && !builds) || !q.y) return QMM_ERR_NULL;
        if (builds && q.k != xb->k) return QMM_ERR_SHAPE;
        int be, bb, wa;
        if (int st = job_geometry(q.type, be, bb, wa)) return st;
        if (q.n <= 0 || q.k <= 0 || q.k % be != 0) return QMM_ERR_SHAPE;
        const long ys = q.y_stride ? q.y_stride : q.n;
        if (ys < q.n || ys > 0x7fffffffl) return QMM_ERR_SHAPE;
        if (reinterpret_cast<uintptr_t>(q.w) % wa != 0 || (!builds && reinterpret_cast<uintptr_t>(q.xq) % 4 != 0) ||
            reinterpret_cast<uintptr_t>(q.y) % 4 != 0)
            return QMM_ERR_ALIGN;
        const long row_bytes = (long)q.k / be * bb;
        if (row_bytes > 48 * 1024) return QMM_ERR_UNSUPPORTED;
        if (q.select) {
            any_sel = true;
            if (q.select_stride_bytes % 16 != 0 || reinterpret_cast<uintptr_t>(q.select) % 4 != 0) return QMM_ERR_ALIGN;
        }
        const int xq_row = q.k / QK8 * Q8_1_BYTES;
        const int units = q.k / (q.type == QMM_TYPE_Q8_0 ? 32 : 64);
        if ((!builds && (reinterpret_cast<uintptr_t>(q.xq) % 16 != 0 || ((long)m * xq_row) % 16 != 0)) || (units + 31) / 32 > nw ||
            (long)m * xq_row > 64 * 1024)
            fits = false;
    }
    if (!fits) {
        if (any_sel || push || builds) return QMM_ERR_UNSUPPORTED;
        for (int i = 0; i < n_jobs; ++i) {
            const qmm_matvec_job& q = jobs[i];
            if (int st = qmatvec_launch_strided(q.type, q.w, q.xq, q.y, q.y_stride ? q.y_stride : q.n, m, q.n, q.k, stream)) return st;
        }
        return QMM_OK;
    }
    const int mt = m;  // register tile = activation rows (1 or 2)
    for (int j0 = 0; j0 < n_jobs; j0 += JOBS_MAX) {
        const int nj = n_jobs - j0 < JOBS_MAX ? n_jobs - j0 : JOBS_MAX;
        JobList L = {};
        L.n_jobs = nj;
        L.m = m;
        L.n_consumers = nw;
        L.any_sel = 0;
        if (push) L.push = *push;
        L.x_mode = x_mode;
        if (builds) L.xb = *xb;
        int slot_max = 0, pstage_max = 0, x_max = 0;
        for (int i = 0; i < nj; ++i) {
            const qmm_matvec_job& q = jobs[j0 + i];
            JobDesc& J = L.job[i];
            int be, bb, wa;
            job_geometry(q.type, be, bb, wa);
            J.w = static_cast<const uint8_t*>(q.w);
            J.xq = static_cast<const uint8_t*>(q.xq);
            J.y = q.y;
            J.sel = q.select;
            J.sel_stride = q.select_stride_bytes;
            if (q.select) L.any_sel = 1;
            J.y_stride = (int)(q.y_stride ? q.y_stride : q.n);
            J.n = q.n, J.k = q.k, J.type = q.type;
            J.row_bytes = q.k / be * bb;
            J.xq_row_bytes = q.k / QK8 * Q8_1_BYTES;
            J.units = q.k / (q.type == QMM_TYPE_Q8_0 ? 32 : 64);
            J.kw = (J.units + 31) / 32;
            J.rg = nw / J.kw;
            const int rows_per_cta = (q.n + sms - 1) / sms;
            int rb = mt == 1 ? 4 : 2;
            while (rb > 1 && (J.rg * rb > rows_per_cta * 2 || rb * J.row_bytes > g_jobs_stage)) rb /= 2;
            J.rb = rb;
            int batches = g_jobs_stage / (rb * J.row_bytes);
            if (batches < 1) batches = 1;
            while (batches > 1 && (batches - 1) * rb >= rows_per_cta) --batches;
            J.rows_stage = rb * batches;
            J.rows_q = q.n / sms, J.rows_r = q.n % sms;
            J.rot = g_jobs_rotate ? (int)(((long)(j0 + i) * 61) % sms) : 0;
            J.push_word = (push && push_words) ? push_words[j0 + i] : -1;
            const int slot = (J.rows_stage * J.row_bytes + 32 + 127) & ~127;
            const int pst = J.rows_stage * J.kw * mt;
            const int xb = (m * J.xq_row_bytes + 127) & ~127;
            if (slot > slot_max) slot_max = slot;
            if (pst > pstage_max) pstage_max = pst;
            if (xb > x_max) x_max = xb;
        }
        constexpr size_t SMEM_LIMIT = 200 * 1024;
        L.slot_bytes = slot_max;
        L.pstage_max = pstage_max;
        L.x_off = (int)((sizeof(JobsSmemHeader) + 127) & ~size_t(127));
        L.partial_off = L.x_off + x_max;
        int nst = g_jobs_ring / slot_max;
        if (nst > JOBS_MAX_STAGES) nst = JOBS_MAX_STAGES;
        for (;; --nst) {
            if (nst < 2) return QMM_ERR_UNSUPPORTED;
            const size_t partial_bytes = (size_t)2 * nst * pstage_max * sizeof(float);
            L.ring_off = (int)((L.partial_off + partial_bytes + 127) & ~size_t(127));
            if ((size_t)L.ring_off + (size_t)nst * slot_max <= SMEM_LIMIT) break;
        }
        L.nst = nst;
        const size_t smem = (size_t)L.ring_off + (size_t)nst * slot_max;
        const int st = mt == 1 ? jobs_launch_inst<1>(L, sms, smem, stream) : jobs_launch_inst<2>(L, sms, smem, stream);
        if (st) return st;
    }
    return QMM_OK;
}

}  // namespace qmm
