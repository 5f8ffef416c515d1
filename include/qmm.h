/*
 * qmm.h — C ABI of libqmm: GGUF-block quantized matmul for NVIDIA B200 (sm_100a).
 *
 * This is the boundary a host program binds (Rust `unsafe extern "C"`, ctypes,
 * cgo ...).  It follows the launcher convention of nm-z/nates-recipe-rs's
 * gpu-core crate: one `launch_<op>` per operator, device pointers first, sizes
 * as `int`/`long`, the stream last (gpu-core/src/kernels/gemm_f64.hip:48-54,
 * gpu-core/src/kernels/f64_infer.hip:19, gpu-core/src/kernels/quantizedx.hip:25-28;
 * Rust declarations gpu-core/src/infer_ops.rs:11-55).  One deliberate difference:
 * every launcher returns an `int` status (0 = launched; negative = an argument
 * was rejected on the host and nothing was launched) where the upstream returns
 * void and relies on `check_launch` (gpu-core/src/kernels.rs:8-13).
 *
 * Conventions shared by all entry points
 *   - every pointer is a DEVICE pointer unless the parameter says `host`;
 *   - the caller owns every buffer; no entry point here allocates device memory;
 *   - weights `w` are row-major (n, k): n rows of k/B packed blocks, exactly the
 *     GGUF tensor bytes (the operand `b` of gpu_gemm_bt_f64_into,
 *     gpu-core/src/infer_ops.rs:224-240);
 *   - activations are row-major (m, k); outputs row-major (m, n), distinct from
 *     the inputs;
 *   - `stream` is a cudaStream_t passed as void*; NULL is the legacy default
 *     stream, which is what the upstream's wrappers pass;
 *   - weight buffers are read in whole 16-byte lines: up to 15 bytes before the
 *     first and after the last byte of `w`, inside the same 16-byte line, may be
 *     read (never written).  Any pointer inside a cudaMalloc allocation satisfies
 *     this.
 *
 * Block formats (little endian; "fp16" = IEEE binary16)
 *   Q8_0   32 elems, 34 B: fp16 d; int8 q[32]                     w = d*q
 *   Q8_1   32 elems, 36 B: fp16 d; fp16 s; int8 q[32]             x = d*q, s = d*sum(q)
 *   Q4_K  256 elems,144 B: fp16 d; fp16 dmin; u8 scales[12]; u8 qs[128]
 *                                                                 w = (d*sc_j)*q - (dmin*m_j)
 *   Q6_K  256 elems,210 B: u8 ql[128]; u8 qh[64]; int8 scales[16]; fp16 d
 *                                                                 w = (d*scale_g)*(q-32)
 */
#ifndef QMM_H
#define QMM_H
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif

/* type tags (GGUF numbering) */
#define QMM_TYPE_Q8_0 8
#define QMM_TYPE_Q8_1 9
#define QMM_TYPE_Q4_K 12
#define QMM_TYPE_Q6_K 14

/* status codes returned by the launchers */
#define QMM_OK 0
#define QMM_ERR_NULL (-1)        /* a required pointer is NULL                         */
#define QMM_ERR_SHAPE (-2)       /* m, n or k is not positive, or k is not a whole number of blocks */
#define QMM_ERR_UNSUPPORTED (-3) /* shape outside what the kernel can stage (see each entry point)  */
#define QMM_ERR_ALIGN (-4)       /* a pointer is not aligned as documented             */
#define QMM_ERR_TYPE (-5)        /* unknown type tag                                   */
#define QMM_ERR_CUDA (-6)        /* the CUDA runtime refused the launch (see qmm_last_cuda_error) */
#define QMM_ERR_SCRATCH (-7)     /* request exceeds a fixed scratch capacity           */
#define QMM_ERR_IO (-8)          /* a file could not be opened, read or written        */
#define QMM_ERR_FORMAT (-9)      /* a file is not what it claims to be (bad magic, truncated, missing tensor) */

const char* qmm_status_string(int status);
/* cudaError_t of the most recent failed runtime call made by this library on this thread */
int qmm_last_cuda_error(void);
/* Reads and clears the device-side status word of the current device (synchronises
 * the device).  0 = no kernel gave up on a bounded wait since the last call. */
int qmm_device_status(int* host_status);
/* bytes of one packed row of k elements, or a negative status */
long qmm_row_bytes(int type, long k);
/* Programmatic dependent launch: when on (default), the matvec kernels are
 * launched so that they may begin streaming weights while the preceding kernel
 * in the stream drains; they still wait for it to complete before touching
 * activations or outputs.  Returns the previous setting. */
int qmm_set_overlap(int on);

/* Tuning hook for the launchers (benchmark sweeps; the defaults are the tuned values):
 * "stage_bytes" (1024..49152), "ring_bytes" (8192..194560), "consumer_warps" (1..24), "q4k_unit" (0 = automatic,
 * 1, 2, 4: 32-byte groups of a Q4_K super-block per lane), "rb_max" (1, 2, 4: rows reduced together per warp),
 * "ctas_per_sm" (1, 2: persistent CTAs per SM of the single-matrix dp4a matvec; 2 needs "ring_bytes" and
 * "consumer_warps" small enough to fit twice), "mma_min_m" (0..16: fewest activation rows that take the
 * tensor-core matvec where type and shape allow it; 0 = never; default 3), "mma_acc_tp1" / "mma_acc_tp2" /
 * "mma_acc_tp4" (2, 4, 8: weight tiles per pass of the tensor-core matvec at up to 8 / 16 / 32 activation rows) and
 * "mma_acc_w1" (8, 16: its warps at up to 8 rows), "umma_min_m" (0..33: fewest activation rows from which Q4_K
 * rows stored back to back take the tcgen05 integer matvec, in groups of up to 32 rows; 0 = never; default 17), "umma_min_k" (a multiple of 256, default 4096: shortest rows that take it; the matrix must also hold
 * 2 * umma_min_k^2 weights) and
 * "umma_ksplit" (0 = automatic, 1, 2, 4: CTAs of a cluster that share its tile of 128 weight rows, each with a
 * part of K), "attn_tc_min_batch" (fewest
 * sequences from which the decode attention runs on the f16 tensor cores; 0 = never; default 4), and for the
 * job-list matvec "jobs_warps" (1..24), "jobs_ring_bytes", "jobs_stage_bytes", "jobs_rotate" (0/1); "decoder_fuse"
 * (0..3, decode engine at batch 1-2: default 0 = every operator its own launch, 1 = Q|K and V as one job list, 2 = also norms built inside the matvec
 * launches, 3 = also the gated activation).
 * "gemm_mb" (0 = automatic, 1, 2: 256-row blocks of x per CTA of the prefill GEMM), "gemm_ksplit" (0 = automatic,
 * 1, 2: CTAs of a cluster that share one output tile of the prefill GEMM, each with a part of K).
 * Every setting computes the same results.  Not thread-safe against concurrent launches.
 * (A library built with -DQMM_TUNING also has instrumentation that is not part of this interface:
 * stream-only probe modes and a per-CTA time-stamp trace, declared in csrc/qmm_tuning.h.) */
int qmm_tune(const char* key, int value);

/* ---- activations -> Q8_1.  No upstream counterpart (its quantizers are affine
 * per-tensor: gpu-core/src/kernels/quantizedx.hip:12-33); rounding follows its
 * half-away-from-zero rule (quantizedx.hip:8).  x (m,k) f32 -> xq m*(k/32)*36 bytes. */
int launch_quantize_q8_1(const float* x, void* xq, int m, int k, void* stream);

/* ---- weights f32 -> packed blocks (deterministic min/max quantizers; used to
 * build synthetic models on the device).  No upstream counterpart. */
int launch_quantize_q8_0(const float* w, void* out, long rows, int k, void* stream);
int launch_quantize_q4_k(const float* w, void* out, long rows, int k, void* stream);
int launch_quantize_q6_k(const float* w, void* out, long rows, int k, void* stream);

/* ---- weight decode.  Replaces launch_widen_bf16_f64 (gpu-core/src/kernels/
 * f64_infer.hip:12-23; Rust gpu_widen_bf16_into, gpu-core/src/infer_ops.rs:85-101):
 * n_elems packed elements -> n_elems decoded values.  n_elems must be a whole
 * number of blocks.  `_bf16` stores the round-to-nearest-even bf16 of the f32 value. */
int launch_dequantize_q8_0_f32(const void* w, float* out, long n_elems, void* stream);
int launch_dequantize_q4_k_f32(const void* w, float* out, long n_elems, void* stream);
int launch_dequantize_q6_k_f32(const void* w, float* out, long n_elems, void* stream);
int launch_dequantize_q8_0_bf16(const void* w, void* out, long n_elems, void* stream);
int launch_dequantize_q4_k_bf16(const void* w, void* out, long n_elems, void* stream);
int launch_dequantize_q6_k_bf16(const void* w, void* out, long n_elems, void* stream);

/* ---- fused dequant-matvec for decode.  Replaces the pair launch_widen_bf16_f64 +
 * launch_gemm_bt_f64 (gpu-core/src/kernels/gemm_f64.hip:14-54; Rust
 * gpu_gemm_bt_f64_into, gpu-core/src/infer_ops.rs:224-240):
 *   y(m,n) = xq(m,k) . w(n,k)^T,  xq = Q8_1 blocks from launch_quantize_q8_1.
 * m >= 1.  One or two activation rows: integer dot products (dp4a), the weights stream once per
 * launch.  Three rows and more, Q4_K and Q6_K: int8 tensor cores (mma.sync), the weights stream once
 * per 16 activation rows; that kernel needs w and xq on 16-byte boundaries and k a multiple of 512
 * (Q4_K) or 2048 (Q6_K); other cases take the dp4a kernel, which streams the weights once per 4 rows.
 * k: whole blocks, at most 131072, and one packed row must fit a 48 KiB stage
 * (QMM_ERR_UNSUPPORTED otherwise).  Bit-identical across reruns (no atomics). */
int launch_qmatvec_q8_0(const void* w, const void* xq, float* y, int m, int n, int k, void* stream);
int launch_qmatvec_q4_k(const void* w, const void* xq, float* y, int m, int n, int k, void* stream);
int launch_qmatvec_q6_k(const void* w, const void* xq, float* y, int m, int n, int k, void* stream);
int launch_qmatvec(int type, const void* w, const void* xq, float* y, int m, int n, int k, void* stream);
/* The same with the weight rows row_pitch_bytes apart instead of back to back (row_pitch_bytes >= the packed row,
 * even; 0 = back to back).  Q6_K and Q8_0 rows are in general not a multiple of 16 bytes long; a loader that pads
 * them (Q6_K: to a multiple of 48 bytes) makes every shape eligible for the tensor-core kernel.  The padding is
 * read and ignored. */
int launch_qmatvec_pitched(int type, const void* w, long row_pitch_bytes, const void* xq, float* y, int m, int n, int k, void* stream);

/* ---- several independent decode projections in ONE launch.  The upstream issues the projections
 * that share an input one launch after the other (q, k, v: examples/gemma4.rs:653-667; gate and up:
 * :675-678; the chosen experts: :726-742) through gpu_gemm_bt_f64_into (gpu-core/src/infer_ops.rs:
 * 224-240); here a list of such jobs is walked by persistent CTAs that keep the weight stream running
 * from one matrix into the next, so a 33 MB matrix costs its bytes and not a launch on top.
 *   y_j(m, n_j) = xq_j(m, k_j) . w_j(n_j, k_j)^T   for every job j, all with the same m.
 * Jobs must be independent of each other's outputs (they run overlapped).  `jobs` is a HOST array,
 * read during the call.  y_stride: floats between the output rows of two activation rows (0 = n).
 * select (optional, device): the job's matrix is w + select[0] * select_stride_bytes, read on the
 * device when the kernel runs (an expert chosen by a router kernel earlier in the stream);
 * select_stride_bytes must be a multiple of 16.
 * The persistent kernel takes m <= 2, xq on a 16-byte boundary and K up to 64 * 32 * 16 elements
 * (Q8_0: half of that); any other list without selectors runs as one launch_qmatvec per job, with
 * selectors it is rejected with QMM_ERR_UNSUPPORTED.  Bit-identical across reruns. */
typedef struct {
    int type;                 /* QMM_TYPE_Q8_0 / Q4_K / Q6_K */
    int n, k;
    const void* w;            /* packed (n, k) rows */
    const void* xq;           /* Q8_1 (m, k) */
    float* y;                 /* (m, n) */
    long y_stride;
    const int* select;
    long select_stride_bytes;
    int tp_sum;               /* launch_qmatvec_batch_tp only: sum this job's outputs over the ranks */
} qmm_matvec_job;
int launch_qmatvec_batch(const qmm_matvec_job* jobs, int n_jobs, int m, void* stream);

/* ---- a job list whose activations are built inside the launch (all jobs share them; the jobs' xq is ignored).
 * launch_norm_qmatvec_batch: xq = Q8_1( rmsnorm(x_in + x_add) * gamma ) for the projections of a block:
 *   the upstream's residual add (gpu-core/src/kernels/elementwise.hip:13), gpu_rmsnorm_f64_into
 *   (gpu-core/src/infer_ops.rs:117-139) and the projections that follow (examples/gemma4.rs:646-667) as ONE
 *   launch.  x_in (m, k) f32; x_add (m, k) or NULL; gamma (k) or NULL; x_out (m, k) or NULL receives
 *   x_in + x_add and must be a buffer other than x_in.  Every job has K = jobs[0].k.
 * launch_glu_qmatvec_batch: xq = Q8_1( act(gate) * up ) from gate_up (m, 2k) = [gate | up] per row
 *   (gpu_glu_gelu_into, infer_ops.rs:206-222) for the projection(s) that consume it (:678); act 0 = tanh-GELU,
 *   1 = SiLU.
 * Both need the persistent kernel (m <= 2, K within its warps, at most 36 jobs); QMM_ERR_UNSUPPORTED otherwise,
 * and the caller uses launch_add_rmsnorm_q8_1 / launch_glu_act_q8_1 followed by launch_qmatvec_batch. */
int launch_norm_qmatvec_batch(const float* x_in, const float* x_add, const float* gamma, float* x_out, float eps, const qmm_matvec_job* jobs,
                              int n_jobs, int m, void* stream);
int launch_glu_qmatvec_batch(const float* gate_up, int act, const qmm_matvec_job* jobs, int n_jobs, int m, void* stream);

/* ---- tensor parallelism over the GPUs of one box: row-parallel projections with the sum over the ranks
 * fused in.  The upstream runs every projection of a layer on one device (examples/gemma4.rs:653-679); when
 * a layer is partitioned, O and down are split by input columns in whole blocks (rank r holds columns
 * [r*k_local, (r+1)*k_local) of the full matrix as its own (n, k_local) matrix and the matching slice of the
 * activations) and their partial outputs must be added.  One process per GPU; no collective library: the
 * matvec kernel of every rank stores its outputs straight into exchange areas that all ranks have mapped
 * (cudaIpc), each value with the sequence number of the exchange in the same 64-bit word, and a small
 * kernel adds the ranks' values in rank order, so every rank ends with bit-identical sums.
 *   qmm_tp_comm_create   on every rank, with that rank's device current.  capacity_floats: the most values
 *                        (m * n, or the total of a job list's summed jobs) one exchange carries.
 *   qmm_tp_comm_export   64 bytes (a cudaIpcMemHandle_t) to hand to the other ranks by any host channel
 *   qmm_tp_comm_import   once per peer with that peer's 64 bytes;  qmm_tp_comm_ready after the last import
 *   launch_qmatvec_tp    y(m,n) = sum over ranks of xq_r(m,k_local) . w_r(n,k_local)^T on every rank.
 *                        Collective: every rank calls it, in the same order as its peers and within the
 *                        wait bound (about two seconds of SM clock) of them; a rank whose peer does not
 *                        arrive leaves y unwritten and raises the device status (qmm_device_status = 5).
 *   launch_qmatvec_batch_tp  a job list (launch_qmatvec_batch) in which the jobs with tp_sum != 0 are
 *                        summed over the ranks as above and the others are local.
 * All ranks must pass a host-side barrier between qmm_tp_comm_ready and the first launch. */
int qmm_tp_comm_create(int rank, int world, long capacity_floats, void** comm);
int qmm_tp_comm_destroy(void* comm);
int qmm_tp_comm_export(void* comm, void* out_handle_64_bytes);
int qmm_tp_comm_import(void* comm, int peer_rank, const void* handle_64_bytes);
int qmm_tp_comm_ready(void* comm);
int launch_qmatvec_tp(void* comm, int type, const void* w, const void* xq, float* y, int m, int n, int k, void* stream);
int launch_qmatvec_batch_tp(void* comm, const qmm_matvec_job* jobs, int n_jobs, int m, void* stream);

/* ---- dequant-GEMM for prefill on the tcgen05 tensor cores.  Same operator shape as
 * launch_gemm_bt_f64 (gpu-core/src/kernels/gemm_f64.hip:48-54; gpu-core/src/infer_ops.rs:224-240) with
 * m in the hundreds:  y(m,n) = bf16( sum_k x(m,k) * bf16(w(n,k)) ), x and y bf16 row-major, w Q4_K
 * rows, fp32 accumulation; bf16(w) is the round-to-nearest-even bf16 of the value
 * launch_dequantize_q4_k_f32 produces.  x and w 16-byte aligned, k a multiple of 256.
 * `_f32acc` stores the fp32 accumulators instead of rounding them (parity instrumentation). */
int launch_qgemm_q4_k_bf16(const void* w, const void* x, void* y, int m, int n, int k, void* stream);
int launch_qgemm_q4_k_bf16_f32acc(const void* w, const void* x, float* yf, int m, int n, int k, void* stream);

/* ---- out(m,n) = a(m,k) . b(n,k)^T with a and b bf16 (row-major), fp32 accumulation: the upstream's
 * gpu_gemm_bt_f64_into (gpu-core/src/infer_ops.rs:224-240, kernels/gemm_f64.hip:14-54) on a DECODED weight
 * window in bf16 - what a caller uses for a weight type that has no fused GEMM here (dequantize with
 * launch_dequantize_*_bf16, then this).  The same tcgen05 kernel as launch_qgemm_q4_k_bf16 with the weight
 * tiles fetched by TMA instead of unpacked.  out bf16, or f32 accumulators (_f32acc).  k a multiple of 256;
 * a, b 16-byte aligned. */
int launch_gemm_bt_bf16(const void* a, const void* b, void* out, int m, int n, int k, void* stream);
int launch_gemm_bt_bf16_f32acc(const void* a, const void* b, float* out, int m, int n, int k, void* stream);

/* ---- decode attention: one query token per sequence against an fp16 KV cache, grouped-query.
 * Counterpart of launch_gqa_masked_attn (gpu-core/src/kernels/f64_infer.hip:49-100; Rust
 * gpu_gqa_attn_into, gpu-core/src/infer_ops.rs:11-55) for the decode case: qkv (batch, (n_q_heads +
 * 2*n_kv_heads)*head_dim) f32, of which the first n_q_heads*head_dim entries of a row are the
 * queries; kcache/vcache (batch, ctx_cap, n_kv_heads, head_dim) fp16; positions [0, len) are
 * attended with scale 1/sqrt(head_dim).  out_f32 (batch, n_q_heads*head_dim) and/or out_q8 (the same
 * values as Q8_1 blocks, ready for the output projection); either may be NULL, not both.
 * scratch: qmm_attn_decode_scratch_bytes(...) bytes of device memory owned by the caller. */
long qmm_attn_decode_scratch_bytes(int batch, int n_q_heads, int head_dim, int len);
int launch_attn_decode(const float* qkv, const void* kcache, const void* vcache, float* scratch, float* out_f32, void* out_q8,
                       int batch, int n_q_heads, int n_kv_heads, int head_dim, int len, int ctx_cap, void* stream);

/* ---- the same attention for callers that cannot allocate.  This entry point has no counterpart in
 * the upstream project.  It takes no scratch pointer: the split results go to a fixed 4 MiB array
 * that lives inside the library on every GPU that loads it (held until the process exits).  It is
 * meant for hosts that must not call an allocator where they need attention: code running inside a
 * frozen no-allocation loop (the upstream aborts on any allocation once its steady state is
 * frozen), a plugin that only owns the buffers its host handed over, a caller that has already
 * handed all of its memory to other uses.  It never calls cudaMalloc, cudaFree or any allocating
 * routine.  Requests whose scratch need (qmm_attn_decode_scratch_bytes) exceeds 4 MiB are rejected
 * with QMM_ERR_SCRATCH and nothing is launched.  The first call on a device looks up the array's
 * device address (a one-time set-up); make that first call outside any stream capture.  All calls
 * share the one array and it keeps what the last call left there: nothing in it needs clearing
 * (each call overwrites every word it reads), but two calls that overlap on the GPU, from any
 * streams or threads, race on it and must be ordered by the caller. */
int launch_attn_decode_static(const float* qkv, const void* kcache, const void* vcache, float* out_f32, void* out_q8, int batch,
                              int n_q_heads, int n_kv_heads, int head_dim, int len, int ctx_cap, void* stream);

/* ---- the small per-layer operators of the decode stack, fp32 with Q8_1 outputs so that the next
 * projection finds its activations ready.  act: 0 = tanh-GELU, 1 = SiLU.
 *
 * launch_add_rmsnorm_q8_1: counterpart of launch_normx_rmsnorm (gpu-core/src/kernels/normx.hip:135-159;
 *   Rust gpu_rmsnorm_f64_into, gpu-core/src/infer_ops.rs:117-139) fused with the residual add before it
 *   (add_kernel, gpu-core/src/kernels/elementwise.hip:13) and the quantization after it:
 *   x(rows,cols) += add (when add != NULL; x is updated in place), then
 *   xq = Q8_1( x / sqrt(mean(x^2) + eps) * gamma ); gamma == NULL is the scale-less variant; out_f32
 *   (optional) receives the normalised values before quantization.  cols a multiple of 32, at most 8192.
 * launch_rope_kv_append: counterpart of launch_rope_partial with rotary_dim == head_dim
 *   (gpu-core/src/kernels/f64_infer.hip:107-132; Rust gpu_rope_partial, infer_ops.rs:61-83) for one new
 *   token per sequence at position pos: rotates the q heads of qkv (batch, (n_q + 2 n_kv) * head_dim) in
 *   place (NeoX rotate-half) and appends the rotated k and the v heads to the fp16 caches
 *   (batch, ctx_cap, n_kv_heads, head_dim) at pos.
 * launch_glu_act_q8_1: counterpart of launch_glu_gelu (gpu-core/src/kernels/f64_infer.hip:150-166; Rust
 *   gpu_glu_gelu_into, infer_ops.rs:206-222): gate_up (rows, 2*half) = [gate | up] per row ->
 *   xq = Q8_1( act(gate) * up ) (rows, half); out_f32 optional.  half a multiple of 32.
 * launch_embed_rows: x[b] = decoded row tokens[b] of a packed (vocab, hidden) table (the upstream example
 *   gathers its bf16 embedding rows on the host: examples/gemma4.rs:951-958); tokens are clamped to the table.
 * launch_argmax_rows: index (lowest on ties) and value of the largest logit of every row (the upstream
 *   example picks the next token on the host: examples/gemma4.rs:1021-1046; greedy here).  scratch:
 *   qmm_argmax_scratch_bytes(batch) bytes of caller-owned device memory, 8-byte aligned.
 * launch_scale_f32: x *= scalar, counterpart of launch_scale_f64 (gpu-core/src/kernels/gemm_f64.hip:57-65;
 *   Rust gpu_scale_f64_inplace, infer_ops.rs:242-248). */
int launch_add_rmsnorm_q8_1(float* x, const float* add, const float* gamma, void* xq, float* out_f32, int rows, int cols, float eps,
                            void* stream);
int launch_rope_kv_append(float* qkv, void* kcache, void* vcache, int batch, int n_q_heads, int n_kv_heads, int head_dim, int pos,
                          int ctx_cap, float theta, void* stream);
int launch_glu_act_q8_1(const float* gate_up, void* xq, float* out_f32, int rows, int half, int act, void* stream);
int launch_embed_rows(int type, const void* table, const int* tokens, float* x, int batch, int hidden, int vocab, void* stream);
long qmm_argmax_scratch_bytes(int batch);
int launch_argmax_rows(const float* logits, void* scratch, int* out_index, float* out_value, int batch, int vocab, void* stream);
int launch_scale_f32(float* x, float scalar, long n, void* stream);

/* ---- attention over a whole sequence: the counterpart of the upstream's gpu_gqa_attn_into
 * (gpu-core/src/infer_ops.rs:160-189 -> launch_gqa_masked_attn, gpu-core/src/kernels/f64_infer.hip:42-100).
 * q (t, n_q_heads*head_dim), k and v (t, n_kv_heads*head_dim), out (t, n_q_heads*head_dim), all f32 row-major
 * (the upstream's are f64); query head h reads kv head h / (n_q_heads / n_kv_heads).  Positions p < prefix are
 * causal (attend sp <= p), positions p >= prefix attend the whole sequence; prefix = t is plain causal
 * attention, prefix = 0 bidirectional.  Scores are q.k * kq_scale (the upstream folds its scale into q: 1).
 * `out` must be distinct from q, k and v (every CTA reads the whole sequence, as upstream).  head_dim 32, 64, 96,
 * 128 or 256; q, k, v 16-byte aligned.  Scores and outputs run on the f16 tensor cores with q (scaled), k, v and
 * the probabilities rounded to f16 (about 1e-3 relative); the t x t scores are never stored. */
int launch_attn_prefill(const float* q, const float* k, const float* v, float* out, int t, int n_q_heads, int n_kv_heads, int head_dim,
                        int prefix, float kq_scale, void* stream);
/* The same with k and v already f16 (2 bytes per element, row-major (t, n_kv_heads*head_dim), 16-byte aligned, n_kv_heads*head_dim
 * a multiple of 8): the rows of a KV cache.  The values the f32 form would round k and v to are read as they are, so both forms
 * give the same bits for k16 = f16(k), v16 = f16(v); the tiles go to shared memory with cp.async, half the traffic, no conversion. */
int launch_attn_prefill_f16kv(const float* q, const void* k16, const void* v16, float* out, int t, int n_q_heads, int n_kv_heads,
                              int head_dim, int prefix, float kq_scale, void* stream);
/* ... and for t queries that continue a sequence: row r of q and out is position q_pos0 + r, k16 and v16 hold positions
 * 0..t_kv-1 (q_pos0 + t <= t_kv); `prefix` counts positions of the sequence as above.  Row for row the same bits as the
 * rows q_pos0.. of one call over the whole sequence. */
int launch_attn_prefill_f16kv_at(const float* q, const void* k16, const void* v16, float* out, int t, int t_kv, int q_pos0, int n_q_heads,
                                 int n_kv_heads, int head_dim, int prefix, float kq_scale, void* stream);

/* ---- quantized dense layer: y(m,n) = act( x(m,k) . w(n,k)^T + bias(n) ), x and y f32, w packed blocks of
 * `type`.  The counterpart of LayerKind::Dense in the upstream's forward pass (recipe-infer/src/forward.rs:
 * 372-431: gpu_linear_into, gpu-core/src/kernels.rs:2589-2640, then one activation launch), the place where a
 * quantized weight plugs into its LayerParams (recipe-infer/src/params.rs:35-59: w, b, in_dim = k,
 * out_dim = n, act, palpha).  Three launches: x -> Q8_1 into xq_scratch, the matvec, bias + activation in
 * place.  From 64 rows on a Q4_K layer takes the tensor-core GEMM instead: x rounded to bf16 into xq_scratch
 * (16-byte aligned), launch_qgemm_q4_k_bf16_f32acc, bias + activation; the product then differs from the
 * small-batch one by the rounding of x (bf16 instead of Q8_1 blocks).  xq_scratch: qmm_qdense_scratch_bytes
 * bytes of caller-owned device memory.  bias may be NULL.  alpha: the negative slope of LEAKY_RELU (upstream:
 * 0.01) and PRELU (the learned scalar), ELU's alpha (upstream: 1.0); ignored otherwise. */
#define QMM_DENSE_LINEAR 0
#define QMM_DENSE_RELU 1
#define QMM_DENSE_SIGMOID 2
#define QMM_DENSE_LEAKY_RELU 3
#define QMM_DENSE_PRELU 4
#define QMM_DENSE_ELU 5
#define QMM_DENSE_SELU 6
#define QMM_DENSE_TANH 7
#define QMM_DENSE_SILU 8
#define QMM_DENSE_GELU 9
long qmm_qdense_scratch_bytes(int type, int m, int k);
int launch_qdense(int type, const void* w, const float* x, const float* bias, float* y, void* xq_scratch, int m, int n, int k, int act,
                  float alpha, void* stream);

/* ---- mixture-of-experts branch of a decode step, on the device.  The upstream example routes on the host:
 * it downloads the activations, computes router logits, softmax and top-k per token in f64 loops, gathers the
 * tokens of every chosen expert, uploads them and runs the experts one after the other
 * (examples/gemma4.rs:684-742).  Here the choice never leaves the device.
 * launch_moe_router_topk: per token p of x (m, hidden) f32:
 *     r = x / sqrt(mean(x^2) + eps) * scale * gain          (gain NULL = 1; the upstream's rnp * 1/sqrt(NE) * gis)
 *     prob = softmax(router_w (n_experts, hidden, f32) . r)
 *     sel[p][0..top_k) = the top_k experts by probability, largest first, lowest index first on ties
 *     weight[p][j] = prob[sel[p][j]] / sum_j prob[sel[p][j]]
 *   probs (optional) receives all probabilities (m, n_experts).  n_experts <= 256, top_k <= 8.
 * launch_moe_experts: for every (token, slot): gu = xq[token] . W_gu[sel]^T, ea = Q8_1(act(gate) * up),
 *     dv = ea . W_dn[sel]^T;  out[token] = sum over slots of weight * expert_scale[sel] * dv (expert_scale NULL = 1).
 *   The experts' matrices lie in two banks, matrix e at bank + e * stride_bytes (strides multiples of 16):
 *   gate_up (2 * ffn_expert, hidden) rows [gate | up], down (hidden, ffn_expert).  xq: Q8_1 (m, hidden).
 *   Each of the two projections is ONE job-list launch whose jobs read their expert index on the device.
 *   scratch: qmm_moe_scratch_bytes(...) bytes of caller-owned device memory, 16-byte aligned.
 *   Decode-sized m: an expert chosen by several tokens is streamed once per token. */
int launch_moe_router_topk(const float* x, const float* gain, const float* router_w, int m, int hidden, int n_experts, int top_k, float scale,
                           float eps, int* sel, float* weight, float* probs, void* stream);
long qmm_moe_scratch_bytes(int m, int top_k, int hidden, int ffn_expert);
int launch_moe_experts(int type_gu, const void* gate_up_bank, long gu_stride_bytes, int type_dn, const void* down_bank, long dn_stride_bytes,
                       const void* xq, const int* sel, const float* weight, const float* expert_scale, float* out, void* scratch, int m,
                       int top_k, int hidden, int ffn_expert, int act, void* stream);

/* ---- per-block integer dot sums (parity instrumentation; same device code as
 * the matvec).  One Q8_1 row xq (k); out int32 (n, k/32) for Q8_0 and Q4_K,
 * (n, k/16) for Q6_K. */
int launch_qblock_dots(int type, const void* w, const void* xq, int32_t* out, int n, int k, void* stream);

#ifdef __cplusplus
}
#endif
#endif
