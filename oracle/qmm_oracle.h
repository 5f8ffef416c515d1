/*
 * qmm_oracle.h — CPU restatement of the GGUF-block quantized-matmul path.
 *
 * TEST INFRASTRUCTURE ONLY.  Nothing in the shipped library may include, link
 * or call this; it exists so the parity tests, the smoke check and the CPU
 * baseline leg of the benchmark have an independent answer to compare with.
 *
 * PARITY UNPINNED: the upstream project (nm-z/nates-recipe-rs) holds no
 * implementation, test, fixture or golden vector for Q8_0 / Q8_1 / Q4_K / Q6_K
 * (gpu-core/tests/suite/prove_quantized.rs:15-20 lists block formats as
 * backlog).  The block layouts below are the public GGUF k-quant layouts as
 * restated from their published description; the ggml/llama.cpp project that
 * defines them is not a dependency of the upstream (no such package in its
 * Cargo.lock) and is not available here, so byte compatibility with real GGUF
 * tensors is unverified.  What the upstream does pin, and this file follows:
 *   - round half away from zero when producing integer codes
 *     (gpu-core/src/kernels/quantizedx.hip:8),
 *   - integer-exact comparison of codes (prove_quantized.rs:349-357),
 *   - operator shape out(m,n) = a(m,k) . b(n,k)^T, row-major, caller-owned out
 *     (gpu-core/src/infer_ops.rs:224-240, kernels/gemm_f64.hip:14-46),
 *   - straight-loop CPU oracle with a max|delta| report (examples/det_probe.rs:49-89).
 *
 * Every float expression is a sequence of single IEEE-754 binary32 operations
 * in the order written (compile with -ffp-contract=off); the device code uses
 * the same order with round-to-nearest intrinsics, which is what makes
 * dequantised values and packed codes comparable bit for bit.
 */
#ifndef QMM_ORACLE_H
#define QMM_ORACLE_H
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif

/* Block geometry (elements per block, bytes per block). */
#define QO_QK8 32
#define QO_QKK 256
#define QO_Q8_0_BYTES 34   /* fp16 d; int8 q[32]                                   */
#define QO_Q8_1_BYTES 36   /* fp16 d; fp16 s; int8 q[32]      (activations)        */
#define QO_Q4_K_BYTES 144  /* fp16 d; fp16 dmin; u8 scales[12]; u8 qs[128]         */
#define QO_Q6_K_BYTES 210  /* u8 ql[128]; u8 qh[64]; int8 scales[16]; fp16 d       */

/* Type tags shared with the device library (GGUF numbering). */
enum { QO_TYPE_Q8_0 = 8, QO_TYPE_Q8_1 = 9, QO_TYPE_Q4_K = 12, QO_TYPE_Q6_K = 14 };

/* scalar conversions (software, round-to-nearest-even) */
uint16_t qo_f32_to_f16(float f);
float    qo_f16_to_f32(uint16_t h);
uint16_t qo_f32_to_bf16(float f);
float    qo_bf16_to_f32(uint16_t h);

/* seeded closed-form generator: out[i] = sigma * z(seed, i), z ~ approx N(0,1)
 * built from integer hashing only (no libm), so C, numpy and CUDA agree bit for bit. */
void qo_fill_normal(float* out, long n, uint64_t seed, float sigma, long first_index);

/* bytes of one packed row of k elements (k must be a multiple of the block size) */
long qo_row_bytes(int type, long k);

/* quantizers: k elements -> packed blocks */
void qo_quantize_row_q8_0(const float* x, void* y, long k);
void qo_quantize_row_q8_1(const float* x, void* y, long k);
void qo_quantize_row_q4_k(const float* x, void* y, long k);
void qo_quantize_row_q6_k(const float* x, void* y, long k);
void qo_quantize_rows(int type, const float* x, void* y, long rows, long k);

/* dequantizers: packed blocks -> k floats (or bf16 = RNE of that float) */
void qo_dequantize_row_q8_0(const void* x, float* y, long k);
void qo_dequantize_row_q8_1(const void* x, float* y, long k);
void qo_dequantize_row_q4_k(const void* x, float* y, long k);
void qo_dequantize_row_q6_k(const void* x, float* y, long k);
void qo_dequantize_rows(int type, const void* x, float* y, long rows, long k);
void qo_dequantize_rows_bf16(int type, const void* x, uint16_t* y, long rows, long k);

/* per-block integer dot sums of weight rows (n,k) against ONE Q8_1 row (k):
 *   Q8_0: one int32 per 32-block        -> out[n][k/32]
 *   Q4_K: one int32 per 32-sub-block    -> out[n][k/32]   (unsigned 4-bit codes)
 *   Q6_K: one int32 per 16-group        -> out[n][k/16]   (codes minus 32)      */
void qo_block_dots(int type, const void* w, const void* xq, int32_t* out, long n, long k);

/* y(m,n) = xq(m,k) . w(n,k)^T with Q8_1 activations, fp32 accumulate */
void qo_matvec(int type, const void* w, const void* xq, float* y, long m, long n, long k);

/* y(m,n) = bf16( sum_k f32(x[m,k]) * f32(bf16(dequant(w[n,k]))) ), x and y bf16;
 * yf (optional, may be NULL) receives the fp32 accumulators before rounding. */
void qo_gemm_bf16(int type, const void* w, const uint16_t* x, uint16_t* y, float* yf,
                  long m, long n, long k);

/* ---- decoder-stack pieces (fp32, straight loops) ---- */
void qo_rmsnorm(const float* x, const float* gamma, float* out, long rows, long cols, float eps);
void qo_rope_neox(float* buf, long rows, long head_dim, long heads_per_tok, long pos0, float theta);
void qo_gelu_mul(const float* gate, const float* up, float* out, long n);
void qo_silu_mul(const float* gate, const float* up, float* out, long n);
/* single-query GQA attention over an fp16 KV cache:
 * q (nqh, hd) f32; kc, vc (ctx_cap, nkv, hd) fp16; attends to positions [0, len) */
void qo_attn_decode(const float* q, const uint16_t* kc, const uint16_t* vc, float* out,
                    long nqh, long nkv, long hd, long len);
void qo_attn_prefill(const float* q, const float* k, const float* v, float* out, long t, long nqh, long nkv, long hd,
                     long prefix, double kq_scale);

int qo_num_threads(void);
void qo_set_num_threads(int n);

#ifdef __cplusplus
}
#endif
#endif
