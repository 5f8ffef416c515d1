/*
 * Development instrumentation of libqmm, compiled only with -DQMM_TUNING (not in the shipped library,
 * not part of the C ABI in include/qmm.h).
 *
 *   qmm_tune("probe", 1)        the single-matrix matvec streams and synchronises but skips its arithmetic
 *   qmm_tune("gemm_probe", 1/2) the prefill GEMM skips its unpack arithmetic / its tensor-core instructions
 *                               (both produce wrong results by design: they time the skeleton)
 *   qmm_trace(buf, stride)      while buf is non-NULL, matvec launch number i (counted from the call) stores
 *                               four global-timer stamps per CTA (start, dependency released, first stage
 *                               landed, end) as 64-bit words at buf + i*stride_words
 */
#ifndef QMM_TUNING_H
#define QMM_TUNING_H
#ifdef __cplusplus
extern "C" {
#endif
int qmm_trace(void* buf, int stride_words);
#ifdef __cplusplus
}
#endif
#endif
