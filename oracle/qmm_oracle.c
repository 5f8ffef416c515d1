/*
 * qmm_oracle.c — CPU restatement of the GGUF-block quantized-matmul path.
 * TEST INFRASTRUCTURE ONLY; see qmm_oracle.h for the parity statement
 * ("parity unpinned": the upstream has no implementation or golden vectors for
 * these block formats) and for the upstream conventions each piece follows.
 *
 * Build: gcc -O3 -march=x86-64-v3 -ffp-contract=off -fopenmp -shared -fPIC
 */
#include "qmm_oracle.h"
#include <math.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

/* The benchmark's CPU legs set the thread count themselves: a launcher may have exported
 * OMP_NUM_THREADS=1 for its children. */
void qo_set_num_threads(int n) {
    if (n > 0) omp_set_num_threads(n);
}

int qo_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* ------------------------------------------------------------------ scalars */

float qo_f16_to_f32(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1Fu;
    uint32_t man = h & 0x3FFu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else { /* subnormal: normalise */
            int e = -1;
            do { man <<= 1; e++; } while (!(man & 0x400u));
            bits = sign | (uint32_t)(127 - 15 - e) << 23 | (man & 0x3FFu) << 13;
        }
    } else if (exp == 31) {
        bits = sign | 0x7F800000u | man << 13;
    } else {
        bits = sign | (exp + 112u) << 23 | man << 13;
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

uint16_t qo_f32_to_f16(float f) {
    uint32_t x;
    memcpy(&x, &f, 4);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t ax = x & 0x7FFFFFFFu;
    if (ax >= 0x7F800000u) /* inf / nan */
        return (uint16_t)(sign | 0x7C00u | (ax > 0x7F800000u ? 0x200u | ((ax >> 13) & 0x3FFu) : 0));
    if (ax >= 0x477FF000u) /* rounds to >= 65520 -> inf */
        return (uint16_t)(sign | 0x7C00u);
    if (ax < 0x38800000u) { /* result is subnormal or zero (|f| < 2^-14) */
        if (ax < 0x33000000u) return (uint16_t)sign; /* < 2^-25 -> 0 */
        uint32_t e = ax >> 23;                         /* biased exponent, 102..112 */
        uint32_t m = (ax & 0x7FFFFFu) | 0x800000u;     /* 24-bit significand */
        uint32_t shift = 126u - e;                     /* 14..24: bits dropped so that unit = 2^-24 */
        uint32_t r = m >> shift;
        uint32_t rem = m & ((1u << shift) - 1u);
        uint32_t half = 1u << (shift - 1u);
        if (rem > half || (rem == half && (r & 1u))) r++;
        return (uint16_t)(sign | r);
    }
    uint32_t e = (ax >> 23) - 112u;
    uint32_t m = ax & 0x7FFFFFu;
    uint32_t r = (e << 10) | (m >> 13);
    uint32_t rem = m & 0x1FFFu;
    if (rem > 0x1000u || (rem == 0x1000u && (r & 1u))) r++;
    return (uint16_t)(sign | r);
}

uint16_t qo_f32_to_bf16(float f) {
    uint32_t x;
    memcpy(&x, &f, 4);
    if ((x & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)((x >> 16) | 0x40u);
    uint32_t lsb = (x >> 16) & 1u;
    x += 0x7FFFu + lsb;
    return (uint16_t)(x >> 16);
}

float qo_bf16_to_f32(uint16_t h) {
    uint32_t x = (uint32_t)h << 16;
    float f;
    memcpy(&f, &x, 4);
    return f;
}

/* ---------------------------------------------------------------- generator */

static inline uint64_t mix64(uint64_t z) {
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

/* Sum of eight 16-bit uniform integers, centred and scaled to unit variance:
 * mean 8*32767.5 = 262140, sd = sqrt(8*(65536^2-1)/12) = 53510.0 (to 7 digits). */
void qo_fill_normal(float* out, long n, uint64_t seed, float sigma, long first_index) {
    const float inv_sd = 1.0f / 53510.0f;
#pragma omp parallel for schedule(static)
    for (long i = 0; i < n; i++) {
        uint64_t h1 = mix64(seed * 0xD1342543DE82EF95ull + (uint64_t)(first_index + i));
        uint64_t h2 = mix64(h1);
        int32_t s = 0;
        for (int c = 0; c < 4; c++) {
            s += (int32_t)((h1 >> (16 * c)) & 0xFFFFu);
            s += (int32_t)((h2 >> (16 * c)) & 0xFFFFu);
        }
        float z = (float)(s - 262140) * inv_sd;
        out[i] = z * sigma;
    }
}

/* ------------------------------------------------------------------ layouts */

long qo_row_bytes(int type, long k) {
    switch (type) {
    case QO_TYPE_Q8_0: return k / QO_QK8 * QO_Q8_0_BYTES;
    case QO_TYPE_Q8_1: return k / QO_QK8 * QO_Q8_1_BYTES;
    case QO_TYPE_Q4_K: return k / QO_QKK * QO_Q4_K_BYTES;
    case QO_TYPE_Q6_K: return k / QO_QKK * QO_Q6_K_BYTES;
    }
    return -1;
}

static inline uint16_t rd16(const uint8_t* p) { return (uint16_t)(p[0] | (p[1] << 8)); }
static inline void wr16(uint8_t* p, uint16_t v) { p[0] = (uint8_t)(v & 0xFF); p[1] = (uint8_t)(v >> 8); }

/* largest finite fp16; scales are clamped to it so a block never stores inf */
#define F16_MAX 65504.0f

static inline int iround_away(float v) { return (int)roundf(v); } /* half away from zero */
static inline int clampi(int v, int lo, int hi) { return v < lo ? lo : (v > hi ? hi : v); }

/* Q4_K 6-bit scale/min codes for sub-block j (0..7) from the 12 packed bytes. */
static inline void q4k_scale_min(int j, const uint8_t* s, int* sc, int* mn) {
    if (j < 4) {
        *sc = s[j] & 63;
        *mn = s[j + 4] & 63;
    } else {
        *sc = (s[j + 4] & 15) | ((s[j - 4] >> 6) << 4);
        *mn = (s[j + 4] >> 4) | ((s[j] >> 6) << 4);
    }
}

static inline void q4k_pack_scales(const int* sc, const int* mn, uint8_t* s) {
    memset(s, 0, 12);
    for (int j = 0; j < 8; j++) {
        if (j < 4) {
            s[j] |= (uint8_t)(sc[j] & 63);
            s[j + 4] |= (uint8_t)(mn[j] & 63);
        } else {
            s[j + 4] |= (uint8_t)((sc[j] & 15) | ((mn[j] & 15) << 4));
            s[j - 4] |= (uint8_t)((sc[j] >> 4) << 6);
            s[j] |= (uint8_t)((mn[j] >> 4) << 6);
        }
    }
}

/* Q4_K: 4-bit code of element e (0..255) of a super-block */
static inline int q4k_code(const uint8_t* qs, int e) {
    int j = e >> 5, l = e & 31;
    uint8_t b = qs[32 * (j >> 1) + l];
    return (j & 1) ? (b >> 4) : (b & 15);
}

/* Q6_K: 6-bit code of element e (0..255): two halves of 128; in a half, the four
 * quarters of 32 take lo/lo/hi/hi nibbles of ql[l], ql[l+32], ql[l], ql[l+32]
 * and bits (2t, 2t+1) of qh[l]. */
static inline int q6k_code(const uint8_t* ql, const uint8_t* qh, int e) {
    int h = e >> 7, r = e & 127, t = r >> 5, l = r & 31;
    uint8_t b = ql[64 * h + l + 32 * (t & 1)];
    int lo = (t < 2) ? (b & 15) : (b >> 4);
    int hi = (qh[32 * h + l] >> (2 * t)) & 3;
    return lo | (hi << 4);
}

/* --------------------------------------------------------------- quantizers */

void qo_quantize_row_q8_0(const float* x, void* vy, long k) {
    uint8_t* y = (uint8_t*)vy;
    for (long b = 0; b < k / QO_QK8; b++, x += QO_QK8, y += QO_Q8_0_BYTES) {
        float amax = 0.0f;
        for (int i = 0; i < QO_QK8; i++) amax = fmaxf(amax, fabsf(x[i]));
        float d = fminf(amax / 127.0f, F16_MAX);
        uint16_t dh = qo_f32_to_f16(d);
        float df = qo_f16_to_f32(dh);
        wr16(y, dh);
        for (int i = 0; i < QO_QK8; i++) {
            int q = (df > 0.0f) ? clampi(iround_away(x[i] / df), -127, 127) : 0;
            y[2 + i] = (uint8_t)(int8_t)q;
        }
    }
}

void qo_quantize_row_q8_1(const float* x, void* vy, long k) {
    uint8_t* y = (uint8_t*)vy;
    for (long b = 0; b < k / QO_QK8; b++, x += QO_QK8, y += QO_Q8_1_BYTES) {
        float amax = 0.0f;
        for (int i = 0; i < QO_QK8; i++) amax = fmaxf(amax, fabsf(x[i]));
        float d = fminf(amax / 127.0f, F16_MAX);
        uint16_t dh = qo_f32_to_f16(d);
        float df = qo_f16_to_f32(dh);
        int sum = 0;
        for (int i = 0; i < QO_QK8; i++) {
            int q = (df > 0.0f) ? clampi(iround_away(x[i] / df), -127, 127) : 0;
            y[4 + i] = (uint8_t)(int8_t)q;
            sum += q;
        }
        wr16(y, dh);
        wr16(y + 2, qo_f32_to_f16(df * (float)sum));
    }
}

/* Q4_K quantizer (this build's own, deterministic):
 *   per 32-sub-block: lo = max(0, -min w), step = (max w + lo) / 15   (both >= 0)
 *   d = max_j step_j / 63, dmin = max_j lo_j / 63, both stored as fp16
 *   sc_j = round(step_j / d), m_j = round(lo_j / dmin), clamped to 0..63
 *   q = clamp(round((w + dmin*m_j) / (d*sc_j)), 0, 15)                           */
void qo_quantize_row_q4_k(const float* x, void* vy, long k) {
    uint8_t* y = (uint8_t*)vy;
    for (long b = 0; b < k / QO_QKK; b++, x += QO_QKK, y += QO_Q4_K_BYTES) {
        float step[8], lo[8], max_step = 0.0f, max_lo = 0.0f;
        for (int j = 0; j < 8; j++) {
            float mn = x[32 * j], mx = x[32 * j];
            for (int i = 1; i < 32; i++) {
                mn = fminf(mn, x[32 * j + i]);
                mx = fmaxf(mx, x[32 * j + i]);
            }
            lo[j] = fmaxf(0.0f, -mn);
            step[j] = fmaxf(0.0f, (mx + lo[j]) / 15.0f);
            max_step = fmaxf(max_step, step[j]);
            max_lo = fmaxf(max_lo, lo[j]);
        }
        uint16_t dh = qo_f32_to_f16(fminf(max_step / 63.0f, F16_MAX));
        uint16_t mh = qo_f32_to_f16(fminf(max_lo / 63.0f, F16_MAX));
        float d = qo_f16_to_f32(dh), dmin = qo_f16_to_f32(mh);
        int sc[8], m[8];
        for (int j = 0; j < 8; j++) {
            sc[j] = (d > 0.0f) ? clampi(iround_away(step[j] / d), 0, 63) : 0;
            m[j] = (dmin > 0.0f) ? clampi(iround_away(lo[j] / dmin), 0, 63) : 0;
        }
        wr16(y, dh);
        wr16(y + 2, mh);
        q4k_pack_scales(sc, m, y + 4);
        uint8_t* qs = y + 16;
        memset(qs, 0, 128);
        for (int j = 0; j < 8; j++) {
            float ds = d * (float)sc[j];
            float off = dmin * (float)m[j];
            for (int i = 0; i < 32; i++) {
                int q = (ds > 0.0f) ? clampi(iround_away((x[32 * j + i] + off) / ds), 0, 15) : 0;
                qs[32 * (j >> 1) + i] |= (uint8_t)((j & 1) ? (q << 4) : q);
            }
        }
    }
}

/* Q6_K quantizer (this build's own, deterministic):
 *   per 16-group: gs = absmax / 31;  d = max_g gs / 127 stored as fp16
 *   scale_g = clamp(round(gs / d), 0, 127);  q = clamp(round(w / (d*scale_g)), -32, 31) + 32 */
void qo_quantize_row_q6_k(const float* x, void* vy, long k) {
    uint8_t* y = (uint8_t*)vy;
    for (long b = 0; b < k / QO_QKK; b++, x += QO_QKK, y += QO_Q6_K_BYTES) {
        float gs[16], max_gs = 0.0f;
        for (int g = 0; g < 16; g++) {
            float amax = 0.0f;
            for (int i = 0; i < 16; i++) amax = fmaxf(amax, fabsf(x[16 * g + i]));
            gs[g] = amax / 31.0f;
            max_gs = fmaxf(max_gs, gs[g]);
        }
        uint16_t dh = qo_f32_to_f16(fminf(max_gs / 127.0f, F16_MAX));
        float d = qo_f16_to_f32(dh);
        uint8_t* ql = y;
        uint8_t* qh = y + 128;
        int8_t* sc = (int8_t*)(y + 192);
        memset(y, 0, 192);
        for (int g = 0; g < 16; g++)
            sc[g] = (int8_t)((d > 0.0f) ? clampi(iround_away(gs[g] / d), 0, 127) : 0);
        wr16(y + 208, dh);
        for (int e = 0; e < QO_QKK; e++) {
            float ds = d * (float)sc[e >> 4];
            int q = ((ds > 0.0f) ? clampi(iround_away(x[e] / ds), -32, 31) : 0) + 32;
            int h = e >> 7, r = e & 127, t = r >> 5, l = r & 31;
            int qi = 64 * h + l + 32 * (t & 1);
            ql[qi] |= (uint8_t)((t < 2) ? (q & 15) : ((q & 15) << 4));
            qh[32 * h + l] |= (uint8_t)((q >> 4) << (2 * t));
        }
    }
}

void qo_quantize_rows(int type, const float* x, void* y, long rows, long k) {
    long rb = qo_row_bytes(type, k);
#pragma omp parallel for schedule(static)
    for (long r = 0; r < rows; r++) {
        const float* xr = x + r * k;
        uint8_t* yr = (uint8_t*)y + r * rb;
        switch (type) {
        case QO_TYPE_Q8_0: qo_quantize_row_q8_0(xr, yr, k); break;
        case QO_TYPE_Q8_1: qo_quantize_row_q8_1(xr, yr, k); break;
        case QO_TYPE_Q4_K: qo_quantize_row_q4_k(xr, yr, k); break;
        case QO_TYPE_Q6_K: qo_quantize_row_q6_k(xr, yr, k); break;
        }
    }
}

/* ------------------------------------------------------------- dequantizers */

void qo_dequantize_row_q8_0(const void* vx, float* y, long k) {
    const uint8_t* x = (const uint8_t*)vx;
    for (long b = 0; b < k / QO_QK8; b++, x += QO_Q8_0_BYTES, y += QO_QK8) {
        float d = qo_f16_to_f32(rd16(x));
        for (int i = 0; i < QO_QK8; i++) y[i] = d * (float)(int8_t)x[2 + i];
    }
}

void qo_dequantize_row_q8_1(const void* vx, float* y, long k) {
    const uint8_t* x = (const uint8_t*)vx;
    for (long b = 0; b < k / QO_QK8; b++, x += QO_Q8_1_BYTES, y += QO_QK8) {
        float d = qo_f16_to_f32(rd16(x));
        for (int i = 0; i < QO_QK8; i++) y[i] = d * (float)(int8_t)x[4 + i];
    }
}

/* w = (d*sc)*q - (dmin*m): three multiplies and one subtract, each rounded */
void qo_dequantize_row_q4_k(const void* vx, float* y, long k) {
    const uint8_t* x = (const uint8_t*)vx;
    for (long b = 0; b < k / QO_QKK; b++, x += QO_Q4_K_BYTES, y += QO_QKK) {
        float d = qo_f16_to_f32(rd16(x)), dmin = qo_f16_to_f32(rd16(x + 2));
        for (int j = 0; j < 8; j++) {
            int sc, m;
            q4k_scale_min(j, x + 4, &sc, &m);
            float ds = d * (float)sc;
            float off = dmin * (float)m;
            for (int i = 0; i < 32; i++) {
                float t = ds * (float)q4k_code(x + 16, 32 * j + i);
                y[32 * j + i] = t - off;
            }
        }
    }
}

/* w = (d*scale)*(q-32): two multiplies, each rounded */
void qo_dequantize_row_q6_k(const void* vx, float* y, long k) {
    const uint8_t* x = (const uint8_t*)vx;
    for (long b = 0; b < k / QO_QKK; b++, x += QO_Q6_K_BYTES, y += QO_QKK) {
        float d = qo_f16_to_f32(rd16(x + 208));
        const int8_t* sc = (const int8_t*)(x + 192);
        for (int e = 0; e < QO_QKK; e++) {
            float ds = d * (float)sc[e >> 4];
            y[e] = ds * (float)(q6k_code(x, x + 128, e) - 32);
        }
    }
}

static void dequantize_row(int type, const void* x, float* y, long k) {
    switch (type) {
    case QO_TYPE_Q8_0: qo_dequantize_row_q8_0(x, y, k); break;
    case QO_TYPE_Q8_1: qo_dequantize_row_q8_1(x, y, k); break;
    case QO_TYPE_Q4_K: qo_dequantize_row_q4_k(x, y, k); break;
    case QO_TYPE_Q6_K: qo_dequantize_row_q6_k(x, y, k); break;
    }
}

void qo_dequantize_rows(int type, const void* x, float* y, long rows, long k) {
    long rb = qo_row_bytes(type, k);
#pragma omp parallel for schedule(static)
    for (long r = 0; r < rows; r++) dequantize_row(type, (const uint8_t*)x + r * rb, y + r * k, k);
}

void qo_dequantize_rows_bf16(int type, const void* x, uint16_t* y, long rows, long k) {
    long rb = qo_row_bytes(type, k);
#pragma omp parallel
    {
        float* tmp = (float*)malloc((size_t)k * sizeof(float));
#pragma omp for schedule(static)
        for (long r = 0; r < rows; r++) {
            dequantize_row(type, (const uint8_t*)x + r * rb, tmp, k);
            for (long i = 0; i < k; i++) y[r * k + i] = qo_f32_to_bf16(tmp[i]);
        }
        free(tmp);
    }
}

/* ------------------------------------------------- integer block dot sums */

static inline const int8_t* q81_q(const uint8_t* xq, long blk) {
    return (const int8_t*)(xq + blk * QO_Q8_1_BYTES + 4);
}
static inline float q81_d(const uint8_t* xq, long blk) { return qo_f16_to_f32(rd16(xq + blk * QO_Q8_1_BYTES)); }
static inline float q81_s(const uint8_t* xq, long blk) { return qo_f16_to_f32(rd16(xq + blk * QO_Q8_1_BYTES + 2)); }

static inline int32_t dot_q8_0(const uint8_t* wb, const int8_t* xq) {
    int32_t s = 0;
    for (int i = 0; i < 32; i++) s += (int32_t)(int8_t)wb[2 + i] * (int32_t)xq[i];
    return s;
}
/* sub-block j of a Q4_K super-block against the matching 32 activations */
static inline int32_t dot_q4_k_sub(const uint8_t* wb, int j, const int8_t* xq) {
    const uint8_t* q = wb + 16 + 32 * (j >> 1);
    int32_t s = 0;
    if (j & 1) for (int i = 0; i < 32; i++) s += (int32_t)(q[i] >> 4) * (int32_t)xq[i];
    else       for (int i = 0; i < 32; i++) s += (int32_t)(q[i] & 15) * (int32_t)xq[i];
    return s;
}
/* 16-group g of a Q6_K super-block against the matching 16 activations */
static inline int32_t dot_q6_k_grp(const uint8_t* wb, int g, const int8_t* xq16) {
    int32_t s = 0;
    for (int i = 0; i < 16; i++) s += (int32_t)(q6k_code(wb, wb + 128, 16 * g + i) - 32) * (int32_t)xq16[i];
    return s;
}

void qo_block_dots(int type, const void* vw, const void* vxq, int32_t* out, long n, long k) {
    const uint8_t* w = (const uint8_t*)vw;
    const uint8_t* xq = (const uint8_t*)vxq;
    long rb = qo_row_bytes(type, k);
#pragma omp parallel for schedule(static)
    for (long r = 0; r < n; r++) {
        const uint8_t* wr = w + r * rb;
        if (type == QO_TYPE_Q8_0) {
            for (long b = 0; b < k / 32; b++) out[r * (k / 32) + b] = dot_q8_0(wr + b * QO_Q8_0_BYTES, q81_q(xq, b));
        } else if (type == QO_TYPE_Q4_K) {
            for (long b = 0; b < k / 256; b++)
                for (int j = 0; j < 8; j++)
                    out[r * (k / 32) + 8 * b + j] = dot_q4_k_sub(wr + b * QO_Q4_K_BYTES, j, q81_q(xq, 8 * b + j));
        } else if (type == QO_TYPE_Q6_K) {
            for (long b = 0; b < k / 256; b++)
                for (int g = 0; g < 16; g++)
                    out[r * (k / 16) + 16 * b + g] =
                        dot_q6_k_grp(wr + b * QO_Q6_K_BYTES, g, q81_q(xq, 8 * b + (g >> 1)) + 16 * (g & 1));
        }
    }
}

/* ------------------------------------------------------------------ matvec */

static float row_dot(int type, const uint8_t* wr, const uint8_t* xq, long k) {
    float y = 0.0f;
    if (type == QO_TYPE_Q8_0) {
        for (long b = 0; b < k / 32; b++) {
            const uint8_t* wb = wr + b * QO_Q8_0_BYTES;
            float dd = qo_f16_to_f32(rd16(wb)) * q81_d(xq, b);
            y += dd * (float)dot_q8_0(wb, q81_q(xq, b));
        }
    } else if (type == QO_TYPE_Q4_K) {
        for (long b = 0; b < k / 256; b++) {
            const uint8_t* wb = wr + b * QO_Q4_K_BYTES;
            float d = qo_f16_to_f32(rd16(wb)), dmin = qo_f16_to_f32(rd16(wb + 2));
            float acc_d = 0.0f, acc_m = 0.0f;
            for (int j = 0; j < 8; j++) {
                int sc, m;
                q4k_scale_min(j, wb + 4, &sc, &m);
                int32_t si = dot_q4_k_sub(wb, j, q81_q(xq, 8 * b + j));
                acc_d += q81_d(xq, 8 * b + j) * (float)(sc * si);
                acc_m += q81_s(xq, 8 * b + j) * (float)m;
            }
            y += d * acc_d - dmin * acc_m;
        }
    } else if (type == QO_TYPE_Q6_K) {
        for (long b = 0; b < k / 256; b++) {
            const uint8_t* wb = wr + b * QO_Q6_K_BYTES;
            float d = qo_f16_to_f32(rd16(wb + 208));
            const int8_t* sc = (const int8_t*)(wb + 192);
            float acc = 0.0f;
            for (int g = 0; g < 16; g++) {
                int32_t si = dot_q6_k_grp(wb, g, q81_q(xq, 8 * b + (g >> 1)) + 16 * (g & 1));
                acc += q81_d(xq, 8 * b + (g >> 1)) * (float)((int32_t)sc[g] * si);
            }
            y += d * acc;
        }
    }
    return y;
}

void qo_matvec(int type, const void* vw, const void* vxq, float* y, long m, long n, long k) {
    const uint8_t* w = (const uint8_t*)vw;
    const uint8_t* xq = (const uint8_t*)vxq;
    long rb = qo_row_bytes(type, k);
    long xb = qo_row_bytes(QO_TYPE_Q8_1, k);
#pragma omp parallel for schedule(static)
    for (long r = 0; r < n; r++)
        for (long i = 0; i < m; i++) y[i * n + r] = row_dot(type, w + r * rb, xq + i * xb, k);
}

/* ---------------------------------------------------------------- bf16 GEMM */

void qo_gemm_bf16(int type, const void* vw, const uint16_t* x, uint16_t* y, float* yf,
                  long m, long n, long k) {
    const uint8_t* w = (const uint8_t*)vw;
    long rb = qo_row_bytes(type, k);
    float* xf = (float*)malloc((size_t)m * k * sizeof(float));
    for (long i = 0; i < m * k; i++) xf[i] = qo_bf16_to_f32(x[i]);
#pragma omp parallel
    {
        float* wf = (float*)malloc((size_t)k * sizeof(float));
#pragma omp for schedule(static)
        for (long r = 0; r < n; r++) {
            dequantize_row(type, w + r * rb, wf, k);
            for (long i = 0; i < k; i++) wf[i] = qo_bf16_to_f32(qo_f32_to_bf16(wf[i]));
            for (long i = 0; i < m; i++) {
                /* 16 interleaved partial sums, then a fixed tree: every product is
                 * exact in binary32, only the additions round */
                float p[16] = {0};
                const float* xr = xf + i * k;
                long kk = 0;
                for (; kk + 16 <= k; kk += 16)
                    for (int l = 0; l < 16; l++) p[l] += xr[kk + l] * wf[kk + l];
                for (; kk < k; kk++) p[kk & 15] += xr[kk] * wf[kk];
                for (int s = 8; s > 0; s >>= 1)
                    for (int l = 0; l < s; l++) p[l] += p[l + s];
                if (yf) yf[i * n + r] = p[0];
                if (y) y[i * n + r] = qo_f32_to_bf16(p[0]);
            }
        }
        free(wf);
    }
    free(xf);
}

/* ------------------------------------------------------------ decoder pieces */

/* out = x * (1/sqrt(mean(x^2) + eps)) * gamma  (gamma optional), cf. the f64
 * normx_rmsnorm_kernel of the upstream (gpu-core/src/kernels/normx.hip:135-159) */
void qo_rmsnorm(const float* x, const float* gamma, float* out, long rows, long cols, float eps) {
    for (long r = 0; r < rows; r++) {
        double ss = 0.0;
        for (long c = 0; c < cols; c++) ss += (double)x[r * cols + c] * (double)x[r * cols + c];
        float inv = (float)(1.0 / sqrt(ss / (double)cols + (double)eps));
        for (long c = 0; c < cols; c++) {
            float v = x[r * cols + c] * inv;
            out[r * cols + c] = gamma ? v * gamma[c] : v;
        }
    }
}

/* NeoX rotate-half over the whole head, row r is head (r % heads_per_tok) of token
 * (r / heads_per_tok) at position pos0 + token; cf. rope_partial
 * (gpu-core/src/kernels/f64_infer.hip:107-132) with rotary_dim == head_dim. */
void qo_rope_neox(float* buf, long rows, long head_dim, long heads_per_tok, long pos0, float theta) {
    long half = head_dim / 2;
    for (long r = 0; r < rows; r++) {
        double pos = (double)(pos0 + r / heads_per_tok);
        float* h = buf + r * head_dim;
        for (long i = 0; i < half; i++) {
            double freq = pow((double)theta, -2.0 * (double)i / (double)head_dim);
            double c = cos(pos * freq), s = sin(pos * freq);
            double a = h[i], b = h[i + half];
            h[i] = (float)(a * c - b * s);
            h[i + half] = (float)(a * s + b * c);
        }
    }
}

static inline double gelu_tanh(double x) {
    return 0.5 * x * (1.0 + tanh(0.7978845608028654 * (x + 0.044715 * x * x * x)));
}
/* gelu_tanh(gate) * up, cf. gelu_mul (gpu-core/src/kernels/f64_infer.hip:134-150) */
void qo_gelu_mul(const float* gate, const float* up, float* out, long n) {
    for (long i = 0; i < n; i++) out[i] = (float)(gelu_tanh((double)gate[i]) * (double)up[i]);
}
void qo_silu_mul(const float* gate, const float* up, float* out, long n) {
    for (long i = 0; i < n; i++) {
        double g = gate[i];
        out[i] = (float)(g / (1.0 + exp(-g)) * (double)up[i]);
    }
}

void qo_attn_decode(const float* q, const uint16_t* kc, const uint16_t* vc, float* out,
                    long nqh, long nkv, long hd, long len) {
    long group = nqh / nkv;
    double scale = 1.0 / sqrt((double)hd);
    double* p = (double*)malloc((size_t)len * sizeof(double));
    for (long h = 0; h < nqh; h++) {
        long kv = h / group;
        double mx = -1e300;
        for (long t = 0; t < len; t++) {
            double s = 0.0;
            for (long i = 0; i < hd; i++)
                s += (double)q[h * hd + i] * (double)qo_f16_to_f32(kc[(t * nkv + kv) * hd + i]);
            p[t] = s * scale;
            if (p[t] > mx) mx = p[t];
        }
        double den = 0.0;
        for (long t = 0; t < len; t++) { p[t] = exp(p[t] - mx); den += p[t]; }
        for (long i = 0; i < hd; i++) {
            double acc = 0.0;
            for (long t = 0; t < len; t++) acc += p[t] * (double)qo_f16_to_f32(vc[(t * nkv + kv) * hd + i]);
            out[h * hd + i] = (float)(acc / den);
        }
    }
    free(p);
}

/* Attention over a whole sequence, the upstream's gqa_masked_attn restated (gpu-core/src/kernels/f64_infer.hip:42-91):
 * one softmax per (position p, head h) over all t keys in double precision; a masked score (p < prefix and
 * sp > p) is -1e30 as upstream; scores are q.k * kq_scale. */
void qo_attn_prefill(const float* q, const float* k, const float* v, float* out, long t, long nqh, long nkv, long hd,
                     long prefix, double kq_scale) {
    long group = nqh / nkv, qd = nqh * hd, kd = nkv * hd;
    double* sc = (double*)malloc((size_t)t * sizeof(double));
    for (long p = 0; p < t; p++)
        for (long h = 0; h < nqh; h++) {
            long kv = h / group;
            const float* qrow = q + p * qd + h * hd;
            double m = -1e300;
            for (long sp = 0; sp < t; sp++) {
                double dot = 0.0;
                for (long x = 0; x < hd; x++) dot += (double)qrow[x] * (double)k[sp * kd + kv * hd + x];
                sc[sp] = (p < prefix && sp > p) ? -1e30 : dot * kq_scale;
                if (sc[sp] > m) m = sc[sp];
            }
            double sum = 0.0;
            for (long sp = 0; sp < t; sp++) { sc[sp] = exp(sc[sp] - m); sum += sc[sp]; }
            for (long x = 0; x < hd; x++) {
                double acc = 0.0;
                for (long sp = 0; sp < t; sp++) acc += sc[sp] * (double)v[sp * kd + kv * hd + x];
                out[p * qd + h * hd + x] = (float)(acc / sum);
            }
        }
    free(sc);
}
