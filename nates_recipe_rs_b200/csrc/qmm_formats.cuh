// Per-format device code shared by the matvec, the block-dot instrumentation,
// the dequantizers and the quantizers.
//
// A "unit" is the slice of one weight row that one lane handles against
// activations it keeps in registers for the whole kernel:
//   Q4_K  64 elements = one 32-byte group of qs = sub-blocks 2g (low nibbles), 2g+1 (high)
//   Q6_K  64 elements = 16 consecutive l of one half: 4 quarter-runs of 16 elements,
//                       each run is exactly one 16-element scale group
//   Q8_0  32 elements = one block
// Every unit therefore yields whole per-block integer sums (the parity quantity)
// with no cross-lane exchange.
#pragma once
#include "qmm_common.cuh"

namespace qmm {

__device__ __forceinline__ int dp4a_u8s8(uint32_t a, int b, int c) {
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

// Exact int -> float without the conversion unit (which runs at a quarter of the
// arithmetic rate): for |i| < 2^22, float(i) = as_float(0x4B400000 + i) - 1.5*2^23.
__device__ __forceinline__ float small_int_to_float(int i) {
    return __int_as_float(0x4B400000 + i) - 12582912.0f;
}

// four consecutive 32-bit words starting at a 2-byte aligned address
__device__ __forceinline__ void ld_words4_align2(const uint8_t* p, uint32_t (&o)[4]) {
    const uintptr_t a = reinterpret_cast<uintptr_t>(p);
    const uint32_t* q = reinterpret_cast<const uint32_t*>(a & ~uintptr_t(3));
    const uint32_t sh = (a & 2u) * 8u;
    uint32_t w0 = q[0], w1 = q[1], w2 = q[2], w3 = q[3], w4 = q[4];
    o[0] = __funnelshift_r(w0, w1, sh);
    o[1] = __funnelshift_r(w1, w2, sh);
    o[2] = __funnelshift_r(w2, w3, sh);
    o[3] = __funnelshift_r(w3, w4, sh);
}
__device__ __forceinline__ uint32_t ld_u16(const uint8_t* p) {
    return *reinterpret_cast<const uint16_t*>(p);
}

// Activation registers of one unit: xw = packed int8 words, xs = float scales,
// xb = integer biases folded into the dot accumulators.
struct XRegs {
    int xw[16];
    float xs[4];
    int xb[4];
};

// Q8_1 accessors (row pointer 4-byte aligned)
__device__ __forceinline__ int q81_word(const uint8_t* xq, int blk, int w) {
    return *reinterpret_cast<const int*>(xq + (size_t)blk * Q8_1_BYTES + 4 + 4 * w);
}
__device__ __forceinline__ float q81_d(const uint8_t* xq, int blk) {
    return f16_bits_to_f32(ld_u16(xq + (size_t)blk * Q8_1_BYTES));
}
__device__ __forceinline__ float q81_s(const uint8_t* xq, int blk) {
    return f16_bits_to_f32(ld_u16(xq + (size_t)blk * Q8_1_BYTES + 2));
}

template <int TYPE>
struct Fmt;

// ----------------------------------------------------------------- Q4_K
template <>
struct Fmt<QMM_TYPE_Q4_K> {
    static constexpr int BLOCK_ELEMS = 256, BLOCK_BYTES = Q4_K_BYTES, UNIT_ELEMS = 64, SUMS_PER_UNIT = 2;
    static constexpr int W_ALIGN = 16;  // required alignment of the weight pointer

    __device__ static __forceinline__ void load_x(const uint8_t* xq, int u, XRegs& r) {
        const int j0 = 2 * u;  // = 8*(u>>2) + 2*(u&3)
#pragma unroll
        for (int w = 0; w < 8; ++w) {
            r.xw[w] = q81_word(xq, j0, w);
            r.xw[8 + w] = q81_word(xq, j0 + 1, w);
        }
        r.xs[0] = q81_d(xq, j0);
        r.xs[1] = q81_d(xq, j0 + 1);
        r.xs[2] = q81_s(xq, j0);
        r.xs[3] = q81_s(xq, j0 + 1);
    }
    __device__ static __forceinline__ void zero_x(XRegs& r) {
#pragma unroll
        for (int w = 0; w < 16; ++w) r.xw[w] = 0;
#pragma unroll
        for (int w = 0; w < 4; ++w) r.xs[w] = 0.f, r.xb[w] = 0;
    }

    struct WRegs {  // the weight words of one unit, fetched once and reused per activation row
        uint4 hdr, qa, qb;
    };
    __device__ static __forceinline__ void load_w(const uint8_t* row, int u, WRegs& wr) {
        const uint8_t* blk = row + (size_t)(u >> 2) * Q4_K_BYTES;
        wr.hdr = *reinterpret_cast<const uint4*>(blk);
        const uint4* q = reinterpret_cast<const uint4*>(blk + 16 + 32 * (u & 3));
        wr.qa = q[0];
        wr.qb = q[1];
    }
    // 6-bit scale / min codes of sub-blocks 2g and 2g+1, packed as two bytes each
    __device__ static __forceinline__ void scale_codes(const uint4& hdr, int g, uint32_t& sc2, uint32_t& m2) {
        const int sh = 16 * (g & 1);
        const uint32_t a = hdr.y >> sh, b = hdr.z >> sh, c = hdr.w >> sh;
        const uint32_t sc_lo = a & 0x3F3Fu, m_lo = b & 0x3F3Fu;
        const uint32_t sc_hi = (c & 0x0F0Fu) | ((a >> 2) & 0x3030u);
        const uint32_t m_hi = ((c >> 4) & 0x0F0Fu) | ((b >> 2) & 0x3030u);
        sc2 = (g < 2) ? sc_lo : sc_hi;
        m2 = (g < 2) ? m_lo : m_hi;
    }
    __device__ static __forceinline__ float dot(const WRegs& wr, int u, const XRegs& x, int* sums) {
        const uint32_t qa[4] = {wr.qa.x, wr.qa.y, wr.qa.z, wr.qa.w};
        const uint32_t qb[4] = {wr.qb.x, wr.qb.y, wr.qb.z, wr.qb.w};
        int s0 = 0, s0b = 0, s1 = 0, s1b = 0;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            s0 = dp4a_ss((int)(qa[w] & 0x0F0F0F0Fu), x.xw[w], s0);
            s0b = dp4a_ss((int)(qb[w] & 0x0F0F0F0Fu), x.xw[4 + w], s0b);
            s1 = dp4a_u8s8(qa[w] & 0xF0F0F0F0u, x.xw[8 + w], s1);  // 16 * (high nibble) . x
            s1b = dp4a_u8s8(qb[w] & 0xF0F0F0F0u, x.xw[12 + w], s1b);
        }
        const int sum0 = s0 + s0b;
        const int sum1 = (s1 + s1b) >> 4;  // exact: a multiple of 16
        if (sums) {
            sums[0] = sum0;
            sums[1] = sum1;
        }
        uint32_t sc2, m2;
        scale_codes(wr.hdr, u & 3, sc2, m2);
        const float d = f16_bits_to_f32(wr.hdr.x & 0xFFFFu), dmin = f16_bits_to_f32(wr.hdr.x >> 16);
        // |sc*sum| <= 63*32*15*127 < 2^22
        const float accd = x.xs[0] * small_int_to_float((int)(sc2 & 0xFFu) * sum0) +
                           x.xs[1] * small_int_to_float((int)(sc2 >> 8) * sum1);
        const float accm = x.xs[2] * small_int_to_float((int)(m2 & 0xFFu)) + x.xs[3] * small_int_to_float((int)(m2 >> 8));
        return d * accd - dmin * accm;
    }
};

// ----------------------------------------------------------------- Q6_K
template <>
struct Fmt<QMM_TYPE_Q6_K> {
    static constexpr int BLOCK_ELEMS = 256, BLOCK_BYTES = Q6_K_BYTES, UNIT_ELEMS = 64, SUMS_PER_UNIT = 4;
    static constexpr int W_ALIGN = 2;

    // unit u: block b = u>>2, half h = (u>>1)&1, l0 = 16*(u&1); run t covers x block 8b+4h+t, elements l0..l0+15
    __device__ static __forceinline__ void load_x(const uint8_t* xq, int u, XRegs& r) {
        const int j0 = 8 * (u >> 2) + 4 * ((u >> 1) & 1);
        const int w0 = 4 * (u & 1);
#pragma unroll
        for (int t = 0; t < 4; ++t) {
            int sx = 0;
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                r.xw[4 * t + w] = q81_word(xq, j0 + t, w0 + w);
                sx = dp4a_ss(0x01010101, r.xw[4 * t + w], sx);
            }
            r.xs[t] = q81_d(xq, j0 + t);
            r.xb[t] = -32 * sx;  // sum((q-32)*x) = sum(q*x) - 32*sum(x)
        }
    }
    __device__ static __forceinline__ void zero_x(XRegs& r) {
#pragma unroll
        for (int w = 0; w < 16; ++w) r.xw[w] = 0;
#pragma unroll
        for (int w = 0; w < 4; ++w) r.xs[w] = 0.f, r.xb[w] = 0;
    }

    struct WRegs {
        uint32_t a[4], b[4], h[4], sc[2], d;
    };
    __device__ static __forceinline__ void load_w(const uint8_t* row, int u, WRegs& wr) {
        const uint8_t* blk = row + (size_t)(u >> 2) * Q6_K_BYTES;
        const int h = (u >> 1) & 1, l0 = 16 * (u & 1);
        ld_words4_align2(blk + 64 * h + l0, wr.a);
        ld_words4_align2(blk + 64 * h + 32 + l0, wr.b);
        ld_words4_align2(blk + 128 + 32 * h + l0, wr.h);
        wr.sc[0] = lds_u32_align2(blk + 192 + 8 * h);
        wr.sc[1] = lds_u32_align2(blk + 196 + 8 * h);
        wr.d = ld_u16(blk + 208);
    }
    __device__ static __forceinline__ float dot(const WRegs& wr, int u, const XRegs& x, int* sums) {
        int s[4] = {x.xb[0], x.xb[1], x.xb[2], x.xb[3]};
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const uint32_t A = wr.a[w], B = wr.b[w], H = wr.h[w];
            const uint32_t q0 = (A & 0x0F0F0F0Fu) | ((H << 4) & 0x30303030u);
            const uint32_t q1 = (B & 0x0F0F0F0Fu) | ((H << 2) & 0x30303030u);
            const uint32_t q2 = ((A >> 4) & 0x0F0F0F0Fu) | (H & 0x30303030u);
            const uint32_t q3 = ((B >> 4) & 0x0F0F0F0Fu) | ((H >> 2) & 0x30303030u);
            s[0] = dp4a_ss((int)q0, x.xw[w], s[0]);
            s[1] = dp4a_ss((int)q1, x.xw[4 + w], s[1]);
            s[2] = dp4a_ss((int)q2, x.xw[8 + w], s[2]);
            s[3] = dp4a_ss((int)q3, x.xw[12 + w], s[3]);
        }
        if (sums) {
#pragma unroll
            for (int t = 0; t < 4; ++t) sums[t] = s[t];
        }
        // scale of run t is byte (u&1) + 2t of the eight scale bytes of this half
        const int bsh = 8 * (u & 1);
        const int c0 = (int)(int8_t)(wr.sc[0] >> bsh), c1 = (int)(int8_t)(wr.sc[0] >> (16 + bsh));
        const int c2 = (int)(int8_t)(wr.sc[1] >> bsh), c3 = (int)(int8_t)(wr.sc[1] >> (16 + bsh));
        // |scale*sum| can reach 2^24, so the two factors are converted separately (each exact)
        // and multiplied in float: the product of two exact integers below 2^24 in magnitude
        // is rounded once, like the int->float conversion of the integer product would be.
        float acc = x.xs[0] * (small_int_to_float(c0) * small_int_to_float(s[0]));
        acc += x.xs[1] * (small_int_to_float(c1) * small_int_to_float(s[1]));
        acc += x.xs[2] * (small_int_to_float(c2) * small_int_to_float(s[2]));
        acc += x.xs[3] * (small_int_to_float(c3) * small_int_to_float(s[3]));
        return f16_bits_to_f32(wr.d) * acc;
    }
};

// ----------------------------------------------------------------- Q8_0
template <>
struct Fmt<QMM_TYPE_Q8_0> {
    static constexpr int BLOCK_ELEMS = 32, BLOCK_BYTES = Q8_0_BYTES, UNIT_ELEMS = 32, SUMS_PER_UNIT = 1;
    static constexpr int W_ALIGN = 2;

    __device__ static __forceinline__ void load_x(const uint8_t* xq, int u, XRegs& r) {
#pragma unroll
        for (int w = 0; w < 8; ++w) r.xw[w] = q81_word(xq, u, w);
        r.xs[0] = q81_d(xq, u);
    }
    __device__ static __forceinline__ void zero_x(XRegs& r) {
#pragma unroll
        for (int w = 0; w < 8; ++w) r.xw[w] = 0;
        r.xs[0] = 0.f;
    }
    struct WRegs {
        uint32_t q[8], d;
    };
    __device__ static __forceinline__ void load_w(const uint8_t* row, int u, WRegs& wr) {
        const uint8_t* blk = row + (size_t)u * Q8_0_BYTES;
        wr.d = ld_u16(blk);
        uint32_t lo[4], hi[4];
        ld_words4_align2(blk + 2, lo);
        ld_words4_align2(blk + 18, hi);
#pragma unroll
        for (int w = 0; w < 4; ++w) wr.q[w] = lo[w], wr.q[4 + w] = hi[w];
    }
    __device__ static __forceinline__ float dot(const WRegs& wr, int, const XRegs& x, int* sums) {
        int s0 = 0, s1 = 0;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            s0 = dp4a_ss((int)wr.q[w], x.xw[w], s0);
            s1 = dp4a_ss((int)wr.q[4 + w], x.xw[4 + w], s1);
        }
        const int sum = s0 + s1;
        if (sums) sums[0] = sum;
        return (f16_bits_to_f32(wr.d) * x.xs[0]) * small_int_to_float(sum);
    }
};

// ------------------------------------------------ element-wise dequantization
// Value of element e of the block at blk, every operation individually rounded
// (no fused multiply-add), so the result equals the CPU oracle's bit for bit.
template <int TYPE>
__device__ __forceinline__ float dequant_elem(const uint8_t* blk, int e);

template <>
__device__ __forceinline__ float dequant_elem<QMM_TYPE_Q8_0>(const uint8_t* blk, int e) {
    return __fmul_rn(f16_bits_to_f32(ld_u16(blk)), (float)(int8_t)blk[2 + e]);
}
template <>
__device__ __forceinline__ float dequant_elem<QMM_TYPE_Q4_K>(const uint8_t* blk, int e) {
    const int j = e >> 5, l = e & 31;
    const uint8_t* s = blk + 4;
    int sc, m;
    if (j < 4) {
        sc = s[j] & 63;
        m = s[j + 4] & 63;
    } else {
        sc = (s[j + 4] & 15) | ((s[j - 4] >> 6) << 4);
        m = (s[j + 4] >> 4) | ((s[j] >> 6) << 4);
    }
    const uint8_t b = blk[16 + 32 * (j >> 1) + l];
    const int q = (j & 1) ? (b >> 4) : (b & 15);
    const float d = f16_bits_to_f32(ld_u16(blk)), dmin = f16_bits_to_f32(ld_u16(blk + 2));
    return __fsub_rn(__fmul_rn(__fmul_rn(d, (float)sc), (float)q), __fmul_rn(dmin, (float)m));
}
template <>
__device__ __forceinline__ float dequant_elem<QMM_TYPE_Q6_K>(const uint8_t* blk, int e) {
    const int h = e >> 7, r = e & 127, t = r >> 5, l = r & 31;
    const uint8_t b = blk[64 * h + l + 32 * (t & 1)];
    const int lo = (t < 2) ? (b & 15) : (b >> 4);
    const int hi = (blk[128 + 32 * h + l] >> (2 * t)) & 3;
    const int q = (lo | (hi << 4)) - 32;
    const float d = f16_bits_to_f32(ld_u16(blk + 208));
    return __fmul_rn(__fmul_rn(d, (float)(int8_t)blk[192 + (e >> 4)]), (float)q);
}

}  // namespace qmm
