// Per-format device code shared by the matvec, the block-dot instrumentation,
// the dequantizers and the quantizers.
//
// A "unit" is the slice of one weight row that one lane handles against
// activations it keeps in registers for the whole kernel:
//   Q4_K  64*UW elements = UW 32-byte groups of qs; group g = sub-blocks 2g (low nibbles), 2g+1 (high)
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

// The same by 32-bit shared-memory address (the matvec's inner loop: no 64-bit address arithmetic)
__device__ __forceinline__ uint32_t sld_u32(uint32_t a) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ uint4 sld_v4(uint32_t a) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
    return v;
}
__device__ __forceinline__ uint32_t sld_u16(uint32_t a) {
    uint32_t v;
    asm volatile("{ .reg .b16 h; ld.shared.u16 h, [%1]; cvt.u32.u16 %0, h; }" : "=r"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ void sld_words4_align2(uint32_t a, uint32_t (&o)[4]) {
    const uint32_t q = a & ~3u, sh = (a & 2u) * 8u;
    const uint32_t w0 = sld_u32(q), w1 = sld_u32(q + 4), w2 = sld_u32(q + 8), w3 = sld_u32(q + 12), w4 = sld_u32(q + 16);
    o[0] = __funnelshift_r(w0, w1, sh);
    o[1] = __funnelshift_r(w1, w2, sh);
    o[2] = __funnelshift_r(w2, w3, sh);
    o[3] = __funnelshift_r(w3, w4, sh);
}
__device__ __forceinline__ uint32_t sld_u32_align2(uint32_t a) {
    const uint32_t q = a & ~3u;
    return __funnelshift_r(sld_u32(q), sld_u32(q + 4), (a & 2u) * 8u);
}

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

// byte `idx` (0..3, may be a run-time value) of w, zero-extended: one PRMT
__device__ __forceinline__ uint32_t byte_of(uint32_t w, uint32_t idx) { return __byte_perm(w, 0u, 0x4440u | idx); }
// float(byte idx of w), exact: PRMT builds the bits of 2^23 + byte, one subtraction removes 2^23
__device__ __forceinline__ float byte_to_float(uint32_t w, uint32_t idx) {
    return __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7540u | idx)) - 8388608.0f;
}

// Fmt<TYPE, UW>: UW is the unit width, used by Q4_K only (UW = 1, 2 or 4 consecutive
// 32-byte groups of qs, i.e. 64, 128 or 256 elements per lane); wider units decode the
// packed 6-bit scales once for more weights at the price of more activation registers.
template <int TYPE, int UW>
struct Fmt;

// ----------------------------------------------------------------- Q4_K
template <int UW>
struct Fmt<QMM_TYPE_Q4_K, UW> {
    static_assert(UW == 1 || UW == 2 || UW == 4, "unit = 1, 2 or 4 groups of a super-block");
    static constexpr int BLOCK_ELEMS = 256, BLOCK_BYTES = Q4_K_BYTES, UNIT_ELEMS = 64 * UW, SUMS_PER_UNIT = 2 * UW;
    static constexpr int W_ALIGN = 16;  // required alignment of the weight pointer
    static constexpr int UNITS_PER_BLOCK = 4 / UW;

    // activations of unit u: the 2*UW Q8_1 blocks 2*UW*u .. of the row
    struct XRegs {
        int xw[16 * UW];
        float xd[2 * UW], xs[2 * UW];
    };
    __device__ static __forceinline__ void load_x(const uint8_t* xq, int u, XRegs& r) {
        const int j0 = 2 * UW * u;
#pragma unroll
        for (int j = 0; j < 2 * UW; ++j) {
#pragma unroll
            for (int w = 0; w < 8; ++w) r.xw[8 * j + w] = q81_word(xq, j0 + j, w);
            r.xd[j] = q81_d(xq, j0 + j);
            r.xs[j] = q81_s(xq, j0 + j);
        }
    }
    __device__ static __forceinline__ void zero_x(XRegs& r) {
#pragma unroll
        for (int w = 0; w < 16 * UW; ++w) r.xw[w] = 0;
#pragma unroll
        for (int w = 0; w < 2 * UW; ++w) r.xd[w] = 0.f, r.xs[w] = 0.f;
    }

    struct WRegs {  // the weight words of one unit, fetched once and reused per activation row
        uint4 hdr, q[2 * UW];
    };
    __device__ static __forceinline__ void load_w(const uint8_t* row, int u, WRegs& wr) {
        const uint8_t* blk = row + (uint32_t)(u / UNITS_PER_BLOCK) * Q4_K_BYTES;
        wr.hdr = *reinterpret_cast<const uint4*>(blk);
        const uint4* q = reinterpret_cast<const uint4*>(blk + 16 + 32 * UW * (u % UNITS_PER_BLOCK));
#pragma unroll
        for (int i = 0; i < 2 * UW; ++i) wr.q[i] = q[i];
    }
    // byte offset of the unit's super-block within a row (loop invariant for a lane)
    __device__ static __forceinline__ uint32_t unit_offset(int u) { return (uint32_t)(u / UNITS_PER_BLOCK) * Q4_K_BYTES; }
    // the same fetch from shared memory: row_s = shared address of the row, blk_off = unit_offset(u)
    __device__ static __forceinline__ void load_w_s(uint32_t row_s, uint32_t blk_off, int u, WRegs& wr) {
        const uint32_t blk = row_s + blk_off;
        wr.hdr = sld_v4(blk);
        const uint32_t q = blk + 16 + 32 * UW * (u % UNITS_PER_BLOCK);
#pragma unroll
        for (int i = 0; i < 2 * UW; ++i) wr.q[i] = sld_v4(q + 16 * i);
    }
    __device__ static __forceinline__ float dot(const WRegs& wr, int u, const XRegs& x, int* sums) {
        // integer sums of the 2*UW sub-blocks
        int sum[2 * UW];
#pragma unroll
        for (int g = 0; g < UW; ++g) {
            const uint32_t qa[4] = {wr.q[2 * g].x, wr.q[2 * g].y, wr.q[2 * g].z, wr.q[2 * g].w};
            const uint32_t qb[4] = {wr.q[2 * g + 1].x, wr.q[2 * g + 1].y, wr.q[2 * g + 1].z, wr.q[2 * g + 1].w};
            const int* xl = x.xw + 16 * g;  // sub-block 2g (low nibbles); +8: sub-block 2g+1 (high nibbles)
            int s0 = 0, s0b = 0, s1 = 0, s1b = 0;
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                s0 = dp4a_ss((int)(qa[w] & 0x0F0F0F0Fu), xl[w], s0);
                s0b = dp4a_ss((int)(qb[w] & 0x0F0F0F0Fu), xl[4 + w], s0b);
                s1 = dp4a_u8s8(qa[w] & 0xF0F0F0F0u, xl[8 + w], s1);  // 16 * (high nibble) . x
                s1b = dp4a_u8s8(qb[w] & 0xF0F0F0F0u, xl[12 + w], s1b);
            }
            sum[2 * g] = s0 + s0b;
            sum[2 * g + 1] = (s1 + s1b) >> 4;  // exact: a multiple of 16
        }
        if (sums) {
#pragma unroll
            for (int j = 0; j < 2 * UW; ++j) sums[j] = sum[j];
        }
        // 6-bit scale / min codes, four per word: A = sub-blocks 0..3, B = sub-blocks 4..7
        const uint32_t scA = wr.hdr.y & 0x3F3F3F3Fu, mA = wr.hdr.z & 0x3F3F3F3Fu;
        const uint32_t scB = (wr.hdr.w & 0x0F0F0F0Fu) | ((wr.hdr.y >> 2) & 0x30303030u);
        const uint32_t mB = ((wr.hdr.w >> 4) & 0x0F0F0F0Fu) | ((wr.hdr.z >> 2) & 0x30303030u);
        float accd = 0.f, accm = 0.f;
        if constexpr (UW == 4) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const uint32_t sc4 = j < 4 ? scA : scB, m4 = j < 4 ? mA : mB;
                accd += x.xd[j] * small_int_to_float((int)byte_of(sc4, j & 3) * sum[j]);  // |sc*sum| < 2^22
                accm += x.xs[j] * byte_to_float(m4, j & 3);
            }
        } else {
            // first sub-block of the unit: j0 = 2*UW*(u % UNITS_PER_BLOCK); lanes differ, a lane never changes
            const int j0 = 2 * UW * (u % UNITS_PER_BLOCK);
            const uint32_t sc4 = j0 < 4 ? scA : scB, m4 = j0 < 4 ? mA : mB;
#pragma unroll
            for (int j = 0; j < 2 * UW; ++j) {
                const uint32_t idx = (uint32_t)(j0 + j) & 3u;
                accd += x.xd[j] * small_int_to_float((int)byte_of(sc4, idx) * sum[j]);
                accm += x.xs[j] * byte_to_float(m4, idx);
            }
        }
        const float d = f16_bits_to_f32(wr.hdr.x & 0xFFFFu), dmin = f16_bits_to_f32(wr.hdr.x >> 16);
        return d * accd - dmin * accm;
    }
};

// ----------------------------------------------------------------- Q6_K
template <int UW>
struct Fmt<QMM_TYPE_Q6_K, UW> {
    static_assert(UW == 1, "Q6_K has one unit width");
    static constexpr int BLOCK_ELEMS = 256, BLOCK_BYTES = Q6_K_BYTES, UNIT_ELEMS = 64, SUMS_PER_UNIT = 4;
    static constexpr int W_ALIGN = 2;

    struct XRegs {
        int xw[16];
        float xd[4];
        int xb[4];  // -32 * sum of the activations of a run, folded into the dot accumulator
    };
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
            r.xd[t] = q81_d(xq, j0 + t);
            r.xb[t] = -32 * sx;  // sum((q-32)*x) = sum(q*x) - 32*sum(x)
        }
    }
    __device__ static __forceinline__ void zero_x(XRegs& r) {
#pragma unroll
        for (int w = 0; w < 16; ++w) r.xw[w] = 0;
#pragma unroll
        for (int w = 0; w < 4; ++w) r.xd[w] = 0.f, r.xb[w] = 0;
    }

    struct WRegs {
        uint32_t a[4], b[4], h[4], sc[2], d;
    };
    __device__ static __forceinline__ void load_w(const uint8_t* row, int u, WRegs& wr) {
        const uint8_t* blk = row + (uint32_t)(u >> 2) * Q6_K_BYTES;
        const int h = (u >> 1) & 1, l0 = 16 * (u & 1);
        ld_words4_align2(blk + 64 * h + l0, wr.a);
        ld_words4_align2(blk + 64 * h + 32 + l0, wr.b);
        ld_words4_align2(blk + 128 + 32 * h + l0, wr.h);
        wr.sc[0] = lds_u32_align2(blk + 192 + 8 * h);
        wr.sc[1] = lds_u32_align2(blk + 196 + 8 * h);
        wr.d = ld_u16(blk + 208);
    }
    __device__ static __forceinline__ uint32_t unit_offset(int u) { return (uint32_t)(u >> 2) * Q6_K_BYTES; }
    __device__ static __forceinline__ void load_w_s(uint32_t row_s, uint32_t blk_off, int u, WRegs& wr) {
        const uint32_t blk = row_s + blk_off;
        const int h = (u >> 1) & 1, l0 = 16 * (u & 1);
        sld_words4_align2(blk + 64 * h + l0, wr.a);
        sld_words4_align2(blk + 64 * h + 32 + l0, wr.b);
        sld_words4_align2(blk + 128 + 32 * h + l0, wr.h);
        wr.sc[0] = sld_u32_align2(blk + 192 + 8 * h);
        wr.sc[1] = sld_u32_align2(blk + 196 + 8 * h);
        wr.d = sld_u16(blk + 208);
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
        // |scale*sum| can reach 2^23, so the two factors are converted separately (each exact)
        // and multiplied in float; the product of two integers stays below 2^24 and is exact.
        float acc = x.xd[0] * (small_int_to_float(c0) * small_int_to_float(s[0]));
        acc += x.xd[1] * (small_int_to_float(c1) * small_int_to_float(s[1]));
        acc += x.xd[2] * (small_int_to_float(c2) * small_int_to_float(s[2]));
        acc += x.xd[3] * (small_int_to_float(c3) * small_int_to_float(s[3]));
        return f16_bits_to_f32(wr.d) * acc;
    }
};

// ----------------------------------------------------------------- Q8_0
template <int UW>
struct Fmt<QMM_TYPE_Q8_0, UW> {
    static_assert(UW == 1, "Q8_0 has one unit width");
    static constexpr int BLOCK_ELEMS = 32, BLOCK_BYTES = Q8_0_BYTES, UNIT_ELEMS = 32, SUMS_PER_UNIT = 1;
    static constexpr int W_ALIGN = 2;

    struct XRegs {
        int xw[8];
        float xd;
    };
    __device__ static __forceinline__ void load_x(const uint8_t* xq, int u, XRegs& r) {
#pragma unroll
        for (int w = 0; w < 8; ++w) r.xw[w] = q81_word(xq, u, w);
        r.xd = q81_d(xq, u);
    }
    __device__ static __forceinline__ void zero_x(XRegs& r) {
#pragma unroll
        for (int w = 0; w < 8; ++w) r.xw[w] = 0;
        r.xd = 0.f;
    }
    struct WRegs {
        uint32_t q[8], d;
    };
    __device__ static __forceinline__ void load_w(const uint8_t* row, int u, WRegs& wr) {
        const uint8_t* blk = row + (uint32_t)u * Q8_0_BYTES;
        wr.d = ld_u16(blk);
        uint32_t lo[4], hi[4];
        ld_words4_align2(blk + 2, lo);
        ld_words4_align2(blk + 18, hi);
#pragma unroll
        for (int w = 0; w < 4; ++w) wr.q[w] = lo[w], wr.q[4 + w] = hi[w];
    }
    __device__ static __forceinline__ uint32_t unit_offset(int u) { return (uint32_t)u * Q8_0_BYTES; }
    __device__ static __forceinline__ void load_w_s(uint32_t row_s, uint32_t blk_off, int, WRegs& wr) {
        const uint32_t blk = row_s + blk_off;
        wr.d = sld_u16(blk);
        uint32_t lo[4], hi[4];
        sld_words4_align2(blk + 2, lo);
        sld_words4_align2(blk + 18, hi);
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
        const int sum = s0 + s1;  // |sum| <= 32*128*127 < 2^22
        if (sums) sums[0] = sum;
        return (f16_bits_to_f32(wr.d) * x.xd) * small_int_to_float(sum);
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
