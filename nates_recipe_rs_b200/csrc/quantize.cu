// Quantizers (activations -> Q8_1, weights -> Q8_0 / Q4_K / Q6_K) and element-wise
// dequantizers.  None of these is on the steady-state decode path except
// quantize_q8_1; they exist for model construction, for the decode of a weight
// window (the upstream's widen step, gpu-core/src/kernels/f64_infer.hip:12-23) and
// for parity checks.  Every float operation is a single correctly rounded IEEE
// operation in the same order as the CPU oracle, so packed bytes and decoded
// values match it bit for bit.  Rounding to integer codes is half away from zero
// (the upstream's convention, gpu-core/src/kernels/quantizedx.hip:8).
#include "qmm_formats.cuh"

namespace qmm {

constexpr float F16_MAX_F = 65504.0f;

__device__ __forceinline__ int clampi(int v, int lo, int hi) { return v < lo ? lo : (v > hi ? hi : v); }
__device__ __forceinline__ uint16_t f32_to_f16_bits(float f) { return __half_as_ushort(__float2half_rn(f)); }
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ void st_u16(uint8_t* p, uint16_t v) { *reinterpret_cast<uint16_t*>(p) = v; }

// ---- 32-element blocks: one warp per block, one element per lane ----
template <bool WITH_SUM>
__global__ void quantize_q8_kernel(const float* __restrict__ x, uint8_t* __restrict__ out, long n_blocks) {
    // Only the activation quantizer takes part in programmatic dependent launch: the kernel after
    // it (a matvec) may start streaming its weights early.  The Q8_0 weight quantizer must not
    // release dependents early, since what follows may read the weights it is still writing.
    if (WITH_SUM) {
        pdl_release_dependents();
        pdl_wait_prior_grids();
    }
    const int lane = threadIdx.x & 31;
    const long blk = ((long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    if (blk >= n_blocks) return;
    const float v = x[blk * 32 + lane];
    const float amax = warp_max(fabsf(v));
    const uint16_t dh = f32_to_f16_bits(fminf(__fdiv_rn(amax, 127.0f), F16_MAX_F));
    const float df = f16_bits_to_f32(dh);
    const int q = (df > 0.0f) ? clampi((int)roundf(__fdiv_rn(v, df)), -127, 127) : 0;
    uint8_t* o = out + blk * (WITH_SUM ? Q8_1_BYTES : Q8_0_BYTES);
    o[(WITH_SUM ? 4 : 2) + lane] = (uint8_t)(int8_t)q;
    if (WITH_SUM) {
        int sum = q;
#pragma unroll
        for (int s = 16; s > 0; s >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, s);
        if (lane == 0) {
            st_u16(o, dh);
            st_u16(o + 2, f32_to_f16_bits(__fmul_rn(df, (float)sum)));
        }
    } else if (lane == 0) {
        st_u16(o, dh);
    }
}

// ---- Q4_K: one warp per super-block; lane l holds elements 8*(l&3).. of sub-block l>>2 ----
__global__ void quantize_q4_k_kernel(const float* __restrict__ x, uint8_t* __restrict__ out, long n_blocks) {
    const int lane = threadIdx.x & 31;
    const long blk = ((long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    if (blk >= n_blocks) return;
    const int j = lane >> 2, i0 = 8 * (lane & 3);
    float v[8];
    const float4* src = reinterpret_cast<const float4*>(x + blk * 256 + 32 * j + i0);
    const float4 a = src[0], b = src[1];
    v[0] = a.x, v[1] = a.y, v[2] = a.z, v[3] = a.w, v[4] = b.x, v[5] = b.y, v[6] = b.z, v[7] = b.w;
    float mn = v[0], mx = v[0];
#pragma unroll
    for (int i = 1; i < 8; ++i) mn = fminf(mn, v[i]), mx = fmaxf(mx, v[i]);
#pragma unroll
    for (int o = 1; o <= 2; o <<= 1) {
        mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    }
    const float lo = fmaxf(0.0f, -mn);
    const float step = fmaxf(0.0f, __fdiv_rn(__fadd_rn(mx, lo), 15.0f));
    float max_step = step, max_lo = lo;
#pragma unroll
    for (int o = 4; o <= 16; o <<= 1) {
        max_step = fmaxf(max_step, __shfl_xor_sync(0xffffffffu, max_step, o));
        max_lo = fmaxf(max_lo, __shfl_xor_sync(0xffffffffu, max_lo, o));
    }
    const uint16_t dh = f32_to_f16_bits(fminf(__fdiv_rn(max_step, 63.0f), F16_MAX_F));
    const uint16_t mh = f32_to_f16_bits(fminf(__fdiv_rn(max_lo, 63.0f), F16_MAX_F));
    const float d = f16_bits_to_f32(dh), dmin = f16_bits_to_f32(mh);
    const int sc = (d > 0.0f) ? clampi((int)roundf(__fdiv_rn(step, d)), 0, 63) : 0;
    const int m = (dmin > 0.0f) ? clampi((int)roundf(__fdiv_rn(lo, dmin)), 0, 63) : 0;
    const float ds = __fmul_rn(d, (float)sc), off = __fmul_rn(dmin, (float)m);
    uint32_t codes = 0;  // eight 4-bit codes
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int q = (ds > 0.0f) ? clampi((int)roundf(__fdiv_rn(__fadd_rn(v[i], off), ds)), 0, 15) : 0;
        codes |= (uint32_t)q << (4 * i);
    }
    uint8_t* o = out + blk * Q4_K_BYTES;
    // low nibbles come from even sub-blocks, high nibbles from the next sub-block (lane + 4)
    const uint32_t hi_codes = __shfl_down_sync(0xffffffffu, codes, 4);
    if ((j & 1) == 0) {
        uint32_t w0 = 0, w1 = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            w0 |= (((codes >> (4 * i)) & 15u) | (((hi_codes >> (4 * i)) & 15u) << 4)) << (8 * i);
            w1 |= (((codes >> (4 * (i + 4))) & 15u) | (((hi_codes >> (4 * (i + 4))) & 15u) << 4)) << (8 * i);
        }
        *reinterpret_cast<uint2*>(o + 16 + 32 * (j >> 1) + i0) = make_uint2(w0, w1);
    }
    // scale / min codes of all eight sub-blocks to lane 0
    int scj[8], mj[8];
#pragma unroll
    for (int t = 0; t < 8; ++t) {
        scj[t] = __shfl_sync(0xffffffffu, sc, 4 * t);
        mj[t] = __shfl_sync(0xffffffffu, m, 4 * t);
    }
    if (lane == 0) {
        uint32_t s[3] = {0, 0, 0};
        uint8_t sb[12];
#pragma unroll
        for (int t = 0; t < 12; ++t) sb[t] = 0;
#pragma unroll
        for (int t = 0; t < 8; ++t) {
            if (t < 4) {
                sb[t] |= (uint8_t)(scj[t] & 63);
                sb[t + 4] |= (uint8_t)(mj[t] & 63);
            } else {
                sb[t + 4] |= (uint8_t)((scj[t] & 15) | ((mj[t] & 15) << 4));
                sb[t - 4] |= (uint8_t)((scj[t] >> 4) << 6);
                sb[t] |= (uint8_t)((mj[t] >> 4) << 6);
            }
        }
#pragma unroll
        for (int t = 0; t < 12; ++t) s[t >> 2] |= (uint32_t)sb[t] << (8 * (t & 3));
        *reinterpret_cast<uint4*>(o) = make_uint4((uint32_t)dh | ((uint32_t)mh << 16), s[0], s[1], s[2]);
    }
}

// ---- Q6_K: one warp per super-block; lane l holds elements 8l..8l+7 (half of scale group l>>1) ----
__global__ void quantize_q6_k_kernel(const float* __restrict__ x, uint8_t* __restrict__ out, long n_blocks) {
    const int lane = threadIdx.x & 31;
    const long blk = ((long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    if (blk >= n_blocks) return;
    float v[8];
    const float4* src = reinterpret_cast<const float4*>(x + blk * 256 + 8 * lane);
    const float4 a = src[0], b = src[1];
    v[0] = a.x, v[1] = a.y, v[2] = a.z, v[3] = a.w, v[4] = b.x, v[5] = b.y, v[6] = b.z, v[7] = b.w;
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    const float gs = __fdiv_rn(amax, 31.0f);
    const float max_gs = warp_max(gs);
    const uint16_t dh = f32_to_f16_bits(fminf(__fdiv_rn(max_gs, 127.0f), F16_MAX_F));
    const float d = f16_bits_to_f32(dh);
    const int sc = (d > 0.0f) ? clampi((int)roundf(__fdiv_rn(gs, d)), 0, 127) : 0;
    const float ds = __fmul_rn(d, (float)sc);
    uint32_t lo4 = 0, hi2 = 0;  // eight low nibbles, eight 2-bit high parts
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int q = ((ds > 0.0f) ? clampi((int)roundf(__fdiv_rn(v[i], ds)), -32, 31) : 0) + 32;
        lo4 |= (uint32_t)(q & 15) << (4 * i);
        hi2 |= (uint32_t)(q >> 4) << (2 * i);
    }
    // lane = 16h + 4t + c holds l = 8c..8c+7 of run t of half h
    const int h = lane >> 4, t = (lane >> 2) & 3, c = lane & 3;
    uint8_t* o = out + blk * Q6_K_BYTES;
    const uint32_t lo4_up = __shfl_down_sync(0xffffffffu, lo4, 8);  // run t+2
    const uint32_t h1 = __shfl_down_sync(0xffffffffu, hi2, 4);
    const uint32_t h2 = __shfl_down_sync(0xffffffffu, hi2, 8);
    const uint32_t h3 = __shfl_down_sync(0xffffffffu, hi2, 12);
    if (t < 2) {
        uint8_t* ql = o + 64 * h + 32 * t + 8 * c;
#pragma unroll
        for (int i = 0; i < 8; ++i) ql[i] = (uint8_t)(((lo4 >> (4 * i)) & 15u) | (((lo4_up >> (4 * i)) & 15u) << 4));
    }
    if (t == 0) {
        uint8_t* qh = o + 128 + 32 * h + 8 * c;
#pragma unroll
        for (int i = 0; i < 8; ++i)
            qh[i] = (uint8_t)(((hi2 >> (2 * i)) & 3u) | (((h1 >> (2 * i)) & 3u) << 2) | (((h2 >> (2 * i)) & 3u) << 4) |
                              (((h3 >> (2 * i)) & 3u) << 6));
    }
    if ((lane & 1) == 0) o[192 + (lane >> 1)] = (uint8_t)(int8_t)sc;
    if (lane == 0) st_u16(o + 208, dh);
}

// ---- element-wise dequantization: one thread per element, coalesced stores ----
template <int TYPE, typename OUT>
__global__ void dequantize_kernel(const uint8_t* __restrict__ w, OUT* __restrict__ out, long n_elems) {
    using F = Fmt<TYPE, 1>;
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n_elems) return;
    const long blk = idx / F::BLOCK_ELEMS;
    const float v = dequant_elem<TYPE>(w + blk * F::BLOCK_BYTES, (int)(idx - blk * F::BLOCK_ELEMS));
    if constexpr (sizeof(OUT) == 4)
        out[idx] = v;
    else
        out[idx] = __float2bfloat16_rn(v);
}

// ---- the same values, eight consecutive elements per thread: 16-bit loads of the packed bytes (a block is only
// 2-byte aligned in general), one 16- or 32-byte store.  Every element goes through the arithmetic of dequant_elem.
template <int TYPE>
__device__ __forceinline__ void dequant8(const uint8_t* blk, int e0, float (&v)[8]);
template <>
__device__ __forceinline__ void dequant8<QMM_TYPE_Q8_0>(const uint8_t* blk, int e0, float (&v)[8]) {
    const float d = f16_bits_to_f32(ld_u16(blk));
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const unsigned w = ld_u16(blk + 2 + e0 + 2 * i);
        v[2 * i] = __fmul_rn(d, (float)(int8_t)(w & 0xFFu));
        v[2 * i + 1] = __fmul_rn(d, (float)(int8_t)(w >> 8));
    }
}
template <>
__device__ __forceinline__ void dequant8<QMM_TYPE_Q4_K>(const uint8_t* blk, int e0, float (&v)[8]) {
    const int j = e0 >> 5, l = e0 & 31;
    const uint8_t* s = blk + 4;
    int sc, m;
    if (j < 4) {
        sc = s[j] & 63;
        m = s[j + 4] & 63;
    } else {
        sc = (s[j + 4] & 15) | ((s[j - 4] >> 6) << 4);
        m = (s[j + 4] >> 4) | ((s[j] >> 6) << 4);
    }
    const float ds = __fmul_rn(f16_bits_to_f32(ld_u16(blk)), (float)sc), mm = __fmul_rn(f16_bits_to_f32(ld_u16(blk + 2)), (float)m);
    const int sh = (j & 1) ? 4 : 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const unsigned w = ld_u16(blk + 16 + 32 * (j >> 1) + l + 2 * i);
        v[2 * i] = __fsub_rn(__fmul_rn(ds, (float)((w >> sh) & 15u)), mm);
        v[2 * i + 1] = __fsub_rn(__fmul_rn(ds, (float)((w >> (8 + sh)) & 15u)), mm);
    }
}
template <>
__device__ __forceinline__ void dequant8<QMM_TYPE_Q6_K>(const uint8_t* blk, int e0, float (&v)[8]) {
    const int h = e0 >> 7, r = e0 & 127, t = r >> 5, l = r & 31;
    const float ds = __fmul_rn(f16_bits_to_f32(ld_u16(blk + 208)), (float)(int8_t)blk[192 + (e0 >> 4)]);
    const int lsh = (t < 2) ? 0 : 4, hsh = 2 * t;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const unsigned wl = ld_u16(blk + 64 * h + l + 32 * (t & 1) + 2 * i), wh = ld_u16(blk + 128 + 32 * h + l + 2 * i);
        const int q0 = (int)(((wl >> lsh) & 15u) | (((wh >> hsh) & 3u) << 4)) - 32;
        const int q1 = (int)(((wl >> (8 + lsh)) & 15u) | (((wh >> (8 + hsh)) & 3u) << 4)) - 32;
        v[2 * i] = __fmul_rn(ds, (float)q0);
        v[2 * i + 1] = __fmul_rn(ds, (float)q1);
    }
}
template <int TYPE, typename OUT>
__global__ void __launch_bounds__(256) dequantize8_kernel(const uint8_t* __restrict__ w, OUT* __restrict__ out, long n_octets) {
    using F = Fmt<TYPE, 1>;
    const long o = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (o >= n_octets) return;
    const long idx = o * 8, blk = idx / F::BLOCK_ELEMS;
    float v[8];
    dequant8<TYPE>(w + blk * F::BLOCK_BYTES, (int)(idx - blk * F::BLOCK_ELEMS), v);
    if constexpr (sizeof(OUT) == 4) {
        float4* d = reinterpret_cast<float4*>(out + idx);
        d[0] = make_float4(v[0], v[1], v[2], v[3]);
        d[1] = make_float4(v[4], v[5], v[6], v[7]);
    } else {
        uint32_t p[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const __nv_bfloat162 b = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
            p[i] = *reinterpret_cast<const uint32_t*>(&b);
        }
        *reinterpret_cast<uint4*>(out + idx) = make_uint4(p[0], p[1], p[2], p[3]);
    }
}

// ------------------------------------------------------------------- host side
int quantize_q8_1_launch(const float* x, void* xq, int m, int k, cudaStream_t stream) {
    if (!x || !xq) return QMM_ERR_NULL;
    if (m <= 0 || k <= 0 || k % 32 != 0) return QMM_ERR_SHAPE;
    if (reinterpret_cast<uintptr_t>(xq) % 4 != 0) return QMM_ERR_ALIGN;
    const long n_blocks = (long)m * (k / 32);
    const int threads = 128;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)((n_blocks * 32 + threads - 1) / threads));
    cfg.blockDim = dim3(threads);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = overlap_enabled() ? 1 : 0;
    QMM_CUDA_TRY(cudaLaunchKernelEx(&cfg, quantize_q8_kernel<true>, x, static_cast<uint8_t*>(xq), n_blocks));
    return QMM_OK;
}

int quantize_weights_launch(int type, const float* w, void* out, long rows, int k, cudaStream_t stream) {
    if (!w || !out) return QMM_ERR_NULL;
    const int be = (type == QMM_TYPE_Q8_0) ? 32 : 256;
    if (rows <= 0 || k <= 0 || k % be != 0) return QMM_ERR_SHAPE;
    const long n_blocks = rows * (k / be);
    const int threads = 128;
    const unsigned grid = (unsigned)((n_blocks * 32 + threads - 1) / threads);
    uint8_t* o = static_cast<uint8_t*>(out);
    switch (type) {
    case QMM_TYPE_Q8_0:
        if (reinterpret_cast<uintptr_t>(out) % 2 != 0) return QMM_ERR_ALIGN;
        quantize_q8_kernel<false><<<grid, threads, 0, stream>>>(w, o, n_blocks);
        break;
    case QMM_TYPE_Q4_K:
        if (reinterpret_cast<uintptr_t>(out) % 16 != 0 || reinterpret_cast<uintptr_t>(w) % 16 != 0) return QMM_ERR_ALIGN;
        quantize_q4_k_kernel<<<grid, threads, 0, stream>>>(w, o, n_blocks);
        break;
    case QMM_TYPE_Q6_K:
        if (reinterpret_cast<uintptr_t>(out) % 2 != 0 || reinterpret_cast<uintptr_t>(w) % 16 != 0) return QMM_ERR_ALIGN;
        quantize_q6_k_kernel<<<grid, threads, 0, stream>>>(w, o, n_blocks);
        break;
    default: return QMM_ERR_TYPE;
    }
    QMM_CUDA_TRY(cudaGetLastError());
    return QMM_OK;
}

template <typename OUT>
static int dequantize_launch_t(int type, const void* w, OUT* out, long n_elems, cudaStream_t stream) {
    if (!w || !out) return QMM_ERR_NULL;
    const int be = (type == QMM_TYPE_Q8_0) ? 32 : 256;
    if (n_elems <= 0 || n_elems % be != 0) return QMM_ERR_SHAPE;
    if (reinterpret_cast<uintptr_t>(w) % 2 != 0) return QMM_ERR_ALIGN;
    const int threads = 256;
    const uint8_t* wb = static_cast<const uint8_t*>(w);
    if (reinterpret_cast<uintptr_t>(out) % 16 == 0) {  // eight elements per thread, whole 16-byte stores
        const long n_octets = n_elems / 8;
        const unsigned grid8 = (unsigned)((n_octets + threads - 1) / threads);
        switch (type) {
        case QMM_TYPE_Q8_0: dequantize8_kernel<QMM_TYPE_Q8_0, OUT><<<grid8, threads, 0, stream>>>(wb, out, n_octets); break;
        case QMM_TYPE_Q4_K: dequantize8_kernel<QMM_TYPE_Q4_K, OUT><<<grid8, threads, 0, stream>>>(wb, out, n_octets); break;
        case QMM_TYPE_Q6_K: dequantize8_kernel<QMM_TYPE_Q6_K, OUT><<<grid8, threads, 0, stream>>>(wb, out, n_octets); break;
        default: return QMM_ERR_TYPE;
        }
        QMM_CUDA_TRY(cudaGetLastError());
        return QMM_OK;
    }
    const unsigned grid = (unsigned)((n_elems + threads - 1) / threads);
    switch (type) {
    case QMM_TYPE_Q8_0: dequantize_kernel<QMM_TYPE_Q8_0, OUT><<<grid, threads, 0, stream>>>(wb, out, n_elems); break;
    case QMM_TYPE_Q4_K: dequantize_kernel<QMM_TYPE_Q4_K, OUT><<<grid, threads, 0, stream>>>(wb, out, n_elems); break;
    case QMM_TYPE_Q6_K: dequantize_kernel<QMM_TYPE_Q6_K, OUT><<<grid, threads, 0, stream>>>(wb, out, n_elems); break;
    default: return QMM_ERR_TYPE;
    }
    QMM_CUDA_TRY(cudaGetLastError());
    return QMM_OK;
}

int dequantize_f32_launch(int type, const void* w, float* out, long n_elems, cudaStream_t stream) {
    return dequantize_launch_t<float>(type, w, out, n_elems, stream);
}
int dequantize_bf16_launch(int type, const void* w, void* out, long n_elems, cudaStream_t stream) {
    return dequantize_launch_t<__nv_bfloat16>(type, w, static_cast<__nv_bfloat16*>(out), n_elems, stream);
}

}  // namespace qmm
