// The small per-layer operators of the decode stack, fused so that every matvec finds its
// activations already in Q8_1: counterparts of the upstream's f64 operators
//   rmsnorm      normx_rmsnorm_kernel   gpu-core/src/kernels/normx.hip:135-159
//   rope         rope_partial           gpu-core/src/kernels/f64_infer.hip:107-132 (rotary_dim == head_dim)
//   attention    gqa_masked_attn        gpu-core/src/kernels/f64_infer.hip:49-100 (one query token, fp16 KV cache)
//   gated act    gelu_mul / glu_gelu    gpu-core/src/kernels/f64_infer.hip:134-166
//   add          add_kernel             gpu-core/src/kernels/elementwise.hip:13
// in fp32 with fp16 KV, as the decode configurations ask.  All of them take part in
// programmatic dependent launch so the following matvec can prefetch its weights.
#include "qmm_formats.cuh"
#include <cooperative_groups.h>

namespace qmm {
namespace cg = cooperative_groups;

__device__ __forceinline__ uint64_t mix64(uint64_t z) {
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

// out[i] = sigma * z(seed, first_index + i): sum of eight 16-bit uniforms, centred and scaled;
// integer hashing only, so the CPU oracle reproduces every value bit for bit.
__global__ void fill_normal_kernel(float* __restrict__ out, long n, uint64_t seed, float sigma, long first_index) {
    const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const uint64_t h1 = mix64(seed * 0xD1342543DE82EF95ull + (uint64_t)(first_index + i));
    const uint64_t h2 = mix64(h1);
    int s = 0;
#pragma unroll
    for (int c = 0; c < 4; ++c) s += (int)((h1 >> (16 * c)) & 0xFFFFu) + (int)((h2 >> (16 * c)) & 0xFFFFu);
    const float z = __fmul_rn((float)(s - 262140), __fdiv_rn(1.0f, 53510.0f));
    out[i] = __fmul_rn(z, sigma);
}

// x[b][:] = decoded row tokens[b] of a packed (vocab, hidden) matrix
template <int TYPE>
__global__ void embed_rows_kernel(const uint8_t* __restrict__ table, const int* __restrict__ tokens, float* __restrict__ x, int hidden,
                                  int row_bytes, int vocab, unsigned* step_counter) {
    using F = Fmt<TYPE, 1>;
    pdl_release_dependents();
    pdl_wait_prior_grids();
    if (step_counter && blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0) *step_counter += 1;  // first kernel of a step
    const int b = blockIdx.y;
    int tok = tokens[b];
    tok = tok < 0 ? 0 : (tok >= vocab ? vocab - 1 : tok);
    const uint8_t* row = table + (size_t)tok * row_bytes;
    for (int e = blockIdx.x * blockDim.x + threadIdx.x; e < hidden; e += gridDim.x * blockDim.x) {
        const int blk = e / F::BLOCK_ELEMS;
        x[(size_t)b * hidden + e] = dequant_elem<TYPE>(row + (size_t)blk * F::BLOCK_BYTES, e - blk * F::BLOCK_ELEMS);
    }
}

__device__ __forceinline__ float block_sum(float v, float* red) {
    v = warp_sum(v);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float t = (lane < nw) ? red[lane] : 0.f;
    t = warp_sum(t);
    __syncthreads();
    return t;
}

__device__ __forceinline__ uint16_t f32_to_f16_bits_rn(float f) { return __half_as_ushort(__float2half_rn(f)); }

// One Q8_1 block from the 32 values held one per lane (same arithmetic as quantize_q8_kernel).
__device__ __forceinline__ void warp_store_q8_1(float v, uint8_t* blk, int lane) {
    float amax = fabsf(v);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const uint16_t dh = f32_to_f16_bits_rn(fminf(__fdiv_rn(amax, 127.0f), 65504.0f));
    const float df = f16_bits_to_f32(dh);
    int q = (df > 0.0f) ? (int)roundf(__fdiv_rn(v, df)) : 0;
    q = q < -127 ? -127 : (q > 127 ? 127 : q);
    blk[4 + lane] = (uint8_t)(int8_t)q;
    int sum = q;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    if (lane == 0) {
        *reinterpret_cast<uint16_t*>(blk) = dh;
        *reinterpret_cast<uint16_t*>(blk + 2) = f32_to_f16_bits_rn(__fmul_rn(df, (float)sum));
    }
}

// Residual update + RMSNorm + Q8_1 in one pass over a row, fused with the tensor-parallel sum:
//   x += part                               (single GPU: the output of the preceding projection, n_parts = 1)
//   x += sum_{r < tp} part_r                (tensor parallel: the partial outputs of the preceding row-parallel
//                                            projection, which every rank's matvec kernel stored into this
//                                            rank's exchange area, one 64-bit word {value, sequence number}
//                                            per output; the words are polled here, in local memory, with a
//                                            bound, and added in rank order - see TpPush / TpRecv)
//   xq = Q8_1( x * rsqrt(mean(x^2) + eps) * gamma )
// One CTA per activation row, one element per thread per pass (hidden <= 8 * blockDim.x).  The last CTA
// to finish advances the exchange counter.
constexpr int NORM_MAX_PER_THREAD = 8;
struct PartPtrs {
    const float* p[8];  // single GPU: p[0] = the projection output to add (or none)
};
__global__ void __launch_bounds__(1024) add_rmsnorm_q8_kernel(float* __restrict__ x, const PartPtrs parts, int n_parts, long part_stride,
                                      const float* __restrict__ gamma, uint8_t* __restrict__ xq, int hidden, float eps, const TpRecv rcv,
                                      float* __restrict__ out_f32, __nv_bfloat16* __restrict__ out_bf16) {
    __shared__ float red[32];
    __shared__ int give_up;
    pdl_release_dependents();
    // gamma is model data: fetched before the wait for the preceding kernel
    float gm[NORM_MAX_PER_THREAD];
#pragma unroll
    for (int i = 0; i < NORM_MAX_PER_THREAD; ++i) {
        const int e = i * blockDim.x + threadIdx.x;
        gm[i] = e < hidden ? (gamma ? gamma[e] : 1.f) : 0.f;  // no gamma: the scale-less variant
    }
    if (threadIdx.x == 0) give_up = 0;
    __syncthreads();
    pdl_wait_prior_grids();
    const int b = blockIdx.x, lane = threadIdx.x & 31;
    const bool exchange = rcv.tp > 1;
    const unsigned seq = exchange ? tp_next_seq(rcv.counter) : 0u;
    float* xr = x + (size_t)b * hidden;
    float v[NORM_MAX_PER_THREAD];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < NORM_MAX_PER_THREAD; ++i) {
        const int e = i * blockDim.x + threadIdx.x;
        v[i] = 0.f;
        if (e < hidden) {
            float t = xr[e];
            if (exchange) {
                for (int r = 0; r < rcv.tp; ++r) {  // rank order: the same sum on every rank
                    float pv = 0.f;
                    if (!tp_poll_word(rcv, seq, r, (long)b * part_stride + e, pv, &give_up)) break;
                    t += pv;
                }
            } else if (n_parts > 0) {
                t += parts.p[0][(size_t)b * part_stride + e];
            }
            v[i] = t;
            ss += t * t;
        }
    }
    ss = block_sum(ss, red);  // (two block-wide barriers: every thread is past its polls after them)
    if (exchange && threadIdx.x == 0) {
        if (give_up) atomicExch(&g_device_status, DEV_TIMEOUT_PEER);
        tp_consumer_done(rcv, seq, gridDim.x);
    }
    if (give_up) return;  // a peer never arrived: leave x and xq as they were
    const float inv = rsqrtf(ss / (float)hidden + eps);
    uint8_t* qrow = xq + (size_t)b * (hidden / 32) * Q8_1_BYTES;
#pragma unroll
    for (int i = 0; i < NORM_MAX_PER_THREAD; ++i) {
        const int e = i * blockDim.x + threadIdx.x;  // a warp covers 32 consecutive elements = one block
        if (e < hidden) {
            if (exchange || n_parts > 0) xr[e] = v[i];
            const float nv = v[i] * inv * gm[i];
            if (out_f32) out_f32[(size_t)b * hidden + e] = nv;
            if (out_bf16) out_bf16[(size_t)b * hidden + e] = __float2bfloat16_rn(nv);
            warp_store_q8_1(nv, qrow + (size_t)(e >> 5) * Q8_1_BYTES, lane);
        }
    }
}

// The same operator with the row split over a cluster of NORM_CLUSTER CTAs (hidden a multiple of 256, at most
// 8192): each CTA owns hidden / NORM_CLUSTER consecutive elements, the partial sums of squares meet through
// distributed shared memory in a fixed order.  A row of 8192 values handled by one CTA is bound by that
// CTA's memory latency (and, tensor parallel, by one SM polling 8 x 8192 exchange words); eight CTAs of 256
// threads keep all their loads in flight at once: every thread first issues the exchange-word loads of all
// its elements and ranks, then checks the sequence numbers and re-polls only what had not arrived.
constexpr int NORM_CLUSTER = 8;
constexpr int NORM_CL_THREADS = 256;
constexpr int NORM_CL_PER_THREAD = 4;   // slice <= 1024 elements
__global__ void __launch_bounds__(NORM_CL_THREADS) add_rmsnorm_q8_cluster_kernel(float* __restrict__ x, const PartPtrs parts, int n_parts,
                                                                                long part_stride, const float* __restrict__ gamma,
                                                                                uint8_t* __restrict__ xq, int hidden, float eps, const TpRecv rcv,
                                                                                float* __restrict__ out_f32, __nv_bfloat16* __restrict__ out_bf16) {
    __shared__ float red[32];
    __shared__ float cl_ss;     // this CTA's sum of squares, read by the other CTAs of the cluster
    __shared__ int cl_bad;      // this CTA gave up on a peer
    __shared__ int give_up;
    cg::cluster_group cluster = cg::this_cluster();
    const int cl = (int)cluster.num_blocks(), cr = (int)cluster.block_rank();
    pdl_release_dependents();
    const int slice = hidden / cl, e0 = cr * slice;
    const int b = blockIdx.y, lane = threadIdx.x & 31;
    float gm[NORM_CL_PER_THREAD];
#pragma unroll
    for (int i = 0; i < NORM_CL_PER_THREAD; ++i) {
        const int o = i * NORM_CL_THREADS + threadIdx.x;
        gm[i] = o < slice ? (gamma ? gamma[e0 + o] : 1.f) : 0.f;
    }
    if (threadIdx.x == 0) give_up = 0;
    __syncthreads();
    pdl_wait_prior_grids();
    const bool exchange = rcv.tp > 1;
    const unsigned seq = exchange ? tp_next_seq(rcv.counter) : 0u;
    float* xr = x + (size_t)b * hidden;
    float v[NORM_CL_PER_THREAD];
    if (exchange) {
        const unsigned long long* p0 = rcv.base + ((seq & 1u) ? rcv.buf_words : 0) + (long)b * part_stride + e0 + threadIdx.x;
        unsigned long long w[NORM_CL_PER_THREAD][QMM_TP_MAX];
#pragma unroll
        for (int i = 0; i < NORM_CL_PER_THREAD; ++i)
#pragma unroll
            for (int r = 0; r < QMM_TP_MAX; ++r)
                if (r < rcv.tp && i * NORM_CL_THREADS + (int)threadIdx.x < slice)
                    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(w[i][r]) : "l"(p0 + (long)r * rcv.src_words + i * NORM_CL_THREADS) : "memory");
#pragma unroll
        for (int i = 0; i < NORM_CL_PER_THREAD; ++i) {
            const int o = i * NORM_CL_THREADS + threadIdx.x;
            v[i] = 0.f;
            if (o < slice) {
                float t = xr[e0 + o];
#pragma unroll
                for (int r = 0; r < QMM_TP_MAX; ++r)  // rank order: the same sum on every rank
                    if (r < rcv.tp) {
                        float pv = __uint_as_float((unsigned)w[i][r]);
                        if ((unsigned)(w[i][r] >> 32) != seq && !tp_poll_word(rcv, seq, r, (long)b * part_stride + e0 + o, pv, &give_up)) pv = 0.f;
                        t += pv;
                    }
                v[i] = t;
            }
        }
    } else {
#pragma unroll
        for (int i = 0; i < NORM_CL_PER_THREAD; ++i) {
            const int o = i * NORM_CL_THREADS + threadIdx.x;
            v[i] = 0.f;
            if (o < slice) {
                float t = xr[e0 + o];
                if (n_parts > 0) t += parts.p[0][(size_t)b * part_stride + e0 + o];
                v[i] = t;
            }
        }
    }
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < NORM_CL_PER_THREAD; ++i) ss += v[i] * v[i];
    ss = block_sum(ss, red);
    if (threadIdx.x == 0) {
        cl_ss = ss;
        cl_bad = give_up;
    }
    cluster.sync();
    float total = 0.f;
    int bad = 0;
    for (int c = 0; c < cl; ++c) {  // fixed order
        total += *cluster.map_shared_rank(&cl_ss, c);
        bad |= *cluster.map_shared_rank(&cl_bad, c);
    }
    cluster.sync();  // nobody leaves while its shared memory may still be read
    if (exchange && threadIdx.x == 0) {
        if (give_up) atomicExch(&g_device_status, DEV_TIMEOUT_PEER);
        tp_consumer_done(rcv, seq, gridDim.x * gridDim.y);
    }
    if (bad) return;  // a peer never arrived: the row keeps its old x and xq
    const float inv = rsqrtf(total / (float)hidden + eps);
    uint8_t* qrow = xq + (size_t)b * (hidden / 32) * Q8_1_BYTES;
#pragma unroll
    for (int i = 0; i < NORM_CL_PER_THREAD; ++i) {
        const int o = i * NORM_CL_THREADS + threadIdx.x;  // a warp covers 32 consecutive elements = one block
        if (o < slice) {
            const int e = e0 + o;
            if (exchange || n_parts > 0) xr[e] = v[i];
            const float nv = v[i] * inv * gm[i];
            if (out_f32) out_f32[(size_t)b * hidden + e] = nv;
            if (out_bf16) out_bf16[(size_t)b * hidden + e] = __float2bfloat16_rn(nv);
            warp_store_q8_1(nv, qrow + (size_t)(e >> 5) * Q8_1_BYTES, lane);
        }
    }
}

// The prompt-path form of the operator: many rows at once, the normalised row wanted only as bf16 (the input of a
// GEMM).  One CTA of 256 threads per row, four consecutive elements per thread per pass (hidden a multiple of 4, at
// most 8192), the row held in registers between the sum of squares and the scaling; no Q8_1 blocks, no exchange.
constexpr int NORM_SEQ_THREADS = 256;
constexpr int NORM_SEQ_PASSES = 8;
__global__ void __launch_bounds__(NORM_SEQ_THREADS) add_rmsnorm_bf16_kernel(float* __restrict__ x, const float* __restrict__ part, long part_stride,
                                                                            const float* __restrict__ gamma, int hidden, float eps,
                                                                            __nv_bfloat16* __restrict__ out_bf16) {
    __shared__ float red[32];
    const int b = blockIdx.x, quads = hidden >> 2;
    float4* xr = reinterpret_cast<float4*>(x + (size_t)b * hidden);
    const float4* pr = part ? reinterpret_cast<const float4*>(part + (size_t)b * part_stride) : nullptr;
    float4 v[NORM_SEQ_PASSES];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < NORM_SEQ_PASSES; ++i) {
        const int q = i * NORM_SEQ_THREADS + threadIdx.x;
        v[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (q < quads) {
            v[i] = xr[q];
            if (pr) {
                const float4 p = pr[q];
                v[i].x += p.x, v[i].y += p.y, v[i].z += p.z, v[i].w += p.w;
                xr[q] = v[i];
            }
            ss += v[i].x * v[i].x + v[i].y * v[i].y + v[i].z * v[i].z + v[i].w * v[i].w;
        }
    }
    ss = block_sum(ss, red);
    const float inv = rsqrtf(ss / (float)hidden + eps);
    uint2* orow = reinterpret_cast<uint2*>(out_bf16 + (size_t)b * hidden);
#pragma unroll
    for (int i = 0; i < NORM_SEQ_PASSES; ++i) {
        const int q = i * NORM_SEQ_THREADS + threadIdx.x;
        if (q < quads) {
            const float4 g = gamma ? reinterpret_cast<const float4*>(gamma)[q] : make_float4(1.f, 1.f, 1.f, 1.f);
            const __nv_bfloat162 lo = __floats2bfloat162_rn(v[i].x * inv * g.x, v[i].y * inv * g.y);
            const __nv_bfloat162 hi = __floats2bfloat162_rn(v[i].z * inv * g.z, v[i].w * inv * g.w);
            orow[q] = make_uint2(*reinterpret_cast<const uint32_t*>(&lo), *reinterpret_cast<const uint32_t*>(&hi));
        }
    }
}
inline bool add_rmsnorm_bf16_fits(int hidden, long part_stride) {
    return hidden % 4 == 0 && part_stride % 4 == 0 && hidden <= 4 * NORM_SEQ_THREADS * NORM_SEQ_PASSES;
}
inline int add_rmsnorm_bf16_launch(float* x, const float* part, long part_stride, const float* gamma, int hidden, float eps, __nv_bfloat16* out_bf16,
                                   int rows, cudaStream_t stream) {
    add_rmsnorm_bf16_kernel<<<rows, NORM_SEQ_THREADS, 0, stream>>>(x, part, part_stride, gamma, hidden, eps, out_bf16);
    QMM_CUDA_TRY(cudaGetLastError());
    return QMM_OK;
}

// Launches the residual + norm + Q8_1 operator: the cluster form when the row splits evenly, else one CTA per row.
inline int add_rmsnorm_launch(float* x, const PartPtrs& parts, int n_parts, long part_stride, const float* gamma, uint8_t* xq, int hidden,
                              float eps, const TpRecv& rcv, float* out_f32, int rows, bool pdl, cudaStream_t stream,
                              __nv_bfloat16* out_bf16 = nullptr) {
    cudaLaunchConfig_t cfg = {};
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int na = 0;
    if (pdl && overlap_enabled()) {
        attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[na].val.programmaticStreamSerializationAllowed = 1;
        ++na;
    }
    // a cluster of eight CTAs per row cuts the latency of a few rows (decode); with many rows (a prompt) one CTA per
    // row fills the GPU anyway and the 16 k tiny CTAs of the clustered form cost 200 instead of 20 us at 2048 rows
    const bool clustered = rows <= 64 && hidden % (NORM_CLUSTER * 32) == 0 && hidden / NORM_CLUSTER <= NORM_CL_THREADS * NORM_CL_PER_THREAD;
    if (clustered) {
        attr[na].id = cudaLaunchAttributeClusterDimension;
        attr[na].val.clusterDim.x = NORM_CLUSTER;
        attr[na].val.clusterDim.y = 1;
        attr[na].val.clusterDim.z = 1;
        ++na;
        cfg.gridDim = dim3(NORM_CLUSTER, rows);
        cfg.blockDim = dim3(NORM_CL_THREADS);
        cfg.attrs = attr;
        cfg.numAttrs = na;
        QMM_CUDA_TRY(cudaLaunchKernelEx(&cfg, add_rmsnorm_q8_cluster_kernel, x, parts, n_parts, part_stride, gamma, xq, hidden, eps, rcv, out_f32, out_bf16));
        return QMM_OK;
    }
    const int passes = (hidden + 1023) / 1024;
    const int threads = (((hidden + passes - 1) / passes) + 31) & ~31;
    cfg.gridDim = dim3(rows);
    cfg.blockDim = dim3(threads);
    cfg.attrs = attr;
    cfg.numAttrs = na;
    QMM_CUDA_TRY(cudaLaunchKernelEx(&cfg, add_rmsnorm_q8_kernel, x, parts, n_parts, part_stride, gamma, xq, hidden, eps, rcv, out_f32, out_bf16));
    return QMM_OK;
}

// The same for a whole sequence (the prefill of a prompt): row r of the buffers is position pos0 + r of sequence
// `seq`.  q (columns [0, nqh*hd) of a row of qk) is rotated in place (f32: the sequence attention reads it there); k
// (columns [nqh*hd, (nqh+nkv)*hd)) is rotated into the fp16 cache, where v goes too and where the attention reads both.
// One CTA per position: a thread keeps one rotation (sine and cosine of pos * theta^(-2i/hd), the costly part) and
// applies it to element pair i of every head of its group of heads.
__global__ void rope_seq_append_kernel(float* __restrict__ qk, long qk_stride, const float* __restrict__ v, long v_stride,
                                       __half* __restrict__ kcache, __half* __restrict__ vcache, int nqh, int nkv, int hd, int pos0, int seq,
                                       int ctx_cap, float theta) {
    const int r = blockIdx.x, pos = pos0 + r;
    const int half = hd / 2;
    float* row = qk + (size_t)r * qk_stride;
    const float* vrow = v + (size_t)r * v_stride;
    const size_t cache_row = ((size_t)seq * ctx_cap + pos) * nkv * hd;
    const int groups = blockDim.x / half;  // (the launcher keeps half <= blockDim.x)
    const int i = threadIdx.x % half, g = threadIdx.x / half;
    if (g < groups) {
        float sn, cs;
        sincosf((float)pos * powf(theta, -2.0f * (float)i / (float)hd), &sn, &cs);
        for (int head = g; head < nqh + nkv; head += groups) {
            float* h = row + (size_t)head * hd;
            const float a = h[i], c = h[i + half];
            const float ra = a * cs - c * sn, rc = a * sn + c * cs;
            if (head < nqh) {
                h[i] = ra;
                h[i + half] = rc;
            } else {
                __half* dst = kcache + cache_row + (size_t)(head - nqh) * hd;
                dst[i] = __float2half_rn(ra);
                dst[i + half] = __float2half_rn(rc);
            }
        }
    }
    const int nv = nkv * hd;  // (a multiple of 4: hd is even and the launcher checks the rest)
    for (int j = threadIdx.x * 4; j < nv; j += blockDim.x * 4) {
        const float4 x = *reinterpret_cast<const float4*>(vrow + j);
        const __half2 lo = __floats2half2_rn(x.x, x.y), hi = __floats2half2_rn(x.z, x.w);
        *reinterpret_cast<uint2*>(vcache + cache_row + j) = make_uint2(*reinterpret_cast<const uint32_t*>(&lo), *reinterpret_cast<const uint32_t*>(&hi));
    }
}

// NeoX rotary embedding of q (in place, fp32) and k, then k and v appended to the fp16 cache at `pos`.
// qkv row layout: [q: nqh*hd | k: nkv*hd | v: nkv*hd].  cache layout: (batch, ctx_cap, nkv, hd).
__global__ void rope_kv_append_kernel(float* __restrict__ qkv, __half* __restrict__ kcache, __half* __restrict__ vcache, int nqh, int nkv,
                                      int hd, int pos, int ctx_cap, float theta) {
    pdl_release_dependents();
    const int b = blockIdx.y;
    const int half = hd / 2;
    const int pairs = (nqh + nkv) * half;
    const int first = blockIdx.x * blockDim.x + threadIdx.x, step = gridDim.x * blockDim.x;
    // the angles depend on nothing the preceding kernel writes: sines and cosines of this thread's first
    // pairs are ready before the wait for it
    constexpr int PRE = 4;
    float psn[PRE], pcs[PRE];
#pragma unroll
    for (int u = 0; u < PRE; ++u) {
        const int idx = first + u * step;
        psn[u] = 0.f, pcs[u] = 1.f;
        if (idx < pairs) {
            const int i = idx % half;
            sincosf((float)pos * powf(theta, -2.0f * (float)i / (float)hd), &psn[u], &pcs[u]);
        }
    }
    pdl_wait_prior_grids();
    float* row = qkv + (size_t)b * (nqh + 2 * nkv) * hd;
    // item idx: a rotation pair of a q or k head (idx < pairs), else one element of v
    auto item = [&](int idx, float sn, float cs) {
        if (idx < pairs) {
            const int head = idx / half, i = idx - head * half;
            float* h = row + (size_t)head * hd;
            const float a = h[i], c = h[i + half];
            const float ra = a * cs - c * sn, rc = a * sn + c * cs;
            if (head < nqh) {
                h[i] = ra;
                h[i + half] = rc;
            } else {
                __half* dst = kcache + (((size_t)b * ctx_cap + pos) * nkv + (head - nqh)) * hd;
                dst[i] = __float2half_rn(ra);
                dst[i + half] = __float2half_rn(rc);
            }
        } else if (idx < pairs + nkv * hd) {
            const int j = idx - pairs;
            vcache[((size_t)b * ctx_cap + pos) * nkv * hd + j] = __float2half_rn(row[(size_t)(nqh + nkv) * hd + j]);
        }
    };
#pragma unroll
    for (int u = 0; u < PRE; ++u) item(first + u * step, psn[u], pcs[u]);
    for (int idx = first + PRE * step; idx < pairs + nkv * hd; idx += step) {  // wider stacks than the grid covers in PRE rounds
        float sn = 0.f, cs = 1.f;
        if (idx < pairs) sincosf((float)pos * powf(theta, -2.0f * (float)(idx % half) / (float)hd), &sn, &cs);
        item(idx, sn, cs);
    }
}

// Single-query GQA attention over the fp16 cache, split over the context: CTA (kv head, batch, split)
// handles ATTN_CHUNK positions for the `group` query heads of its kv head.  The K and V rows of
// the chunk are staged in shared memory with coalesced 16-byte loads (all in flight at once), the
// scores are one thread per (position, half of the heads), the outputs one thread per head
// dimension.  Per query head the CTA writes the running maximum, the sum of exponentials and
// the unnormalised output (hd floats); attn_combine_q8_kernel merges the splits.
// scratch layout: (batch, nqh, splits, hd + 2) floats.
constexpr int ATTN_THREADS = 128;
constexpr int ATTN_MAX_GROUP = 8;
constexpr int ATTN_CHUNK = 64;
// 16-byte asynchronous copy global -> shared (no register in between, so a thread keeps all its copies
// of a chunk in flight at once); `valid` false writes zeros instead
__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc, bool valid) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(valid ? 16 : 0) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.commit_group;\n\tcp.async.wait_group 0;" ::: "memory"); }
__global__ void __launch_bounds__(ATTN_THREADS) attn_decode_split_kernel(const float* __restrict__ qkv, const __half* __restrict__ kcache,
                                                                        const __half* __restrict__ vcache, float* __restrict__ scratch,
                                                                        int nqh, int nkv, int hd, int len, int ctx_cap, int splits) {
    extern __shared__ __align__(16) uint8_t att_raw[];
    // layout: K rows (ATTN_CHUNK x (hd+8) halves, padded against bank conflicts) | V rows (ATTN_CHUNK x hd halves)
    //         | q (group x hd floats) | p (group x ATTN_CHUNK floats) | stats (2 x group floats)
    const int kpitch = hd + 8;
    __half* ks = reinterpret_cast<__half*>(att_raw);
    __half* vs = ks + ATTN_CHUNK * kpitch;
    float* qs = reinterpret_cast<float*>(vs + ATTN_CHUNK * hd);
    const int group = nqh / nkv;
    float* ps = qs + group * hd;
    float* stat = ps + group * ATTN_CHUNK;
    pdl_release_dependents();
    pdl_wait_prior_grids();
    const int kvh = blockIdx.x, b = blockIdx.y, sp = blockIdx.z;
    const int t0 = sp * ATTN_CHUNK, nt = max(min(len - t0, ATTN_CHUNK), 0);
    const int tid = threadIdx.x;
    const float scale = rsqrtf((float)hd);
    const float* qrow = qkv + (size_t)b * (nqh + 2 * nkv) * hd + (size_t)kvh * group * hd;
    // stage K and V: hd/8 16-byte pieces per row
    const int pieces = hd / 8;
    const size_t row_stride = (size_t)nkv * hd;  // halves between consecutive positions
    const __half* kbase = kcache + (((size_t)b * ctx_cap + t0) * nkv + kvh) * hd;
    const __half* vbase = vcache + (((size_t)b * ctx_cap + t0) * nkv + kvh) * hd;
    // (V rows past the end of the context are multiplied by zero probabilities below: zeros, so that they are finite)
    for (int i = tid; i < ATTN_CHUNK * pieces; i += ATTN_THREADS) {
        const int t = i / pieces, c = i - t * pieces;
        const bool in = t < nt;
        if (in) cp_async16(ks + t * kpitch + 8 * c, kbase + t * row_stride + 8 * c, true);
        cp_async16(vs + t * hd + 8 * c, in ? vbase + t * row_stride + 8 * c : vbase, in);
    }
    for (int i = tid; i < group * hd; i += ATTN_THREADS) qs[i] = qrow[i] * scale;
    cp_async_wait_all();
    __syncthreads();
    // scores: thread = (position t, head parity): heads g = par, par+2, ...; eight elements per step, the
    // K row as one 16-byte load, q as 16-byte broadcast loads
    {
        const int t = tid & (ATTN_CHUNK - 1), par = tid / ATTN_CHUNK;
        float acc[ATTN_MAX_GROUP / 2];
#pragma unroll
        for (int g = 0; g < ATTN_MAX_GROUP / 2; ++g) acc[g] = 0.f;
        if (t < nt) {
            const uint4* kr = reinterpret_cast<const uint4*>(ks + t * kpitch);
            for (int c = 0; c < hd / 8; ++c) {
                const uint4 kk = kr[c];
                const float2 k0 = __half22float2(*reinterpret_cast<const __half2*>(&kk.x));
                const float2 k1 = __half22float2(*reinterpret_cast<const __half2*>(&kk.y));
                const float2 k2 = __half22float2(*reinterpret_cast<const __half2*>(&kk.z));
                const float2 k3 = __half22float2(*reinterpret_cast<const __half2*>(&kk.w));
#pragma unroll
                for (int g = 0; g < ATTN_MAX_GROUP / 2; ++g) {
                    const int head = 2 * g + par;
                    if (head < group) {
                        const float4 qa = *reinterpret_cast<const float4*>(qs + head * hd + 8 * c);
                        const float4 qb = *reinterpret_cast<const float4*>(qs + head * hd + 8 * c + 4);
                        acc[g] += k0.x * qa.x + k0.y * qa.y + k1.x * qa.z + k1.y * qa.w + k2.x * qb.x + k2.y * qb.y + k3.x * qb.z + k3.y * qb.w;
                    }
                }
            }
        }
#pragma unroll
        for (int g = 0; g < ATTN_MAX_GROUP / 2; ++g) {
            const int head = 2 * g + par;
            if (head < group) ps[head * ATTN_CHUNK + t] = (t < nt) ? acc[g] : -INFINITY;
        }
    }
    __syncthreads();
    // per head: max, exponentials, sum; warp w handles heads w, w+4, ... (ATTN_CHUNK = 64 = two values per lane)
    {
        const int warp = tid >> 5, lane = tid & 31;
        for (int head = warp; head < group; head += ATTN_THREADS / 32) {
            float a = ps[head * ATTN_CHUNK + lane], c = ps[head * ATTN_CHUNK + 32 + lane];
            float m = fmaxf(a, c);
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
            a = (lane < nt) ? __expf(a - m) : 0.f;
            c = (32 + lane < nt) ? __expf(c - m) : 0.f;
            ps[head * ATTN_CHUNK + lane] = a;
            ps[head * ATTN_CHUNK + 32 + lane] = c;
            const float sum = warp_sum(a + c);
            if (lane == 0) stat[2 * head] = m, stat[2 * head + 1] = sum;
        }
    }
    __syncthreads();
    // outputs, head dimensions up to the thread count: thread = (pair of head dimensions, half of the
    // positions); four positions per step, the probabilities as 16-byte broadcast loads; the two halves
    // meet in shared memory (the K area is free)
    if (hd <= ATTN_THREADS) {
        float* osum = reinterpret_cast<float*>(ks);  // (group x hd) floats of the upper half
        const int pairs = hd / 2;
        const int th = tid / pairs >= 1 ? 1 : 0, dp = tid - th * pairs;
        const bool worker = tid < 2 * pairs;
        float2 o[ATTN_MAX_GROUP];
#pragma unroll
        for (int g = 0; g < ATTN_MAX_GROUP; ++g) o[g] = make_float2(0.f, 0.f);
        if (worker) {
            const int tb = th * (ATTN_CHUNK / 2);
            for (int t = tb; t < tb + ATTN_CHUNK / 2; t += 4) {  // probabilities past nt are zero, V rows past nt hold finite stale values
                float2 vv[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) vv[u] = __half22float2(*reinterpret_cast<const __half2*>(vs + (t + u) * hd + 2 * dp));
#pragma unroll
                for (int g = 0; g < ATTN_MAX_GROUP; ++g)
                    if (g < group) {
                        const float4 pp = *reinterpret_cast<const float4*>(ps + g * ATTN_CHUNK + t);
                        o[g].x += pp.x * vv[0].x + pp.y * vv[1].x + pp.z * vv[2].x + pp.w * vv[3].x;
                        o[g].y += pp.x * vv[0].y + pp.y * vv[1].y + pp.z * vv[2].y + pp.w * vv[3].y;
                    }
            }
        }
        __syncthreads();  // everybody is done with K
        if (worker && th == 1) {
#pragma unroll
            for (int g = 0; g < ATTN_MAX_GROUP; ++g)
                if (g < group) *reinterpret_cast<float2*>(osum + g * hd + 2 * dp) = o[g];
        }
        __syncthreads();
        if (worker && th == 0) {
#pragma unroll
            for (int g = 0; g < ATTN_MAX_GROUP; ++g)
                if (g < group) {
                    const float2 u = *reinterpret_cast<const float2*>(osum + g * hd + 2 * dp);
                    float* dst = scratch + (((size_t)b * nqh + kvh * group + g) * splits + sp) * (hd + 2);
                    dst[2 + 2 * dp] = o[g].x + u.x;
                    dst[3 + 2 * dp] = o[g].y + u.y;
                    if (dp == 0) dst[0] = stat[2 * g], dst[1] = stat[2 * g + 1];
                }
        }
        return;
    }
    // wider heads: thread d accumulates over the positions for every head of the group
    for (int d = tid; d < hd; d += ATTN_THREADS) {
        float o[ATTN_MAX_GROUP];
#pragma unroll
        for (int g = 0; g < ATTN_MAX_GROUP; ++g) o[g] = 0.f;
        for (int t = 0; t < nt; ++t) {
            const float vv = __half2float(vs[t * hd + d]);
#pragma unroll
            for (int g = 0; g < ATTN_MAX_GROUP; ++g)
                if (g < group) o[g] += ps[g * ATTN_CHUNK + t] * vv;
        }
#pragma unroll
        for (int g = 0; g < ATTN_MAX_GROUP; ++g)
            if (g < group) {
                float* dst = scratch + (((size_t)b * nqh + kvh * group + g) * splits + sp) * (hd + 2);
                dst[2 + d] = o[g];
                if (d == 0) dst[0] = stat[2 * g], dst[1] = stat[2 * g + 1];
            }
    }
}

// The same split attention on the f16 tensor cores, for batches of several sequences, where the scalar
// kernel above is bound by its own arithmetic (2.2 TB/s of K and V at batch 16): scores S = Q K^T and
// outputs O = P V as mma.sync.m16n8k16 (f16 operands, f32 accumulation).  The group's query heads (<= 8)
// are the rows 0..7 of the 16-row A operand (rows 8..15 stay zero), q (scaled) and the probabilities
// are rounded to f16 - the only numerical difference to the scalar kernel, about 1e-3 relative.  K rows
// are B fragments as they lie in shared memory, V rows go through ldmatrix.trans.  Same scratch layout
// and merge kernel as above.  hd a multiple of 32.
__device__ __forceinline__ void mma_f16_k16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// from this many sequences on the tensor-core form is used (below it the scalar kernel is not the bottleneck
// and keeps f32 q and probabilities)
static int g_attn_tc_min_batch = 4;  // tunable "attn_tc_min_batch"; 0: never
int attn_set_tc_min_batch(int v) {
    if (v < 0 || v > 1 << 20) return QMM_ERR_UNSUPPORTED;
    g_attn_tc_min_batch = v;
    return QMM_OK;
}
inline bool attn_use_tc(int batch, int hd) { return g_attn_tc_min_batch > 0 && batch >= g_attn_tc_min_batch && hd % 32 == 0; }
__host__ __device__ inline size_t attn_tc_smem_bytes(int hd) {
    return (size_t)(2 * ATTN_CHUNK * (hd + 8) + 8 * (hd + 8) + 8 * (ATTN_CHUNK + 8)) * sizeof(__half) + (size_t)(8 * ATTN_CHUNK + 16) * sizeof(float);
}
__global__ void __launch_bounds__(ATTN_THREADS) attn_decode_split_tc_kernel(const float* __restrict__ qkv, const __half* __restrict__ kcache,
                                                                           const __half* __restrict__ vcache, float* __restrict__ scratch,
                                                                           int nqh, int nkv, int hd, int len, int ctx_cap, int splits) {
    extern __shared__ __align__(16) uint8_t att_raw[];
    // layout (halves unless noted): K rows 64 x (hd+8) | V rows 64 x (hd+8) | Q 8 x (hd+8) | P 8 x 72 |
    //                               S/P floats 8 x 64 | stats 2 x 8 floats
    const int pitch = hd + 8;
    constexpr int PPITCH = ATTN_CHUNK + 8;
    __half* ks = reinterpret_cast<__half*>(att_raw);
    __half* vs = ks + ATTN_CHUNK * pitch;
    __half* qh = vs + ATTN_CHUNK * pitch;
    __half* ph = qh + 8 * pitch;
    float* ps = reinterpret_cast<float*>(ph + 8 * PPITCH);
    float* stat = ps + 8 * ATTN_CHUNK;
    const int group = nqh / nkv;
    pdl_release_dependents();
    pdl_wait_prior_grids();
    const int kvh = blockIdx.x, b = blockIdx.y, sp = blockIdx.z;
    const int t0 = sp * ATTN_CHUNK, nt = max(min(len - t0, ATTN_CHUNK), 0);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, q = lane >> 2, pq = lane & 3;
    const float scale = rsqrtf((float)hd);
    const float* qrow = qkv + (size_t)b * (nqh + 2 * nkv) * hd + (size_t)kvh * group * hd;
    const int pieces = hd / 8;
    const size_t row_stride = (size_t)nkv * hd;
    const __half* kbase = kcache + (((size_t)b * ctx_cap + t0) * nkv + kvh) * hd;
    const __half* vbase = vcache + (((size_t)b * ctx_cap + t0) * nkv + kvh) * hd;
    // stage K and V (rows past the end of the context as zeros: they meet zero probabilities)
    for (int i = tid; i < ATTN_CHUNK * pieces; i += ATTN_THREADS) {
        const int t = i / pieces, c = i - t * pieces;
        const bool in = t < nt;
        cp_async16(ks + t * pitch + 8 * c, in ? kbase + t * row_stride + 8 * c : kbase, in);
        cp_async16(vs + t * pitch + 8 * c, in ? vbase + t * row_stride + 8 * c : vbase, in);
    }
    for (int i = tid; i < 8 * hd; i += ATTN_THREADS) {
        const int g = i / hd, d = i - g * hd;
        qh[g * pitch + d] = __float2half_rn(g < group ? qrow[i] * scale : 0.f);
    }
    cp_async_wait_all();
    __syncthreads();
    // scores: warp w owns positions 16w .. 16w+15 (two n-tiles), k runs over the head dimension
    {
        float c0[4] = {0.f, 0.f, 0.f, 0.f}, c1[4] = {0.f, 0.f, 0.f, 0.f};
        const __half* qa = qh + q * pitch + 2 * pq;
        const __half* kb0 = ks + (16 * warp + q) * pitch + 2 * pq;
        const __half* kb1 = kb0 + 8 * pitch;
        for (int kk = 0; kk < hd; kk += 16) {
            const uint32_t a0 = *reinterpret_cast<const uint32_t*>(qa + kk), a2 = *reinterpret_cast<const uint32_t*>(qa + kk + 8);
            mma_f16_k16(c0, a0, 0u, a2, 0u, *reinterpret_cast<const uint32_t*>(kb0 + kk), *reinterpret_cast<const uint32_t*>(kb0 + kk + 8));
            mma_f16_k16(c1, a0, 0u, a2, 0u, *reinterpret_cast<const uint32_t*>(kb1 + kk), *reinterpret_cast<const uint32_t*>(kb1 + kk + 8));
        }
        // c[0], c[1]: head q, positions 16w + 8n + 2pq, +1
        if (q < group) {
            const int p0 = 16 * warp + 2 * pq;
            ps[q * ATTN_CHUNK + p0] = p0 < nt ? c0[0] : -INFINITY;
            ps[q * ATTN_CHUNK + p0 + 1] = p0 + 1 < nt ? c0[1] : -INFINITY;
            ps[q * ATTN_CHUNK + p0 + 8] = p0 + 8 < nt ? c1[0] : -INFINITY;
            ps[q * ATTN_CHUNK + p0 + 9] = p0 + 9 < nt ? c1[1] : -INFINITY;
        }
    }
    __syncthreads();
    // per head: max, exponentials, sum (as in the scalar kernel), the probabilities also as f16 A operand
    for (int head = warp; head < 8; head += ATTN_THREADS / 32) {
        float a = 0.f, c = 0.f;
        if (head < group) {
            a = ps[head * ATTN_CHUNK + lane], c = ps[head * ATTN_CHUNK + 32 + lane];
            float m = fmaxf(a, c);
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
            a = (lane < nt) ? __expf(a - m) : 0.f;
            c = (32 + lane < nt) ? __expf(c - m) : 0.f;
            const float sum = warp_sum(a + c);
            if (lane == 0) stat[2 * head] = m, stat[2 * head + 1] = sum;
        }
        ph[head * PPITCH + lane] = __float2half_rn(a);
        ph[head * PPITCH + 32 + lane] = __float2half_rn(c);
    }
    __syncthreads();
    // outputs: warp w owns head dimensions w*hd/4 .. (w+1)*hd/4 - 1 in n-tiles of eight, k runs over the positions
    {
        const int nw = hd / 4;  // dimensions per warp
        const __half* pa = ph + q * PPITCH + 2 * pq;
        uint32_t a0[4], a2[4];
#pragma unroll
        for (int k4 = 0; k4 < 4; ++k4) a0[k4] = *reinterpret_cast<const uint32_t*>(pa + 16 * k4), a2[k4] = *reinterpret_cast<const uint32_t*>(pa + 16 * k4 + 8);
        for (int n0 = warp * nw; n0 < (warp + 1) * nw; n0 += 8) {
            float o[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int k4 = 0; k4 < 4; ++k4) {
                // two 8x8 blocks of V (positions 16*k4 + 0..7 and + 8..15, dimensions n0..n0+7), transposed on load
                const uint32_t addr = smem_u32(vs + (16 * k4 + (lane & 15)) * pitch + n0);
                uint32_t b0, b1;
                asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];" : "=r"(b0), "=r"(b1) : "r"(addr));
                mma_f16_k16(o, a0[k4], 0u, a2[k4], 0u, b0, b1);
            }
            if (q < group) {
                float* dst = scratch + (((size_t)b * nqh + kvh * group + q) * splits + sp) * (hd + 2);
                dst[2 + n0 + 2 * pq] = o[0];
                dst[3 + n0 + 2 * pq] = o[1];
            }
        }
        if (tid < group) {
            float* dst = scratch + (((size_t)b * nqh + kvh * group + tid) * splits + sp) * (hd + 2);
            dst[0] = stat[2 * tid], dst[1] = stat[2 * tid + 1];
        }
    }
}

// Opt-in to more than 48 KiB of dynamic shared memory for the two split kernels.  cudaFuncSetAttribute
// REPLACES the limit, so every caller (the stand-alone entry points and every decoder) goes through this
// one per-device high-water mark and the limit is only ever raised.
inline int attn_opt_in_smem(bool tensor_core, size_t bytes) {
    static size_t high[2][64] = {};
    int dev = 0;
    QMM_CUDA_TRY(cudaGetDevice(&dev));
    const bool track = dev >= 0 && dev < 64;
    if (track && bytes <= high[tensor_core ? 1 : 0][dev]) return QMM_OK;
    if (tensor_core)
        QMM_CUDA_TRY(cudaFuncSetAttribute(attn_decode_split_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
    else
        QMM_CUDA_TRY(cudaFuncSetAttribute(attn_decode_split_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
    if (track) high[tensor_core ? 1 : 0][dev] = bytes;
    return QMM_OK;
}

// Merge of the context splits + Q8_1 of the attention output (the activations of the O projection).
// One CTA per (query head, batch): the split weights are computed once into shared memory, then
// every thread merges its output element with independent loads.
constexpr int ATTN_MAX_SPLITS = 512;
__global__ void attn_combine_q8_kernel(const float* __restrict__ scratch, uint8_t* __restrict__ xq, float* __restrict__ out_f32, int nqh,
                                       int hd, int splits) {
    __shared__ float wgt[ATTN_MAX_SPLITS];
    __shared__ float red[32];
    pdl_release_dependents();
    pdl_wait_prior_grids();
    const int head = blockIdx.x, b = blockIdx.y, lane = threadIdx.x & 31;
    const float* src = scratch + ((size_t)b * nqh + head) * splits * (hd + 2);
    // maxima and sums of all splits in one round of loads (the sums wait in wgt[])
    float m = -INFINITY;
    for (int s = threadIdx.x; s < splits; s += blockDim.x) {
        const float2 ml = *reinterpret_cast<const float2*>(src + (size_t)s * (hd + 2));
        wgt[s] = ml.y;
        m = fmaxf(m, ml.x);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if (lane == 0) red[threadIdx.x >> 5] = m;
    __syncthreads();
    m = red[0];
    for (int w = 1; w < (int)(blockDim.x >> 5); ++w) m = fmaxf(m, red[w]);
    __syncthreads();
    float den = 0.f;
    for (int s = threadIdx.x; s < splits; s += blockDim.x) {
        const float l = wgt[s];
        const float w = l > 0.f ? __expf(src[(size_t)s * (hd + 2)] - m) : 0.f;
        wgt[s] = w;
        den += w * l;
    }
    den = block_sum(den, red);
    const float inv = den > 0.f ? 1.0f / den : 0.f;
    for (int d = threadIdx.x; d < hd; d += blockDim.x) {  // hd is a multiple of 32: whole warps
        float num = 0.f;
#pragma unroll 8
        for (int s = 0; s < splits; ++s) num += wgt[s] * src[(size_t)s * (hd + 2) + 2 + d];
        const float v = num * inv;
        const int e = head * hd + d;
        if (out_f32) out_f32[(size_t)b * nqh * hd + e] = v;
        warp_store_q8_1(v, xq + ((size_t)b * (nqh * hd / 32) + (e >> 5)) * Q8_1_BYTES, lane);
    }
}

__device__ __forceinline__ float gelu_tanh_f(float x) {
    return 0.5f * x * (1.0f + tanhf(0.7978845608028654f * (x + 0.044715f * x * x * x)));
}

// gated activation on the fused [gate | up] projection output + Q8_1: act(gate) * up -> xq (ffn per row)
// out = act(gate) * up for many rows (the prompt path: only the f32 values are needed), four elements per thread
__global__ void act_mul_f32_kernel(const float* __restrict__ gate_up, float* __restrict__ out, __nv_bfloat16* __restrict__ out_bf16, int ffn, int act,
                                   long quads) {
    const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= quads) return;
    const int per_row = ffn / 4;
    const long b = i / per_row;
    const int c = (int)(i - b * per_row) * 4;
    const float* row = gate_up + (size_t)b * 2 * ffn;
    const float4 g = *reinterpret_cast<const float4*>(row + c), u = *reinterpret_cast<const float4*>(row + ffn + c);
    float4 r;
    r.x = (act == 0 ? gelu_tanh_f(g.x) : g.x / (1.0f + __expf(-g.x))) * u.x;
    r.y = (act == 0 ? gelu_tanh_f(g.y) : g.y / (1.0f + __expf(-g.y))) * u.y;
    r.z = (act == 0 ? gelu_tanh_f(g.z) : g.z / (1.0f + __expf(-g.z))) * u.z;
    r.w = (act == 0 ? gelu_tanh_f(g.w) : g.w / (1.0f + __expf(-g.w))) * u.w;
    if (out) *reinterpret_cast<float4*>(out + (size_t)b * ffn + c) = r;
    if (out_bf16) {
        const __nv_bfloat162 lo = __floats2bfloat162_rn(r.x, r.y), hi = __floats2bfloat162_rn(r.z, r.w);
        *reinterpret_cast<uint2*>(out_bf16 + (size_t)b * ffn + c) = make_uint2(*reinterpret_cast<const uint32_t*>(&lo), *reinterpret_cast<const uint32_t*>(&hi));
    }
}

__global__ void act_mul_q8_kernel(const float* __restrict__ gate_up, uint8_t* __restrict__ xq, int ffn, int act, float* __restrict__ out_f32) {
    pdl_release_dependents();
    pdl_wait_prior_grids();
    const int b = blockIdx.y, lane = threadIdx.x & 31;
    const int blk = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (blk >= ffn / 32) return;
    const float* row = gate_up + (size_t)b * 2 * ffn;
    const float g = row[blk * 32 + lane], u = row[ffn + blk * 32 + lane];
    const float a = act == 0 ? gelu_tanh_f(g) : g / (1.0f + __expf(-g));
    if (out_f32) out_f32[(size_t)b * ffn + blk * 32 + lane] = a * u;
    warp_store_q8_1(a * u, xq + ((size_t)b * (ffn / 32) + blk) * Q8_1_BYTES, lane);
}

// argmax over rows of logits (lowest index wins ties), two stages: grid (parts, batch) CTAs each scan a
// contiguous slice and write one candidate {value, index}; the second kernel reduces the candidates.
struct Candidate {
    float value;
    int index;
};
__device__ __forceinline__ void better(float& bv, int& bi, float v, int i) {
    if (v > bv || (v == bv && i < bi)) bv = v, bi = i;
}
__device__ __forceinline__ void block_argmax(float& bv, int& bi, float* sv, int* si) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        better(bv, bi, ov, oi);
    }
    if ((threadIdx.x & 31) == 0) sv[threadIdx.x >> 5] = bv, si[threadIdx.x >> 5] = bi;
    __syncthreads();
    if (threadIdx.x == 0)
        for (int w = 1; w < (int)(blockDim.x >> 5); ++w) better(bv, bi, sv[w], si[w]);
}
__global__ void argmax_partial_kernel(const float* __restrict__ logits, Candidate* __restrict__ cand, int vocab) {
    __shared__ float sv[32];
    __shared__ int si[32];
    pdl_release_dependents();
    pdl_wait_prior_grids();
    const int b = blockIdx.y, parts = gridDim.x;
    const int per = (vocab + parts - 1) / parts;
    const int i0 = blockIdx.x * per, i1 = min(vocab, i0 + per);
    const float* row = logits + (size_t)b * vocab;
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = i0 + threadIdx.x; i < i1; i += blockDim.x) better(bv, bi, row[i], i);
    block_argmax(bv, bi, sv, si);
    if (threadIdx.x == 0) cand[(size_t)b * parts + blockIdx.x] = Candidate{bv, bi};
}
__global__ void argmax_final_kernel(const Candidate* __restrict__ cand, int parts, int* __restrict__ out, int index_offset,
                                    float* __restrict__ best_val) {
    __shared__ float sv[32];
    __shared__ int si[32];
    pdl_release_dependents();
    pdl_wait_prior_grids();
    const int b = blockIdx.x;
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < parts; i += blockDim.x) better(bv, bi, cand[(size_t)b * parts + i].value, cand[(size_t)b * parts + i].index);
    block_argmax(bv, bi, sv, si);
    if (threadIdx.x == 0) {
        out[b] = bi + index_offset;
        if (best_val) best_val[b] = bv;
    }
}

// Tensor-parallel greedy pick: every rank has the argmax of its vocabulary slice (global index and value);
// it pushes both as two exchange words per sequence into every rank's area, then reads all ranks' pairs
// from its own area (bounded polls) and keeps the best (lowest index on ties), so all ranks continue with
// the same token.  One CTA, one thread per sequence.  A rank whose peer never arrives stores -1.
__global__ void tp_pick_token_kernel(const float* __restrict__ best_val, int* __restrict__ tokens_io, const TpPush push, const TpRecv rcv,
                                     int batch) {
    __shared__ int give_up;
    pdl_release_dependents();
    if (threadIdx.x == 0) give_up = 0;
    __syncthreads();
    pdl_wait_prior_grids();
    const unsigned seq = tp_next_seq(rcv.counter);
    const int b = threadIdx.x;
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    bool ok = true;
    if (b < batch) {
        tp_push_word(push, seq, 2l * b, best_val[b]);
        tp_push_word(push, seq, 2l * b + 1, __int_as_float(tokens_io[b]));
        for (int r = 0; r < rcv.tp && ok; ++r) {
            float v = 0.f, fi = 0.f;
            ok = tp_poll_word(rcv, seq, r, 2l * b, v, &give_up) && tp_poll_word(rcv, seq, r, 2l * b + 1, fi, &give_up);
            const int i = __float_as_int(fi);
            if (ok && (v > bv || (v == bv && i < bi))) bv = v, bi = i;
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        if (give_up) atomicExch(&g_device_status, DEV_TIMEOUT_PEER);
        tp_consumer_done(rcv, seq, 1u);
    }
    if (b < batch) tokens_io[b] = ok ? bi : -1;
}

}  // namespace qmm
