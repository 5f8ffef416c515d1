"""ctypes binding of ``libqmm_oracle.so`` (the C oracle).  Test infrastructure only."""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "_build", "libqmm_oracle.so")

Q8_0, Q8_1, Q4_K, Q6_K = 8, 9, 12, 14
BLOCK_ELEMS = {Q8_0: 32, Q8_1: 32, Q4_K: 256, Q6_K: 256}
BLOCK_BYTES = {Q8_0: 34, Q8_1: 36, Q4_K: 144, Q6_K: 210}
TYPE_NAMES = {Q8_0: "q8_0", Q8_1: "q8_1", Q4_K: "q4_k", Q6_K: "q6_k"}
# integer dot sums reported per this many elements
DOT_GROUP = {Q8_0: 32, Q4_K: 32, Q6_K: 16}


def build(force=False):
    """Compile the C oracle with its Makefile if the shared object is missing or stale."""
    src = [os.path.join(_HERE, f) for f in ("qmm_oracle.c", "qmm_oracle.h", "Makefile")]
    stale = not os.path.exists(_SO) or any(os.path.getmtime(s) > os.path.getmtime(_SO) for s in src)
    if force or stale:
        subprocess.check_call(["make", "-C", _HERE, "-s"] + (["-B"] if force else []))
    return _SO


_lib = None


def lib():
    global _lib
    if _lib is None:
        build()  # compiles only when the shared object is missing or older than its sources
        L = C.CDLL(_SO)
        vp, i64, i32, f32, u64 = C.c_void_p, C.c_long, C.c_int, C.c_float, C.c_uint64
        L.qo_fill_normal.argtypes = [vp, i64, u64, f32, i64]
        L.qo_row_bytes.argtypes = [i32, i64]
        L.qo_row_bytes.restype = i64
        L.qo_quantize_rows.argtypes = [i32, vp, vp, i64, i64]
        L.qo_dequantize_rows.argtypes = [i32, vp, vp, i64, i64]
        L.qo_dequantize_rows_bf16.argtypes = [i32, vp, vp, i64, i64]
        L.qo_block_dots.argtypes = [i32, vp, vp, vp, i64, i64]
        L.qo_matvec.argtypes = [i32, vp, vp, vp, i64, i64, i64]
        L.qo_gemm_bf16.argtypes = [i32, vp, vp, vp, vp, i64, i64, i64]
        L.qo_rmsnorm.argtypes = [vp, vp, vp, i64, i64, f32]
        L.qo_rope_neox.argtypes = [vp, i64, i64, i64, i64, f32]
        L.qo_gelu_mul.argtypes = [vp, vp, vp, i64]
        L.qo_silu_mul.argtypes = [vp, vp, vp, i64]
        L.qo_attn_decode.argtypes = [vp, vp, vp, vp, i64, i64, i64, i64]
        L.qo_attn_prefill.argtypes = [vp, vp, vp, vp, i64, i64, i64, i64, i64, C.c_double]
        L.qo_f32_to_f16.argtypes = [f32]
        L.qo_f32_to_f16.restype = C.c_uint16
        L.qo_f16_to_f32.argtypes = [C.c_uint16]
        L.qo_f16_to_f32.restype = f32
        L.qo_f32_to_bf16.argtypes = [f32]
        L.qo_f32_to_bf16.restype = C.c_uint16
        L.qo_num_threads.restype = i32
        L.qo_set_num_threads.argtypes = [i32]
        _lib = L
    return _lib


def _p(a):
    return a.ctypes.data_as(C.c_void_p)


def _c(a, dt):
    a = np.ascontiguousarray(a, dtype=dt)
    return a


def row_bytes(qtype, k):
    assert k % BLOCK_ELEMS[qtype] == 0, (qtype, k)
    return k // BLOCK_ELEMS[qtype] * BLOCK_BYTES[qtype]


def num_threads():
    return lib().qo_num_threads()


def set_num_threads(n):
    """OpenMP threads of the C oracle (overrides an inherited OMP_NUM_THREADS)."""
    lib().qo_set_num_threads(int(n))


def fill_normal(n, seed, sigma, first_index=0):
    out = np.empty(n, dtype=np.float32)
    lib().qo_fill_normal(_p(out), n, seed, sigma, first_index)
    return out


def quantize(qtype, x):
    """x (rows, k) float32 -> packed uint8 (rows, row_bytes)."""
    x = _c(x, np.float32)
    if x.ndim == 1:
        x = x[None]
    rows, k = x.shape
    out = np.empty((rows, row_bytes(qtype, k)), dtype=np.uint8)
    lib().qo_quantize_rows(qtype, _p(x), _p(out), rows, k)
    return out


def dequantize(qtype, w, k):
    w = _c(w, np.uint8).reshape(-1, row_bytes(qtype, k))
    out = np.empty((w.shape[0], k), dtype=np.float32)
    lib().qo_dequantize_rows(qtype, _p(w), _p(out), w.shape[0], k)
    return out


def dequantize_bf16(qtype, w, k):
    """Returns the bf16 bit patterns (uint16)."""
    w = _c(w, np.uint8).reshape(-1, row_bytes(qtype, k))
    out = np.empty((w.shape[0], k), dtype=np.uint16)
    lib().qo_dequantize_rows_bf16(qtype, _p(w), _p(out), w.shape[0], k)
    return out


def block_dots(qtype, w, xq, k):
    w = _c(w, np.uint8).reshape(-1, row_bytes(qtype, k))
    xq = _c(xq, np.uint8).reshape(-1)
    assert xq.size == row_bytes(Q8_1, k)
    out = np.empty((w.shape[0], k // DOT_GROUP[qtype]), dtype=np.int32)
    lib().qo_block_dots(qtype, _p(w), _p(xq), _p(out), w.shape[0], k)
    return out


def matvec(qtype, w, xq, k):
    """w (n, row_bytes) packed, xq (m, q8_1 row bytes) packed -> y (m, n) float32."""
    w = _c(w, np.uint8).reshape(-1, row_bytes(qtype, k))
    xq = _c(xq, np.uint8).reshape(-1, row_bytes(Q8_1, k))
    y = np.empty((xq.shape[0], w.shape[0]), dtype=np.float32)
    lib().qo_matvec(qtype, _p(w), _p(xq), _p(y), xq.shape[0], w.shape[0], k)
    return y


def gemm_bf16(qtype, w, x_bf16, k):
    """x_bf16 (m, k) uint16 bit patterns -> (y bf16 bits (m, n), y fp32 accumulators (m, n))."""
    w = _c(w, np.uint8).reshape(-1, row_bytes(qtype, k))
    x = _c(x_bf16, np.uint16).reshape(-1, k)
    m, n = x.shape[0], w.shape[0]
    y = np.empty((m, n), dtype=np.uint16)
    yf = np.empty((m, n), dtype=np.float32)
    lib().qo_gemm_bf16(qtype, _p(w), _p(x), _p(y), _p(yf), m, n, k)
    return y, yf


def f32_to_bf16_bits(a):
    a = _c(a, np.float32)
    u = a.view(np.uint32).astype(np.uint64)
    nan = (u & 0x7FFFFFFF) > 0x7F800000
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
    r[nan] = ((u[nan] >> 16) | 0x40).astype(np.uint16)
    return r


def bf16_bits_to_f32(b):
    return (_c(b, np.uint16).astype(np.uint32) << 16).view(np.float32)


def rmsnorm(x, gamma, eps):
    x = _c(x, np.float32)
    rows, cols = x.shape
    out = np.empty_like(x)
    g = None if gamma is None else _c(gamma, np.float32)
    lib().qo_rmsnorm(_p(x), None if g is None else _p(g), _p(out), rows, cols, eps)
    return out


def rope_neox(buf, head_dim, heads_per_tok, pos0, theta):
    b = _c(buf, np.float32).copy().reshape(-1, head_dim)
    lib().qo_rope_neox(_p(b), b.shape[0], head_dim, heads_per_tok, pos0, theta)
    return b


def gelu_mul(gate, up):
    g, u = _c(gate, np.float32), _c(up, np.float32)
    out = np.empty_like(g)
    lib().qo_gelu_mul(_p(g), _p(u), _p(out), g.size)
    return out


def silu_mul(gate, up):
    g, u = _c(gate, np.float32), _c(up, np.float32)
    out = np.empty_like(g)
    lib().qo_silu_mul(_p(g), _p(u), _p(out), g.size)
    return out


def attn_prefill(q, k, v, nqh, nkv, hd, prefix, kq_scale=1.0):
    """q (t, nqh*hd), k, v (t, nkv*hd) f32 -> out (t, nqh*hd): the upstream's gqa_masked_attn."""
    q, k, v = _c(q, np.float32), _c(k, np.float32), _c(v, np.float32)
    t = q.shape[0]
    out = np.empty((t, nqh * hd), dtype=np.float32)
    lib().qo_attn_prefill(_p(q), _p(k), _p(v), _p(out), t, nqh, nkv, hd, prefix, float(kq_scale))
    return out


DENSE_ACTS = ("linear", "relu", "sigmoid", "leaky_relu", "prelu", "elu", "selu", "tanh", "silu", "gelu")


def dense(qtype, w, x, bias, act, alpha, k, via="q8_1"):
    """Quantized dense layer y = act(x . w^T + bias): the composition the upstream runs for LayerKind::Dense
    (recipe-infer/src/forward.rs:372-431) with the product taken through the Q8_1 form of x and the packed
    weight (quantize + matvec above), or through bf16(x) and the bf16 form of the weight (via="bf16").  The activations follow the upstream's kernels (elementwise.hip:1521-1560,
    gapact.hip:6-18), evaluated in float64 and rounded to float32."""
    x = _c(x, np.float32)
    if via == "bf16":   # many rows: x rounded to bf16, exact products, f32 accumulators (gemm_bf16 above)
        y = gemm_bf16(qtype, w, f32_to_bf16_bits(x), k)[1]
    else:
        y = matvec(qtype, w, quantize(Q8_1, x), k)
    z = y if bias is None else (y + _c(bias, np.float32)[None, :]).astype(np.float32)
    z = z.astype(np.float64)
    if act == "linear":
        r = z
    elif act == "relu":
        r = np.maximum(z, 0.0)
    elif act == "sigmoid":
        r = 1.0 / (1.0 + np.exp(-z))
    elif act in ("leaky_relu", "prelu"):
        r = np.where(z > 0, z, alpha * z)
    elif act == "elu":
        r = np.where(z > 0, z, alpha * (np.exp(z) - 1.0))
    elif act == "selu":
        r = 1.0507009873554804934193349852946 * np.where(z > 0, z, 1.6732632423543772848170429916717 * (np.exp(z) - 1.0))
    elif act == "tanh":
        r = np.tanh(z)
    elif act == "silu":
        r = z / (1.0 + np.exp(-z))
    elif act == "gelu":
        r = 0.5 * z * (1.0 + np.tanh(0.7978845608028654 * (z + 0.044715 * z ** 3)))
    else:
        raise ValueError(act)
    return r.astype(np.float32)


def attn_decode(q, kc, vc, nqh, nkv, hd, length):
    """q (nqh, hd) f32; kc/vc (cap, nkv, hd) fp16 bit patterns (uint16 or float16)."""
    q = _c(q, np.float32)
    kc = np.ascontiguousarray(kc).view(np.uint16)
    vc = np.ascontiguousarray(vc).view(np.uint16)
    out = np.empty((nqh, hd), dtype=np.float32)
    lib().qo_attn_decode(_p(q), _p(kc), _p(vc), _p(out), nqh, nkv, hd, length)
    return out
