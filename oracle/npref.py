"""numpy restatement of the block formats, written independently of ``qmm_oracle.c``.

TEST INFRASTRUCTURE ONLY.  It exists so the C oracle is not its own judge: the
two are compared bit for bit on dequantised values, packed codes and integer
block sums, and this module generates the known-answer fixtures committed under
``tests/golden``.  Parity with the upstream project is unpinned (it has no
implementation of these formats); see ``qmm_oracle.h``.
"""
import numpy as np

Q8_0, Q8_1, Q4_K, Q6_K = 8, 9, 12, 14
_M64 = (1 << 64) - 1


def _mix64(z):
    z = (z + np.uint64(0x9E3779B97F4A7C15))
    z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
    z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
    return z ^ (z >> np.uint64(31))


def fill_normal(n, seed, sigma, first_index=0):
    with np.errstate(over="ignore"):
        idx = np.arange(first_index, first_index + n, dtype=np.uint64)
        h1 = _mix64(np.uint64((seed * 0xD1342543DE82EF95) & _M64) + idx)
        h2 = _mix64(h1)
    s = np.zeros(n, dtype=np.int64)
    for c in range(4):
        s += ((h1 >> np.uint64(16 * c)) & np.uint64(0xFFFF)).astype(np.int64)
        s += ((h2 >> np.uint64(16 * c)) & np.uint64(0xFFFF)).astype(np.int64)
    z = (s - 262140).astype(np.float32) * (np.float32(1.0) / np.float32(53510.0))
    return z * np.float32(sigma)


def _f16(b):
    """(..., 2) uint8 little-endian -> float32 value of the fp16."""
    return np.ascontiguousarray(b).view(np.float16)[..., 0].astype(np.float32)


def _round_away(v):
    v = np.asarray(v, dtype=np.float64)  # |v| + 0.5 is exact in binary64 for every binary32 v
    return (np.sign(v) * np.floor(np.abs(v) + 0.5)).astype(np.int32)


def quantize_q8_1(x):
    x = np.asarray(x, dtype=np.float32).reshape(-1, 32)
    amax = np.abs(x).max(axis=1)
    d = np.minimum(amax / np.float32(127.0), np.float32(65504.0)).astype(np.float16)
    df = d.astype(np.float32)
    with np.errstate(divide="ignore", invalid="ignore"):
        q = np.where(df[:, None] > 0, np.clip(_round_away(x / df[:, None]), -127, 127), 0).astype(np.int8)
    s = (df * q.sum(axis=1, dtype=np.int32).astype(np.float32)).astype(np.float16)
    out = np.empty((x.shape[0], 36), dtype=np.uint8)
    out[:, 0:2] = d.view(np.uint8).reshape(-1, 2)
    out[:, 2:4] = s.view(np.uint8).reshape(-1, 2)
    out[:, 4:] = q.view(np.uint8)
    return out.reshape(-1)


def q8_1_parts(xq):
    b = np.asarray(xq, dtype=np.uint8).reshape(-1, 36)
    return _f16(b[:, 0:2]), _f16(b[:, 2:4]), b[:, 4:].view(np.int8).astype(np.int32)


def q4k_scales(sb):
    """(nb, 12) packed -> (nb, 8) scale codes, (nb, 8) min codes."""
    s = sb.astype(np.int32)
    sc = np.empty((s.shape[0], 8), dtype=np.int32)
    mn = np.empty_like(sc)
    sc[:, :4] = s[:, 0:4] & 63
    mn[:, :4] = s[:, 4:8] & 63
    sc[:, 4:] = (s[:, 8:12] & 15) | ((s[:, 0:4] >> 6) << 4)
    mn[:, 4:] = (s[:, 8:12] >> 4) | ((s[:, 4:8] >> 6) << 4)
    return sc, mn


def q4k_codes(qs):
    """(nb, 128) -> (nb, 256) codes in element order."""
    g = qs.reshape(-1, 4, 32).astype(np.int32)
    return np.stack([g & 15, g >> 4], axis=2).reshape(-1, 256)


def q6k_codes(ql, qh):
    """(nb, 128), (nb, 64) -> (nb, 256) codes in element order."""
    l = ql.reshape(-1, 2, 2, 32).astype(np.int32)      # half, which 32-run of ql, l
    h = qh.reshape(-1, 2, 32).astype(np.int32)
    out = np.empty((l.shape[0], 2, 4, 32), dtype=np.int32)
    out[:, :, 0] = (l[:, :, 0] & 15) | (((h >> 0) & 3) << 4)
    out[:, :, 1] = (l[:, :, 1] & 15) | (((h >> 2) & 3) << 4)
    out[:, :, 2] = (l[:, :, 0] >> 4) | (((h >> 4) & 3) << 4)
    out[:, :, 3] = (l[:, :, 1] >> 4) | (((h >> 6) & 3) << 4)
    return out.reshape(-1, 256)


def dequantize(qtype, w):
    """Packed bytes (any shape, whole blocks) -> flat float32 values."""
    w = np.asarray(w, dtype=np.uint8)
    if qtype == Q8_0:
        b = w.reshape(-1, 34)
        return (_f16(b[:, 0:2])[:, None] * b[:, 2:].view(np.int8).astype(np.float32)).reshape(-1)
    if qtype == Q8_1:
        d, _, q = q8_1_parts(w)
        return (d[:, None] * q.astype(np.float32)).reshape(-1)
    if qtype == Q4_K:
        b = w.reshape(-1, 144)
        d, dmin = _f16(b[:, 0:2]), _f16(b[:, 2:4])
        sc, mn = q4k_scales(b[:, 4:16])
        q = q4k_codes(b[:, 16:]).reshape(-1, 8, 32).astype(np.float32)
        ds = d[:, None] * sc.astype(np.float32)
        off = dmin[:, None] * mn.astype(np.float32)
        return (ds[:, :, None] * q - off[:, :, None]).astype(np.float32).reshape(-1)
    if qtype == Q6_K:
        b = w.reshape(-1, 210)
        d = _f16(b[:, 208:210])
        sc = b[:, 192:208].view(np.int8).astype(np.float32)
        q = (q6k_codes(b[:, 0:128], b[:, 128:192]) - 32).reshape(-1, 16, 16).astype(np.float32)
        ds = d[:, None] * sc
        return (ds[:, :, None] * q).astype(np.float32).reshape(-1)
    raise ValueError(qtype)


def block_dots(qtype, w, xq, k):
    """Integer sums per 32 (Q8_0, Q4_K) or 16 (Q6_K) elements; w holds n rows of k."""
    _, _, qx = q8_1_parts(xq)
    qx = qx.reshape(-1)[:k]
    w = np.asarray(w, dtype=np.uint8)
    if qtype == Q8_0:
        qw = w.reshape(-1, 34)[:, 2:].view(np.int8).astype(np.int32).reshape(-1, k)
        return (qw * qx).reshape(qw.shape[0], k // 32, 32).sum(axis=2, dtype=np.int32)
    if qtype == Q4_K:
        qw = q4k_codes(w.reshape(-1, 144)[:, 16:]).reshape(-1, k)
        return (qw * qx).reshape(qw.shape[0], k // 32, 32).sum(axis=2, dtype=np.int32)
    if qtype == Q6_K:
        b = w.reshape(-1, 210)
        qw = (q6k_codes(b[:, 0:128], b[:, 128:192]) - 32).reshape(-1, k)
        return (qw * qx).reshape(qw.shape[0], k // 16, 16).sum(axis=2, dtype=np.int32)
    raise ValueError(qtype)
