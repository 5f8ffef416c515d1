"""Host-side mirror of the upstream operator API for the quantized path.

The upstream's operators are Rust functions `gpu_<op>_into(inputs: &GpuBuffer..,
out: &GpuBuffer, dims..)` that pass raw device pointers to an `extern "C"
launch_<op>` on the null stream and then call `check_launch()`
(gpu-core/src/infer_ops.rs:224-240, gpu-core/src/kernels.rs:8-13); an allocating
twin `gpu_<op>(..) -> GpuBuffer` allocates and calls the `_into` form
(gpu-core/src/infer_ops.rs:105-115).  The functions below keep those names,
argument order and the caller-owns-the-output rule, with torch CUDA tensors
standing in for `GpuBuffer` (device memory + byte length) and the current torch
stream standing in for the null stream.  Sizes are trusted exactly as upstream
("caller must ensure buffer sizes match the declared dimensions",
gpu-core/src/kernels.rs:1-2) except that obviously short buffers raise.

Everything here launches CUDA kernels from libqmm.so; there is no CPU path.
"""
import torch

from . import _lib
from ._lib import Q4_K, Q6_K, Q8_0, Q8_1, BLOCK_BYTES, BLOCK_ELEMS, TYPE_NAMES, check, lib

__all__ = [
    "Q8_0", "Q8_1", "Q4_K", "Q6_K", "row_bytes", "check_launch",
    "gpu_quantize_q8_1_into", "gpu_quantize_q8_1", "gpu_quantize_weights_into", "gpu_quantize_weights",
    "gpu_dequantize_into", "gpu_dequantize", "gpu_qmatvec_into", "gpu_qmatvec", "gpu_qblock_dots",
    "MatvecJobs", "gpu_qmatvec_batch_into",
    "gpu_qgemm_q4_k_bf16_into", "gpu_qgemm_q4_k_bf16",
    "gpu_qlinear",
]


def _ptr(t):
    return t.data_ptr()


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _need(t, nbytes, name):
    if not t.is_cuda or not t.is_contiguous():
        raise ValueError(f"{name}: expected a contiguous CUDA tensor")
    if t.numel() * t.element_size() < nbytes:
        raise ValueError(f"{name}: buffer holds {t.numel() * t.element_size()} bytes, needs {nbytes}")


def row_bytes(qtype, k):
    r = lib().qmm_row_bytes(qtype, k)
    check(r if r < 0 else 0, f"row_bytes({TYPE_NAMES.get(qtype, qtype)}, {k})")
    return r


def check_launch():
    """Counterpart of the upstream's post-launch assert (gpu-core/src/kernels.rs:8-13):
    raises if a kernel of this library gave up on a bounded wait.  Synchronises the device."""
    import ctypes
    v = ctypes.c_int(0)
    check(lib().qmm_device_status(ctypes.byref(v)), "qmm_device_status")
    if v.value != 0:
        raise RuntimeError(f"libqmm device status {v.value}: a kernel abandoned a bounded wait")


# ---- activations ----------------------------------------------------------------
def gpu_quantize_q8_1_into(x, xq, m, k):
    """x (m,k) f32 -> xq, m*(k/32) Q8_1 blocks."""
    _need(x, m * k * 4, "x")
    _need(xq, m * row_bytes(Q8_1, k), "xq")
    check(lib().launch_quantize_q8_1(_ptr(x), _ptr(xq), m, k, _stream()), "launch_quantize_q8_1")


def gpu_quantize_q8_1(x):
    x = x.contiguous()
    m, k = (1, x.numel()) if x.dim() == 1 else x.shape
    xq = torch.empty(m * row_bytes(Q8_1, k), dtype=torch.uint8, device=x.device)
    gpu_quantize_q8_1_into(x, xq, m, k)
    return xq


# ---- weights ----------------------------------------------------------------------
_QUANT = {Q8_0: "launch_quantize_q8_0", Q4_K: "launch_quantize_q4_k", Q6_K: "launch_quantize_q6_k"}


def gpu_quantize_weights_into(qtype, w, out, rows, k):
    _need(w, rows * k * 4, "w")
    _need(out, rows * row_bytes(qtype, k), "out")
    check(getattr(lib(), _QUANT[qtype])(_ptr(w), _ptr(out), rows, k, _stream()), _QUANT[qtype])


def gpu_quantize_weights(qtype, w):
    w = w.contiguous()
    rows, k = w.shape
    out = torch.empty(rows * row_bytes(qtype, k), dtype=torch.uint8, device=w.device)
    gpu_quantize_weights_into(qtype, w, out, rows, k)
    return out


def gpu_dequantize_into(qtype, w, out, n_elems):
    """Decode n_elems packed elements into `out` (float32 or bfloat16): the upstream's
    gpu_widen_bf16_into (gpu-core/src/infer_ops.rs:96-101) for block formats."""
    _need(w, n_elems // BLOCK_ELEMS[qtype] * BLOCK_BYTES[qtype], "w")
    _need(out, n_elems * out.element_size(), "out")
    suffix = {torch.float32: "f32", torch.bfloat16: "bf16"}[out.dtype]
    name = f"launch_dequantize_{TYPE_NAMES[qtype]}_{suffix}"
    check(getattr(lib(), name)(_ptr(w), _ptr(out), n_elems, _stream()), name)


def gpu_dequantize(qtype, w, n_elems, dtype=torch.float32):
    out = torch.empty(n_elems, dtype=dtype, device=w.device)
    gpu_dequantize_into(qtype, w, out, n_elems)
    return out


# ---- the operator -------------------------------------------------------------------
def gpu_qmatvec_into(qtype, w, xq, out, m, n, k):
    """out(m,n) = xq(m,k) . w(n,k)^T; w packed `qtype` rows, xq Q8_1 rows, out f32.
    Same shape contract as gpu_gemm_bt_f64_into (gpu-core/src/infer_ops.rs:224-240):
    all row-major, `out` caller-owned and distinct from the inputs."""
    _need(w, n * row_bytes(qtype, k), "w")
    _need(xq, m * row_bytes(Q8_1, k), "xq")
    _need(out, m * n * 4, "out")
    check(lib().launch_qmatvec(qtype, _ptr(w), _ptr(xq), _ptr(out), m, n, k, _stream()),
          f"launch_qmatvec_{TYPE_NAMES.get(qtype, qtype)}")


def gpu_qmatvec(qtype, w, xq, m, n, k):
    out = torch.empty((m, n), dtype=torch.float32, device=w.device)
    gpu_qmatvec_into(qtype, w, xq, out, m, n, k)
    return out


class MatvecJobs:
    """A host-side list of independent projections for gpu_qmatvec_batch_into (one launch for all).
    Holds references to the tensors so the device pointers stay valid while the list is in use."""

    def __init__(self):
        self._jobs, self._keep = [], []

    def add(self, qtype, w, xq, out, n, k, y_stride=0, select=None, select_stride_bytes=0):
        """out(m,n) = xq(m,k) . w(n,k)^T, as gpu_qmatvec_into; `select` (int32 device tensor) makes the
        matrix w + select[0] * select_stride_bytes, resolved on the device when the kernel runs."""
        self._jobs.append(_lib.MatvecJob(qtype, n, k, _ptr(w), _ptr(xq), _ptr(out), y_stride,
                                         _ptr(select) if select is not None else None, select_stride_bytes))
        self._keep.append((w, xq, out, select))
        return self

    def __len__(self):
        return len(self._jobs)

    def array(self):
        return (_lib.MatvecJob * len(self._jobs))(*self._jobs)


def gpu_qmatvec_batch_into(jobs, m):
    """Every job of `jobs` (MatvecJobs) in one launch: persistent CTAs walk from one matrix into the
    next.  The upstream issues such projections as consecutive gpu_gemm_bt_f64_into calls on one
    input (examples/gemma4.rs:653-667, 675-678, 726-742)."""
    arr = jobs.array()
    check(lib().launch_qmatvec_batch(arr, len(jobs), m, _stream()), "launch_qmatvec_batch")


def gpu_qblock_dots(qtype, w, xq, n, k):
    group = 16 if qtype == Q6_K else 32
    out = torch.empty((n, k // group), dtype=torch.int32, device=w.device)
    check(lib().launch_qblock_dots(qtype, _ptr(w), _ptr(xq), _ptr(out), n, k, _stream()), "launch_qblock_dots")
    return out


def gpu_qgemm_q4_k_bf16_into(w, x, out, m, n, k):
    """out(m,n) = x(m,k) . bf16(w(n,k))^T on the tensor cores; x bf16, w Q4_K rows, out bf16 (or
    float32: the unrounded accumulators).  The prefill form of gpu_gemm_bt_f64_into."""
    _need(w, n * row_bytes(Q4_K, k), "w")
    _need(x, m * k * 2, "x")
    if x.dtype != torch.bfloat16:
        raise ValueError("x must be bfloat16")
    _need(out, m * n * out.element_size(), "out")
    name = "launch_qgemm_q4_k_bf16" if out.dtype == torch.bfloat16 else "launch_qgemm_q4_k_bf16_f32acc"
    if out.dtype not in (torch.bfloat16, torch.float32):
        raise ValueError("out must be bfloat16 or float32")
    check(getattr(lib(), name)(_ptr(w), _ptr(x), _ptr(out), m, n, k, _stream()), name)


def gpu_qgemm_q4_k_bf16(w, x, n, k, dtype=torch.bfloat16):
    x = x.contiguous()
    m = x.shape[0]
    out = torch.empty((m, n), dtype=dtype, device=x.device)
    gpu_qgemm_q4_k_bf16_into(w, x, out, m, n, k)
    return out


def gpu_qlinear(qtype, w, x, n, k):
    """Convenience: f32 activations (m,k) -> quantize to Q8_1 -> matvec.  Allocates."""
    x = x.contiguous()
    m = 1 if x.dim() == 1 else x.shape[0]
    return gpu_qmatvec(qtype, w, gpu_quantize_q8_1(x.reshape(m, k)), m, n, k)
