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
    "MatvecJobs", "gpu_qmatvec_batch_into", "gpu_norm_qmatvec_batch_into", "gpu_glu_qmatvec_batch_into", "TpComm", "gpu_qmatvec_tp_into", "gpu_qmatvec_batch_tp_into",
    "gpu_qgemm_q4_k_bf16_into", "gpu_qgemm_q4_k_bf16", "gpu_qdense_into", "DENSE_ACTS", "gpu_gqa_attn_into", "gpu_gqa_attn_at_into", "gpu_gemm_bt_bf16_into",
    "gpu_qlinear",
    "gpu_rmsnorm_q8_1_into", "gpu_rope_kv_append", "gpu_glu_act_q8_1_into", "gpu_embed_rows_into", "gpu_argmax_rows",
    "gpu_scale_f32_inplace", "gpu_moe_router_topk", "gpu_moe_experts_into",
]


def _ptr(t):
    return t.data_ptr()


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _opt(t):
    return _ptr(t) if t is not None else None


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

    def add(self, qtype, w, xq, out, n, k, y_stride=0, select=None, select_stride_bytes=0, tp_sum=False):
        """out(m,n) = xq(m,k) . w(n,k)^T, as gpu_qmatvec_into; `select` (int32 device tensor) makes the
        matrix w + select[0] * select_stride_bytes, resolved on the device when the kernel runs; tp_sum
        (gpu_qmatvec_batch_tp_into only): the outputs are summed over the tensor-parallel ranks."""
        self._jobs.append(_lib.MatvecJob(qtype, n, k, _ptr(w), _opt(xq), _ptr(out), y_stride,
                                         _ptr(select) if select is not None else None, select_stride_bytes, 1 if tp_sum else 0))
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


def gpu_norm_qmatvec_batch_into(x_in, x_add, gamma, x_out, eps, jobs, m):
    """Residual add + RMSNorm + Q8_1 built inside the job-list launch that consumes them (the jobs' xq is
    not used): examples/gemma4.rs:646-667 as one launch.  x_out (or None) receives x_in + x_add."""
    arr = jobs.array()
    check(lib().launch_norm_qmatvec_batch(_ptr(x_in), _opt(x_add), _opt(gamma), _opt(x_out), eps, arr, len(jobs), m, _stream()),
          "launch_norm_qmatvec_batch")


def gpu_glu_qmatvec_batch_into(gate_up, act, jobs, m):
    """Gated activation + Q8_1 built inside the job-list launch that consumes them (examples/gemma4.rs:677-678)."""
    arr = jobs.array()
    check(lib().launch_glu_qmatvec_batch(_ptr(gate_up), act, arr, len(jobs), m, _stream()), "launch_glu_qmatvec_batch")


class TpComm:
    """One rank's end of the tensor-parallel sum (qmm_tp_comm_* of include/qmm.h).  The 64-byte handles of
    the ranks' exchange areas travel through torch.distributed (any host channel would do)."""

    def __init__(self, capacity_floats, group=None):
        import ctypes as C
        import torch.distributed as dist
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.h = C.c_void_p()
        check(lib().qmm_tp_comm_create(self.rank, self.world, capacity_floats, C.byref(self.h)), "qmm_tp_comm_create")
        buf = C.create_string_buffer(64)
        check(lib().qmm_tp_comm_export(self.h, buf), "qmm_tp_comm_export")
        handles = [None] * self.world
        dist.all_gather_object(handles, bytes(buf.raw), group=group)
        for r, hb in enumerate(handles):
            if r != self.rank:
                check(lib().qmm_tp_comm_import(self.h, r, C.create_string_buffer(hb, 64)), "qmm_tp_comm_import")
        check(lib().qmm_tp_comm_ready(self.h), "qmm_tp_comm_ready")
        dist.barrier(group=group)

    def close(self):
        if self.h:
            lib().qmm_tp_comm_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def gpu_qmatvec_tp_into(comm, qtype, w, xq, out, m, n, k):
    """Row-parallel projection: this rank's (n, k) column shard against its slice of the activations;
    out(m,n) receives the sum over the ranks (bit-identical on all of them).  Collective."""
    _need(w, n * row_bytes(qtype, k), "w")
    _need(xq, m * row_bytes(Q8_1, k), "xq")
    _need(out, m * n * 4, "out")
    check(lib().launch_qmatvec_tp(comm.h, qtype, _ptr(w), _ptr(xq), _ptr(out), m, n, k, _stream()), "launch_qmatvec_tp")


def gpu_qmatvec_batch_tp_into(comm, jobs, m):
    """A job list in which the jobs added with tp_sum=True are summed over the ranks.  Collective."""
    arr = jobs.array()
    check(lib().launch_qmatvec_batch_tp(comm.h, arr, len(jobs), m, _stream()), "launch_qmatvec_batch_tp")


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


# ---- the small per-layer operators -----------------------------------------------------
def gpu_rmsnorm_q8_1_into(x, gamma, xq, rows, cols, eps, add=None, out_f32=None):
    """x (rows, cols) f32 [+= add, in place] -> xq = Q8_1(rmsnorm(x) * gamma); the upstream's
    gpu_rmsnorm_f64_into (gpu-core/src/infer_ops.rs:117-139) fused with the residual add before it and
    the activation quantization after it.  gamma None: the scale-less variant; out_f32 (optional)
    receives the normalised values."""
    _need(x, rows * cols * 4, "x")
    _need(xq, rows * row_bytes(Q8_1, cols), "xq")
    check(lib().launch_add_rmsnorm_q8_1(_ptr(x), _opt(add), _opt(gamma), _ptr(xq), _opt(out_f32), rows, cols, eps, _stream()),
          "launch_add_rmsnorm_q8_1")


def gpu_rope_kv_append(qkv, kcache, vcache, batch, n_q_heads, n_kv_heads, head_dim, pos, ctx_cap, theta):
    """NeoX rotary embedding of the q heads in place and append of the rotated k and the v heads to the fp16
    caches at `pos`: the upstream's gpu_rope_partial (gpu-core/src/infer_ops.rs:61-83) with rotary_dim ==
    head_dim, for one new token per sequence."""
    check(lib().launch_rope_kv_append(_ptr(qkv), _ptr(kcache), _ptr(vcache), batch, n_q_heads, n_kv_heads, head_dim, pos, ctx_cap, theta,
                                      _stream()), "launch_rope_kv_append")


def gpu_glu_act_q8_1_into(gate_up, xq, rows, half, act, out_f32=None):
    """gate_up (rows, 2*half) = [gate | up] -> xq = Q8_1(act(gate) * up): the upstream's gpu_glu_gelu_into
    (gpu-core/src/infer_ops.rs:206-222) with the quantization fused; act 0 = tanh-GELU, 1 = SiLU."""
    _need(gate_up, rows * 2 * half * 4, "gate_up")
    _need(xq, rows * row_bytes(Q8_1, half), "xq")
    check(lib().launch_glu_act_q8_1(_ptr(gate_up), _ptr(xq), _opt(out_f32), rows, half, act, _stream()), "launch_glu_act_q8_1")


def gpu_embed_rows_into(qtype, table, tokens, x, batch, hidden, vocab):
    """x[b] = decoded row tokens[b] of the packed (vocab, hidden) table."""
    _need(x, batch * hidden * 4, "x")
    check(lib().launch_embed_rows(qtype, _ptr(table), _ptr(tokens), _ptr(x), batch, hidden, vocab, _stream()), "launch_embed_rows")


def gpu_argmax_rows(logits):
    """(index int32, value f32) of the largest entry of every row; the lowest index wins ties.  Allocates."""
    batch, vocab = logits.shape
    scratch = torch.empty(lib().qmm_argmax_scratch_bytes(batch), dtype=torch.uint8, device=logits.device)
    idx = torch.empty(batch, dtype=torch.int32, device=logits.device)
    val = torch.empty(batch, dtype=torch.float32, device=logits.device)
    check(lib().launch_argmax_rows(_ptr(logits), _ptr(scratch), _ptr(idx), _ptr(val), batch, vocab, _stream()), "launch_argmax_rows")
    return idx, val


def gpu_scale_f32_inplace(x, scalar):
    """x *= scalar: the upstream's gpu_scale_f64_inplace (gpu-core/src/infer_ops.rs:242-248)."""
    check(lib().launch_scale_f32(_ptr(x), scalar, x.numel(), _stream()), "launch_scale_f32")


def gpu_gemm_bt_bf16_into(a, b, out, m, n, k):
    """out(m,n) = a(m,k) . b(n,k)^T, a and b bf16, out bf16 or f32: the upstream's gpu_gemm_bt_f64_into
    (gpu-core/src/infer_ops.rs:224-240) on a bf16 weight window."""
    _need(a, m * k * 2, "a")
    _need(b, n * k * 2, "b")
    _need(out, m * n * out.element_size(), "out")
    name = "launch_gemm_bt_bf16" if out.dtype == torch.bfloat16 else "launch_gemm_bt_bf16_f32acc"
    check(getattr(lib(), name)(_ptr(a), _ptr(b), _ptr(out), m, n, k, _stream()), name)


def gpu_gqa_attn_into(q, k, v, out, t, nqh, nkv, hd, prefix, kq_scale=1.0):
    """Attention over a whole sequence into a caller-owned out (t, nqh*hd), the upstream's gpu_gqa_attn_into
    (gpu-core/src/infer_ops.rs:160-189): positions below `prefix` causal, the others bidirectional.  q and out f32;
    k and v f32, or both float16 (the rows of a KV cache)."""
    if k.dtype != v.dtype or k.dtype not in (torch.float32, torch.float16):
        raise TypeError("k and v must both be float32 or both float16")
    _need(q, t * nqh * hd * 4, "q")
    _need(k, t * nkv * hd * k.element_size(), "k")
    _need(v, t * nkv * hd * v.element_size(), "v")
    _need(out, t * nqh * hd * 4, "out")
    name = "launch_attn_prefill" if k.dtype == torch.float32 else "launch_attn_prefill_f16kv"
    check(getattr(lib(), name)(_ptr(q), _ptr(k), _ptr(v), _ptr(out), t, nqh, nkv, hd, prefix, float(kq_scale), _stream()), name)


def gpu_gqa_attn_at_into(q, k16, v16, out, t, t_kv, q_pos0, nqh, nkv, hd, prefix, kq_scale=1.0):
    """The same for t queries that continue a sequence: row r of q / out is position q_pos0 + r, k16 and v16 (float16)
    hold positions 0..t_kv-1 (the rows of a KV cache)."""
    _need(q, t * nqh * hd * 4, "q")
    _need(k16, t_kv * nkv * hd * 2, "k16")
    _need(v16, t_kv * nkv * hd * 2, "v16")
    _need(out, t * nqh * hd * 4, "out")
    if k16.dtype != torch.float16 or v16.dtype != torch.float16:
        raise TypeError("k16 and v16 must be float16")
    check(lib().launch_attn_prefill_f16kv_at(_ptr(q), _ptr(k16), _ptr(v16), _ptr(out), t, t_kv, q_pos0, nqh, nkv, hd, prefix, float(kq_scale), _stream()),
          "launch_attn_prefill_f16kv_at")


# ---- quantized dense layer ---------------------------------------------------------------
DENSE_ACTS = {"linear": 0, "relu": 1, "sigmoid": 2, "leaky_relu": 3, "prelu": 4, "elu": 5, "selu": 6, "tanh": 7, "silu": 8, "gelu": 9}


def gpu_qdense_into(qtype, w, x, bias, out, m, n, k, act="linear", alpha=0.0, xq_scratch=None):
    """out(m,n) = act(x(m,k) . w(n,k)^T + bias): LayerKind::Dense of the upstream's forward pass
    (recipe-infer/src/forward.rs:372-431) with the weight in packed `qtype` blocks.  x, out f32.  Up to 63 rows
    (and every type but Q4_K) through the Q8_1 matvec, from 64 rows on Q4_K through the bf16 tensor-core GEMM."""
    _need(w, n * row_bytes(qtype, k), "w")
    _need(x, m * k * 4, "x")
    _need(out, m * n * 4, "out")
    if bias is not None:
        _need(bias, n * 4, "bias")
    need = lib().qmm_qdense_scratch_bytes(qtype, m, k)
    if xq_scratch is None:
        xq_scratch = torch.empty(need, dtype=torch.uint8, device=x.device)
    _need(xq_scratch, need, "xq_scratch")
    check(lib().launch_qdense(qtype, _ptr(w), _ptr(x), _ptr(bias) if bias is not None else None, _ptr(out), _ptr(xq_scratch), m, n, k,
                              DENSE_ACTS[act] if isinstance(act, str) else int(act), float(alpha), _stream()), "launch_qdense")


# ---- mixture of experts ---------------------------------------------------------------------
def gpu_moe_router_topk(x, router_w, top_k, scale=1.0, eps=1e-6, gain=None, want_probs=False):
    """Router of a mixture-of-experts layer, on the device (the upstream routes on the host:
    examples/gemma4.rs:694-711): per row of x (m, hidden) the top_k experts of softmax(router_w . r),
    r = rms_normalise(x) * scale * gain.  Returns (sel int32 (m, top_k), weight f32 (m, top_k)[, probs])."""
    m, hidden = x.shape
    n_experts = router_w.shape[0]
    sel = torch.empty(m, top_k, dtype=torch.int32, device=x.device)
    weight = torch.empty(m, top_k, dtype=torch.float32, device=x.device)
    probs = torch.empty(m, n_experts, dtype=torch.float32, device=x.device) if want_probs else None
    check(lib().launch_moe_router_topk(_ptr(x), _opt(gain), _ptr(router_w), m, hidden, n_experts, top_k, scale, eps, _ptr(sel), _ptr(weight),
                                       _opt(probs), _stream()), "launch_moe_router_topk")
    return (sel, weight, probs) if want_probs else (sel, weight)


def gpu_moe_experts_into(type_gu, gate_up_bank, type_dn, down_bank, xq, sel, weight, out, hidden, ffn_expert, act, expert_scale=None):
    """The chosen experts' gated FFN for every token and their weighted sum into out (m, hidden); the
    banks hold n_experts matrices back to back (gate_up: (2*ffn_expert, hidden) each, down: (hidden,
    ffn_expert) each).  The upstream runs the experts one by one from the host
    (examples/gemma4.rs:713-737).  Allocates its scratch."""
    m, top_k = sel.shape
    gu_stride = 2 * ffn_expert * row_bytes(type_gu, hidden)
    dn_stride = hidden * row_bytes(type_dn, ffn_expert)
    scratch = torch.empty(lib().qmm_moe_scratch_bytes(m, top_k, hidden, ffn_expert), dtype=torch.uint8, device=out.device)
    check(lib().launch_moe_experts(type_gu, _ptr(gate_up_bank), gu_stride, type_dn, _ptr(down_bank), dn_stride, _ptr(xq), _ptr(sel),
                                   _ptr(weight), _opt(expert_scale), _ptr(out), _ptr(scratch), m, top_k, hidden, ffn_expert, act, _stream()),
          "launch_moe_experts")
    return scratch
