"""Quantized dense layers behind the upstream's layer-list interface.

The upstream describes a network as a list of ``LayerParams`` (recipe-infer/src/params.rs:35-59:
kind, w, b, in_dim, out_dim, act, palpha) and runs it with ``forward_into``
(recipe-infer/src/forward.rs:272-460), which for ``LayerKind::Dense`` calls ``gpu_linear_into`` and
one activation launch (forward.rs:372-431).  ``QuantDense`` is that record with the weight kept in
packed GGUF blocks (out_dim rows of in_dim elements, the layout the matvec streams), and
``forward_into`` the same loop over ``launch_qdense``.  Weights come from f32 matrices (quantized on
the device) or from the tensors of a GGUF file.
"""
import torch

from . import quant_ops as ops
from ._lib import Q8_1, TYPE_NAMES

LEAKY_ALPHA = 0.01  # recipe-infer/src/params.rs:11
ELU_ALPHA = 1.0     # recipe-infer/src/params.rs:14


class QuantDense:
    """One dense layer: w (out_dim, in_dim) packed blocks of `qtype`, b (out_dim,) f32 or None, an activation
    name of ``quant_ops.DENSE_ACTS`` and, for "prelu", its slope."""

    def __init__(self, qtype, w, b, in_dim, out_dim, act="linear", palpha=0.25):
        if act not in ops.DENSE_ACTS:
            raise ValueError(f"unknown activation {act!r}")
        if w.numel() < out_dim * ops.row_bytes(qtype, in_dim):
            raise ValueError("w is smaller than out_dim rows of packed blocks")
        self.qtype, self.w, self.b = qtype, w, b
        self.in_dim, self.out_dim, self.act, self.palpha = in_dim, out_dim, act, palpha

    @classmethod
    def from_f32(cls, qtype, w_f32, b=None, act="linear", palpha=0.25):
        """w_f32 (out_dim, in_dim) on the device; quantized there (deterministic min/max quantizers)."""
        out_dim, in_dim = w_f32.shape
        return cls(qtype, ops.gpu_quantize_weights(qtype, w_f32.contiguous()), b, in_dim, out_dim, act, palpha)

    @classmethod
    def from_gguf(cls, gf, weight_name, bias_name=None, act="linear", palpha=0.25, device="cuda"):
        """The layer of a GGUF file (``gguf.GgufFile``): a 2-D packed tensor (dims = [in_dim, out_dim], in_dim
        fastest) and an optional f32 bias of out_dim elements."""
        i = gf.find(weight_name)
        if i < 0:
            raise KeyError(weight_name)
        info = gf.info(i)
        in_dim, out_dim = info["dims"][0], info["dims"][1]
        w = torch.empty(info["bytes"], dtype=torch.uint8, device=device)
        gf.upload(i, w)
        b = None
        if bias_name:
            b = torch.empty(out_dim, dtype=torch.float32, device=device)
            gf.upload(bias_name, b)
        return cls(info["type"], w, b, in_dim, out_dim, act, palpha)

    def alpha(self):
        return {"leaky_relu": LEAKY_ALPHA, "prelu": self.palpha, "elu": ELU_ALPHA}.get(self.act, 0.0)

    def __repr__(self):
        return f"QuantDense({TYPE_NAMES.get(self.qtype, self.qtype)}, {self.in_dim} -> {self.out_dim}, {self.act})"


class Scratch:
    """Activations of every layer for n rows, and the Q8_1 staging of the widest input (allocated once)."""

    def __init__(self, layers, n, device="cuda"):
        self.n = n
        self.acts = [torch.empty(n, l.out_dim, dtype=torch.float32, device=device) for l in layers]
        from ._lib import lib
        self.xq = torch.empty(max(lib().qmm_qdense_scratch_bytes(l.qtype, n, l.in_dim) for l in layers), dtype=torch.uint8, device=device)


def forward_into(layers, x, scratch):
    """Runs the dense stack on x (n, in_dim of the first layer) f32; returns the last layer's activations
    (a view of the scratch).  Three launches per layer, all on the current stream."""
    n = x.shape[0]
    if n != scratch.n:
        raise ValueError("scratch was sized for another batch")
    prev = x.contiguous()
    for l, out in zip(layers, scratch.acts):
        if prev.shape[1] != l.in_dim:
            raise ValueError(f"{l!r} fed {prev.shape[1]} features")
        ops.gpu_qdense_into(l.qtype, l.w, prev, l.b, out, n, l.out_dim, l.in_dim, l.act, l.alpha(), scratch.xq)
        prev = out
    return prev
