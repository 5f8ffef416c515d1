"""Python binding of the decode engine (include/qmm_decoder.h) for tests and the benchmark.

The engine itself is C++/CUDA inside libqmm.so; this class only holds the handle, the token
buffers and, for tensor parallelism, exchanges the IPC handles of the ranks' exchange areas
through torch.distributed."""
import ctypes as C

import torch

from ._lib import Q4_K, Q6_K, Q8_0, check, lib

ACT_GELU_TANH, ACT_SILU = 0, 1
T_ATTN_NORM, T_WQK, T_WV, T_WO, T_FFN_NORM, T_WGU, T_WDOWN, T_FINAL_NORM, T_HEAD, T_EMBED = 0, 1, 3, 4, 5, 6, 8, 9, 10, 11


class DecoderConfig(C.Structure):
    _fields_ = [(n, C.c_int) for n in ("n_layers", "hidden", "n_q_heads", "n_kv_heads", "head_dim", "ffn", "vocab", "ctx_len")] + \
               [("rope_theta", C.c_float), ("rms_eps", C.c_float), ("act", C.c_int)] + \
               [(n, C.c_int) for n in ("type_attn_qk", "type_attn_v", "type_attn_o", "type_ffn_gate_up", "type_ffn_down", "type_head")] + \
               [("max_batch", C.c_int), ("tp_rank", C.c_int), ("tp_size", C.c_int), ("seed", C.c_ulonglong)]


def config_8b(**kw):
    """BASELINE config 4: 8B-class Gemma/Llama-style decoder in a Q4_K_M-like mix."""
    c = dict(n_layers=32, hidden=4096, n_q_heads=32, n_kv_heads=8, head_dim=128, ffn=14336, vocab=256000, ctx_len=2048,
             rope_theta=10000.0, rms_eps=1e-6, act=ACT_GELU_TANH, type_attn_qk=Q4_K, type_attn_v=Q6_K, type_attn_o=Q4_K,
             type_ffn_gate_up=Q4_K, type_ffn_down=Q6_K, type_head=Q6_K, max_batch=1, tp_rank=0, tp_size=1, seed=0x5EED)
    c.update(kw)
    return DecoderConfig(**c)


def config_70b(**kw):
    """BASELINE config 5: 70B-class decoder in Q4_K with a Q6_K head."""
    c = dict(n_layers=80, hidden=8192, n_q_heads=64, n_kv_heads=8, head_dim=128, ffn=28672, vocab=128256, ctx_len=4096,
             rope_theta=10000.0, rms_eps=1e-6, act=ACT_SILU, type_attn_qk=Q4_K, type_attn_v=Q4_K, type_attn_o=Q4_K,
             type_ffn_gate_up=Q4_K, type_ffn_down=Q4_K, type_head=Q6_K, max_batch=1, tp_rank=0, tp_size=1, seed=0x5EED)
    c.update(kw)
    return DecoderConfig(**c)


_bound = False


def _bind():
    global _bound
    L = lib()
    if not _bound:
        vp, i32 = C.c_void_p, C.c_int
        L.qmm_decoder_create.argtypes = [C.POINTER(DecoderConfig), C.POINTER(vp)]
        L.qmm_decoder_destroy.argtypes = [vp]
        L.qmm_decoder_weight_bytes.argtypes = [vp]
        L.qmm_decoder_weight_bytes.restype = C.c_long
        L.qmm_decoder_get_tensor.argtypes = [vp, i32, i32, C.POINTER(vp), C.POINTER(C.c_long)]
        L.qmm_decoder_read_tensor.argtypes = [vp, i32, i32, vp, C.c_long]
        L.qmm_decoder_fill_cache.argtypes = [vp, C.c_ulonglong, vp]
        L.qmm_decoder_ipc_export.argtypes = [vp, vp]
        L.qmm_decoder_ipc_import.argtypes = [vp, i32, vp]
        L.qmm_decoder_tp_ready.argtypes = [vp]
        L.qmm_decoder_step.argtypes = [vp, vp, i32, i32, vp, vp, vp, vp]
        L.qmm_decoder_prefill.argtypes = [vp, vp, i32, i32, vp, vp, vp]
        L.qmm_decoder_prefill_at.argtypes = [vp, vp, i32, i32, i32, vp, vp, vp]
        L.qmm_decoder_create_from_gguf.argtypes = [C.c_char_p, i32, i32, i32, i32, C.POINTER(vp)]
        L.qmm_decoder_export_gguf.argtypes = [vp, C.c_char_p, C.c_char_p]
        _bound = True
    return L


class Decoder:
    def __init__(self, cfg, group=None, gguf_path=None):
        """cfg: a DecoderConfig (weights: the seeded model).  With gguf_path the weights and the shapes come
        from that file; of cfg only max_batch, ctx_len (0 = the file's), tp_rank and tp_size are used."""
        self.L = _bind()
        self.cfg = cfg
        self.h = C.c_void_p()
        if gguf_path is None:
            check(self.L.qmm_decoder_create(C.byref(cfg), C.byref(self.h)), "qmm_decoder_create")
        else:
            check(self.L.qmm_decoder_create_from_gguf(str(gguf_path).encode(), cfg.max_batch, cfg.ctx_len, cfg.tp_rank, cfg.tp_size,
                                                      C.byref(self.h)), "qmm_decoder_create_from_gguf")
        dev = torch.device("cuda", torch.cuda.current_device())
        self.tokens = torch.zeros(cfg.max_batch, dtype=torch.int32, device=dev)
        self.next_tokens = torch.zeros(cfg.max_batch, dtype=torch.int32, device=dev)
        self.best = torch.zeros(cfg.max_batch, dtype=torch.float32, device=dev)
        self.group = group
        if cfg.tp_size > 1:
            self._wire_peers()

    def _wire_peers(self):
        import torch.distributed as dist
        buf = C.create_string_buffer(64)
        check(self.L.qmm_decoder_ipc_export(self.h, buf), "qmm_decoder_ipc_export")
        handles = [None] * self.cfg.tp_size
        dist.all_gather_object(handles, bytes(buf.raw), group=self.group)
        for r, hb in enumerate(handles):
            if r != self.cfg.tp_rank:
                check(self.L.qmm_decoder_ipc_import(self.h, r, C.create_string_buffer(hb, 64)), "qmm_decoder_ipc_import")
        check(self.L.qmm_decoder_tp_ready(self.h), "qmm_decoder_tp_ready")
        dist.barrier(group=self.group)

    @property
    def weight_bytes(self):
        return self.L.qmm_decoder_weight_bytes(self.h)

    def tensor(self, layer, which):
        """uint8 copy (host, numpy) of a tensor's bytes."""
        p, n = C.c_void_p(), C.c_long()
        check(self.L.qmm_decoder_get_tensor(self.h, layer, which, C.byref(p), C.byref(n)), "qmm_decoder_get_tensor")
        import numpy as np
        out = np.empty(n.value, dtype=np.uint8)
        check(self.L.qmm_decoder_read_tensor(self.h, layer, which, out.ctypes.data_as(C.c_void_p), n.value), "qmm_decoder_read_tensor")
        return out

    def export_gguf(self, path, architecture="llama"):
        """Writes this (single-GPU) decoder's model as a GGUF file."""
        check(self.L.qmm_decoder_export_gguf(self.h, str(path).encode(), architecture.encode()), "qmm_decoder_export_gguf")

    def fill_cache(self, seed=1):
        check(self.L.qmm_decoder_fill_cache(self.h, seed, torch.cuda.current_stream().cuda_stream), "qmm_decoder_fill_cache")

    def step(self, batch, pos, logits=None):
        check(self.L.qmm_decoder_step(self.h, self.tokens.data_ptr(), batch, pos, self.next_tokens.data_ptr(),
                                      logits.data_ptr() if logits is not None else None, self.best.data_ptr(),
                                      torch.cuda.current_stream().cuda_stream), "qmm_decoder_step")

    def prefill(self, prompt, seq=0, logits=None, pos0=0):
        """All positions of `prompt` (int32 CUDA tensor) through the stack at once; fills the KV cache of sequence
        `seq` for positions pos0..pos0+len-1 (the cache must already hold 0..pos0-1) and returns the greedy token
        after the last position (int32 CUDA tensor of one element); `logits` (vocab floats) optionally receives that
        position's logits.  Decode goes on with step(batch, pos=pos0+len(prompt))."""
        out = torch.empty(1, dtype=torch.int32, device=prompt.device)
        check(self.L.qmm_decoder_prefill_at(self.h, prompt.data_ptr(), prompt.numel(), seq, pos0, out.data_ptr(),
                                            logits.data_ptr() if logits is not None else None, torch.cuda.current_stream().cuda_stream),
              "qmm_decoder_prefill_at")
        return out

    def close(self):
        if self.h:
            self.L.qmm_decoder_destroy(self.h)
            self.h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
