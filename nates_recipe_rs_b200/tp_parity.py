"""Tensor-parallel self-check of the decode engine, called with one process per GPU after
torch.distributed is initialised (backend nccl).

Every rank builds its shard of a small decoder (the shards of all layouts come from one seeded
model: element (r, c) of a full matrix is a function of the seed and r*K + c), rank 0 also builds
the unsharded model, and both decode the same tokens for a few steps.  Checked: the gathered
logits slices equal the single-GPU logits within the decoder tolerance (2e-2 of the logit scale;
a rounding-order difference flips a few Q8_1 codes, most steps are bit-equal), every rank ends
each step with the same greedy token, and that token is the argmax of the gathered logits.
"""
import torch
import torch.distributed as dist

from . import decoder as dec, quant_ops as ops
from ._lib import Q4_K, Q6_K

LOGIT_TOL = 2e-2  # of the logit scale


def shapes(world, wide):
    base = dict(n_layers=3, hidden=512, n_q_heads=8, n_kv_heads=8, head_dim=64, ffn=2048, vocab=4096, ctx_len=40,
                rope_theta=10000.0, rms_eps=1e-6, act=dec.ACT_GELU_TANH, type_attn_qk=Q4_K, type_attn_v=Q6_K, type_attn_o=Q4_K,
                type_ffn_gate_up=Q4_K, type_ffn_down=Q6_K, type_head=Q6_K, max_batch=2, seed=4242)
    if wide:  # five sequences, 2048-wide layers: the projections take the tensor-core matvec
        base.update(n_layers=2, hidden=2048, n_q_heads=16, head_dim=128, ffn=8192, max_batch=5)
    if (base["n_q_heads"] * base["head_dim"]) % (256 * world) or base["ffn"] % (256 * world) or base["n_kv_heads"] % world or \
            base["vocab"] % world:
        raise ValueError(f"tp_parity: world size {world} does not divide the test model")
    return base


def tp_parity(wide=False, steps=5, verbose=False):
    """Returns {"n", "wide", "max_logit_diff", "logit_scale", "tokens_agree", "ok"} (same on every rank)."""
    rank, world = dist.get_rank(), dist.get_world_size()
    base = shapes(world, wide)
    tp = dec.Decoder(dec.DecoderConfig(tp_rank=rank, tp_size=world, **base))
    ref = dec.Decoder(dec.DecoderConfig(tp_rank=0, tp_size=1, **base)) if rank == 0 else None
    B, V = base["max_batch"], base["vocab"]
    toks = torch.tensor([17, 3001, 5, 4000, 999][:B], dtype=torch.int32, device="cuda")
    worst, scale_at_worst, agree = 0.0, 1.0, True
    for pos in range(steps):
        lg = torch.empty(B, V // world, device="cuda")
        tp.tokens.copy_(toks)
        tp.step(B, pos, lg)
        ops.check_launch()
        slices = [torch.empty_like(lg) for _ in range(world)]
        dist.all_gather(slices, lg)
        mine = tp.next_tokens.clone()
        all_tok = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(all_tok, mine)
        if rank == 0:
            full = torch.cat(slices, dim=1)
            rl = torch.empty(B, V, device="cuda")
            ref.tokens.copy_(toks)
            ref.step(B, pos, rl)
            ops.check_launch()
            scale = float(rl.abs().max())
            err = float((full - rl).abs().max())
            same = all(torch.equal(t, all_tok[0]) for t in all_tok)
            is_argmax = torch.equal(all_tok[0], full.argmax(dim=1).to(torch.int32))
            if verbose:
                print(f"pos {pos}: max |logit diff| {err:.3e} (scale {scale:.3f}), ranks agree on token: {same}, "
                      f"token = argmax of gathered logits: {is_argmax}")
            if err / scale > worst / scale_at_worst:
                worst, scale_at_worst = err, scale
            agree = agree and same and is_argmax
            toks = ref.next_tokens.clone()
        dist.broadcast(toks, 0)
    res = torch.tensor([worst, scale_at_worst, 1.0 if agree else 0.0], device="cuda", dtype=torch.float64)
    dist.broadcast(res, 0)
    tp.close()
    if ref:
        ref.close()
    dist.barrier()
    worst, scale_at_worst, agree = float(res[0]), float(res[1]), bool(res[2] > 0.5)
    return {"n": world, "wide": bool(wide), "max_logit_diff": worst, "logit_scale": scale_at_worst, "tokens_agree": agree,
            "ok": bool(agree and worst <= LOGIT_TOL * scale_at_worst)}
