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


def tp_matvec_parity(verbose=False):
    """The row-parallel projections with the fused sum (launch_qmatvec_tp, launch_qmatvec_batch_tp) against
    the same shards computed one by one on rank 0 and added in rank order: bit-identical, and the same bits on
    every rank.  Returns {"n", "cases", "ok"}."""
    from ._lib import Q8_0
    rank, world = dist.get_rank(), dist.get_world_size()
    dev = torch.device("cuda", torch.cuda.current_device())
    n_max, m_max = 8192, 32
    comm = ops.TpComm(4 * m_max * n_max)
    ok, cases = True, 0

    def shard(qt, n, kl, r, seed):
        g = torch.Generator(device=dev)
        g.manual_seed(seed * 131 + r)
        w = ops.gpu_quantize_weights(qt, torch.randn(n, kl, device=dev, generator=g) * 0.02)
        xq = ops.gpu_quantize_q8_1(torch.randn(m_max, kl, device=dev, generator=g))
        return w, xq

    def reference(qt, n, kl, m, seed):
        """Sum over ranks of the single-GPU result of every shard, in rank order (computed on this rank)."""
        acc = torch.zeros(m, n, device=dev)
        for r in range(world):
            w, xq = shard(qt, n, kl, r, seed)
            acc += ops.gpu_qmatvec(qt, w, xq, m, n, kl)
        return acc

    def same_everywhere(y):
        ys = [torch.empty_like(y) for _ in range(world)]
        dist.all_gather(ys, y.contiguous())
        return all(torch.equal(ys[0], t) for t in ys)

    for seed, (qt, n, kl, m) in enumerate([(Q4_K, 4096, 1792, 1), (Q6_K, 4096, 1792, 1), (Q4_K, 512, 3584, 2), (Q8_0, 300, 512, 1),
                                           (Q4_K, 4096, 2048, 5), (Q6_K, 2048, 2048, 16), (Q6_K, 1000, 1792, 9), (Q4_K, 37, 256, 3),
                                           (Q4_K, 4096, 2048, 32), (Q4_K, 1000, 1792, 20), (Q4_K, 8192, 4096, 32), (Q4_K, 1000, 4096, 20)]):
        w, xq = shard(qt, n, kl, rank, seed)
        for rep in range(2):   # two exchanges in a row use the two alternating buffers
            y = torch.full((m, n), float("nan"), device=dev)
            ops.gpu_qmatvec_tp_into(comm, qt, w, xq, y, m, n, kl)
            torch.cuda.synchronize()
            ops.check_launch()
            want = reference(qt, n, kl, m, seed)
            good = torch.equal(y, want) and same_everywhere(y)
            if verbose and rank == 0:
                print(f"launch_qmatvec_tp type {qt} n {n} k_local {kl} m {m} rep {rep}: {'ok' if good else 'MISMATCH'} "
                      f"(max diff {float((y - want).abs().max()):.3e})")
            ok, cases = ok and good, cases + 1
    # a job list: two local projections and three summed ones of different shapes
    for m in (1, 2, 5):
        specs = [(Q4_K, 1024, 1024, False), (Q4_K, 2048, 1792, True), (Q6_K, 512, 1792, True), (Q8_0, 256, 512, False), (Q4_K, 4096, 512, True)]
        jobs = ops.MatvecJobs()
        outs, wants = [], []
        for i, (qt, n, kl, summed) in enumerate(specs):
            w, xq = shard(qt, n, kl, rank, 100 + i)
            y = torch.full((m, n), float("nan"), device=dev)
            jobs.add(qt, w, xq, y, n, kl, tp_sum=summed)
            outs.append(y)
            wants.append(reference(qt, n, kl, m, 100 + i) if summed else ops.gpu_qmatvec(qt, w, xq, m, n, kl))
        ops.gpu_qmatvec_batch_tp_into(comm, jobs, m)
        torch.cuda.synchronize()
        ops.check_launch()
        for i, (y, want) in enumerate(zip(outs, wants)):
            good = torch.equal(y, want) and (not specs[i][3] or same_everywhere(y))
            if verbose and rank == 0:
                print(f"launch_qmatvec_batch_tp m {m} job {i} {specs[i]}: {'ok' if good else 'MISMATCH'}")
            ok, cases = ok and good, cases + 1
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    comm.close()
    dist.barrier()
    return {"n": world, "cases": cases, "ok": bool(int(flag.item()))}
