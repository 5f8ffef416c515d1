"""Tensor-parallel self-check, one process per GPU:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        -m nates_recipe_rs_b200.tp_check

Every rank builds its shard of a small decoder (the shards of all layouts come from one seeded
model), rank 0 also builds the unsharded model, and both decode the same tokens for a few steps:
the gathered logits slices must match the single-GPU logits within the matvec tolerance and every
rank must end each step with the same greedy token.  Prints "tp_check ok" on rank 0."""
import os
import sys

import torch
import torch.distributed as dist

from . import decoder as dec, quant_ops as ops
from ._lib import Q4_K, Q6_K


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    for kv in os.environ.get("QMM_TUNE", "").split(","):  # e.g. QMM_TUNE=attn_tc_min_batch=0,mma_min_m=0
        if kv:
            from ._lib import check, lib
            check(lib().qmm_tune(kv.split("=")[0].encode(), int(kv.split("=")[1])), "qmm_tune")
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    base = dict(n_layers=3, hidden=512, n_q_heads=8, n_kv_heads=8, head_dim=64, ffn=2048, vocab=4096, ctx_len=40,
                rope_theta=10000.0, rms_eps=1e-6, act=dec.ACT_GELU_TANH, type_attn_qk=Q4_K, type_attn_v=Q6_K, type_attn_o=Q4_K,
                type_ffn_gate_up=Q4_K, type_ffn_down=Q6_K, type_head=Q6_K, max_batch=2, seed=4242)
    if "wide" in sys.argv[1:]:  # five sequences, 2048-wide layers: the projections take the tensor-core matvec
        base.update(n_layers=2, hidden=2048, n_q_heads=16, head_dim=128, ffn=8192, max_batch=5)
    if (base["n_q_heads"] * base["head_dim"]) % (256 * world) or base["ffn"] % (256 * world) or base["n_kv_heads"] % world:
        raise SystemExit(f"tp_check supports world sizes dividing 2 (got {world})" if world > 2 else "bad world size")
    tp = dec.Decoder(dec.DecoderConfig(tp_rank=rank, tp_size=world, **base))
    ref = dec.Decoder(dec.DecoderConfig(tp_rank=0, tp_size=1, **base)) if rank == 0 else None
    B, V = base["max_batch"], base["vocab"]
    toks = torch.tensor([17, 3001, 5, 4000, 999][:B], dtype=torch.int32, device="cuda")
    ok = True
    for pos in range(5):
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
            agrees = torch.equal(all_tok[0], full.argmax(dim=1).to(torch.int32))
            print(f"pos {pos}: max |logit diff| {err:.3e} (scale {scale:.3f}), ranks agree on token: {same}, token = argmax of gathered logits: {agrees}")
            ok = ok and err <= 2e-2 * scale and same and agrees
            toks = ref.next_tokens.clone()
        dist.broadcast(toks, 0)
    flag = torch.tensor([1 if ok else 0], device="cuda")
    dist.broadcast(flag, 0)
    tp.close()
    if ref:
        ref.close()
    dist.barrier()
    dist.destroy_process_group()
    if rank == 0:
        print("tp_check ok" if ok else "tp_check FAILED")
    sys.exit(0 if int(flag.item()) else 1)


if __name__ == "__main__":
    main()
