"""Tensor-parallel check on real GPUs, one process per GPU (not collected by pytest: it needs torchrun):

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        tests/tp_check.py [wide | matvec]

Runs nates_recipe_rs_b200.tp_parity: the decode engine's shards against the unsharded model (default; `wide`:
the shapes that take the tensor-core matvec), or (`matvec`) the row-parallel projections with the fused sum
against the shards computed one by one.  Exits non-zero on a mismatch."""
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402


def main():
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    from nates_recipe_rs_b200.tp_parity import tp_matvec_parity, tp_parity
    if "matvec" in sys.argv[1:]:
        res = tp_matvec_parity(verbose=True)
    else:
        res = tp_parity(wide="wide" in sys.argv[1:], verbose=True)
    if dist.get_rank() == 0:
        print(res)
        print("tp_check ok" if res["ok"] else "tp_check FAILED")
    dist.destroy_process_group()
    sys.exit(0 if res["ok"] else 1)


if __name__ == "__main__":
    main()
