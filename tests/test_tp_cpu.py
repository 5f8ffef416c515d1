"""Host-side tensor-parallel logic on CPU with two gloo ranks: the sharding rule the engine uses
(Q/K/V/gate/up by output rows, O/down by input columns in whole 256-blocks, partial outputs summed)
reproduces the unsharded projections when each shard is quantized independently.  No GPU."""
import os
import socket
import subprocess
import sys
import textwrap

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = textwrap.dedent("""
    import os, sys
    import numpy as np
    import torch
    import torch.distributed as dist
    sys.path.insert(0, %r)
    import oracle
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo")
    H, F = 512, 1024
    x = oracle.fill_normal(H, 5, 1.0)
    xq = oracle.quantize(oracle.Q8_1, x)
    w_up_full = oracle.fill_normal(F * H, 6, 0.02).reshape(F, H)
    w_dn_full = oracle.fill_normal(H * F, 7, 0.02).reshape(H, F)
    # column-parallel (rows of W_up): this rank's slice of the intermediate
    fl = F // world
    up_l = oracle.matvec(oracle.Q4_K, oracle.quantize(oracle.Q4_K, w_up_full[rank * fl:(rank + 1) * fl]), xq, H)[0]
    hq_l = oracle.quantize(oracle.Q8_1, up_l)                     # Q8_1 blocks of 32 never straddle a shard
    # row-parallel (columns of W_down in whole 256-blocks) + sum of the partial outputs
    part = oracle.matvec(oracle.Q6_K, oracle.quantize(oracle.Q6_K, np.ascontiguousarray(w_dn_full[:, rank * fl:(rank + 1) * fl])), hq_l, fl)[0]
    t = torch.from_numpy(part.copy())
    dist.all_reduce(t)
    if rank == 0:
        up = oracle.matvec(oracle.Q4_K, oracle.quantize(oracle.Q4_K, w_up_full), xq, H)[0]
        full = oracle.matvec(oracle.Q6_K, oracle.quantize(oracle.Q6_K, w_dn_full), oracle.quantize(oracle.Q8_1, up), F)[0]
        err = np.abs(t.numpy() - full).max()
        assert err <= 1e-4 + 1e-3 * np.abs(full).max(), err
        # the shards hold exactly the bytes of the corresponding rows / block columns of the full matrices
        q_full = oracle.quantize(oracle.Q6_K, w_dn_full).reshape(H, F // 256, 210)
        q_l = oracle.quantize(oracle.Q6_K, np.ascontiguousarray(w_dn_full[:, :fl])).reshape(H, fl // 256, 210)
        assert np.array_equal(q_full[:, :fl // 256], q_l)
        print("tp cpu ok")
    dist.barrier()
    dist.destroy_process_group()
""") % ROOT


def test_two_rank_gloo_sharding_matches_unsharded(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    procs = []
    for r in range(2):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE="2", MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), OMP_NUM_THREADS="2")
        procs.append(subprocess.Popen([sys.executable, str(script)], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    outs = [p.communicate(timeout=240)[0] for p in procs]
    assert all(p.returncode == 0 for p in procs), "\n".join(outs)
    assert "tp cpu ok" in outs[0]
