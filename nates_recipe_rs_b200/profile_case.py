"""Small driver for profiler captures of one matvec or GEMM shape.

    python -m nates_recipe_rs_b200.profile_case <q8_0|q4_k|q6_k> <n> <k> <m> [launches]
    python -m nates_recipe_rs_b200.profile_case gemm <n> <k> <m> [launches]      (Q4_K x bf16 prefill GEMM)

Allocates enough distinct random weight matrices to exceed L2 (about 300 MB in
total, never more), quantizes random activations and launches the matvec on the
matrices in rotation.  Tuning overrides: QMM_TUNE="key=value,key=value".
"""
import os
import sys

import torch

from . import _lib, quant_ops as ops


def main(argv):
    names = {"q8_0": _lib.Q8_0, "q4_k": _lib.Q4_K, "q6_k": _lib.Q6_K, "gemm": _lib.Q4_K}
    qt = names[argv[0]]
    gemm = argv[0] == "gemm"
    n, k, m = int(argv[1]), int(argv[2]), int(argv[3])
    reps = int(argv[4]) if len(argv) > 4 else 4
    torch.cuda.set_device(0)
    L = _lib.lib()
    for kv in os.environ.get("QMM_TUNE", "").split(","):
        if kv:
            key, val = kv.split("=")
            _lib.check(L.qmm_tune(key.encode(), int(val)), f"qmm_tune({key})")
    rb = ops.row_bytes(qt, k)
    ncopy = max(2, int(300e6 // (n * rb)) + 1)
    ws = [torch.randint(0, 255, (n * rb,), dtype=torch.uint8, device="cuda") for _ in range(ncopy)]
    for w in ws:  # finite fp16 scales
        ops.gpu_quantize_weights_into(qt, torch.randn(n, k, device="cuda") * 0.02, w, n, k)
    if gemm:
        x = torch.randn(m, k, device="cuda").to(torch.bfloat16)
        y = torch.empty(m, n, device="cuda", dtype=torch.bfloat16)
        torch.cuda.synchronize()
        for i in range(reps):
            ops.gpu_qgemm_q4_k_bf16_into(ws[i % ncopy], x, y, m, n, k)
    else:
        xq = ops.gpu_quantize_q8_1(torch.randn(m, k, device="cuda"))
        y = torch.empty(m, n, device="cuda")
        torch.cuda.synchronize()
        for i in range(reps):
            ops.gpu_qmatvec_into(qt, ws[i % ncopy], xq, y, m, n, k)
    torch.cuda.synchronize()
    ops.check_launch()
    print("done")


if __name__ == "__main__":
    main(sys.argv[1:])
