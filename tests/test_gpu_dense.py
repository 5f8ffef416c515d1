"""Quantized dense layer (launch_qdense) and the layer-list forward, against the CPU oracle.  Needs a B200.

The product is the quantized matvec (same tolerance as its own tests: the order of the fp32 additions); bias and
activation are evaluated by the oracle in float64 as the upstream does, so the f32 kernel must agree within a few
ulp of float32."""
import numpy as np
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    if not torch.cuda.is_available():
        pytest.fail("these tests need a CUDA device")
    from nates_recipe_rs_b200 import quant_ops
    return quant_ops


def close(got, want):
    err = np.abs(got.astype(np.float64) - want.astype(np.float64))
    return bool((err <= 2e-4 + 1e-3 * np.abs(want)).all()), float(err.max())


@pytest.mark.parametrize("act", oracle.DENSE_ACTS)
@pytest.mark.parametrize("qtype,m,n,k", [(oracle.Q4_K, 1, 300, 1024), (oracle.Q6_K, 5, 129, 512), (oracle.Q8_0, 2, 64, 256), (oracle.Q4_K, 40, 200, 768)])
def test_dense_matches_oracle(ops, act, qtype, m, n, k):
    w = oracle.quantize(qtype, oracle.fill_normal(n * k, 40 + n, 0.05).reshape(n, k))
    x = oracle.fill_normal(m * k, 41 + k, 1.0).reshape(m, k)
    bias = oracle.fill_normal(n, 42, 0.5)
    alpha = {"leaky_relu": 0.01, "prelu": 0.2, "elu": 1.0}.get(act, 0.0)
    want = oracle.dense(qtype, w, x, bias, act, alpha, k)
    out = torch.full((m, n), float("nan"), device="cuda")
    ops.gpu_qdense_into(qtype, torch.from_numpy(w).cuda(), torch.from_numpy(x).cuda(), torch.from_numpy(bias).cuda(), out, m, n, k, act, alpha)
    ops.check_launch()
    ok, worst = close(out.cpu().numpy(), want)
    assert ok, f"{act}: max err {worst:.3e}"


@pytest.mark.parametrize("act", ["linear", "gelu", "selu"])
@pytest.mark.parametrize("m,n,k", [(64, 300, 1024), (200, 129, 512), (700, 256, 768)])
def test_dense_many_rows_takes_the_gemm(ops, act, m, n, k):
    """From 64 rows on a Q4_K layer runs on the tcgen05 GEMM with x rounded to bf16."""
    w = oracle.quantize(oracle.Q4_K, oracle.fill_normal(n * k, 90 + n, 0.05).reshape(n, k))
    x = oracle.fill_normal(m * k, 91 + k, 1.0).reshape(m, k)
    bias = oracle.fill_normal(n, 92, 0.5)
    want = oracle.dense(oracle.Q4_K, w, x, bias, act, 0.0, k, via="bf16")
    out = torch.full((m, n), float("nan"), device="cuda")
    ops.gpu_qdense_into(oracle.Q4_K, torch.from_numpy(w).cuda(), torch.from_numpy(x).cuda(), torch.from_numpy(bias).cuda(), out, m, n, k, act)
    ops.check_launch()
    ok, worst = close(out.cpu().numpy(), want)
    assert ok, f"{act}: max err {worst:.3e}"


def test_dense_without_bias_is_the_matvec(ops):
    m, n, k = 3, 257, 1024
    w = oracle.quantize(oracle.Q4_K, oracle.fill_normal(n * k, 7, 0.05).reshape(n, k))
    x = oracle.fill_normal(m * k, 8, 1.0).reshape(m, k)
    wd, xd = torch.from_numpy(w).cuda(), torch.from_numpy(x).cuda()
    out = torch.empty(m, n, device="cuda")
    ops.gpu_qdense_into(oracle.Q4_K, wd, xd, None, out, m, n, k)
    y = ops.gpu_qmatvec(oracle.Q4_K, wd, ops.gpu_quantize_q8_1(xd), m, n, k)
    ops.check_launch()
    assert torch.equal(out, y)


def test_dense_rejects_bad_arguments(ops):
    from nates_recipe_rs_b200 import _lib
    L = _lib.lib()   # QMM_ERR_NULL -1, QMM_ERR_SHAPE -2, QMM_ERR_UNSUPPORTED -3 (include/qmm.h)
    w = torch.zeros(144 * 4, dtype=torch.uint8, device="cuda")
    x = torch.zeros(256, device="cuda")
    y = torch.zeros(4, device="cuda")
    xq = torch.zeros(288, dtype=torch.uint8, device="cuda")
    assert L.launch_qdense(oracle.Q4_K, w.data_ptr(), x.data_ptr(), None, y.data_ptr(), xq.data_ptr(), 1, 4, 256, 99, 0.0, None) == -3
    assert L.launch_qdense(oracle.Q4_K, None, x.data_ptr(), None, y.data_ptr(), xq.data_ptr(), 1, 4, 256, 0, 0.0, None) == -1
    assert L.launch_qdense(oracle.Q4_K, w.data_ptr(), x.data_ptr(), None, y.data_ptr(), xq.data_ptr(), 1, 4, 100, 0, 0.0, None) == -2
    ops.check_launch()


def test_layer_list_forward_and_gguf_round_trip(ops, tmp_path):
    """A three-layer stack (the upstream's LayerParams list, recipe-infer/src/params.rs:35-59) built from f32
    weights, run, written to a GGUF file, loaded back and run again: same bits; and against the oracle layer by layer."""
    from nates_recipe_rs_b200 import gguf, layers
    dims = [(512, 1024, "gelu", oracle.Q4_K), (1024, 256, "leaky_relu", oracle.Q6_K), (256, 3, "linear", oracle.Q8_0)]
    n = 6
    stack, host = [], []
    for i, (k, o, act, qt) in enumerate(dims):
        wq = oracle.quantize(qt, oracle.fill_normal(o * k, 60 + i, 0.05).reshape(o, k))
        b = oracle.fill_normal(o, 70 + i, 0.1)
        host.append((qt, wq, b, act, k, o))
        stack.append(layers.QuantDense(qt, torch.from_numpy(wq).cuda(), torch.from_numpy(b).cuda(), k, o, act))
    x = oracle.fill_normal(n * dims[0][0], 80, 1.0).reshape(n, dims[0][0])
    scratch = layers.Scratch(stack, n)
    y = layers.forward_into(stack, torch.from_numpy(x).cuda(), scratch).clone()
    ops.check_launch()
    ref = x
    for l, (qt, wq, b, act, k, o) in zip(stack, host):
        ref = oracle.dense(qt, wq, ref, b, act, l.alpha(), k)
    ok, worst = close(y.cpu().numpy(), ref)
    assert ok, f"stack: max err {worst:.3e}"
    path = tmp_path / "mlp.gguf"
    wr = gguf.GgufWriter(path)
    wr.meta("general.architecture", "mlp")
    for i, (qt, wq, b, act, k, o) in enumerate(host):
        wr.tensor(f"layers.{i}.weight", qt, [k, o], wq)
        wr.tensor(f"layers.{i}.bias", gguf.F32, [o], b)
    wr.finish()
    with gguf.GgufFile(path) as gf:
        loaded = [layers.QuantDense.from_gguf(gf, f"layers.{i}.weight", f"layers.{i}.bias", act) for i, (_, _, _, act, _, _) in enumerate(host)]
    torch.cuda.synchronize()
    y2 = layers.forward_into(loaded, torch.from_numpy(x).cuda(), layers.Scratch(loaded, n))
    ops.check_launch()
    assert torch.equal(y, y2)
