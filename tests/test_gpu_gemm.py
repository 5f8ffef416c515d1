"""Q4_K dequant-GEMM (tcgen05) against the CPU oracle, through the C ABI.  Needs a B200.

The oracle's product is exact per term (bf16 x bf16 fits binary32); only the order of the fp32
additions differs, so the accumulators must agree within 1e-3 relative / 1e-4 absolute and the
bf16 outputs within one bf16 step of the oracle's."""
import numpy as np
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu
REL_TOL, ABS_TOL = 1e-3, 1e-4


@pytest.fixture(scope="module")
def ops():
    if not torch.cuda.is_available():
        pytest.fail("these tests need a CUDA device")
    from nates_recipe_rs_b200 import quant_ops
    return quant_ops


def make_case(m, n, k, seed):
    w = oracle.quantize(oracle.Q4_K, oracle.fill_normal(n * k, seed, 0.02).reshape(n, k))
    x = oracle.f32_to_bf16_bits(oracle.fill_normal(m * k, seed + 1, 1.0).reshape(m, k))
    return w, x


def bf16_tensor(bits):
    return torch.from_numpy(bits.astype(np.int16)).cuda().view(torch.bfloat16)


SHAPES = [(1, 128, 256), (128, 128, 256), (129, 128, 512), (300, 256, 1024), (512, 384, 768), (640, 128, 512),
          (77, 200, 256), (1100, 128, 256)]


@pytest.mark.parametrize("m,n,k", SHAPES)
def test_gemm_matches_oracle(ops, m, n, k):
    w, x = make_case(m, n, k, 100 + m + n)
    y_ref, yf_ref = oracle.gemm_bf16(oracle.Q4_K, w, x, k)
    wd, xd = torch.from_numpy(w).cuda(), bf16_tensor(x)
    yf = ops.gpu_qgemm_q4_k_bf16(wd, xd, n, k, torch.float32)
    y = ops.gpu_qgemm_q4_k_bf16(wd, xd, n, k)
    ops.check_launch()
    got_f = yf.cpu().numpy()
    err = np.abs(got_f.astype(np.float64) - yf_ref.astype(np.float64))
    assert (err <= ABS_TOL + REL_TOL * np.abs(yf_ref)).all(), f"max err {err.max():.3e}"
    got = y.view(torch.int16).cpu().numpy().view(np.uint16)
    # bf16 of the GPU's own accumulators, exactly; and within one bf16 step of the oracle's output
    assert np.array_equal(got, oracle.f32_to_bf16_bits(got_f))
    step = np.abs(oracle.bf16_bits_to_f32(y_ref)) * 2.0 ** -7 + 2 * ABS_TOL   # one bf16 step, or the accumulator tolerance near zero
    assert (np.abs(oracle.bf16_bits_to_f32(got) - oracle.bf16_bits_to_f32(y_ref)) <= step).all()


@pytest.mark.parametrize("m,n,k", [(100, 300, 1024), (256, 128, 2048), (77, 200, 512), (129, 384, 4096), (300, 256, 1024)])
@pytest.mark.parametrize("ksplit", [1, 2])
def test_gemm_split_k_over_a_cluster(ops, m, n, k, ksplit):
    """K split over the two CTAs of a cluster (partial tiles joined through distributed shared memory) and not
    split, forced by the tunable: both against the oracle, reruns bit identical, f32 and bf16 outputs."""
    from nates_recipe_rs_b200 import _lib
    L = _lib.lib()
    w, x = make_case(m, n, k, 500 + m + n)
    y_ref, yf_ref = oracle.gemm_bf16(oracle.Q4_K, w, x, k)
    wd, xd = torch.from_numpy(w).cuda(), bf16_tensor(x)
    try:
        _lib.check(L.qmm_tune(b"gemm_mb", 1), "tune")
        _lib.check(L.qmm_tune(b"gemm_ksplit", ksplit), "tune")
        yf = ops.gpu_qgemm_q4_k_bf16(wd, xd, n, k, torch.float32)
        yf2 = ops.gpu_qgemm_q4_k_bf16(wd, xd, n, k, torch.float32)
        y = ops.gpu_qgemm_q4_k_bf16(wd, xd, n, k)
        ops.check_launch()
    finally:
        _lib.check(L.qmm_tune(b"gemm_mb", 0), "tune")
        _lib.check(L.qmm_tune(b"gemm_ksplit", 0), "tune")
    assert torch.equal(yf, yf2)
    got_f = yf.cpu().numpy()
    err = np.abs(got_f.astype(np.float64) - yf_ref.astype(np.float64))
    assert (err <= ABS_TOL + REL_TOL * np.abs(yf_ref)).all(), f"max err {err.max():.3e}"
    got = y.view(torch.int16).cpu().numpy().view(np.uint16)
    assert np.array_equal(got, oracle.f32_to_bf16_bits(got_f))


def test_gemm_weights_are_the_bf16_dequant(ops):
    """With x = identity rows the GEMM returns the bf16 weights themselves: bit-exact vs the oracle."""
    n, k = 128, 256
    w, _ = make_case(1, n, k, 7)
    eye = np.eye(k, dtype=np.float32)
    y = ops.gpu_qgemm_q4_k_bf16(torch.from_numpy(w).cuda(), bf16_tensor(oracle.f32_to_bf16_bits(eye)), n, k, torch.float32)
    want = oracle.bf16_bits_to_f32(oracle.dequantize_bf16(oracle.Q4_K, w, k))   # (n, k)
    assert np.array_equal(y.cpu().numpy().view(np.uint32), np.ascontiguousarray(want.T).view(np.uint32))


def test_gemm_twice_bit_identical_and_padding_untouched(ops):
    m, n, k = 200, 256, 512
    w, x = make_case(m, n, k, 3)
    wd, xd = torch.from_numpy(w).cuda(), bf16_tensor(x)
    buf = torch.full((m * n + 256,), 7.0, dtype=torch.bfloat16, device="cuda")
    ops.gpu_qgemm_q4_k_bf16_into(wd, xd, buf[128:128 + m * n], m, n, k)
    a = buf.clone()
    ops.gpu_qgemm_q4_k_bf16_into(wd, xd, buf[128:128 + m * n], m, n, k)
    ops.check_launch()
    assert torch.equal(a.view(torch.int16), buf.view(torch.int16))
    assert bool((buf[:128] == 7.0).all()) and bool((buf[128 + m * n:] == 7.0).all())


@pytest.mark.parametrize("m,n,k", [(512, 4096, 4096), (2048, 4096, 4096), (512, 14336, 4096)])
def test_gemm_full_size_against_torch(ops, m, n, k):
    """BASELINE config 3 shapes: every output against a float32 matmul of the dequantised operands."""
    g = torch.Generator(device="cuda").manual_seed(m + n)
    wq = ops.gpu_quantize_weights(oracle.Q4_K, torch.randn(n, k, device="cuda", generator=g) * 0.02)
    x = torch.randn(m, k, device="cuda", generator=g).to(torch.bfloat16)
    yf = ops.gpu_qgemm_q4_k_bf16(wq, x, n, k, torch.float32)
    ops.check_launch()
    wb = ops.gpu_dequantize(oracle.Q4_K, wq, n * k, torch.bfloat16).reshape(n, k)
    ref = x.float() @ wb.float().T
    mag = x.float().abs() @ wb.float().abs().T
    assert bool(((yf - ref).abs() <= ABS_TOL + REL_TOL * mag).all()), float((yf - ref).abs().max())


@pytest.mark.parametrize("qtype", [oracle.Q6_K, oracle.Q8_0, oracle.Q4_K])
@pytest.mark.parametrize("m,n,k", [(70, 300, 1024), (512, 256, 768), (129, 128, 256)])
def test_gemm_bt_on_a_bf16_weight_window(ops, qtype, m, n, k):
    """launch_gemm_bt_bf16 on weights dequantised to bf16 by the library (the route of a block type without a fused
    GEMM) against the oracle's GEMM on the same packed weights: the bf16 weights are bit-identical by construction."""
    w = oracle.quantize(qtype, oracle.fill_normal(n * k, 300 + n, 0.02).reshape(n, k))
    x = oracle.f32_to_bf16_bits(oracle.fill_normal(m * k, 301 + m, 1.0).reshape(m, k))
    y_ref, yf_ref = oracle.gemm_bf16(qtype, w, x, k)
    wb = ops.gpu_dequantize(qtype, torch.from_numpy(w).cuda(), n * k, torch.bfloat16)
    xd = bf16_tensor(x)
    yf = torch.full((m, n), float("nan"), device="cuda")
    ops.gpu_gemm_bt_bf16_into(xd, wb, yf, m, n, k)
    y = torch.empty(m, n, device="cuda", dtype=torch.bfloat16)
    ops.gpu_gemm_bt_bf16_into(xd, wb, y, m, n, k)
    ops.check_launch()
    got_f = yf.cpu().numpy()
    err = np.abs(got_f.astype(np.float64) - yf_ref.astype(np.float64))
    assert (err <= ABS_TOL + REL_TOL * np.abs(yf_ref)).all(), f"max err {err.max():.3e}"
    assert np.array_equal(y.view(torch.int16).cpu().numpy().view(np.uint16), oracle.f32_to_bf16_bits(got_f))
