"""The CPU oracle against the committed known-answer fixtures, closed-form block
values, and its independent numpy restatement.  No GPU.

Follows the upstream's test conventions for quantization: integer-exact codes,
tie-free probes (gpu-core/tests/suite/prove_quantized.rs:168-173, 349-357)."""
import numpy as np
import pytest

import oracle
from oracle import npref

TYPES = [oracle.Q8_0, oracle.Q4_K, oracle.Q6_K]


def _bits(hexstr, dt):
    return np.frombuffer(bytes.fromhex(hexstr), dtype=dt)


def test_golden_blocks_dequantize_bit_exact(golden):
    for case in golden["blocks"]:
        t = case["type"]
        blk = _bits(case["bytes"], np.uint8)
        want = _bits(case["f32_bits"], np.uint32)
        got = oracle.dequantize(t, blk, oracle.BLOCK_ELEMS[t]).view(np.uint32).reshape(-1)
        assert np.array_equal(got, want), case["name"]
        want_bf16 = oracle.f32_to_bf16_bits(want.view(np.float32))
        got_bf16 = oracle.dequantize_bf16(t, blk, oracle.BLOCK_ELEMS[t]).reshape(-1)
        assert np.array_equal(got_bf16, want_bf16), case["name"]


def test_closed_form_values(golden):
    by = {c["name"]: c for c in golden["blocks"]}

    def deq(name):
        c = by[name]
        return oracle.dequantize(c["type"], _bits(c["bytes"], np.uint8), oracle.BLOCK_ELEMS[c["type"]]).reshape(-1)

    assert np.all(deq("q4_k_closed_form") == 1.0 * 2 * 15 - 0.5 * 3)          # 28.5
    assert np.all(deq("q4_k_allmax") == 63 * 15 - 0.5 * 63)                    # 913.5
    assert np.all(deq("q4_k_zero") == 0) and np.all(deq("q6_k_zero") == 0) and np.all(deq("q8_0_zero") == 0)
    for pos in (0, 31, 32, 100, 255):
        v = deq(f"q4_k_onehot_{pos}")
        want = np.zeros(256, dtype=np.float32)
        want[pos] = 2.0 * (pos // 32 + 1) * 9
        assert np.array_equal(v, want), pos
    assert np.all(deq("q6_k_allmax") == 127 * 31)
    assert np.all(deq("q6_k_allmin_negscale") == 0.5 * -128 * -32)
    for pos in (0, 15, 16, 127, 128, 200, 255):
        v = deq(f"q6_k_onehot_{pos}")
        want = np.zeros(256, dtype=np.float32)
        want[pos] = (pos // 16 + 1) * 31
        assert np.array_equal(v, want), pos
    assert np.array_equal(deq("q8_0_ramp"), 0.5 * np.arange(-16, 16, dtype=np.float32))
    assert np.array_equal(deq("q8_0_extremes_negd"), -1.25 * np.array([-128, 127] * 16, dtype=np.float32))


def test_golden_q8_1_quantizer(golden):
    for case in golden["q8_1"]:
        x = _bits(case["x_bits"], np.uint32).view(np.float32)
        got = oracle.quantize(oracle.Q8_1, x).reshape(-1)
        assert np.array_equal(got, _bits(case["bytes"], np.uint8)), case["name"]


def test_golden_block_dots(golden):
    for case in golden["dots"]:
        t, k = case["type"], case["k"]
        got = oracle.block_dots(t, _bits(case["w"], np.uint8), _bits(case["xq"], np.uint8), k)
        assert np.array_equal(got.reshape(-1), _bits(case["sums"], np.int32))


def test_generator_pinned(golden):
    g = golden["generator"]
    sigma = np.array([g["sigma_bits"]], dtype=np.uint32).view(np.float32)[0]
    got = oracle.fill_normal(16, g["seed"], float(sigma), g["first_index"])
    assert np.array_equal(got.view(np.uint32), _bits(g["f32_bits"], np.uint32))
    big = oracle.fill_normal(1 << 16, 3, 1.0)
    assert abs(float(big.mean())) < 0.02 and abs(float(big.std()) - 1.0) < 0.02
    assert np.array_equal(big, npref.fill_normal(1 << 16, 3, 1.0))


@pytest.mark.parametrize("qtype", TYPES)
def test_c_and_numpy_agree_on_seeded_rows(qtype):
    k, n = 1024, 24
    w = oracle.quantize(qtype, oracle.fill_normal(n * k, 0x5EED + qtype, 0.02).reshape(n, k))
    assert np.array_equal(oracle.dequantize(qtype, w, k).reshape(-1).view(np.uint32),
                          npref.dequantize(qtype, w).view(np.uint32))
    x = oracle.fill_normal(k, 99, 1.0)
    xq = oracle.quantize(oracle.Q8_1, x).reshape(-1)
    assert np.array_equal(xq, npref.quantize_q8_1(x))
    assert np.array_equal(oracle.block_dots(qtype, w, xq, k), npref.block_dots(qtype, w, xq, k))


@pytest.mark.parametrize("qtype", TYPES)
def test_quantize_roundtrip_error_bound(qtype):
    k, n = 2048, 16
    x = oracle.fill_normal(n * k, 5, 0.02).reshape(n, k)
    d = oracle.dequantize(qtype, oracle.quantize(qtype, x), k)
    rel = float(np.sqrt(((d - x) ** 2).mean()) / x.std())
    assert rel < {oracle.Q8_0: 0.01, oracle.Q4_K: 0.10, oracle.Q6_K: 0.03}[qtype]
    # quantizing the dequantised values again reproduces the same values (idempotence of the grid)
    if qtype == oracle.Q8_0:
        d2 = oracle.dequantize(qtype, oracle.quantize(qtype, d), k)
        assert np.allclose(d2, d, rtol=0, atol=float(np.abs(x).max()) / 127)


@pytest.mark.parametrize("qtype", TYPES)
def test_matvec_matches_float_reference(qtype):
    """y from integer block dots == dequant(w) . dequant(xq) up to fp32 accumulation noise."""
    k, n, m = 1536, 40, 3
    w = oracle.quantize(qtype, oracle.fill_normal(n * k, 21, 0.02).reshape(n, k))
    xq = oracle.quantize(oracle.Q8_1, oracle.fill_normal(m * k, 22, 1.0).reshape(m, k))
    y = oracle.matvec(qtype, w, xq, k)
    wf = oracle.dequantize(qtype, w, k).astype(np.float64)
    xf = oracle.dequantize(oracle.Q8_1, xq, k).astype(np.float64)
    ref = xf @ wf.T
    # Q4_K uses the fp16 block sum s of the activations for the -dmin*m term, which is coarser
    tol = 2e-2 if qtype == oracle.Q4_K else 1e-4
    assert np.abs(y - ref).max() < tol * max(1.0, np.abs(ref).max())


def test_matvec_linearity_in_rows():
    """Row r of the output depends only on row r of the weights."""
    k = 512
    w = oracle.quantize(oracle.Q4_K, oracle.fill_normal(8 * k, 1, 0.02).reshape(8, k))
    xq = oracle.quantize(oracle.Q8_1, oracle.fill_normal(k, 2, 1.0))
    full = oracle.matvec(oracle.Q4_K, w, xq, k)
    part = oracle.matvec(oracle.Q4_K, w[3:5], xq, k)
    assert np.array_equal(full[:, 3:5], part)


def test_gemm_bf16_against_float64():
    k, n, m = 512, 32, 9
    w = oracle.quantize(oracle.Q4_K, oracle.fill_normal(n * k, 31, 0.02).reshape(n, k))
    x = oracle.f32_to_bf16_bits(oracle.fill_normal(m * k, 32, 1.0).reshape(m, k))
    y, yf = oracle.gemm_bf16(oracle.Q4_K, w, x, k)
    wf = oracle.bf16_bits_to_f32(oracle.dequantize_bf16(oracle.Q4_K, w, k)).astype(np.float64)
    ref = oracle.bf16_bits_to_f32(x).astype(np.float64) @ wf.T
    assert np.abs(yf - ref).max() < 1e-4
    assert np.array_equal(y, oracle.f32_to_bf16_bits(yf))


def test_scalar_conversions_against_numpy():
    rng = np.random.default_rng(0)
    vals = np.concatenate([rng.normal(size=2000) * 10.0 ** rng.integers(-9, 6, 2000),
                           [0.0, -0.0, 65504.0, 65519.9, 65520.0, 1e9, 2.0 ** -24, 2.0 ** -25, 2.0 ** -25 * 1.0001,
                            2.0 ** -14, 6.1e-5, np.inf, -np.inf]]).astype(np.float32)
    L = oracle.lib()
    with np.errstate(over="ignore"):
        want = vals.astype(np.float16).view(np.uint16)
    for v, wv in zip(vals, want):
        assert L.qo_f32_to_f16(float(v)) == int(wv), float(v)
    allh = np.arange(0, 0x7C01, dtype=np.uint16)  # every non-negative finite fp16 and +inf
    for h in allh[::37]:
        assert L.qo_f16_to_f32(int(h)) == float(np.array([h], dtype=np.uint16).view(np.float16)[0])
    bf = oracle.f32_to_bf16_bits(vals)
    for v, b in zip(vals, bf):
        assert L.qo_f32_to_bf16(float(v)) == int(b)
