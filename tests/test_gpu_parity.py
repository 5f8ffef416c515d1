"""CUDA kernels against the CPU oracle, through the C ABI.  Needs a B200.

Bars: bit-exact for packed codes, dequantised values and per-block integer sums;
fp32 matvec outputs within 1e-3 relative / 1e-4 absolute."""
import numpy as np
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu

REL_TOL, ABS_TOL = 1e-3, 1e-4
TYPES = [oracle.Q8_0, oracle.Q4_K, oracle.Q6_K]


@pytest.fixture(scope="module")
def ops():
    if not torch.cuda.is_available():
        pytest.fail("these tests need a CUDA device")
    from nates_recipe_rs_b200 import quant_ops
    return quant_ops


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def assert_close(got, want, what=""):
    err = np.abs(got.astype(np.float64) - want.astype(np.float64))
    bound = ABS_TOL + REL_TOL * np.abs(want.astype(np.float64))
    bad = err > bound
    assert not bad.any(), f"{what}: {bad.sum()} of {bad.size} outside tolerance, max err {err.max():.3e}"


def seeded_weights(qtype, n, k, seed):
    return oracle.quantize(qtype, oracle.fill_normal(n * k, seed, 0.02).reshape(n, k))


def random_byte_weights(qtype, n, k, seed):
    """Raw random bytes with finite fp16 scales: reaches every code and scale pattern."""
    rng = np.random.default_rng(seed)
    bb = oracle.BLOCK_BYTES[qtype]
    w = rng.integers(0, 256, (n * k // oracle.BLOCK_ELEMS[qtype], bb), dtype=np.uint8)
    scale = (rng.normal(size=w.shape[0]) * 0.01).astype(np.float16).view(np.uint8).reshape(-1, 2)
    if qtype == oracle.Q8_0:
        w[:, 0:2] = scale
    elif qtype == oracle.Q4_K:
        w[:, 0:2] = scale
        w[:, 2:4] = (rng.normal(size=w.shape[0]) * 0.01).astype(np.float16).view(np.uint8).reshape(-1, 2)
    else:
        w[:, 208:210] = scale
    return w.reshape(n, -1)


# ------------------------------------------------------------------ golden fixtures
def test_golden_blocks_dequantize_bit_exact(ops, golden):
    for case in golden["blocks"]:
        t = case["type"]
        blk = np.frombuffer(bytes.fromhex(case["bytes"]), dtype=np.uint8)
        want = np.frombuffer(bytes.fromhex(case["f32_bits"]), dtype=np.uint32)
        pad = np.zeros(256, dtype=np.uint8)          # the library reads whole 16-byte lines
        buf = dev(np.concatenate([blk, pad]))
        got = ops.gpu_dequantize(t, buf, oracle.BLOCK_ELEMS[t]).cpu().numpy().view(np.uint32)
        assert np.array_equal(got, want), case["name"]
        got16 = ops.gpu_dequantize(t, buf, oracle.BLOCK_ELEMS[t], torch.bfloat16).view(torch.int16).cpu().numpy().view(np.uint16)
        assert np.array_equal(got16, oracle.f32_to_bf16_bits(want.view(np.float32))), case["name"]


def test_golden_q8_1_quantizer(ops, golden):
    for case in golden["q8_1"]:
        x = np.frombuffer(bytes.fromhex(case["x_bits"]), dtype=np.uint32).view(np.float32)
        got = ops.gpu_quantize_q8_1(dev(x)).cpu().numpy()
        assert np.array_equal(got, np.frombuffer(bytes.fromhex(case["bytes"]), dtype=np.uint8)), case["name"]


def test_golden_block_dots(ops, golden):
    for case in golden["dots"]:
        t, k = case["type"], case["k"]
        w = np.frombuffer(bytes.fromhex(case["w"]), dtype=np.uint8)
        xq = np.frombuffer(bytes.fromhex(case["xq"]), dtype=np.uint8)
        n = w.size // oracle.row_bytes(t, k)
        got = ops.gpu_qblock_dots(t, dev(w), dev(xq), n, k).cpu().numpy()
        assert np.array_equal(got.reshape(-1), np.frombuffer(bytes.fromhex(case["sums"]), dtype=np.int32))


# ------------------------------------------------------------------ quantizers
@pytest.mark.parametrize("m,k", [(1, 32), (1, 4096), (3, 14336), (16, 4096)])
def test_quantize_q8_1_bit_exact(ops, m, k):
    x = oracle.fill_normal(m * k, 17 + m, 1.0).reshape(m, k)
    x[0, :32] = 0.0  # an all-zero block
    got = ops.gpu_quantize_q8_1(dev(x)).cpu().numpy()
    assert np.array_equal(got, oracle.quantize(oracle.Q8_1, x).reshape(-1))


@pytest.mark.parametrize("qtype", TYPES)
def test_weight_quantizers_bit_exact(ops, qtype):
    n, k = 37, 2048
    x = oracle.fill_normal(n * k, 0x5EED + qtype, 0.02).reshape(n, k)
    x[3] = 0.0
    x[5, :256] = np.abs(x[5, :256])      # a super-block with no negative value
    x[6, :256] = -np.abs(x[6, :256])     # and one with no positive value
    got = ops.gpu_quantize_weights(qtype, dev(x)).cpu().numpy()
    assert np.array_equal(got, oracle.quantize(qtype, x).reshape(-1))


# ------------------------------------------------------------------ dequantize
@pytest.mark.parametrize("qtype", TYPES)
@pytest.mark.parametrize("maker", [seeded_weights, random_byte_weights])
def test_dequantize_bit_exact(ops, qtype, maker):
    n, k = 64, 1024
    w = maker(qtype, n, k, 123)
    got = ops.gpu_dequantize(qtype, dev(w), n * k).cpu().numpy().view(np.uint32)
    want = oracle.dequantize(qtype, w, k).reshape(-1).view(np.uint32)
    assert np.array_equal(got, want)
    got16 = ops.gpu_dequantize(qtype, dev(w), n * k, torch.bfloat16).view(torch.int16).cpu().numpy().view(np.uint16)
    assert np.array_equal(got16, oracle.dequantize_bf16(qtype, w, k).reshape(-1))


@pytest.mark.parametrize("qtype", TYPES)
def test_dequantize_into_an_unaligned_window(ops, qtype):
    """An output that does not start on a 16-byte line takes the one-element-per-thread kernel: the same bits."""
    n, k = 8, 1024
    w = random_byte_weights(qtype, n, k, 321)
    for dtype, want in ((torch.float32, oracle.dequantize(qtype, w, k).reshape(-1).view(np.uint32)),
                        (torch.bfloat16, oracle.dequantize_bf16(qtype, w, k).reshape(-1))):
        buf = torch.zeros(n * k + 1, dtype=dtype, device="cuda")
        ops.gpu_dequantize_into(qtype, dev(w), buf[1:], n * k)
        got = buf[1:].contiguous().view(torch.int32 if dtype == torch.float32 else torch.int16).cpu().numpy()
        assert np.array_equal(got.view(want.dtype), want)
        assert float(buf[0]) == 0.0


# ------------------------------------------------------------------ integer block sums
@pytest.mark.parametrize("qtype", TYPES)
@pytest.mark.parametrize("maker", [seeded_weights, random_byte_weights])
def test_block_dots_bit_exact(ops, qtype, maker):
    n, k = 48, 2048
    w = maker(qtype, n, k, 7)
    xq = oracle.quantize(oracle.Q8_1, oracle.fill_normal(k, 8, 1.0)).reshape(-1)
    got = ops.gpu_qblock_dots(qtype, dev(w), dev(xq), n, k).cpu().numpy()
    assert np.array_equal(got, oracle.block_dots(qtype, w, xq, k))


# ------------------------------------------------------------------ matvec
SHAPES = [
    # (m, n, k)
    (1, 1, 256), (1, 7, 256), (1, 33, 512), (1, 300, 1024), (2, 129, 2048), (3, 64, 4096),
    (1, 1000, 4096), (4, 515, 4096), (1, 257, 14336), (5, 96, 8192), (1, 40, 28672), (9, 200, 1792),
    # three rows and more: Q4_K takes the tensor-core kernel where the shape allows (one or two tiles of
    # eight activation rows, one or several K chunks, ragged last row tile and last chunk), else dp4a
    (8, 300, 4096), (16, 1000, 4096), (13, 257, 14336), (21, 100, 8192), (16, 40, 28672), (7, 17, 256),
    (6, 50, 1024), (12, 50, 1024), (3, 4099, 2048), (10, 333, 4608),
    # 17..32 rows in one pass of the tensor-core kernel (four tiles of eight), more rows in groups of 32
    (17, 300, 4096), (32, 1000, 4096), (25, 257, 14336), (32, 2500, 2048), (40, 130, 4096), (70, 64, 1024),
]


@pytest.mark.parametrize("qtype", TYPES)
@pytest.mark.parametrize("m,n,k", SHAPES)
def test_matvec_matches_oracle(ops, qtype, m, n, k):
    w = seeded_weights(qtype, n, k, 1000 + n)
    xq = oracle.quantize(oracle.Q8_1, oracle.fill_normal(m * k, 2000 + k, 1.0).reshape(m, k))
    y = torch.full((m, n), float("nan"), device="cuda")
    ops.gpu_qmatvec_into(qtype, dev(w), dev(xq), y, m, n, k)
    ops.check_launch()
    assert_close(y.cpu().numpy(), oracle.matvec(qtype, w, xq, k), f"{oracle.TYPE_NAMES[qtype]} {m}x{n}x{k}")


@pytest.mark.parametrize("qtype", [oracle.Q4_K, oracle.Q6_K])
@pytest.mark.parametrize("m,n,k", [(3, 515, 4096), (8, 4096, 4096), (16, 1031, 14336), (11, 2048, 8192), (16, 77, 6144)])
def test_small_batch_tensor_core_kernel_matches_dp4a_kernel(ops, qtype, m, n, k):
    """The same launch through both kernels of a type (the threshold is a tunable), twice each."""
    from nates_recipe_rs_b200 import _lib
    L = _lib.lib()
    w = dev(seeded_weights(qtype, n, k, 77))
    xq = ops.gpu_quantize_q8_1(torch.from_numpy(oracle.fill_normal(m * k, 78, 1.0).reshape(m, k)).cuda())
    try:
        _lib.check(L.qmm_tune(b"mma_min_m", 0), "tune")
        y_dp4a = ops.gpu_qmatvec(qtype, w, xq, m, n, k)
        _lib.check(L.qmm_tune(b"mma_min_m", 1), "tune")
        y_mma = ops.gpu_qmatvec(qtype, w, xq, m, n, k)
        y_mma2 = ops.gpu_qmatvec(qtype, w, xq, m, n, k)
    finally:
        _lib.check(L.qmm_tune(b"mma_min_m", 3), "tune")
    ops.check_launch()
    assert torch.equal(y_mma, y_mma2)
    assert_close(y_mma.cpu().numpy(), y_dp4a.cpu().numpy())


@pytest.mark.parametrize("qtype", [oracle.Q4_K, oracle.Q6_K])
@pytest.mark.parametrize("m,n,k", [(5, 20000, 2048), (16, 20000, 1024), (29, 20000, 1024), (8, 3000, 14336), (32, 700, 8192)])
def test_tensor_core_kernel_tiles_per_pass(ops, qtype, m, n, k):
    """Every instantiation of the tensor-core kernel (2, 4 or 8 weight tiles per pass; 8 or 16 warps for up
    to eight rows) against the oracle; the tall matrices have nine row tiles per CTA, more than any pass takes."""
    from nates_recipe_rs_b200 import _lib
    L = _lib.lib()
    w = seeded_weights(qtype, n, k, 31 + n)
    xq = oracle.quantize(oracle.Q8_1, oracle.fill_normal(m * k, 32 + k, 1.0).reshape(m, k))
    want = oracle.matvec(qtype, w, xq, k)
    wd, xd = dev(w), dev(xq)
    try:
        for warps in (8, 16):
            _lib.check(L.qmm_tune(b"mma_acc_w1", warps), "tune")
            for tp in (2, 4, 8):
                for key in (b"mma_acc_tp1", b"mma_acc_tp2"):
                    _lib.check(L.qmm_tune(key, tp), "tune")
                _lib.check(L.qmm_tune(b"mma_acc_tp4", min(tp, 4)), "tune")
                y = torch.full((m, n), float("nan"), device="cuda")
                ops.gpu_qmatvec_into(qtype, wd, xd, y, m, n, k)
                ops.check_launch()
                assert_close(y.cpu().numpy(), want, f"warps {warps} tiles/pass {tp}")
    finally:
        _lib.check(L.qmm_tune(b"mma_acc_w1", 16), "tune")
        _lib.check(L.qmm_tune(b"mma_acc_tp1", 8), "tune")
        _lib.check(L.qmm_tune(b"mma_acc_tp2", 8), "tune")
        _lib.check(L.qmm_tune(b"mma_acc_tp4", 4), "tune")


@pytest.mark.parametrize("maker", [seeded_weights, random_byte_weights])
@pytest.mark.parametrize("m,n,k", [(17, 1000, 1024), (32, 4096, 4096), (24, 300, 14336), (12, 2048, 2048), (40, 640, 8192)])
def test_tcgen05_integer_matvec(ops, maker, m, n, k):
    """The tcgen05 kind::i8 form of the Q4_K matvec (int32 sums in tensor memory, scales in the epilogue) against the
    oracle: both widths of the instruction (16 and 32 activation rows; 12 rows reach it through the tunable), ragged
    last tiles, K split over clusters of 1, 2 and 4 CTAs, a second group of rows past 32; reruns give the same bits."""
    from nates_recipe_rs_b200 import _lib
    L = _lib.lib()
    w = maker(oracle.Q4_K, n, k, 77 + n)
    xq = oracle.quantize(oracle.Q8_1, oracle.fill_normal(m * k, 78 + k, 1.0).reshape(m, k))
    want = oracle.matvec(oracle.Q4_K, w, xq, k)
    wd, xd = dev(w), dev(xq)
    try:
        _lib.check(L.qmm_tune(b"umma_min_m", 8), "tune")
        _lib.check(L.qmm_tune(b"umma_min_k", 256), "tune")
        for ksplit in (0, 1, 2, 4):
            _lib.check(L.qmm_tune(b"umma_ksplit", ksplit), "tune")
            y = torch.full((m, n), float("nan"), device="cuda")
            ops.gpu_qmatvec_into(oracle.Q4_K, wd, xd, y, m, n, k)
            y2 = torch.full((m, n), float("nan"), device="cuda")
            ops.gpu_qmatvec_into(oracle.Q4_K, wd, xd, y2, m, n, k)
            ops.check_launch()
            assert_close(y.cpu().numpy(), want, f"ksplit {ksplit}")
            assert torch.equal(y, y2)
    finally:
        _lib.check(L.qmm_tune(b"umma_min_m", 17), "tune")
        _lib.check(L.qmm_tune(b"umma_min_k", 4096), "tune")
        _lib.check(L.qmm_tune(b"umma_ksplit", 0), "tune")


# per-rank projection shapes of the 8B- and 70B-class stacks under tensor parallelism 4 and 8
TP_SHARD_SHAPES = [
    (oracle.Q4_K, 1280, 4096), (oracle.Q6_K, 256, 4096), (oracle.Q4_K, 4096, 1024), (oracle.Q4_K, 7168, 4096), (oracle.Q6_K, 4096, 3584),
    (oracle.Q4_K, 640, 4096), (oracle.Q6_K, 128, 4096), (oracle.Q4_K, 4096, 512), (oracle.Q4_K, 3584, 4096), (oracle.Q6_K, 4096, 1792),
    (oracle.Q4_K, 2560, 8192), (oracle.Q4_K, 8192, 2048), (oracle.Q4_K, 8192, 7168), (oracle.Q4_K, 8192, 1024), (oracle.Q4_K, 8192, 3584),
    (oracle.Q6_K, 16032, 8192),
]


@pytest.mark.parametrize("qtype,n,k", TP_SHARD_SHAPES)
def test_tensor_parallel_shard_shapes_both_kernels(ops, qtype, n, k):
    """Decode batch sizes 1, 8, 16 and 32 on every shard shape: the launcher's own choice of kernel
    against the dp4a kernel alone, every output written (NaN sentinel)."""
    from nates_recipe_rs_b200 import _lib
    L = _lib.lib()
    gen = torch.Generator(device="cuda").manual_seed(n + k)
    w = ops.gpu_quantize_weights(qtype, torch.randn(n, k, device="cuda", generator=gen) * 0.02)
    try:
        for m in (1, 8, 16, 32):
            xq = ops.gpu_quantize_q8_1(torch.randn(m, k, device="cuda", generator=gen))
            _lib.check(L.qmm_tune(b"mma_min_m", 0), "tune")
            y_dp4a = ops.gpu_qmatvec(qtype, w, xq, m, n, k)
            _lib.check(L.qmm_tune(b"mma_min_m", 3), "tune")
            y = torch.full((m, n), float("nan"), device="cuda")
            ops.gpu_qmatvec_into(qtype, w, xq, y, m, n, k)
            ops.check_launch()
            assert not torch.isnan(y).any()
            assert_close(y.cpu().numpy(), y_dp4a.cpu().numpy(), f"m={m}")
    finally:
        _lib.check(L.qmm_tune(b"mma_min_m", 3), "tune")


def test_tall_head_with_several_k_chunks_takes_the_tensor_core_kernel(ops):
    """The 70B-class output head (128256 x 8192, Q6_K) at 16 activation rows: several K chunks and 55 row tiles per CTA,
    i.e. seven passes of eight tiles.  Against the dp4a kernel on every output and against the oracle on a row sample."""
    from nates_recipe_rs_b200 import _lib
    L = _lib.lib()
    qtype, n, k, m = oracle.Q6_K, 128256, 8192, 16
    gen = torch.Generator(device="cuda").manual_seed(99)
    w = torch.empty(n * oracle.row_bytes(qtype, k), dtype=torch.uint8, device="cuda")
    rb = oracle.row_bytes(qtype, k)
    for r0 in range(0, n, 16032):   # quantized in pieces: the f32 source of the whole matrix would be 4 GB
        ops.gpu_quantize_weights_into(qtype, torch.randn(16032, k, device="cuda", generator=gen) * 0.02, w[r0 * rb:(r0 + 16032) * rb], 16032, k)
    xq = ops.gpu_quantize_q8_1(torch.randn(m, k, device="cuda", generator=gen))
    try:
        _lib.check(L.qmm_tune(b"mma_min_m", 0), "tune")
        y_dp4a = ops.gpu_qmatvec(qtype, w, xq, m, n, k)
        _lib.check(L.qmm_tune(b"mma_min_m", 3), "tune")
        y = torch.full((m, n), float("nan"), device="cuda")
        ops.gpu_qmatvec_into(qtype, w, xq, y, m, n, k)
        ops.check_launch()
    finally:
        _lib.check(L.qmm_tune(b"mma_min_m", 3), "tune")
    assert not torch.isnan(y).any()
    assert_close(y.cpu().numpy(), y_dp4a.cpu().numpy(), "all rows")
    rows = np.concatenate([np.arange(0, n, 4099), np.arange(66290, 66320), [n - 1]])
    wn = w.cpu().numpy().reshape(n, rb)[rows]
    want = oracle.matvec(qtype, wn, xq.cpu().numpy(), k)
    assert_close(y.cpu().numpy()[:, rows], want, "row sample")


@pytest.mark.parametrize("qtype,n,k,pitch_to", [(oracle.Q6_K, 300, 7168, 48), (oracle.Q6_K, 513, 1792, 48), (oracle.Q6_K, 200, 3584, 48),
                                                (oracle.Q8_0, 129, 4224, 16), (oracle.Q4_K, 64, 2048, 256), (oracle.Q6_K, 64, 2048, 48)])
def test_matvec_with_padded_rows(ops, qtype, n, k, pitch_to):
    """launch_qmatvec_pitched: the rows of the matrix lie further apart than their packed length (the padding
    filled with 0xFF).  Q6_K shards of a tensor-parallel down projection (K = 14336 / 2, / 4, / 8) are padded to a
    multiple of 48 bytes so that the tensor-core kernel can fetch them; results as for back-to-back rows."""
    from nates_recipe_rs_b200._lib import check, lib
    rb = oracle.row_bytes(qtype, k)
    pitch = (rb + pitch_to - 1) // pitch_to * pitch_to + (pitch_to if qtype == oracle.Q4_K else 0)
    w = oracle.quantize(qtype, oracle.fill_normal(n * k, 31, 0.02).reshape(n, k))
    padded = np.full((n, pitch), 0xFF, dtype=np.uint8)
    padded[:, :rb] = w
    wd, wp = dev(w), dev(padded)
    for m in (1, 2, 5, 16, 32):
        x = oracle.fill_normal(m * k, 32 + m, 1.0).reshape(m, k)
        xq = oracle.quantize(oracle.Q8_1, x)
        xqd = dev(xq)
        y = torch.full((m, n), float("nan"), device="cuda")
        check(lib().launch_qmatvec_pitched(qtype, wp.data_ptr(), pitch, xqd.data_ptr(), y.data_ptr(), m, n, k, torch.cuda.current_stream().cuda_stream),
              "launch_qmatvec_pitched")
        ops.check_launch()
        assert not torch.isnan(y).any()
        assert_close(y.cpu().numpy(), oracle.matvec(qtype, w, xq, k), f"m={m} against the oracle")
        assert_close(y.cpu().numpy(), ops.gpu_qmatvec(qtype, wd, xqd, m, n, k).cpu().numpy(), f"m={m} against back-to-back rows")
    assert lib().launch_qmatvec_pitched(qtype, wp.data_ptr(), rb - 2, xqd.data_ptr(), y.data_ptr(), 1, n, k, None) == -2


@pytest.mark.parametrize("qtype", TYPES)
@pytest.mark.parametrize("m", [2, 8, 16])
def test_matvec_random_byte_weights(ops, qtype, m):
    n, k = 77, 2048
    w = random_byte_weights(qtype, n, k, 5)
    xq = oracle.quantize(oracle.Q8_1, oracle.fill_normal(m * k, 6, 1.0).reshape(m, k))
    y = ops.gpu_qmatvec(qtype, dev(w), dev(xq), m, n, k)
    want = oracle.matvec(qtype, w, xq, k)
    # terms cancel in these rows, so the bound is relative to the magnitude of the terms
    wf = np.abs(oracle.dequantize(qtype, w, k)).astype(np.float64)
    xf = np.abs(oracle.dequantize(oracle.Q8_1, xq, k)).astype(np.float64)
    bound = ABS_TOL + REL_TOL * (xf @ wf.T)
    assert (np.abs(y.cpu().numpy() - want) <= bound).all()


@pytest.mark.parametrize("qtype", TYPES)
def test_matvec_unaligned_row_views(ops, qtype):
    """Rows taken from the middle of a matrix: for Q6_K / Q8_0 the view starts on a
    2-byte boundary only; the padding bytes around the output stay untouched."""
    n, k, skip = 40, 1792 if qtype != oracle.Q8_0 else 1056, 3
    w = seeded_weights(qtype, n + skip, k, 9)
    xq = oracle.quantize(oracle.Q8_1, oracle.fill_normal(k, 10, 1.0))
    wd = dev(w).reshape(-1)
    rb = oracle.row_bytes(qtype, k)
    view = wd[skip * rb:]
    ybuf = torch.full((n + 64,), 12345.0, device="cuda")
    from nates_recipe_rs_b200._lib import check, lib
    check(lib().launch_qmatvec(qtype, view.data_ptr(), dev(xq).data_ptr(), ybuf[32:].data_ptr(), 1, n, k,
                               torch.cuda.current_stream().cuda_stream), "launch_qmatvec")
    ops.check_launch()
    out = ybuf.cpu().numpy()
    assert (out[:32] == 12345.0).all() and (out[32 + n:] == 12345.0).all()
    assert_close(out[32:32 + n][None], oracle.matvec(qtype, w[skip:], xq, k))


@pytest.mark.parametrize("qtype", TYPES)
def test_matvec_twice_bit_identical(ops, qtype):
    """Rerun determinism, as examples/det_probe.rs:125-134 checks for the upstream's GEMM."""
    m, n, k = 2, 4096, 4096
    w = dev(seeded_weights(qtype, n, k, 3))
    xq = dev(oracle.quantize(oracle.Q8_1, oracle.fill_normal(m * k, 4, 1.0).reshape(m, k)))
    a = ops.gpu_qmatvec(qtype, w, xq, m, n, k)
    b = ops.gpu_qmatvec(qtype, w, xq, m, n, k)
    assert torch.equal(a.view(torch.int32), b.view(torch.int32))


def test_config1_q8_0_4096(ops):
    """BASELINE config 1: Q8_0 4096x4096, batch 1, x ~ N(0,1), w ~ N(0,0.02)."""
    n = k = 4096
    w = seeded_weights(oracle.Q8_0, n, k, 0x5EED)
    x = oracle.fill_normal(k, 0x5EED + 1, 1.0)
    xq = ops.gpu_quantize_q8_1(dev(x))
    assert np.array_equal(xq.cpu().numpy(), oracle.quantize(oracle.Q8_1, x).reshape(-1))
    y = ops.gpu_qmatvec(oracle.Q8_0, dev(w), xq, 1, n, k)
    assert_close(y.cpu().numpy(), oracle.matvec(oracle.Q8_0, w, xq.cpu().numpy(), k))


@pytest.mark.parametrize("qtype,n,k", [(oracle.Q4_K, 14336, 4096), (oracle.Q4_K, 4096, 14336), (oracle.Q6_K, 4096, 14336)])
def test_config2_full_size(ops, qtype, n, k):
    """BASELINE config 2 at full size: weights quantised on the device, checked against the
    oracle on a sample of rows and through linearity: W.(x1) + W.(x2) vs rows of a 2-row batch."""
    wf = torch.from_numpy(oracle.fill_normal(n * k, 0x5EED + n, 0.02).reshape(n, k)).cuda()
    w = ops.gpu_quantize_weights(qtype, wf)
    x = oracle.fill_normal(2 * k, 77, 1.0).reshape(2, k)
    xq = ops.gpu_quantize_q8_1(dev(x))
    y2 = ops.gpu_qmatvec(qtype, w, xq, 2, n, k)
    rb = oracle.row_bytes(oracle.Q8_1, k)
    y_a = ops.gpu_qmatvec(qtype, w, xq[:rb], 1, n, k)
    y_b = ops.gpu_qmatvec(qtype, w, xq[rb:], 1, n, k)
    ops.check_launch()
    # batch rows are independent (the batched launch may use another summation order, hence a tolerance)
    assert_close(y2[0].cpu().numpy(), y_a[0].cpu().numpy())
    assert_close(y2[1].cpu().numpy(), y_b[0].cpu().numpy())
    rows = np.r_[0:64, n // 2:n // 2 + 64, n - 64:n]
    wrows = w.reshape(n, -1)[torch.from_numpy(rows).cuda()].cpu().numpy()
    assert_close(y2.cpu().numpy()[:, rows], oracle.matvec(qtype, wrows, xq.cpu().numpy(), k))


@pytest.mark.parametrize("qtype,n,k", [(oracle.Q4_K, 14336, 4096), (oracle.Q4_K, 4096, 14336), (oracle.Q6_K, 4096, 14336),
                                       (oracle.Q8_0, 4096, 4096), (oracle.Q4_K, 28672, 8192)])
def test_full_size_every_row_back_to_back(ops, qtype, n, k):
    """Every output row of full-size launches issued back to back over rotating weight buffers
    (so each launch overlaps the tail of the previous one) against float64 products of the
    dequantised operands; the dequantisers are checked bit for bit against the oracle elsewhere."""
    copies = 4
    ws, refs = [], []
    x = torch.from_numpy(oracle.fill_normal(k, 91, 1.0)).cuda()
    xq = ops.gpu_quantize_q8_1(x)
    # Q8_1 decode on the host (small): d * q
    xf = torch.from_numpy(oracle.dequantize(oracle.Q8_1, xq.cpu().numpy(), k).reshape(-1)).cuda().double()
    for c in range(copies):
        wf = torch.randn(n, k, device="cuda", generator=torch.Generator(device="cuda").manual_seed(c)) * 0.02
        w = ops.gpu_quantize_weights(qtype, wf)
        wd = ops.gpu_dequantize(qtype, w, n * k).reshape(n, k)
        refs.append(((wd.double() @ xf), (wd.double().abs() @ xf.abs())))
        ws.append(w)
        del wf, wd
    ys = [torch.empty(1, n, device="cuda") for _ in range(3 * copies)]
    for i, y in enumerate(ys):
        ops.gpu_qmatvec_into(qtype, ws[i % copies], xq, y, 1, n, k)
    ops.check_launch()
    for i, y in enumerate(ys):
        ref, mag = refs[i % copies]
        # Q4_K subtracts dmin*m*s with the fp16-rounded block sums s of Q8_1: bound relative to the term magnitudes
        bound = ABS_TOL + (4e-3 if qtype == oracle.Q4_K else REL_TOL) * mag
        err = (y[0].double() - ref).abs()
        assert bool((err <= bound).all()), f"launch {i}: {int((err > bound).sum())} rows off, max err {float(err.max()):.3e}"


def test_bad_arguments_are_rejected_not_launched(ops):
    w = torch.zeros(4096, dtype=torch.uint8, device="cuda")
    y = torch.zeros(16, device="cuda")
    from nates_recipe_rs_b200._lib import QmmError
    with pytest.raises(QmmError):
        ops.gpu_qmatvec_into(oracle.Q4_K, w, w, y, 1, 1, 100)
    with pytest.raises(ValueError):
        ops.gpu_qmatvec_into(oracle.Q4_K, w[:100], w, y, 1, 1, 256)
    ops.check_launch()
