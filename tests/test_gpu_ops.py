"""The small per-layer operators (norm, rotary + cache append, gated activation, embedding rows, argmax,
scale) one by one against the CPU oracle, through the C ABI.  Needs a B200.

Bars: f32 values within 1e-5 relative (plus 1e-6 absolute) of the oracle; Q8_1 bytes bit-exact given the
kernel's own f32 values (the oracle's quantizer applied to them); decoded embedding rows, argmax indices
and scaled values bit-exact."""
import numpy as np
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu

REL, ABS = 1e-5, 1e-6


@pytest.fixture(scope="module")
def ops():
    if not torch.cuda.is_available():
        pytest.fail("these tests need a CUDA device")
    from nates_recipe_rs_b200 import quant_ops
    return quant_ops


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def close(got, want, what):
    err = np.abs(got.astype(np.float64) - want.astype(np.float64))
    bound = ABS + REL * np.abs(want.astype(np.float64))
    assert (err <= bound).all(), f"{what}: max err {err.max():.3e} at value {np.abs(want).flat[err.argmax()]:.3e}"


@pytest.mark.parametrize("rows,cols", [(1, 256), (3, 4096), (2, 4352), (5, 8192), (1, 96)])
@pytest.mark.parametrize("with_add", [False, True])
@pytest.mark.parametrize("with_gamma", [True, False])
def test_add_rmsnorm_q8_1(ops, rows, cols, with_add, with_gamma):
    x = oracle.fill_normal(rows * cols, 3, 1.5).reshape(rows, cols)
    add = oracle.fill_normal(rows * cols, 4, 0.7).reshape(rows, cols) if with_add else None
    gamma = (oracle.fill_normal(cols, 5, 0.1) + np.float32(1.0)) if with_gamma else None
    xd = dev(x)
    xq = torch.zeros(rows * oracle.row_bytes(oracle.Q8_1, cols), dtype=torch.uint8, device="cuda")
    out = torch.full((rows, cols), float("nan"), device="cuda")
    ops.gpu_rmsnorm_q8_1_into(xd, dev(gamma) if with_gamma else None, xq, rows, cols, 1e-6, add=dev(add) if with_add else None, out_f32=out)
    ops.check_launch()
    xs = x + add if with_add else x               # one correctly rounded f32 addition, as on the device
    assert np.array_equal(xd.cpu().numpy(), xs), "residual not updated in place"
    got = out.cpu().numpy()
    close(got, oracle.rmsnorm(xs, gamma, 1e-6), "normalised values")
    assert np.array_equal(xq.cpu().numpy(), oracle.quantize(oracle.Q8_1, got).reshape(-1)), "Q8_1 bytes"


@pytest.mark.parametrize("batch,nq,nkv,hd,pos", [(1, 4, 2, 64, 0), (3, 32, 8, 128, 17), (2, 8, 8, 32, 2047), (1, 64, 8, 128, 4095)])
def test_rope_kv_append(ops, batch, nq, nkv, hd, pos):
    cap = pos + 2
    theta = 10000.0
    qkv = oracle.fill_normal(batch * (nq + 2 * nkv) * hd, 21, 1.0).reshape(batch, (nq + 2 * nkv) * hd)
    qd = dev(qkv)
    kc = torch.zeros(batch, cap, nkv, hd, dtype=torch.float16, device="cuda")
    vc = torch.zeros_like(kc)
    ops.gpu_rope_kv_append(qd, kc, vc, batch, nq, nkv, hd, pos, cap, theta)
    ops.check_launch()
    got = qd.cpu().numpy()
    for b in range(batch):
        q_want = oracle.rope_neox(qkv[b, :nq * hd], hd, nq, pos, theta).reshape(-1)
        k_want = oracle.rope_neox(qkv[b, nq * hd:(nq + nkv) * hd], hd, nkv, pos, theta).reshape(-1)
        # the angle pos * theta^(-2i/hd) is evaluated in f32 on the device: at position 4095 its rounding
        # and that of the f32 power move sin/cos by a few 1e-7 per unit of position, so the bound scales with it
        tol = 2e-6 + 5e-7 * pos
        assert np.abs(got[b, :nq * hd] - q_want).max() <= tol * max(1.0, np.abs(q_want).max()), "rotated q"
        kgot = kc[b, pos].float().cpu().numpy().reshape(-1)
        assert np.abs(kgot - k_want).max() <= tol * np.abs(k_want).max() + 2.0 ** -10 * np.abs(k_want).max(), "rotated k in the cache (fp16)"
        vgot = vc[b, pos].cpu().numpy().reshape(-1)
        assert np.array_equal(vgot, qkv[b, (nq + nkv) * hd:].astype(np.float16)), "v in the cache"
        assert np.array_equal(got[b, nq * hd:], qkv[b, nq * hd:]), "k and v of the row are left as they were"
    if pos > 0:
        assert float(kc[:, :pos].abs().max()) == 0.0 and float(vc[:, pos + 1:].abs().max()) == 0.0, "other positions untouched"


@pytest.mark.parametrize("rows,half", [(1, 32), (2, 14336), (5, 2048)])
@pytest.mark.parametrize("act", [0, 1])
def test_glu_act_q8_1(ops, rows, half, act):
    gu = oracle.fill_normal(rows * 2 * half, 31, 2.0).reshape(rows, 2 * half)
    xq = torch.zeros(rows * oracle.row_bytes(oracle.Q8_1, half), dtype=torch.uint8, device="cuda")
    out = torch.full((rows, half), float("nan"), device="cuda")
    ops.gpu_glu_act_q8_1_into(dev(gu), xq, rows, half, act, out_f32=out)
    ops.check_launch()
    got = out.cpu().numpy()
    fn = oracle.gelu_mul if act == 0 else oracle.silu_mul
    want = fn(gu[:, :half].copy(), gu[:, half:].copy())
    # SiLU uses the fast exponential (2 ulp): 1e-5 relative still holds with the absolute floor below
    err = np.abs(got.astype(np.float64) - want.astype(np.float64))
    assert (err <= 2e-6 + 1e-5 * np.abs(want)).all(), f"max err {err.max():.3e}"
    assert np.array_equal(xq.cpu().numpy(), oracle.quantize(oracle.Q8_1, got).reshape(-1)), "Q8_1 bytes"


@pytest.mark.parametrize("qtype", [oracle.Q8_0, oracle.Q4_K, oracle.Q6_K])
def test_embed_rows_bit_exact(ops, qtype):
    vocab, hidden = 300, 1024
    table = oracle.quantize(qtype, oracle.fill_normal(vocab * hidden, 41, 0.02).reshape(vocab, hidden))
    toks = np.array([0, 299, 17, 500, -3], dtype=np.int32)       # the last two are clamped to the table
    x = torch.full((len(toks), hidden), float("nan"), device="cuda")
    ops.gpu_embed_rows_into(qtype, dev(table), dev(toks), x, len(toks), hidden, vocab)
    ops.check_launch()
    want = oracle.dequantize(qtype, table, hidden)[np.clip(toks, 0, vocab - 1)]
    assert np.array_equal(x.cpu().numpy().view(np.uint32), want.view(np.uint32))


def test_argmax_rows(ops):
    rng = np.random.default_rng(5)
    for batch, vocab in [(1, 100), (4, 128256), (3, 256000), (2, 255)]:
        lg = rng.normal(size=(batch, vocab)).astype(np.float32)
        lg[0, vocab // 2] = 50.0
        if batch > 1:
            lg[1, [7, vocab - 1]] = 60.0                         # a tie: the lowest index wins
        idx, val = ops.gpu_argmax_rows(dev(lg))
        ops.check_launch()
        assert np.array_equal(idx.cpu().numpy(), lg.argmax(axis=1).astype(np.int32))
        assert np.array_equal(val.cpu().numpy(), lg.max(axis=1))


def test_scale_f32(ops):
    x = oracle.fill_normal(100003, 51, 3.0)
    xd = dev(x)
    ops.gpu_scale_f32_inplace(xd, 0.37)
    ops.check_launch()
    assert np.array_equal(xd.cpu().numpy(), x * np.float32(0.37))


def test_entries_reject_bad_arguments(ops):
    from nates_recipe_rs_b200._lib import lib
    L = lib()
    assert L.launch_add_rmsnorm_q8_1(None, None, None, 16, None, 1, 256, 1e-6, None) == -1
    assert L.launch_add_rmsnorm_q8_1(16, None, None, 16, None, 1, 100, 1e-6, None) == -2
    assert L.launch_add_rmsnorm_q8_1(16, None, None, 16, None, 1, 8192 + 32, 1e-6, None) == -3
    assert L.launch_glu_act_q8_1(16, 16, None, 1, 48, 0, None) == -2
    assert L.launch_glu_act_q8_1(16, 16, None, 1, 64, 7, None) == -3
    assert L.launch_rope_kv_append(16, 16, 16, 1, 4, 2, 64, 5, 5, 1e4, None) == -2
    assert L.launch_embed_rows(77, 16, 16, 16, 1, 256, 10, None) == -5
    assert L.launch_argmax_rows(16, None, 16, None, 1, 10, None) == -1
    assert L.launch_scale_f32(None, 1.0, 5, None) == -1


@pytest.mark.parametrize("t,nqh,nkv,hd,prefix", [(1, 4, 2, 64, 1), (70, 8, 2, 128, 70), (130, 4, 4, 32, 0), (200, 8, 2, 128, 77), (300, 16, 4, 96, 300),
                                                  (129, 2, 1, 256, 64), (513, 4, 1, 128, 400), (64, 4, 2, 64, 10)])
def test_sequence_attention_matches_oracle(ops, t, nqh, nkv, hd, prefix):
    """launch_attn_prefill (the upstream's gqa_masked_attn: causal below `prefix`, bidirectional from it on) against the
    oracle's double-precision loops.  q, k, v and the probabilities pass through f16 on the tensor cores (2^-11 each)."""
    rng = np.random.default_rng(t * 7 + hd)
    q = rng.normal(size=(t, nqh * hd)).astype(np.float32)
    k = rng.normal(size=(t, nkv * hd)).astype(np.float32)
    v = rng.normal(size=(t, nkv * hd)).astype(np.float32)
    scale = 1.0 / np.sqrt(hd)
    want = oracle.attn_prefill(q, k, v, nqh, nkv, hd, prefix, scale)
    out = torch.full((t, nqh * hd), float("nan"), device="cuda")
    ops.gpu_gqa_attn_into(torch.from_numpy(q).cuda(), torch.from_numpy(k).cuda(), torch.from_numpy(v).cuda(), out, t, nqh, nkv, hd, prefix, scale)
    ops.check_launch()
    got = out.cpu().numpy()
    assert not np.isnan(got).any()
    assert np.abs(got - want).max() <= 1e-4 + 4e-3 * np.abs(want).max()
    # twice: identical bits
    out2 = torch.empty_like(out)
    ops.gpu_gqa_attn_into(torch.from_numpy(q).cuda(), torch.from_numpy(k).cuda(), torch.from_numpy(v).cuda(), out2, t, nqh, nkv, hd, prefix, scale)
    assert torch.equal(out, out2)
    # k and v handed over as f16 (the rows of a KV cache): the values the f32 form rounds to, so the same bits
    out3 = torch.full_like(out, float("nan"))
    ops.gpu_gqa_attn_into(torch.from_numpy(q).cuda(), torch.from_numpy(k).cuda().half(), torch.from_numpy(v).cuda().half(), out3, t, nqh, nkv, hd, prefix, scale)
    ops.check_launch()
    assert torch.equal(out, out3)


@pytest.mark.parametrize("t_kv,q_pos0,t,nqh,nkv,hd,prefix", [(200, 64, 136, 8, 2, 128, 200), (200, 77, 100, 8, 2, 128, 200), (513, 500, 13, 4, 1, 64, 513),
                                                          (300, 100, 150, 4, 4, 32, 120), (130, 129, 1, 2, 1, 256, 130)])
def test_sequence_attention_continuing_a_cache(ops, t_kv, q_pos0, t, nqh, nkv, hd, prefix):
    """Queries that continue a sequence whose earlier keys and values sit in an f16 cache: row for row the bits of one
    call over the whole sequence (also when the piece does not start on a tile of 64 positions)."""
    rng = np.random.default_rng(t_kv + q_pos0)
    q = torch.from_numpy(rng.normal(size=(t_kv, nqh * hd)).astype(np.float32)).cuda()
    k = torch.from_numpy(rng.normal(size=(t_kv, nkv * hd)).astype(np.float32)).cuda().half()
    v = torch.from_numpy(rng.normal(size=(t_kv, nkv * hd)).astype(np.float32)).cuda().half()
    scale = 1.0 / np.sqrt(hd)
    whole = torch.empty(t_kv, nqh * hd, device="cuda")
    ops.gpu_gqa_attn_into(q, k, v, whole, t_kv, nqh, nkv, hd, prefix, scale)
    # the piece sees only the keys up to its own end when it is causal throughout; with bidirectional positions it needs all
    kv_len = t_kv if prefix < t_kv else q_pos0 + t
    piece = torch.full((t, nqh * hd), float("nan"), device="cuda")
    ops.gpu_gqa_attn_at_into(q[q_pos0:q_pos0 + t].contiguous(), k[:kv_len].contiguous(), v[:kv_len].contiguous(), piece, t, kv_len, q_pos0, nqh, nkv, hd,
                             prefix, scale)
    ops.check_launch()
    assert torch.equal(piece, whole[q_pos0:q_pos0 + t])
    from nates_recipe_rs_b200._lib import lib
    L = lib()
    assert L.launch_attn_prefill_f16kv_at(q.data_ptr(), k.data_ptr(), v.data_ptr(), piece.data_ptr(), t, q_pos0 + t - 1, q_pos0, nqh, nkv, hd, prefix, 1.0, None) == -2


def test_sequence_attention_rejects_bad_arguments(ops):
    from nates_recipe_rs_b200._lib import lib
    L = lib()
    x = torch.zeros(64 * 64, device="cuda")
    o = torch.zeros(64 * 64, device="cuda")
    p = lambda a: a.data_ptr()
    assert L.launch_attn_prefill(p(x), p(x), p(x), p(o), 4, 4, 3, 64, 0, 1.0, None) == -2      # heads do not divide
    assert L.launch_attn_prefill(p(x), p(x), p(x), p(x), 4, 4, 2, 64, 0, 1.0, None) == -2      # out aliases an input
    assert L.launch_attn_prefill(p(x), p(x), p(x), p(o), 4, 4, 2, 80, 0, 1.0, None) == -3      # head_dim not instantiated
    assert L.launch_attn_prefill(None, p(x), p(x), p(o), 4, 4, 2, 64, 0, 1.0, None) == -1
    assert L.launch_attn_prefill_f16kv(p(x), p(x), None, p(o), 4, 4, 2, 64, 0, 1.0, None) == -1
    assert L.launch_attn_prefill_f16kv(p(x), p(x), p(x), p(o), 4, 4, 2, 80, 0, 1.0, None) == -3
    ops.check_launch()
