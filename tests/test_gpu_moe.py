"""Mixture-of-experts branch on the device (router + top-k, experts chosen by device-side selectors, weighted
sum) against a numpy composition of the CPU oracle's pieces, through the C ABI.  Needs a B200."""
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


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def ref_router(x, gain, rw, top_k, scale, eps):
    x = x.astype(np.float64)
    r = x / np.sqrt((x * x).mean(axis=1, keepdims=True) + eps) * scale * (gain.astype(np.float64) if gain is not None else 1.0)
    logits = r @ rw.astype(np.float64).T
    p = np.exp(logits - logits.max(axis=1, keepdims=True))
    p /= p.sum(axis=1, keepdims=True)
    sel = np.argsort(-p, axis=1, kind="stable")[:, :top_k]
    w = np.take_along_axis(p, sel, axis=1)
    return sel.astype(np.int32), (w / w.sum(axis=1, keepdims=True)).astype(np.float32), p


@pytest.mark.parametrize("m,hidden,n_experts,top_k,with_gain", [(1, 2816, 128, 8, True), (4, 1024, 64, 2, False), (3, 4096, 256, 4, True),
                                                                (2, 512, 8, 8, False), (1, 256, 3, 1, True)])
def test_router_topk(ops, m, hidden, n_experts, top_k, with_gain):
    x = oracle.fill_normal(m * hidden, 1, 1.0).reshape(m, hidden)
    gain = (oracle.fill_normal(hidden, 2, 0.2) + np.float32(1.0)) if with_gain else None
    rw = oracle.fill_normal(n_experts * hidden, 3, 0.05).reshape(n_experts, hidden)
    scale = 1.0 / np.sqrt(hidden)
    sel, w, probs = ops.gpu_moe_router_topk(dev(x), dev(rw), top_k, scale=scale, eps=1e-6, gain=dev(gain) if with_gain else None, want_probs=True)
    ops.check_launch()
    want_sel, want_w, want_p = ref_router(x, gain, rw, top_k, scale, 1e-6)
    assert np.abs(probs.cpu().numpy() - want_p).max() <= 1e-5 * want_p.max() + 1e-7
    got_sel = sel.cpu().numpy()
    # the order may only differ where two probabilities are closer than the f32 evaluation can tell apart
    for p in range(m):
        if not np.array_equal(got_sel[p], want_sel[p]):
            assert np.abs(np.sort(want_p[p, got_sel[p]]) - np.sort(want_p[p, want_sel[p]])).max() <= 1e-6, (p, got_sel[p], want_sel[p])
    gp = np.take_along_axis(want_p, got_sel.astype(np.int64), axis=1)
    assert np.abs(w.cpu().numpy() - gp / gp.sum(axis=1, keepdims=True)).max() <= 1e-5
    assert np.abs(w.cpu().numpy().sum(axis=1) - 1.0).max() <= 1e-5


def test_router_ties_take_the_lowest_index(ops):
    hidden, n_experts = 256, 16
    x = oracle.fill_normal(hidden, 7, 1.0).reshape(1, hidden)
    row = oracle.fill_normal(hidden, 8, 0.05)
    rw = np.tile(row, (n_experts, 1))          # every expert has the same logit
    sel, w = ops.gpu_moe_router_topk(dev(x), dev(rw), 4)
    assert sel.cpu().numpy().tolist() == [[0, 1, 2, 3]]
    assert np.allclose(w.cpu().numpy(), 0.25)


@pytest.mark.parametrize("m,hidden,ffn_e,n_experts,top_k,act,tgu,tdn", [
    (1, 1024, 512, 8, 2, 0, oracle.Q4_K, oracle.Q6_K),
    (3, 2048, 768, 16, 4, 1, oracle.Q4_K, oracle.Q4_K),
    (2, 512, 256, 4, 4, 0, oracle.Q8_0, oracle.Q8_0),
    (5, 2816 - 2816 % 256 + 256, 704 - 704 % 256 + 256, 32, 8, 0, oracle.Q4_K, oracle.Q6_K)])   # 40 (token, slot) pairs: more than one launch per projection
def test_expert_branch(ops, m, hidden, ffn_e, n_experts, top_k, act, tgu, tdn):
    rng = np.random.default_rng(11)
    gu_bank = [oracle.quantize(tgu, oracle.fill_normal(2 * ffn_e * hidden, 100 + e, 0.02).reshape(2 * ffn_e, hidden)) for e in range(n_experts)]
    dn_bank = [oracle.quantize(tdn, oracle.fill_normal(hidden * ffn_e, 500 + e, 0.02).reshape(hidden, ffn_e)) for e in range(n_experts)]
    x = oracle.fill_normal(m * hidden, 5, 1.0).reshape(m, hidden)
    xq = oracle.quantize(oracle.Q8_1, x)
    sel = np.stack([rng.permutation(n_experts)[:top_k] for _ in range(m)]).astype(np.int32)
    w = rng.random((m, top_k)).astype(np.float32)
    w /= w.sum(axis=1, keepdims=True)
    scale = (rng.random(n_experts) + 0.5).astype(np.float32)
    out = torch.full((m, hidden), float("nan"), device="cuda")
    ops.gpu_moe_experts_into(tgu, dev(np.stack(gu_bank)), tdn, dev(np.stack(dn_bank)), dev(xq), dev(sel), dev(w), out, hidden, ffn_e, act,
                             expert_scale=dev(scale))
    ops.check_launch()
    want = np.zeros((m, hidden), dtype=np.float64)
    fn = oracle.gelu_mul if act == 0 else oracle.silu_mul
    for p in range(m):
        for j in range(top_k):
            e = int(sel[p, j])
            gu = oracle.matvec(tgu, gu_bank[e], xq[p], hidden)[0]
            ea = oracle.quantize(oracle.Q8_1, fn(gu[:ffn_e].copy(), gu[ffn_e:].copy()))
            want[p] += float(w[p, j]) * float(scale[e]) * oracle.matvec(tdn, dn_bank[e], ea, ffn_e)[0].astype(np.float64)
    got = out.cpu().numpy()
    assert not np.isnan(got).any()
    # activations differ by an ulp between device and host, which may flip a Q8_1 code of the expert's hidden
    # values: bound relative to the output scale
    assert np.abs(got - want).max() <= 3e-3 * np.abs(want).max(), float(np.abs(got - want).max() / np.abs(want).max())


def test_moe_entries_reject_bad_arguments(ops):
    from nates_recipe_rs_b200._lib import lib
    L = lib()
    assert L.launch_moe_router_topk(None, None, 16, 1, 256, 8, 2, 1.0, 1e-6, 16, 16, None, None) == -1
    assert L.launch_moe_router_topk(16, None, 16, 1, 256, 8, 9, 1.0, 1e-6, 16, 16, None, None) == -2      # top_k > n_experts
    assert L.launch_moe_router_topk(16, None, 16, 1, 256, 300, 2, 1.0, 1e-6, 16, 16, None, None) == -3
    assert L.qmm_moe_scratch_bytes(1, 2, 256, 100) == -2
    assert L.launch_moe_experts(12, 16, 24, 12, 16, 32, 16, 16, 16, None, 16, 16, 1, 2, 256, 256, 0, None) == -4     # stride not a multiple of 16
