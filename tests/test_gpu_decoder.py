"""Decode engine against a numpy composition of the CPU oracle's pieces on the engine's own
packed weights.  Needs a B200."""
import numpy as np
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu


def tiny_cfg(dec, **kw):
    c = dict(n_layers=2, hidden=256, n_q_heads=4, n_kv_heads=2, head_dim=64, ffn=512, vocab=1024, ctx_len=48,
             rope_theta=10000.0, rms_eps=1e-6, act=dec.ACT_GELU_TANH, type_attn_qk=oracle.Q4_K, type_attn_v=oracle.Q6_K,
             type_attn_o=oracle.Q4_K, type_ffn_gate_up=oracle.Q4_K, type_ffn_down=oracle.Q6_K, type_head=oracle.Q6_K,
             max_batch=3, tp_rank=0, tp_size=1, seed=77)
    c.update(kw)
    return dec.DecoderConfig(**c)


class RefModel:
    """Straight-loop restatement of one decode step from oracle pieces."""

    def __init__(self, d, dec):
        c = d.cfg
        self.c, self.dec = c, dec
        H = c.hidden
        f32 = lambda b: b.view(np.float32)
        self.layers = []
        for l in range(c.n_layers):
            self.layers.append(dict(
                attn_norm=f32(d.tensor(l, dec.T_ATTN_NORM)), ffn_norm=f32(d.tensor(l, dec.T_FFN_NORM)),
                wqk=d.tensor(l, dec.T_WQK), wv=d.tensor(l, dec.T_WV), wo=d.tensor(l, dec.T_WO), wgu=d.tensor(l, dec.T_WGU),
                wdown=d.tensor(l, dec.T_WDOWN)))
        self.final_norm = f32(d.tensor(-1, dec.T_FINAL_NORM))
        self.head = d.tensor(-1, dec.T_HEAD)
        hd = c.head_dim
        self.kc = np.zeros((c.n_layers, c.max_batch, c.ctx_len, c.n_kv_heads, hd), dtype=np.float16)
        self.vc = np.zeros_like(self.kc)

    def q8(self, v):
        return oracle.quantize(oracle.Q8_1, v.reshape(1, -1)).reshape(-1)

    def step(self, b, token, pos):
        c = self.c
        H, hd, nq, nkv = c.hidden, c.head_dim, c.n_q_heads, c.n_kv_heads
        rb = oracle.row_bytes(c.type_head, H)
        x = oracle.dequantize(c.type_head, self.head[token * rb:(token + 1) * rb], H).reshape(-1).copy()
        for l, L in enumerate(self.layers):
            xq = self.q8(oracle.rmsnorm(x[None], L["attn_norm"], c.rms_eps)[0])
            qk = oracle.matvec(c.type_attn_qk, L["wqk"], xq, H)[0]
            v = oracle.matvec(c.type_attn_v, L["wv"], xq, H)[0]
            q = oracle.rope_neox(qk[:nq * hd], hd, nq, pos, c.rope_theta)           # rows = heads of one token at `pos`
            k = oracle.rope_neox(qk[nq * hd:], hd, nkv, pos, c.rope_theta)
            self.kc[l, b, pos] = k.reshape(nkv, hd).astype(np.float16)
            self.vc[l, b, pos] = v.reshape(nkv, hd).astype(np.float16)
            att = oracle.attn_decode(q, self.kc[l, b], self.vc[l, b], nq, nkv, hd, pos + 1)
            x = x + oracle.matvec(c.type_attn_o, L["wo"], self.q8(att), nq * hd)[0]
            xq = self.q8(oracle.rmsnorm(x[None], L["ffn_norm"], c.rms_eps)[0])
            gu = oracle.matvec(c.type_ffn_gate_up, L["wgu"], xq, H)[0]
            act = oracle.gelu_mul if c.act == self.dec.ACT_GELU_TANH else oracle.silu_mul
            hq = self.q8(act(gu[:c.ffn], gu[c.ffn:]))
            x = x + oracle.matvec(c.type_ffn_down, L["wdown"], hq, c.ffn)[0]
        xq = self.q8(oracle.rmsnorm(x[None], self.final_norm, c.rms_eps)[0])
        return oracle.matvec(c.type_head, self.head, xq, H)[0]


@pytest.fixture(scope="module")
def dec():
    if not torch.cuda.is_available():
        pytest.fail("these tests need a CUDA device")
    from nates_recipe_rs_b200 import decoder
    return decoder


def test_model_bytes_are_the_seeded_quantized_normal(dec):
    """The engine's weights are reproducible on the CPU: fill_normal(seed, index) quantized by the oracle."""
    d = dec.Decoder(tiny_cfg(dec))
    c = d.cfg
    seed = lambda layer, which: (c.seed * 1000003 + (layer + 1) * 64 + which) & ((1 << 64) - 1)
    got = d.tensor(1, dec.T_WDOWN)
    want = oracle.quantize(c.type_ffn_down, oracle.fill_normal(c.hidden * c.ffn, seed(1, 8), 0.02).reshape(c.hidden, c.ffn)).reshape(-1)
    assert np.array_equal(got, want)
    got = d.tensor(0, dec.T_WQK)
    rows_q = c.n_q_heads * c.head_dim
    wq = oracle.quantize(c.type_attn_qk, oracle.fill_normal(rows_q * c.hidden, seed(0, 1), 0.02).reshape(rows_q, c.hidden)).reshape(-1)
    assert np.array_equal(got[:wq.size], wq)
    g = d.tensor(0, dec.T_ATTN_NORM).view(np.float32)
    assert np.array_equal(g, oracle.fill_normal(c.hidden, seed(0, 0), 0.1) + np.float32(1.0))
    d.close()


FIRST_POSITION_TOL = 1e-5   # of the logit scale: with one position in the context no rounding order differs enough to flip a code


@pytest.mark.parametrize("act,wide", [("gelu", False), ("silu", False), ("gelu", True), ("silu", True), ("gelu", "odd")])
def test_decode_steps_match_reference(dec, act, wide):
    """wide: five sequences and 2048-wide layers, so that every projection of the engine takes the
    tensor-core matvec (Q4_K and Q6_K, one and two K chunks); otherwise the dp4a kernel.
    odd: a hidden width (17 * 256) that no block size of the norm kernel divides."""
    kw = dict(act=dec.ACT_GELU_TANH if act == "gelu" else dec.ACT_SILU)
    if wide == "odd":
        kw.update(n_layers=1, hidden=4352, vocab=1024, max_batch=2)
        wide = False
    elif wide:
        kw.update(n_layers=1, hidden=2048, n_q_heads=16, n_kv_heads=4, head_dim=128, ffn=4096, vocab=2048, max_batch=5)
    d = dec.Decoder(tiny_cfg(dec, **kw))
    c = d.cfg
    ref = RefModel(d, dec)
    from nates_recipe_rs_b200 import quant_ops as ops
    B = c.max_batch
    toks = np.array([5, 700, 123, 1999, 42][:B], dtype=np.int32)
    logits = torch.empty(B, c.vocab, device="cuda")
    for pos in range(3 if wide else 6):
        d.tokens.copy_(torch.from_numpy(toks))
        d.step(B, pos, logits)
        ops.check_launch()
        got = logits.cpu().numpy()
        nxt = d.next_tokens.cpu().numpy()
        new = []
        for b in range(B):
            want = ref.step(b, int(toks[b]), pos)
            scale = np.abs(want).max()
            bound = FIRST_POSITION_TOL if pos == 0 else 2e-2
            assert np.abs(got[b] - want).max() <= bound * scale, (pos, b, float(np.abs(got[b] - want).max()), float(scale))
            assert int(nxt[b]) == int(np.argmax(got[b]))
            top2 = np.sort(want)[-2:]
            if top2[1] - top2[0] > 4e-2 * scale:
                assert int(nxt[b]) == int(np.argmax(want))
            new.append(int(np.argmax(want)))      # both sides continue from the reference's token
        toks = np.array(new, dtype=np.int32)
    d.close()


def test_step_rejects_bad_arguments(dec):
    d = dec.Decoder(tiny_cfg(dec))
    from nates_recipe_rs_b200._lib import QmmError
    with pytest.raises(QmmError):
        d.step(4, 0)            # batch above max_batch
    with pytest.raises(QmmError):
        d.step(1, 48)           # position beyond the context
    d.close()
    for bad in (dict(head_dim=80, n_q_heads=16, n_kv_heads=2), dict(head_dim=16, n_q_heads=16, n_kv_heads=2), dict(hidden=8448)):
        with pytest.raises(QmmError):    # head_dim must be a multiple of 32; hidden at most 8192
            dec.Decoder(tiny_cfg(dec, **bad))


@pytest.mark.parametrize("batch,nqh,nkv,hd,length", [(1, 4, 2, 64, 1), (2, 8, 2, 128, 70), (3, 32, 8, 128, 300), (1, 8, 8, 32, 129),
                                                     (4, 8, 2, 128, 70), (5, 32, 8, 128, 300), (4, 8, 8, 64, 129), (6, 64, 8, 128, 1),
                                                     (4, 16, 4, 96, 200),
                                                     # more work items than persistent CTAs: several chunks per CTA through the ring of buffers
                                                     (16, 32, 8, 128, 700), (8, 8, 1, 128, 4096), (4, 4, 2, 256, 100), (32, 8, 1, 128, 1300)])
def test_attention_entry_matches_oracle(dec, batch, nqh, nkv, hd, length):
    """launch_attn_decode through the C ABI against the oracle's straight-loop attention.  From four
    sequences on the library computes scores and outputs on the f16 tensor cores with q and the
    probabilities rounded to f16 (2^-11 relative each), hence the wider bound there."""
    from nates_recipe_rs_b200._lib import check, lib
    L = lib()
    cap = length + 5
    rng = np.random.default_rng(batch * 1000 + length)
    qkv = rng.normal(size=(batch, (nqh + 2 * nkv) * hd)).astype(np.float32)
    kc = rng.normal(size=(batch, cap, nkv, hd)).astype(np.float16)
    vc = rng.normal(size=(batch, cap, nkv, hd)).astype(np.float16)
    dq, dk, dv = (torch.from_numpy(a).cuda() for a in (qkv, kc, vc))
    nbytes = L.qmm_attn_decode_scratch_bytes(batch, nqh, hd, length)
    scratch = torch.empty(nbytes // 4, dtype=torch.float32, device="cuda")
    out = torch.full((batch, nqh * hd), float("nan"), device="cuda")
    q8 = torch.zeros(batch * (nqh * hd // 32) * 36, dtype=torch.uint8, device="cuda")
    check(L.launch_attn_decode(dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), scratch.data_ptr(), out.data_ptr(), q8.data_ptr(), batch, nqh, nkv,
                               hd, length, cap, torch.cuda.current_stream().cuda_stream), "launch_attn_decode")
    got = out.cpu().numpy()
    for b in range(batch):
        want = oracle.attn_decode(qkv[b, :nqh * hd].reshape(nqh, hd), kc[b], vc[b], nqh, nkv, hd, length).reshape(-1)
        rel = 1e-3 if batch < 4 else 4e-3
        assert np.abs(got[b] - want).max() <= 1e-4 + rel * np.abs(want).max()
    # the Q8_1 output is the library's own quantization of the f32 output
    from nates_recipe_rs_b200 import quant_ops as ops
    assert torch.equal(q8, ops.gpu_quantize_q8_1(out))


def test_gguf_round_trip_gives_the_same_decoder(dec, tmp_path):
    """The seeded model written as a GGUF file and loaded back decodes bit-identically; a tensor-parallel
    rank that loads its shard from the file holds the same bytes as the seeded shard."""
    from nates_recipe_rs_b200 import gguf, quant_ops as ops
    cfg = tiny_cfg(dec, n_layers=2, max_batch=2)
    a = dec.Decoder(cfg)
    path = tmp_path / "tiny.gguf"
    a.export_gguf(path, "gemma")
    with gguf.GgufFile(path) as f:
        assert f.meta_int("gemma.block_count") == 2 and f.meta_int("gemma.embedding_length") == cfg.hidden
        assert f.find("blk.1.ffn_down.weight") >= 0 and f.find("output.weight") == -1      # tied head
        buf = torch.zeros(f.info(f.find("blk.0.attn_v.weight"))["bytes"], dtype=torch.uint8, device="cuda")
        f.upload("blk.0.attn_v.weight", buf)
        assert np.array_equal(buf.cpu().numpy(), a.tensor(0, dec.T_WV))
    b = dec.Decoder(dec.DecoderConfig(max_batch=2, ctx_len=0, tp_rank=0, tp_size=1), gguf_path=path)
    for which in (dec.T_ATTN_NORM, dec.T_WQK, dec.T_WV, dec.T_WO, dec.T_FFN_NORM, dec.T_WGU, dec.T_WDOWN):
        assert np.array_equal(a.tensor(1, which), b.tensor(1, which)), which
    assert np.array_equal(a.tensor(-1, dec.T_HEAD), b.tensor(-1, dec.T_HEAD))
    toks = torch.tensor([5, 700], dtype=torch.int32, device="cuda")
    la, lb = torch.empty(2, cfg.vocab, device="cuda"), torch.empty(2, cfg.vocab, device="cuda")
    for pos in range(4):
        for d, lg in ((a, la), (b, lb)):
            d.tokens.copy_(toks)
            d.step(2, pos, lg)
        ops.check_launch()
        assert torch.equal(la, lb), pos
        assert torch.equal(a.next_tokens, b.next_tokens)
        toks = a.next_tokens.clone()
    a.close()
    b.close()
    # rank 1 of 2: row ranges of Q/K/V/gate/up/head, whole-block column ranges of O and down
    kw = dict(n_layers=2, max_batch=2, tp_rank=1, tp_size=2, hidden=512, n_q_heads=8, n_kv_heads=2, head_dim=64, ffn=1024)
    full = dec.Decoder(tiny_cfg(dec, **{**kw, "tp_rank": 0, "tp_size": 1}))
    full.export_gguf(path, "llama")
    full.close()
    seeded = dec.Decoder.__new__(dec.Decoder)      # shards without wiring peers: only the tensors are compared
    loaded = dec.Decoder.__new__(dec.Decoder)
    import ctypes as C
    L = dec._bind()
    from nates_recipe_rs_b200._lib import check
    for obj, make in ((seeded, lambda h: L.qmm_decoder_create(C.byref(tiny_cfg(dec, **kw)), C.byref(h))),
                      (loaded, lambda h: L.qmm_decoder_create_from_gguf(str(path).encode(), 2, 0, 1, 2, C.byref(h)))):
        obj.L, obj.h, obj.cfg = L, C.c_void_p(), None
        check(make(obj.h), "create shard")
    for layer, which in [(0, dec.T_WQK), (0, dec.T_WV), (1, dec.T_WO), (1, dec.T_WGU), (0, dec.T_WDOWN), (-1, dec.T_HEAD), (-1, dec.T_EMBED),
                         (1, dec.T_FFN_NORM), (-1, dec.T_FINAL_NORM)]:
        assert np.array_equal(seeded.tensor(layer, which), loaded.tensor(layer, which)), (layer, which)
    seeded.close()
    loaded.close()


def test_gguf_decoder_rejects_what_it_cannot_run(dec, tmp_path):
    from nates_recipe_rs_b200 import gguf
    from nates_recipe_rs_b200._lib import QmmError
    path = tmp_path / "bad.gguf"
    w = gguf.GgufWriter(path)
    w.meta("general.architecture", "llama").meta("llama.block_count", 1).meta("llama.embedding_length", 256)
    w.tensor("token_embd.weight", oracle.Q6_K, [256, 4], oracle.quantize(oracle.Q6_K, oracle.fill_normal(1024, 1, 0.02).reshape(4, 256)))
    w.finish()
    with pytest.raises(QmmError) as e:       # the layer tensors are missing
        dec.Decoder(dec.DecoderConfig(max_batch=1, ctx_len=16, tp_rank=0, tp_size=1), gguf_path=path)
    assert e.value.status == -9
    with pytest.raises(QmmError) as e:
        dec.Decoder(dec.DecoderConfig(max_batch=1, ctx_len=16, tp_rank=0, tp_size=1), gguf_path=tmp_path / "none.gguf")
    assert e.value.status == -8


def test_fused_and_separate_launches_agree(dec):
    """Batch 1-2 on one GPU: the levels of the tunable decoder_fuse (Q|K and V as one job list; norms and
    gated activations built inside the matvec launches) against every operator as its own launch (0)."""
    from nates_recipe_rs_b200 import quant_ops as ops
    from nates_recipe_rs_b200._lib import check, lib
    cfg = tiny_cfg(dec, n_layers=3, hidden=1024, n_q_heads=8, n_kv_heads=2, head_dim=64, ffn=2048, vocab=2048, max_batch=2)
    results = []
    for fuse in (3, 2, 1, 0):
        check(lib().qmm_tune(b"decoder_fuse", fuse), "qmm_tune")
        try:
            d = dec.Decoder(cfg)
            toks = torch.tensor([9, 1500], dtype=torch.int32, device="cuda")
            seq = []
            for pos in range(5):
                lg = torch.empty(2, cfg.vocab, device="cuda")
                d.tokens.copy_(toks)
                d.step(2, pos, lg)
                ops.check_launch()
                seq.append(lg.cpu().numpy())
                toks = torch.tensor([100 + pos, 200 + pos], dtype=torch.int32, device="cuda")
            results.append(seq)
            d.close()
        finally:
            check(lib().qmm_tune(b"decoder_fuse", 1), "qmm_tune")
    for level, seq in zip((3, 2, 1), results[:3]):
        for pos, (a, b) in enumerate(zip(seq, results[3])):
            scale = np.abs(b).max()
            assert np.abs(a - b).max() <= (1e-5 if pos == 0 else 2e-2) * scale, (level, pos, float(np.abs(a - b).max()), float(scale))


def ref_prefill(ref, tokens):
    """The prompt path restated from oracle pieces: every projection a quantized dense over all positions (bf16 GEMM
    route from 64 rows on - fused for Q4_K, on the decoded bf16 matrix for the other types - and the Q8_1 matvec route
    below), attention over the whole sequence, causal.  Fills the reference cache of sequence 0 and returns the
    logits of the last position."""
    c = ref.c
    t = len(tokens)
    H, hd, nq, nkv, ffn = c.hidden, c.head_dim, c.n_q_heads, c.n_kv_heads, c.ffn

    def dense(qt, w, x, k):
        via = "bf16" if (t >= 64 and k % 256 == 0) else "q8_1"
        return oracle.dense(qt, w, x, None, "linear", 0.0, k, via=via)

    rb = oracle.row_bytes(c.type_head, H)
    x = np.stack([oracle.dequantize(c.type_head, ref.head[tok * rb:(tok + 1) * rb], H).reshape(-1) for tok in tokens]).astype(np.float32)
    for l, L in enumerate(ref.layers):
        xn = oracle.rmsnorm(x, L["attn_norm"], c.rms_eps)
        qk = dense(c.type_attn_qk, L["wqk"], xn, H)
        v = dense(c.type_attn_v, L["wv"], xn, H)
        q = oracle.rope_neox(qk[:, :nq * hd].copy(), hd, nq, 0, c.rope_theta).reshape(t, nq * hd)
        k = oracle.rope_neox(qk[:, nq * hd:].copy(), hd, nkv, 0, c.rope_theta).reshape(t, nkv * hd)
        ref.kc[l, 0, :t] = k.reshape(t, nkv, hd).astype(np.float16)
        ref.vc[l, 0, :t] = v.reshape(t, nkv, hd).astype(np.float16)
        att = oracle.attn_prefill(q, k, v, nq, nkv, hd, t, 1.0 / np.sqrt(hd))
        x = x + dense(c.type_attn_o, L["wo"], att, nq * hd)
        xn = oracle.rmsnorm(x, L["ffn_norm"], c.rms_eps)
        gu = dense(c.type_ffn_gate_up, L["wgu"], xn, H)
        act = oracle.gelu_mul if c.act == ref.dec.ACT_GELU_TANH else oracle.silu_mul
        x = x + dense(c.type_ffn_down, L["wdown"], act(gu[:, :ffn].copy(), gu[:, ffn:].copy()), ffn)
    xq = ref.q8(oracle.rmsnorm(x[-1:], ref.final_norm, c.rms_eps)[0])
    return oracle.matvec(c.type_head, ref.head, xq, H)[0]


@pytest.mark.parametrize("t", [1, 20, 70, 130])
def test_prefill_matches_reference_and_decode_continues(dec, t):
    """qmm_decoder_prefill on a prompt of t tokens (below and above the 64 rows from which Q4_K projections take the
    tensor-core GEMM) against the oracle composition; then one decode step from the filled cache."""
    from nates_recipe_rs_b200 import quant_ops as ops
    d = dec.Decoder(tiny_cfg(dec, ctx_len=160, max_batch=2))
    c = d.cfg
    ref = RefModel(d, dec)
    rng = np.random.default_rng(t)
    prompt = rng.integers(0, c.vocab, size=t).astype(np.int32)
    logits = torch.empty(c.vocab, device="cuda")
    nxt = d.prefill(torch.from_numpy(prompt).cuda(), 0, logits)
    ops.check_launch()
    want = ref_prefill(ref, prompt)
    got = logits.cpu().numpy()
    scale = np.abs(want).max()
    assert np.abs(got - want).max() <= 2e-2 * scale, (float(np.abs(got - want).max()), float(scale))
    assert int(nxt.item()) == int(got.argmax())
    # the cache the engine filled continues the sequence: one decode step at position t
    tok = int(nxt.item())
    d.tokens[:1] = tok
    step_logits = torch.empty(c.max_batch, c.vocab, device="cuda")
    d.step(1, t, step_logits)
    ops.check_launch()
    want2 = ref.step(0, tok, t)
    got2 = step_logits[0].cpu().numpy()
    assert np.abs(got2 - want2).max() <= 2e-2 * np.abs(want2).max()
    d.close()


def test_prefill_agrees_with_token_by_token_decoding(dec):
    """The same prompt through the decode path one token at a time: the logits after the last token agree with the
    prompt path within the difference of the activation formats (bf16 / f16 against Q8_1 blocks)."""
    from nates_recipe_rs_b200 import quant_ops as ops
    t = 80
    d = dec.Decoder(tiny_cfg(dec, ctx_len=96, max_batch=2))
    c = d.cfg
    prompt = np.random.default_rng(5).integers(0, c.vocab, size=t).astype(np.int32)
    a = torch.empty(c.vocab, device="cuda")
    d.prefill(torch.from_numpy(prompt).cuda(), 1, a)      # sequence 1
    b = torch.empty(c.max_batch, c.vocab, device="cuda")
    for pos in range(t):
        d.tokens[:1] = int(prompt[pos])
        d.step(1, pos, b)                                  # sequence 0
    ops.check_launch()
    scale = float(b[0].abs().max())
    assert float((a - b[0]).abs().max()) <= 5e-2 * scale
    d.close()


@pytest.mark.parametrize("pieces", [(70, 70), (60, 64, 30), (20, 30), (64, 1, 75)])
def test_prefill_in_pieces_continues_the_cache(dec, pieces):
    """A prompt fed in pieces (qmm_decoder_prefill_at: each piece attends to the cached positions before it) against the
    same prompt in one call: the last position's logits agree (the pieces may take the matvec route where the whole
    prompt takes the GEMM route, hence the decoder tolerance), and decode continues from either cache alike."""
    from nates_recipe_rs_b200 import quant_ops as ops
    t = sum(pieces)
    d = dec.Decoder(tiny_cfg(dec, ctx_len=160, max_batch=2))
    c = d.cfg
    prompt = torch.from_numpy(np.random.default_rng(t).integers(0, c.vocab, size=t).astype(np.int32)).cuda()
    whole = torch.empty(c.vocab, device="cuda")
    nxt_whole = d.prefill(prompt, 0, whole)                       # sequence 0: one call
    part = torch.empty(c.vocab, device="cuda")
    pos = 0
    for n in pieces:                                              # sequence 1: piece by piece
        nxt_part = d.prefill(prompt[pos:pos + n].contiguous(), 1, part, pos0=pos)
        pos += n
    ops.check_launch()
    scale = float(whole.abs().max())
    same_route = all((n >= 64) == (t >= 64) for n in pieces)
    assert float((whole - part).abs().max()) <= (2e-3 if same_route else 5e-2) * scale
    if same_route:
        assert int(nxt_whole.item()) == int(nxt_part.item())
    # one decode step for both sequences from their caches
    d.tokens[:2] = int(nxt_whole.item())
    step_logits = torch.empty(c.max_batch, c.vocab, device="cuda")
    d.step(2, t, step_logits)
    ops.check_launch()
    assert float((step_logits[0] - step_logits[1]).abs().max()) <= (2e-3 if same_route else 5e-2) * float(step_logits[0].abs().max())
    d.close()


def test_prefill_rejects_bad_arguments(dec):
    from nates_recipe_rs_b200._lib import QmmError
    d = dec.Decoder(tiny_cfg(dec))
    toks = torch.zeros(100, dtype=torch.int32, device="cuda")
    with pytest.raises(QmmError):
        d.prefill(toks, 0)            # longer than the context (48)
    with pytest.raises(QmmError):
        d.prefill(toks[:4], 7)        # no such sequence
    with pytest.raises(QmmError):
        d.prefill(toks[:10], 0, pos0=40)   # runs past the context (48)
    with pytest.raises(QmmError):
        d.prefill(toks[:4], 0, pos0=-1)
    d.close()
