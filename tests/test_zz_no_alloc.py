"""The allocation-free attention entry point (launch_attn_decode_static) against the regular one.

Some hosts of the library cannot allocate device memory at the point where they need attention
(a frozen no-allocation steady state, a plugin that only owns the buffers it was given), so the
library carries a fixed scratch array of its own for them.  The variant must give exactly what
launch_attn_decode gives with caller-owned scratch, call after call: the array is shared by all
calls and keeps the previous call's contents, so the second call below uses other shapes and
data than the first on purpose.  Collected last (file name) so a stop-at-first-failure run has
already run every other test.  Needs a B200."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def run_both(L, check, batch, nqh, nkv, hd, length, seed):
    cap = length + 3
    g = torch.Generator(device="cuda").manual_seed(seed)
    qkv = torch.randn(batch, (nqh + 2 * nkv) * hd, device="cuda", generator=g)
    kc = torch.randn(batch, cap, nkv, hd, device="cuda", generator=g).half()
    vc = torch.randn(batch, cap, nkv, hd, device="cuda", generator=g).half()
    stream = torch.cuda.current_stream().cuda_stream
    nblk = batch * (nqh * hd // 32) * 36
    ref_f, ref_q = torch.full((batch, nqh * hd), float("nan"), device="cuda"), torch.zeros(nblk, dtype=torch.uint8, device="cuda")
    got_f, got_q = torch.full_like(ref_f, float("nan")), torch.zeros_like(ref_q)
    scratch = torch.empty(L.qmm_attn_decode_scratch_bytes(batch, nqh, hd, length) // 4, device="cuda")
    check(L.launch_attn_decode(qkv.data_ptr(), kc.data_ptr(), vc.data_ptr(), scratch.data_ptr(), ref_f.data_ptr(), ref_q.data_ptr(),
                               batch, nqh, nkv, hd, length, cap, stream), "launch_attn_decode")
    check(L.launch_attn_decode_static(qkv.data_ptr(), kc.data_ptr(), vc.data_ptr(), got_f.data_ptr(), got_q.data_ptr(),
                                      batch, nqh, nkv, hd, length, cap, stream), "launch_attn_decode_static")
    torch.cuda.synchronize()
    return ref_f, ref_q, got_f, got_q


def test_static_scratch_attention_matches_regular_entry_twice():
    if not torch.cuda.is_available():
        pytest.fail("this test needs a CUDA device")
    from nates_recipe_rs_b200._lib import check, lib
    from nates_recipe_rs_b200 import quant_ops as ops
    L = lib()
    # two calls in a row: the second is larger in one dimension and smaller in another than the first,
    # so stale words of the first call lie both inside and beyond what the second one uses
    for call, (batch, nqh, nkv, hd, length) in enumerate([(2, 32, 8, 128, 1000), (3, 8, 2, 64, 257)]):
        ref_f, ref_q, got_f, got_q = run_both(L, check, batch, nqh, nkv, hd, length, 100 + call)
        assert not torch.isnan(got_f).any()
        # same kernels, same order of operations: the tolerance of the other tests is met with zero to spare
        assert torch.allclose(got_f, ref_f, rtol=1e-3, atol=1e-4), f"call {call}: max diff {float((got_f - ref_f).abs().max())}"
        assert torch.equal(got_q, ref_q), f"call {call}: Q8_1 bytes differ"
    ops.check_launch()


def test_static_scratch_attention_rejects_what_does_not_fit():
    if not torch.cuda.is_available():
        pytest.fail("this test needs a CUDA device")
    from nates_recipe_rs_b200._lib import lib
    L = lib()
    batch, nqh, nkv, hd, length = 16, 64, 8, 128, 4096     # needs 16*64*64*130 floats = 34 MB > 4 MiB
    assert L.qmm_attn_decode_scratch_bytes(batch, nqh, hd, length) > 4 << 20
    dummy = torch.zeros(64, device="cuda")
    rc = L.launch_attn_decode_static(dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(), None, batch, nqh, nkv, hd,
                                     length, length, None)
    assert rc == -7 and b"scratch" in L.qmm_status_string(rc)
