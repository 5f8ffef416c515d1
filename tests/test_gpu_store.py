"""The tiered weight store on a GPU: blobs fetched from device memory, pinned host memory and a file hold the
same bytes; a matvec on a staged weight equals the resident one; prefetch and the slot cache.  Needs a B200."""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle
from nates_recipe_rs_b200 import store

pytestmark = pytest.mark.gpu


def as_tensor(addr, nbytes):
    """uint8 CUDA tensor over raw device memory (no ownership)."""
    class _Holder:
        pass
    h = _Holder()
    h.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (addr, False), "version": 2}
    return torch.as_tensor(h, device="cuda")


def test_three_tiers_fetch_prefetch_and_cache(tmp_path):
    if not torch.cuda.is_available():
        pytest.fail("this test needs a CUDA device")
    from nates_recipe_rs_b200 import quant_ops as ops
    n, k = 512, 2048
    rb = oracle.row_bytes(oracle.Q4_K, k)
    mats = [oracle.quantize(oracle.Q4_K, oracle.fill_normal(n * k, 60 + i, 0.02).reshape(n, k)) for i in range(6)]
    nbytes = n * rb
    path = tmp_path / "bank.bin"
    path.write_bytes(b"".join(m.tobytes() for m in mats))
    s = store.WeightStore(vram_budget=2 * nbytes + 512, ram_budget=2 * nbytes, stage_bytes=nbytes, cache_slots=2, cache_slot_bytes=nbytes)
    homes = [s.place_file(f"w{i}", path, i * nbytes, nbytes) for i in range(6)]
    assert homes == [store.VRAM, store.VRAM, store.RAM, store.RAM, store.DISK, store.DISK]
    xq = ops.gpu_quantize_q8_1(torch.from_numpy(oracle.fill_normal(k, 9, 1.0)).cuda())
    xq_ref = oracle.quantize(oracle.Q8_1, oracle.fill_normal(k, 9, 1.0))

    def check_blob(i, addr):
        w = as_tensor(addr, nbytes)
        assert np.array_equal(w.cpu().numpy(), mats[i].reshape(-1)), f"w{i}: bytes differ"
        y = ops.gpu_qmatvec(oracle.Q4_K, w, xq, 1, n, k).cpu().numpy()
        want = oracle.matvec(oracle.Q4_K, mats[i], xq_ref, k)
        assert np.all(np.abs(y - want) <= 1e-4 + 1e-3 * np.abs(want)), f"w{i}: matvec"

    for i in range(6):
        check_blob(i, s.fetch(f"w{i}"))
    st = s.stats()
    assert (st["fetches_vram"], st["fetches_ram"], st["fetches_disk"]) == (2, 2, 2) and st["staged_bytes"] == 4 * nbytes
    a0, a1 = s.fetch("w0"), s.fetch("w0")
    assert a0 == a1, "a resident blob is used in place"
    # prefetch: the copy runs on the store's stream; the fetch that follows only waits for it
    s.prefetch("w5")
    y_before = ops.gpu_qmatvec(oracle.Q4_K, as_tensor(s.fetch("w1"), nbytes), xq, 1, n, k)   # resident: does not disturb the prefetch
    check_blob(5, s.fetch("w5"))
    check_blob(3, s.fetch("w3"))
    assert y_before.shape == (1, n)
    # slot cache: two slots, least recently used goes first
    base = s.stats()
    check_blob(4, s.fetch_cached("w4"))
    check_blob(2, s.fetch_cached("w2"))
    p4 = s.fetch_cached("w4")
    check_blob(4, p4)
    assert s.stats()["cache_hits"] == base["cache_hits"] + 1
    check_blob(5, s.fetch_cached("w5"))          # evicts w2 (w4 was used more recently)
    assert s.fetch_cached("w4") == p4
    assert s.stats()["cache_hits"] == base["cache_hits"] + 2
    check_blob(2, s.fetch_cached("w2"))          # staged again
    assert s.stats()["cache_hits"] == base["cache_hits"] + 2
    check_blob(0, s.fetch_cached("w0"))          # resident: in place, no slot used
    torch.cuda.synchronize()
    s.close()
