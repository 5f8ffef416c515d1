"""Placement policy of the tiered weight store (include/qmm_store.h) without a GPU: host memory while its
budget lasts, the rest stays in its file and is not read at placement."""
import numpy as np
import pytest

from nates_recipe_rs_b200 import store
from nates_recipe_rs_b200._lib import QmmError


def test_placement_overflows_from_host_memory_to_disk(tmp_path):
    blob = np.arange(1000, dtype=np.uint8)
    path = tmp_path / "w.bin"
    path.write_bytes(bytes(blob) * 4)
    s = store.WeightStore(ram_budget=2500)
    assert s.place_file("a", path, 0, 1000) == store.RAM
    assert s.place_host("b", blob) == store.RAM
    assert s.place_file("c", path, 2000, 1000) == store.DISK          # 3000 > 2500: stays in the file
    assert s.place_file("d", tmp_path / "never_opened.bin", 0, 10 ** 9) == store.DISK   # a disk placement reads nothing
    with pytest.raises(QmmError):
        s.place_host("e", blob)                                        # no budget left and no file behind it
    with pytest.raises(QmmError):
        s.place_file("a", path, 0, 10)                                 # placed already
    with pytest.raises(QmmError):
        s.place_file("f", tmp_path / "missing.bin", 0, 10)             # would fit in memory, but cannot be read
    st = s.stats()
    assert (st["vram_bytes"], st["ram_bytes"], st["disk_bytes"]) == (0, 2000, 1000 + 10 ** 9)
    assert s.home("c") == store.DISK
    with pytest.raises(QmmError):
        s.home("unknown")
    s.close()
