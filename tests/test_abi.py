"""The C-ABI library loads and exports every symbol include/qmm.h declares.  No GPU."""
import ctypes
import os
import re

import pytest

from nates_recipe_rs_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    names = []
    for fn in sorted(os.listdir(os.path.join(ROOT, "include"))):
        if fn.endswith(".h"):
            text = open(os.path.join(ROOT, "include", fn)).read()
            text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
            names += re.findall(r"\b((?:launch_|qmm_)\w+)\s*\(", text)
    return sorted(set(names))


def test_header_declares_something():
    assert len(_declared()) >= 20


def test_every_declared_symbol_is_exported_and_bound():
    if not os.path.exists(_lib.LIB_PATH):
        pytest.fail("libqmm.so is not built: run python -m nates_recipe_rs_b200.build")
    raw = ctypes.CDLL(_lib.LIB_PATH)
    for name in _declared():
        assert hasattr(raw, name), f"{name} declared in include/ but not exported"
        if not name.startswith("qmm_decoder_"):  # the engine is bound in nates_recipe_rs_b200/decoder.py
            assert name in _lib.SIGNATURES, f"{name} has no ctypes signature"
    for name in _lib.SIGNATURES:
        assert name in _declared(), f"{name} bound but not declared in include/"
    from nates_recipe_rs_b200 import decoder
    L = decoder._bind()
    for name in _declared():
        if name.startswith("qmm_decoder_") and name != "qmm_decoder_config":
            assert getattr(L, name).argtypes is not None, f"{name} has no ctypes signature"


def test_host_side_argument_checks_need_no_gpu():
    L = _lib.lib()
    assert L.qmm_row_bytes(_lib.Q4_K, 4096) == 2304
    assert L.qmm_row_bytes(_lib.Q6_K, 14336) == 11760
    assert L.qmm_row_bytes(_lib.Q8_0, 4096) == 4352
    assert L.qmm_row_bytes(_lib.Q8_1, 4096) == 4608
    assert L.qmm_row_bytes(_lib.Q4_K, 100) == -2
    assert L.qmm_row_bytes(77, 256) == -5
    # rejected before any CUDA call
    assert L.launch_qmatvec(_lib.Q4_K, None, None, None, 1, 8, 256, None) == -1
    assert L.launch_qmatvec(_lib.Q4_K, 16, 16, 16, 1, 8, 100, None) == -2
    assert L.launch_qmatvec(_lib.Q4_K, 16, 16, 16, 0, 8, 256, None) == -2
    assert L.launch_qmatvec(99, 16, 16, 16, 1, 8, 256, None) == -5
    assert L.launch_qmatvec(_lib.Q4_K, 8, 16, 16, 1, 8, 256, None) == -4     # Q4_K rows must be 16-byte aligned
    assert L.launch_qmatvec(_lib.Q4_K, 16, 16, 16, 1, 8, 256 * 1024, None) == -3  # row does not fit a stage
    assert L.launch_quantize_q8_1(16, 16, 1, 48, None) == -2
    assert L.launch_dequantize_q4_k_f32(16, 16, 100, None) == -2
    assert b"aligned" in L.qmm_status_string(-4)
