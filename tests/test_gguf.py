"""GGUF container reader and writer (include/qmm_gguf.h) on the CPU: files written by the writer follow the
published layout (checked by an independent struct parse here) and read back byte for byte; malformed
files are rejected.  No GPU."""
import struct

import numpy as np
import pytest

import oracle
from nates_recipe_rs_b200 import gguf
from nates_recipe_rs_b200._lib import QmmError


def sample_tensors():
    k = 512
    w = oracle.fill_normal(5 * k, 3, 0.02).reshape(5, k)
    return [
        ("token_embd.weight", oracle.Q6_K, [k, 5], oracle.quantize(oracle.Q6_K, w)),
        ("blk.0.attn_q.weight", oracle.Q4_K, [k, 5], oracle.quantize(oracle.Q4_K, w)),
        ("blk.0.attn_v.weight", oracle.Q8_0, [k, 5], oracle.quantize(oracle.Q8_0, w)),
        ("blk.0.attn_norm.weight", gguf.F32, [k], oracle.fill_normal(k, 4, 0.1)),
    ]


def write_sample(path):
    w = gguf.GgufWriter(path)
    w.meta("general.architecture", "llama").meta("llama.block_count", 1).meta("llama.rope.freq_base", 10000.0)
    for name, t, dims, data in sample_tensors():
        w.tensor(name, t, dims, data)
    w.finish()


def test_round_trip(tmp_path):
    path = tmp_path / "m.gguf"
    write_sample(path)
    with gguf.GgufFile(path) as f:
        assert len(f) == 4
        assert f.meta_str("general.architecture") == "llama"
        assert f.meta_int("llama.block_count") == 1
        assert f.meta_float("llama.rope.freq_base") == 10000.0
        assert f.meta_int("general.alignment") == 32
        with pytest.raises(QmmError):
            f.meta_int("no.such.key")
        with pytest.raises(QmmError):
            f.meta_int("general.architecture")       # a string, not a number
        for i, (name, t, dims, data) in enumerate(sample_tensors()):
            info = f.info(i)
            assert info["name"] == name and info["type"] == t and info["dims"] == dims
            assert info["file_offset"] % 32 == 0
            raw = np.ascontiguousarray(data).view(np.uint8).reshape(-1)
            assert info["bytes"] == raw.size
            assert f.find(name) == i
            assert np.array_equal(f.read(name), raw)
        assert f.find("missing") == -1


def test_written_file_follows_the_published_layout(tmp_path):
    """Independent parse of the bytes: magic, version 3, counts, key/value records, tensor infos (name, rank,
    dims innermost first, type, offset relative to the aligned data section)."""
    path = tmp_path / "m.gguf"
    write_sample(path)
    b = path.read_bytes()
    pos = 0

    def take(fmt):
        nonlocal pos
        v = struct.unpack_from("<" + fmt, b, pos)
        pos += struct.calcsize("<" + fmt)
        return v[0] if len(v) == 1 else v

    def take_str():
        nonlocal pos
        n = take("Q")
        s = b[pos:pos + n].decode()
        pos += n
        return s

    assert take("I") == 0x46554747 and b[:4] == b"GGUF"
    assert take("I") == 3
    n_tensors, n_kv = take("Q"), take("Q")
    assert (n_tensors, n_kv) == (4, 4)
    kv = {}
    for _ in range(n_kv):
        key, vt = take_str(), take("I")
        kv[key] = {4: lambda: take("I"), 6: lambda: take("f"), 8: take_str}[vt]()
    assert kv == {"general.alignment": 32, "general.architecture": "llama", "llama.block_count": 1, "llama.rope.freq_base": 10000.0}
    infos = []
    for _ in range(n_tensors):
        name, nd = take_str(), take("I")
        dims = [take("Q") for _ in range(nd)]
        infos.append((name, dims, take("I"), take("Q")))
    data_start = (pos + 31) // 32 * 32
    for (name, dims, t, off), (wname, wt, wdims, data) in zip(infos, sample_tensors()):
        assert (name, dims, t) == (wname, wdims, wt) and off % 32 == 0
        raw = np.ascontiguousarray(data).view(np.uint8).reshape(-1)
        assert b[data_start + off:data_start + off + raw.size] == raw.tobytes()


def test_malformed_files_are_rejected(tmp_path):
    good = tmp_path / "m.gguf"
    write_sample(good)
    b = good.read_bytes()
    cases = {"magic": b"GGUX" + b[4:], "version": b[:4] + struct.pack("<I", 9) + b[8:], "truncated header": b[:40],
             "truncated data": b[:-100], "empty": b""}
    for what, data in cases.items():
        p = tmp_path / "bad.gguf"
        p.write_bytes(data)
        with pytest.raises(QmmError) as e:
            gguf.GgufFile(p)
        assert e.value.status == -9, what
    with pytest.raises(QmmError) as e:
        gguf.GgufFile(tmp_path / "nowhere.gguf")
    assert e.value.status == -8
    w = gguf.GgufWriter(tmp_path / "x.gguf")
    with pytest.raises(QmmError):
        w.tensor("t", oracle.Q4_K, [512, 2], np.zeros(100, dtype=np.uint8))       # byte count does not match the shape
    with pytest.raises(QmmError):
        w.tensor("t", oracle.Q4_K, [100, 2], np.zeros(100, dtype=np.uint8))       # row is not whole blocks
    w.finish()


def test_unknown_tensor_types_are_listed_but_not_read(tmp_path):
    """A file may hold tensors of types this library does not decode: they appear in the table with bytes = 0."""
    path = tmp_path / "m.gguf"
    write_sample(path)
    b = bytearray(path.read_bytes())
    # patch the type field of the last tensor info (F32 = 0) to 30
    name = b"blk.0.attn_norm.weight"
    at = b.find(name) + len(name) + 4 + 8          # name bytes, n_dims (u32), one dim (u64)
    assert struct.unpack_from("<I", b, at)[0] == 0
    struct.pack_into("<I", b, at, 30)
    path.write_bytes(bytes(b))
    with gguf.GgufFile(path) as f:
        info = f.info(3)
        assert info["type"] == 30 and info["bytes"] == 0
        with pytest.raises(QmmError):
            f.read(3)
        assert np.array_equal(f.read(0), sample_tensors()[0][3].reshape(-1))
