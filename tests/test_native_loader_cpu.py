"""The memory-mapped safetensors reader of the host library against the ``safetensors`` package."""
import gc
import json
import struct

import pytest
import torch
from safetensors.torch import load_file as st_load_file, save_file

from rmlx_b200.loader import native_st
from rmlx_b200.loader.safetensors_loader import load_tensors

pytestmark = pytest.mark.skipif(not native_st.available(), reason="host library not available")


def _same_bytes(a, b):
    if a.numel() == 0:
        return a.shape == b.shape
    return torch.equal(a.reshape(-1).view(torch.uint8), b.reshape(-1).view(torch.uint8))


def _sample():
    g = torch.Generator().manual_seed(0)
    return {
        "model.embed_tokens.weight": torch.randn(50, 16, generator=g).to(torch.bfloat16),
        "model.layers.0.self_attn.q_proj.weight": torch.randint(-2**31, 2**31 - 1, (8, 4), generator=g, dtype=torch.int64).to(torch.int32),
        "model.layers.0.self_attn.q_proj.scales": torch.randn(8, 1, generator=g).to(torch.float16),
        "model.norm.weight": torch.randn(16, generator=g),
        "scalar": torch.tensor(3.5),
        "flags": torch.tensor([True, False, True]),
        "bytes": torch.arange(7, dtype=torch.uint8),
        "empty": torch.zeros(0, 4),
        "big": torch.randn(3 * 1024 * 1024 + 5, generator=g),            # > 8 MiB: threaded copy path
    }


def test_native_reader_matches_safetensors_package(tmp_path):
    tensors = _sample()
    path = tmp_path / "model.safetensors"
    save_file(tensors, str(path), metadata={"format": "pt", "note": "with \"quotes\" and {braces}"})
    want = st_load_file(str(path))
    f = native_st.SafetensorsFile(str(path))
    assert sorted(f.keys()) == sorted(want.keys())
    for name, w in want.items():
        assert name in f
        dtype, shape, nbytes = f.info(name)
        assert dtype == w.dtype and shape == tuple(w.shape) and nbytes == w.numel() * w.element_size()
        got = f.tensor(name)
        assert got.dtype == w.dtype and got.shape == w.shape
        assert _same_bytes(got, w), name
    assert "missing" not in f
    with pytest.raises(KeyError):
        f.tensor("missing")
    # copy into a caller buffer (the pinned-memory path), single- and multi-threaded
    for name in ("big", "model.norm.weight"):
        for threads in (1, 4):
            dst = torch.empty_like(want[name])
            f.read_into(name, dst, threads=threads)
            assert torch.equal(dst, want[name])
    with pytest.raises(ValueError):
        f.read_into("big", torch.empty(3))


def test_views_outlive_the_file_object(tmp_path):
    path = tmp_path / "m.safetensors"
    save_file({"w": torch.arange(1000, dtype=torch.float32)}, str(path))
    t = native_st.load_file(str(path))["w"]
    derived = t.view(torch.int32)[10:20]
    del t
    gc.collect()
    assert derived.view(torch.float32).tolist() == [float(i) for i in range(10, 20)]


def test_malformed_files_are_refused(tmp_path):
    bad = tmp_path / "bad.safetensors"
    bad.write_bytes(b"\x01\x02")
    with pytest.raises(ValueError, match="too small"):
        native_st.SafetensorsFile(str(bad))
    bad.write_bytes(struct.pack("<Q", 10_000) + b"{}")
    with pytest.raises(ValueError, match="header length"):
        native_st.SafetensorsFile(str(bad))
    hdr = json.dumps({"w": {"dtype": "F32", "shape": [4], "data_offsets": [0, 16]}}).encode()
    bad.write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\x00" * 8)          # data shorter than claimed
    with pytest.raises(ValueError, match="past the end"):
        native_st.SafetensorsFile(str(bad))
    hdr = b'{"w": {"dtype": "F32", "shape": [4], "data_offsets": [0, 16]'   # unterminated
    bad.write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\x00" * 16)
    with pytest.raises(ValueError):
        native_st.SafetensorsFile(str(bad))
    with pytest.raises(ValueError, match="cannot open"):
        native_st.SafetensorsFile(str(tmp_path / "nope.safetensors"))


def test_load_tensors_uses_the_native_reader_for_sharded_checkpoints(tmp_path, monkeypatch):
    tensors = _sample()
    names = sorted(tensors)
    a, b = {n: tensors[n] for n in names[:4]}, {n: tensors[n] for n in names[4:]}
    save_file(a, str(tmp_path / "model-00001-of-00002.safetensors"))
    save_file(b, str(tmp_path / "model-00002-of-00002.safetensors"))
    weight_map = {n: "model-00001-of-00002.safetensors" for n in a}
    weight_map.update({n: "model-00002-of-00002.safetensors" for n in b})
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"weight_map": weight_map}))
    got = load_tensors(str(tmp_path))
    monkeypatch.setenv("RMLX_NATIVE_LOADER", "0")
    want = load_tensors(str(tmp_path))
    assert sorted(got) == sorted(want) == names
    for n in names:
        assert got[n].dtype == want[n].dtype and got[n].shape == want[n].shape
        assert _same_bytes(got[n], want[n]), n


_SCALE_FIELDS = {"F16": [0], "Q4_0": [0], "Q4_1": [0, 2], "Q5_0": [0], "Q5_1": [0, 2], "Q8_0": [0],
                 "Q2_K": [80, 82], "Q3_K": [108], "Q4_K": [0, 2], "Q5_K": [0, 2], "Q6_K": [208]}


def _random_blocks(rng, nblocks, bb, type_name):
    import numpy as np
    raw = rng.integers(0, 256, size=(nblocks, bb), dtype=np.uint8)
    for off in _SCALE_FIELDS.get(type_name, []):
        hi = raw[:, off + 1]
        hi[(hi & 0x7C) == 0x7C] &= 0xBF                  # exponent 31 (inf / nan) -> finite
    return raw


@pytest.mark.parametrize("type_name", ["F32", "F16", "BF16", "Q4_0", "Q4_1", "Q5_0", "Q5_1", "Q8_0",
                                       "Q2_K", "Q3_K", "Q4_K", "Q5_K", "Q6_K"])
@pytest.mark.parametrize("nblocks", [1, 37, 9000])
def test_native_ggml_dequantisers_match_numpy_bit_for_bit(type_name, nblocks):
    """Random block bytes (every scale field a finite fp16, subnormals included) through the native
    dequantisers and the numpy restatement; 9000 K-quant blocks take the threaded path."""
    import numpy as np
    from rmlx_b200.loader import gguf
    t = gguf._T[type_name]
    _, be, bb = gguf.GGML_TYPES[t]
    rng = np.random.default_rng(nblocks)
    raw = _random_blocks(rng, nblocks, bb, type_name)
    if type_name == "F32":
        raw = rng.standard_normal(nblocks).astype(np.float32).view(np.uint8).reshape(nblocks, 4)
    raw = raw.reshape(-1)
    assert gguf._native_lib() is not None
    got = gguf.dequantize(raw, t)
    want = gguf.dequantize_numpy(raw, t)
    assert got.dtype == np.float32 and got.shape == want.shape == (nblocks * be,)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def test_ggml_dequantize_rejects_partial_blocks():
    import numpy as np
    from rmlx_b200.loader import gguf
    with pytest.raises(ValueError):
        gguf.dequantize(np.zeros(17, np.uint8), gguf._T["Q4_0"])


@pytest.mark.parametrize("type_name", ["Q4_0", "Q4_1", "Q5_0", "Q5_1", "Q8_0", "Q2_K", "Q3_K", "Q4_K", "Q5_K", "Q6_K"])
def test_ggml_dequantisers_agree_with_the_gguf_package(type_name):
    """Independent oracle for the block layouts: the ``gguf`` package's own dequantisers on the same
    random blocks (skipped where that package is not installed)."""
    import numpy as np
    gguf_pkg = pytest.importorskip("gguf")
    from rmlx_b200.loader import gguf
    t = gguf._T[type_name]
    _, be, bb = gguf.GGML_TYPES[t]
    qt = getattr(gguf_pkg.GGMLQuantizationType, type_name)
    assert tuple(gguf_pkg.GGML_QUANT_SIZES[qt]) == (be, bb)
    raw = _random_blocks(np.random.default_rng(7), 64, bb, type_name)
    want = gguf_pkg.quants.dequantize(raw, qt).reshape(-1)
    for fn in (gguf.dequantize, gguf.dequantize_numpy):
        got = fn(raw.reshape(-1), t)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), fn.__name__


def test_dtype_table_matches_the_gguf_type_table():
    from rmlx_b200 import dtypes
    from rmlx_b200.loader import gguf
    for _, (name, be, bb) in gguf.GGML_TYPES.items():
        d = dtypes.from_name(name)
        assert (d.block_elems, d.block_bytes) == (be, bb), name
    assert dtypes.Q3_K.nbytes(512) == 220 and dtypes.Q5_K.is_quantized
