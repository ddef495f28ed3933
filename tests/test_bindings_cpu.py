"""Every entry point that a Python wrapper registers exists in the built CUDA library, and its
registered argument string has as many entries as the C prototype has parameters (the library loads
without a GPU, so this runs on CPU)."""
import importlib
import pathlib
import pkgutil
import re

import rmlx_b200
from rmlx_b200 import _lib

CSRC = pathlib.Path(rmlx_b200.__file__).parent / "csrc"


def _cuda_lib():
    """The CUDA library (it loads without a GPU); skip where it cannot be built (no nvcc)."""
    import pytest
    try:
        return _lib.cuda()
    except Exception as e:                         # noqa: BLE001
        pytest.skip(f"CUDA library not available: {e}")


def _import_everything():
    for m in pkgutil.walk_packages(rmlx_b200.__path__, "rmlx_b200."):
        if not m.name.endswith("__main__"):
            importlib.import_module(m.name)


def _prototypes():
    """name -> parameter count, from the ``extern "C"`` definitions in the .cu / .cpp sources."""
    out = {}
    # either prefixed with extern "C", or a definition at the start of a line inside an extern "C" block
    pat = re.compile(r'(?:extern\s+"C"\s+[A-Za-z_][\w\s\*]*?|^(?:const\s+)?[A-Za-z_]\w*[\s\*]+)\b(rmlx_\w+)\s*\(',
                     re.MULTILINE)
    for path in list(CSRC.rglob("*.cu")) + list(CSRC.rglob("*.cpp")):
        src = path.read_text()
        for m in pat.finditer(src):
            i, depth, start = m.end(), 1, m.end()
            while depth:
                c = src[i]
                depth += (c == "(") - (c == ")")
                i += 1
            params = src[start:i - 1].strip()
            out[m.group(1)] = [] if params in ("", "void") else [_kind(p) for p in params.split(",")]
    return out


def _kind(param: str) -> str:
    """The registration code a C parameter should have: p pointer / stream, f float, d double,
    q 64-bit integer, i other integers."""
    param = " ".join(param.split())
    if "*" in param or "cudaStream_t" in param:
        return "p"
    ctype = param.rsplit(" ", 1)[0]
    if ctype.endswith("double"):
        return "d"
    if ctype.endswith("float"):
        return "f"
    if any(t in ctype for t in ("int64_t", "uint64_t", "size_t", "long long")):
        return "q"
    return "i"


def test_registered_entry_points_exist_and_match_their_prototypes():
    lib = _cuda_lib()
    _import_everything()
    protos = _prototypes()
    assert len(_lib._CUDA_SIGS) >= 50
    for name, (args, _ret) in _lib._CUDA_SIGS.items():
        assert hasattr(lib, name), f"{name} is registered but not exported by the library"
        assert name in protos, f"no extern \"C\" definition found for {name}"
        want = "".join(protos[name])
        assert len(args) == len(want), f"{name}: {len(args)} registered arguments, {len(want)} in the prototype"
        got = args.replace("Q", "q").replace("l", "q")
        assert got == want, f"{name}: registered {args!r}, prototype reads {want!r}"


def test_host_library_bindings_match_their_prototypes():
    """The same check for the host library (allocator, serving core, safetensors reader, GGML
    dequantisers), whose wrappers set ctypes argtypes directly."""
    import ctypes
    from rmlx_b200.loader import gguf, native_st
    from rmlx_b200.runtime import alloc
    from rmlx_b200.serve import native
    lib = native._host()
    native_st._host()
    alloc._host()
    assert gguf._native_lib() is not None
    protos = {n: k for n, k in _prototypes().items()
              if any(n.startswith(p) for p in ("rmlx_bm_", "rmlx_pc_", "rmlx_sched_", "rmlx_st_", "rmlx_ggml_",
                                               "rmlx_bfc_", "rmlx_alloc_", "rmlx_crc32"))}
    assert len(protos) > 60

    def kind(t) -> str:
        if t in (ctypes.c_void_p, ctypes.c_char_p) or isinstance(t, type) and issubclass(t, ctypes._Pointer):
            return "p"
        if t in (ctypes.c_int64, ctypes.c_uint64, ctypes.c_longlong, ctypes.c_ulonglong, ctypes.c_size_t):
            return "q"
        if t in (ctypes.c_float,):
            return "f"
        return "i"

    checked = 0
    for name, want in protos.items():
        assert hasattr(lib, name), name
        argtypes = getattr(lib, name).argtypes
        if argtypes is None:
            continue                                   # exported but not wrapped
        got = "".join(kind(t) for t in argtypes)
        assert got == "".join(want), f"{name}: bound as {got!r}, prototype reads {''.join(want)!r}"
        checked += 1
    assert checked > 55


def test_prefill_kernel_choice_is_a_host_decision(monkeypatch):
    """Which attention kernel a prompt gets is decided on the host from head_dim, window and the
    override variable; no GPU is needed to ask."""
    from rmlx_b200.ops.attention import prefill_kernel_choice
    lib = _cuda_lib()
    monkeypatch.delenv("RMLX_FLASH_PREFILL", raising=False)
    assert prefill_kernel_choice(128, 0) == "tc"
    assert prefill_kernel_choice(64, 0) == "mma" and prefill_kernel_choice(128, 4096) == "tc"
    monkeypatch.setenv("RMLX_FLASH_PREFILL", "mma")
    assert prefill_kernel_choice(128, 0) == "mma"
    assert lib.rmlx_qgemm_supported(4096) == 1 and lib.rmlx_qgemm_supported(4096 + 64) == 0
    assert lib.rmlx_gemm_pick_bn(8192, 4096) in (32, 64, 128, 256)
