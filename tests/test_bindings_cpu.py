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


def _import_everything():
    for m in pkgutil.walk_packages(rmlx_b200.__path__, "rmlx_b200."):
        if not m.name.endswith("__main__"):
            importlib.import_module(m.name)


def _prototypes():
    """name -> parameter count, from the ``extern "C"`` definitions in the .cu / .cpp sources."""
    out = {}
    pat = re.compile(r'extern\s+"C"\s+[A-Za-z_][\w\s\*]*?\b(rmlx_\w+)\s*\(')
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
    _import_everything()
    lib = _lib.cuda()
    protos = _prototypes()
    assert len(_lib._CUDA_SIGS) >= 50
    for name, (args, _ret) in _lib._CUDA_SIGS.items():
        assert hasattr(lib, name), f"{name} is registered but not exported by the library"
        assert name in protos, f"no extern \"C\" definition found for {name}"
        want = "".join(protos[name])
        assert len(args) == len(want), f"{name}: {len(args)} registered arguments, {len(want)} in the prototype"
        got = args.replace("Q", "q").replace("l", "q")
        assert got == want, f"{name}: registered {args!r}, prototype reads {want!r}"
