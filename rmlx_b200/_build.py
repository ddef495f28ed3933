"""In-tree native build: every ``.cu`` under ``csrc/kernels``, ``csrc/comm`` and ``csrc/runtime`` is compiled for
sm_100a and linked into ``lib/librmlx_b200_cuda.so``; every ``.cpp`` under ``csrc/host`` goes into
``lib/librmlx_b200_host.so`` (pure C++, loadable without a GPU).

Objects are rebuilt only when the content hash of the source, of every header in ``csrc`` and of
the flags changes, so a built tree that is copied to another machine is used as it is (no
dependence on file times). This plays the role of the reference's AOT metallib build plus its
pipeline caches (crates/rmlx-core/build.rs:31-138, crates/rmlx-metal/src/pipeline_cache.rs:84-210):
kernels are compiled ahead of time into one fat binary and looked up by exported symbol.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
OBJ = ROOT / "build"
LIB = ROOT / "lib"

CUDA_LIB = LIB / "librmlx_b200_cuda.so"
# The same sources compiled with -DRMLX_BOUNDS: device-side index checks that record the first
# offender and skip the access (build(kinds=("cuda_bounds",)); loaded when RMLX_BOUNDS=1).
CUDA_BOUNDS_LIB = LIB / "librmlx_b200_cuda_bounds.so"
# RMLX_HOST_LIB=<file>: load that build of the host runtime instead (a sanitizer build, say: the
# sources compile on their own, `g++ -shared -fPIC -pthread -fsanitize=address,undefined csrc/host/*.cpp`)
HOST_LIB = Path(os.environ["RMLX_HOST_LIB"]) if os.environ.get("RMLX_HOST_LIB") else LIB / "librmlx_b200_host.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xptxas", "-v", "--expt-relaxed-constexpr",
    "-Xcudafe", "--diag_suppress=177",
]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-Wall", "-pthread"]


def _nvcc() -> str | None:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    return cand if os.path.exists(cand) else None


def _headers_digest() -> str:
    h = hashlib.sha256()
    for p in sorted(CSRC.rglob("*")):
        if p.suffix in (".cuh", ".h", ".hpp"):
            h.update(p.name.encode())
            h.update(p.read_bytes())
    return h.hexdigest()


def _digest(src: Path, flags: list[str], hdr: str) -> str:
    h = hashlib.sha256()
    h.update(src.read_bytes())
    h.update(" ".join(flags).encode())
    h.update(hdr.encode())
    return h.hexdigest()


def _compile_one(args) -> tuple[Path, bool, str]:
    src, obj, cmd, digest = args
    stamp = obj.with_suffix(".hash")
    if obj.exists() and stamp.exists() and stamp.read_text() == digest:
        return obj, False, ""
    proc = subprocess.run(cmd, capture_output=True, text=True)
    log = proc.stdout + proc.stderr
    obj.with_suffix(".log").write_text(log)
    if proc.returncode != 0:
        raise RuntimeError(f"compile failed: {' '.join(cmd)}\n{log}")
    stamp.write_text(digest)
    return obj, True, log


def _sources(kind: str) -> list[Path]:
    if kind in ("cuda", "cuda_bounds"):
        return sorted((CSRC / "kernels").glob("*.cu")) + sorted((CSRC / "comm").glob("*.cu")) + \
            sorted((CSRC / "runtime").glob("*.cu"))
    return sorted((CSRC / "host").glob("*.cpp"))


def build(kinds=("host", "cuda"), verbose: bool = False, force: bool = False) -> dict[str, Path]:
    """Compile and link whatever is out of date. Returns the library paths."""
    OBJ.mkdir(exist_ok=True)
    LIB.mkdir(exist_ok=True)
    hdr = _headers_digest()
    out: dict[str, Path] = {}
    for kind in kinds:
        srcs = _sources(kind)
        lib = {"cuda": CUDA_LIB, "cuda_bounds": CUDA_BOUNDS_LIB}.get(kind, HOST_LIB)
        if not srcs:
            continue
        if kind in ("cuda", "cuda_bounds"):
            nvcc = _nvcc()
            if nvcc is None:
                raise RuntimeError("nvcc not found; cannot build the CUDA library")
            flags = NVCC_FLAGS + (["-DRMLX_BOUNDS"] if kind == "cuda_bounds" else [])
            mk = lambda s, o: [nvcc, *flags, "-I", str(CSRC), "-c", str(s), "-o", str(o)]
        else:
            cxx = shutil.which("g++") or "g++"
            flags = CXX_FLAGS
            mk = lambda s, o: [cxx, *flags, "-I", str(CSRC), "-c", str(s), "-o", str(o)]
        jobs = []
        for s in srcs:
            o = OBJ / f"{kind}_{s.stem}.o"
            d = _digest(s, flags, hdr)
            if force and o.exists():
                o.unlink()
            jobs.append((s, o, mk(s, o), d))
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            results = list(ex.map(_compile_one, jobs))
        rebuilt = any(r[1] for r in results)
        if verbose:
            for o, did, log in results:
                if did:
                    print(f"[build] compiled {o.name}", file=sys.stderr)
        link_stamp = OBJ / f"{kind}.linkhash"
        link_digest = hashlib.sha256(
            "".join(sorted(j[3] for j in jobs)).encode()).hexdigest()
        if rebuilt or not lib.exists() or not link_stamp.exists() or \
                link_stamp.read_text() != link_digest:
            objs = [str(r[0]) for r in results]
            if kind in ("cuda", "cuda_bounds"):
                cmd = [_nvcc(), "-shared", "-o", str(lib), *objs, "-lpthread", "-ldl"]
            else:
                cmd = [shutil.which("g++") or "g++", "-shared", "-o", str(lib), *objs, "-pthread"]
            proc = subprocess.run(cmd, capture_output=True, text=True)
            if proc.returncode != 0:
                raise RuntimeError(f"link failed: {' '.join(cmd)}\n{proc.stdout}{proc.stderr}")
            link_stamp.write_text(link_digest)
            if verbose:
                print(f"[build] linked {lib.name}", file=sys.stderr)
        out[kind] = lib
    return out


def ptxas_report() -> str:
    """Registers / spills / shared memory per kernel as printed by ``-Xptxas -v``."""
    lines = []
    for log in sorted(OBJ.glob("cuda_*.log")):
        lines.append(f"== {log.stem}")
        txt = log.read_text().splitlines()
        for i, ln in enumerate(txt):
            if "Used" in ln and "registers" in ln:
                name = ""
                for back in range(i, max(-1, i - 4), -1):
                    if "Compiling entry function" in txt[back]:
                        name = txt[back].split("'")[1]
                        break
                lines.append(f"{name}: {ln.split(':', 1)[-1].strip()}")
    return "\n".join(lines)


if __name__ == "__main__":
    libs = build(verbose=True, force="--force" in sys.argv)
    for k, v in libs.items():
        print(k, v)
    if "--report" in sys.argv:
        print(ptxas_report())
