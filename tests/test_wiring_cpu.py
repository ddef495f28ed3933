"""Wiring proof, static part: every runtime component that claims a product caller is named in that
caller's source (the idea of the reference's check that its asynchronous paths are reachable from
product code, .github/workflows/ci.yml:96-101 and tools/check_runtime_wiring.sh there). The
dynamic part lives with the features: counters such as ``GraphCache.native_captures``,
``Group.native_calls`` or ``StreamManager.waits_inserted`` are asserted in their own tests."""
import pathlib
import re

import pytest

import rmlx_b200

PKG = pathlib.Path(rmlx_b200.__file__).parent

# component -> files of the package (not its own module, not tests) that must use it
WIRED = {
    "GraphCache": ["models/decode_engine.py", "models/prefill.py", "parallel/ep_fused.py"],
    "bucket_for": ["models/decode_engine.py", "models/prefill.py"],
    "NativeGraphStore": ["runtime/graph.py"],
    "HAZARDS": ["runtime/streams.py"],
    "StreamManager": ["nn/moe_pipeline.py"],
    "MoePipeline": ["nn/moe.py"],
    "MoePolicy": ["nn/moe.py"],
    "LayerPipeline": ["models/weights.py"],
    "PrefillPlan": ["models/prefill.py"],
    "Warmup": ["serve/engine.py"],
    "PrecisionGuard": ["serve/engine.py"],
    "default_heap": ["parallel/comm.py"],
    "SymmetricRegion": ["parallel/tp_gemm.py", "parallel/ep_fused.py"],
    "PeerChannel": ["parallel/group.py"],
    "NativeScheduler": ["serve/engine.py"],
    "NativePrefixCache": ["serve/engine.py"],
    "drop_front": ["serve/engine.py"],
    "fp8_quant_rows": ["parallel/ep.py"],
    "SparseGuard": ["parallel/ep.py"],
    "NativeSampler": ["serve/engine.py", "serve/speculative.py"],
    "narrow_expert_ffn": ["ops/grouped.py"],
}


@pytest.mark.parametrize("name", sorted(WIRED))
def test_component_has_its_product_callers(name):
    pat = re.compile(r"\b" + re.escape(name) + r"\b")
    for rel in WIRED[name]:
        src = (PKG / rel).read_text()
        # a use, not only an import line or a mention in a docstring
        uses = [ln for ln in src.splitlines()
                if pat.search(ln) and not ln.lstrip().startswith(("from ", "import ", "#", '"""'))]
        assert uses, f"{name} is not used in rmlx_b200/{rel}"


def test_every_extern_c_launcher_is_named_by_a_wrapper():
    """Every ``extern "C"`` entry point of the CUDA sources is named by some Python module of the
    package (an entry point nothing names is code no product path can reach), the allocation-free
    attention entry apart: it is a C interface with its own header."""
    defined = set()
    pat = re.compile(r'extern\s+"C"\s+[A-Za-z_][\w\s\*]*?\b(rmlx_\w+)\s*\(')
    for path in (PKG / "csrc").rglob("*.cu"):
        defined.update(pat.findall(path.read_text()))
    assert len(defined) > 100
    python = "\n".join(p.read_text() for p in PKG.rglob("*.py"))
    c_only = {"rmlx_flash_decode_paged_noalloc", "rmlx_flash_decode_noalloc_error"}
    missing = sorted(n for n in defined - c_only if not re.search(r"\b" + n + r"\b", python))
    assert not missing, f"entry points no Python module names: {missing}"
