"""Documentation hygiene: every source file the documents name in backticks exists (a document
that points at a file that was moved or deleted is worse than no pointer)."""
import pathlib
import re

import pytest

ROOT = pathlib.Path(__file__).resolve().parent.parent
DOCS = [ROOT / "README.md", ROOT / "CHANGELOG.md", ROOT / "profiles" / "README.md"] + sorted((ROOT / "docs").glob("*.md"))
PATH = re.compile(r"`([A-Za-z0-9_./-]+\.(?:py|cu|cuh|cpp|h|md|json|toml|yml))(?:::[A-Za-z0-9_.]+)?`")
# where a short path may live
BASES = [ROOT, ROOT / "rmlx_b200", ROOT / "rmlx_b200" / "csrc", ROOT / "profiles", ROOT / "docs"]
# names of files that are not in the tree by design: the reference's files, driver-written files, patterns
SKIP = re.compile(r"^(crates/|\.github/|tools/|scripts/|docs/reports|MEASURED_PEAKS|BENCH_|SCALE_|GPUTEST|config\.json|"
                  r"model\.safetensors|.*\*.*|benchmarks/\*|bench/|shaders/)")


@pytest.mark.parametrize("doc", DOCS, ids=lambda p: p.name)
def test_named_files_exist(doc):
    missing = []
    for m in PATH.finditer(doc.read_text()):
        name = m.group(1)
        if SKIP.match(name) or name.endswith(".rs"):
            continue
        if not any((b / name).exists() for b in BASES):
            # a bare file name: anywhere in the package, the tests, the benchmarks or the examples
            if "/" not in name and any(ROOT.glob(f"**/{name}")):
                continue
            missing.append(name)
    assert not missing, f"{doc.name} names files that do not exist: {sorted(set(missing))}"
