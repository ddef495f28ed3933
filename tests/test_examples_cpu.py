"""The scripts under examples/ run end to end on CPU."""
import importlib
import os
import sys

import pytest

EX = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "examples")


@pytest.fixture()
def examples_on_path():
    sys.path.insert(0, EX)
    yield
    sys.path.remove(EX)
    for m in ("generate", "serve_requests", "speculative", "deepseek_paged"):
        sys.modules.pop(m, None)


def test_generate_example(examples_on_path):
    toks = importlib.import_module("generate").main(["--steps", "5", "--device", "cpu"])
    assert len(toks) == 5


def test_serve_requests_example(examples_on_path):
    outs = importlib.import_module("serve_requests").main(
        ["--requests", "3", "--max-batch", "1", "--max-new", "3", "--device", "cpu"])
    assert len(outs) == 3 and all(len(v) == 3 for v in outs.values())


def test_speculative_example(examples_on_path):
    out = importlib.import_module("speculative").main(["--k", "3", "--steps", "9"])
    assert len(out) == 9


def test_deepseek_paged_example(examples_on_path):
    out = importlib.import_module("deepseek_paged").main(["--steps", "4"])
    assert len(out) == 2 and all(len(o) == 4 for o in out)
