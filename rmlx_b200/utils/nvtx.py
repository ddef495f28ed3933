"""NVTX ranges around layers and kernels (visible in Nsight Systems timelines), no-ops on CPU or
when disabled. The reference's counterpart is its capture scope / per-dispatch breakdown hooks
(crates/rmlx-metal/src/capture.rs:46-105, crates/rmlx-nn/src/transformer.rs:3215-3600)."""
from __future__ import annotations

import contextlib
import os

import torch

_ENABLED = os.environ.get("RMLX_NVTX", "0") not in ("", "0", "false", "False")


def enable(on: bool = True) -> None:
    global _ENABLED
    _ENABLED = on


def enabled() -> bool:
    return _ENABLED and torch.cuda.is_available()


@contextlib.contextmanager
def range(name: str):
    if not enabled():
        yield
        return
    torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        torch.cuda.nvtx.range_pop()


def mark(name: str) -> None:
    if enabled():
        torch.cuda.nvtx.mark(name)
