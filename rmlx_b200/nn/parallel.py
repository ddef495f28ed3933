"""Megatron-style tensor-parallel linears over a ``Group``.

``ColumnParallelLinear``: every rank holds a slice of the output rows; forward = local GEMM then
all-gather of the outputs (skipped with ``gather_output=False`` when a row-parallel layer follows).
``RowParallelLinear``: every rank holds a slice of the input columns; forward = local GEMM on its
input shard then all-reduce, bias added once. Quantised shards re-slice packed words, scales and
biases together. Same contracts as crates/rmlx-nn/src/parallel.rs:31-1130. These are the general
layers (prefill, tests, baselines); decode uses the fused kernels in ``parallel.comm``."""
from __future__ import annotations

from typing import Optional

import torch

from ..ops.weights import LinearWeight
from ..parallel.group import Group
from .layers import Linear


def shard_column(w: LinearWeight, rank: int, world: int) -> LinearWeight:
    assert w.n % world == 0
    n = w.n // world
    return w.rows(rank * n, (rank + 1) * n)


def shard_row(w: LinearWeight, rank: int, world: int) -> LinearWeight:
    assert w.k % world == 0
    k = w.k // world
    return w.cols(rank * k, (rank + 1) * k)


def shard_column_segments(w: LinearWeight, segments, rank: int, world: int) -> LinearWeight:
    """Merged weights (e.g. Q|K|V or gate|up): shard every segment separately and re-merge."""
    parts, lo = [], 0
    for seg in segments:
        assert seg % world == 0
        n = seg // world
        parts.append(w.rows(lo + rank * n, lo + (rank + 1) * n))
        lo += seg
    return LinearWeight.cat_rows(parts)


class ColumnParallelLinear:
    def __init__(self, full: LinearWeight, group: Group, bias: Optional[torch.Tensor] = None,
                 gather_output: bool = True):
        self.group = group
        r, w = group.local_rank, group.world_size
        self.local = Linear(shard_column(full, r, w),
                            None if bias is None else bias[r * full.n // w:(r + 1) * full.n // w])
        self.gather_output = gather_output
        self.out_features = full.n

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        y = self.local(x)
        if not self.gather_output or self.group.single:
            return y
        return self.group.allgather(y, dim=-1) if y.dim() == 1 else \
            self.group.allgather(y.reshape(-1, y.shape[-1]).t().contiguous(), dim=0).t().reshape(
                *y.shape[:-1], self.out_features)

    __call__ = forward


class RowParallelLinear:
    def __init__(self, full: LinearWeight, group: Group, bias: Optional[torch.Tensor] = None,
                 input_is_parallel: bool = True):
        self.group = group
        r, w = group.local_rank, group.world_size
        self.local = Linear(shard_row(full, r, w))
        self.bias = bias
        self.input_is_parallel = input_is_parallel
        self.k_local = full.k // w

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if not self.input_is_parallel:
            r = self.group.local_rank
            x = x[..., r * self.k_local:(r + 1) * self.k_local]
        y = self.local(x.contiguous())
        y = self.group.allreduce(y)
        if self.bias is not None:
            y = y + self.bias.to(y.dtype)
        return y

    __call__ = forward
