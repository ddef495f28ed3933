"""Stand-alone collectives over peer-mapped memory (csrc/comm/collectives.cu): all-gather,
all-to-all, reduce-scatter, two-shot all-reduce and broadcast, each one kernel launch with no host
work between ranks. ``parallel.group.Group`` offers the same operations on ``torch.distributed``
(NCCL on GPUs, gloo on CPU); that is the baseline and the oracle for these.

Counterpart of the reference's ``Group`` algorithms executed on the CPU over RDMA
(crates/rmlx-distributed/src/group.rs:648-1393).
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from .. import _lib
from ..ops.gemm import GemmStatus
from .comm import SymmetricRegion

_lib.register_cuda_sigs({
    "rmlx_coll": ("ppiiiippqqiipp", "i"),
    "rmlx_coll_area_bytes": ("iq", "q"),
})

ALL_GATHER, ALL_TO_ALL, REDUCE_SCATTER, ALL_REDUCE, BROADCAST = range(5)


class PeerCollectives:
    """``max_chunk_bytes``: the largest per-rank piece any call will move (an all-reduce of n bytes
    moves pieces of n / world)."""

    def __init__(self, max_chunk_bytes: int, group=None, device=None, blocks: int = 32):
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.cap = (max_chunk_bytes + 255) // 256 * 256
        self.blocks = blocks
        area = int(_lib.cuda().rmlx_coll_area_bytes(self.world, self.cap))
        self.region = SymmetricRegion(area + 256, group)
        self._buf = self.region.peer_array(0)
        self._ctl = self.region.peer_array(area)

    def _run(self, op: int, src: torch.Tensor, dst: torch.Tensor, chunk_bytes: int, root: int = 0) -> torch.Tensor:
        assert src.is_contiguous() and dst.is_contiguous() and src.is_cuda and dst.is_cuda
        if chunk_bytes % 16 or chunk_bytes > self.cap:
            raise ValueError(f"piece of {chunk_bytes} bytes: must be a multiple of 16 and at most {self.cap}")
        bf16 = 1 if src.dtype == torch.bfloat16 else 0
        if op in (REDUCE_SCATTER, ALL_REDUCE) and src.dtype not in (torch.bfloat16, torch.float32):
            raise ValueError("sums are implemented for bf16 and fp32")
        blocks = max(4, min(self.blocks, chunk_bytes * self.world // 65536))   # small messages: few CTAs
        rc = _lib.cuda().rmlx_coll(self._buf, self._ctl, self.rank, self.world, op, bf16, src.data_ptr(),
                                   dst.data_ptr(), chunk_bytes, self.cap, root, blocks,
                                   GemmStatus.get(self.device).data_ptr(), _lib.stream_ptr())
        _lib.check(rc, "coll")
        return dst

    def all_gather(self, x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """x [n, ...] -> [world*n, ...] in rank order."""
        x = x.contiguous()
        out = out if out is not None else x.new_empty((self.world * x.shape[0],) + tuple(x.shape[1:]))
        return self._run(ALL_GATHER, x, out, x.numel() * x.element_size())

    def all_to_all(self, x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """x [world*n, ...]: piece p goes to rank p; the result holds the pieces in source order."""
        x = x.contiguous()
        out = out if out is not None else torch.empty_like(x)
        return self._run(ALL_TO_ALL, x, out, x.numel() * x.element_size() // self.world)

    def reduce_scatter(self, x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """x [world*n, ...] -> sum over ranks of piece ``rank``: [n, ...]."""
        x = x.contiguous()
        out = out if out is not None else x.new_empty((x.shape[0] // self.world,) + tuple(x.shape[1:]))
        return self._run(REDUCE_SCATTER, x, out, x.numel() * x.element_size() // self.world)

    def all_reduce(self, x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Sum over ranks (two-shot: reduce-scatter then all-gather inside one kernel). The element
        count must split into ``world`` pieces of whole 16-byte vectors."""
        x = x.contiguous()
        out = out if out is not None else torch.empty_like(x)
        return self._run(ALL_REDUCE, x, out, x.numel() * x.element_size() // self.world)

    def broadcast(self, x: torch.Tensor, root: int = 0, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        x = x.contiguous()
        out = out if out is not None else torch.empty_like(x)
        return self._run(BROADCAST, x, out, x.numel() * x.element_size(), root)

    def status(self) -> int:
        return int(GemmStatus.get(self.device).item())

    def close(self) -> None:
        self.region.close()
