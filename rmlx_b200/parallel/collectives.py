"""Stand-alone collectives over peer-mapped memory (csrc/comm/collectives.cu): all-gather,
all-to-all, reduce-scatter, two-shot all-reduce and broadcast, each one kernel launch with no host
work between ranks. ``parallel.group.Group`` offers the same operations on ``torch.distributed``
(NCCL on GPUs, gloo on CPU); that is the baseline and the oracle for these.

Counterpart of the reference's ``Group`` algorithms executed on the CPU over RDMA
(crates/rmlx-distributed/src/group.rs:648-1393).
"""
from __future__ import annotations

import ctypes

from typing import Optional

import torch
import torch.distributed as dist

from .. import _lib
from ..ops.gemm import GemmStatus
from .comm import SymmetricRegion

_lib.register_cuda_sigs({
    "rmlx_coll": ("ppiiiippqqiipp", "i"),
    "rmlx_coll_area_bytes": ("iq", "q"),
    "rmlx_nvls_allreduce": ("pqipiiip", "i"),
    "rmlx_nvls_flag_bytes": ("", "i"),
    "rmlx_nvls_status": ("", "i"),
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
        # in-switch all-reduce: an operand buffer and a flag area in the symmetric heap, usable
        # when the heap is bound to NVLink multicast objects (RMLX_SYMM_MULTICAST=1)
        self._nvls = None
        if getattr(self.region, "mc", 0):
            self.nvls_cap = self.cap * self.world
            flag_bytes = int(_lib.cuda().rmlx_nvls_flag_bytes())
            self._nvls = SymmetricRegion(self.nvls_cap + 256 + flag_bytes, group)
            self._nvls_flags = self._nvls.peer_array(self.nvls_cap + 256)

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

    @property
    def nvls_available(self) -> bool:
        return self._nvls is not None

    def nvls_buffer(self, dtype: torch.dtype, numel: int) -> torch.Tensor:
        """View of this rank's copy of the in-switch all-reduce operand: a producer that writes
        its partial result here saves the staging copy of ``all_reduce_nvls``."""
        from .tp_gemm import _RawCuda
        nbytes = numel * torch.empty(0, dtype=dtype).element_size()
        if nbytes > self.nvls_cap:
            raise ValueError(f"{nbytes} bytes exceed the operand buffer of {self.nvls_cap}")
        raw = torch.as_tensor(_RawCuda(self._nvls.local, nbytes), device=self.device)
        return raw.view(dtype)

    def all_reduce_nvls(self, x: Optional[torch.Tensor] = None, numel: Optional[int] = None,
                        dtype: Optional[torch.dtype] = None, out: Optional[torch.Tensor] = None):
        """Sum over ranks done by the NVLink switch (``multimem.ld_reduce`` + ``multimem.st``,
        csrc/comm/nvls.cu). With ``x`` the operand is staged into the heap buffer first; without it
        the buffer (``nvls_buffer(dtype, numel)``) is reduced in place and returned as a view."""
        if self._nvls is None:
            raise _lib.NativeError("the symmetric heap is not bound to NVLink multicast "
                                   "(RMLX_SYMM_MULTICAST=1 on a box that supports it)")
        if x is not None:
            x = x.contiguous()
            numel, dtype = x.numel(), x.dtype
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError("sums are implemented for bf16 and fp32")
        buf = self.nvls_buffer(dtype, numel)
        nbytes = buf.numel() * buf.element_size()
        if nbytes % 16:
            raise ValueError("the operand must be a whole number of 16-byte vectors")
        if x is not None:
            buf.copy_(x.view(-1))
        rc = _lib.cuda().rmlx_nvls_allreduce(ctypes.c_void_p(self._nvls.mc), nbytes,
                                             int(dtype == torch.bfloat16), self._nvls_flags, self.rank,
                                             self.world, 0, _lib.stream_ptr())
        _lib.check(rc, "nvls_allreduce")
        if x is None:
            return buf
        out = out if out is not None else torch.empty_like(x)
        out.view(-1).copy_(buf)
        return out

    def broadcast(self, x: torch.Tensor, root: int = 0, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        x = x.contiguous()
        out = out if out is not None else torch.empty_like(x)
        return self._run(BROADCAST, x, out, x.numel() * x.element_size(), root)

    def status(self) -> int:
        return int(GemmStatus.get(self.device).item()) or int(_lib.cuda().rmlx_nvls_status())

    def close(self) -> None:
        if self._nvls is not None:
            self._nvls.close()
            self._nvls = None
        self.region.close()
