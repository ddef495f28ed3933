"""MPI-style process group over ``torch.distributed`` (NCCL on GPUs, gloo on CPU).

API of the reference's ``Group`` (crates/rmlx-distributed/src/group.rs:166-848): ``allreduce`` with
Sum / Max / Min, ``allgather``, ``broadcast``, ``send`` / ``recv`` / ``sendrecv``, ``all_to_all``,
``reduce_scatter``, ``barrier``, ``split(color, key)``. A group of one rank returns identities
without touching any backend (the reference's single-rank stub mode, group.rs:348-356,837-847).
Reductions of bf16 / fp16 accumulate in fp32 (group.rs:1094-1160); unlike the reference's
``allreduce_sum`` (group.rs:648-675 sums raw half-precision bytes as fp32 words) every path here is
dtype-correct.

The hot paths do not go through this class: decode uses the fused peer-memory kernels of
``parallel.comm``. This is the general-purpose / bootstrap / baseline layer.
"""
from __future__ import annotations

import os

from enum import Enum
from typing import List, Optional, Sequence

import torch
import torch.distributed as dist


class DistributedError(RuntimeError):
    pass


class ReduceOp(Enum):
    SUM = "sum"
    MAX = "max"
    MIN = "min"


_OPS = {ReduceOp.SUM: dist.ReduceOp.SUM, ReduceOp.MAX: dist.ReduceOp.MAX, ReduceOp.MIN: dist.ReduceOp.MIN}


class Group:
    """Collectives of one process group. CUDA tensors go through this package's peer-memory
    kernels (``parallel.collectives.PeerCollectives`` over the symmetric heap: all-reduce,
    all-gather, reduce-scatter, all-to-all, broadcast) whenever the call fits them (sum, bf16 or
    fp32, pieces of whole 16-byte vectors); everything else, and every CPU tensor, goes to
    ``torch.distributed`` (NCCL / gloo), the last resort. ``RMLX_GROUP_NATIVE=0`` switches the
    native path off; ``native_calls`` / ``library_calls`` count which way calls went.
    Reference: crates/rmlx-distributed/src/group.rs:348-964 (ring / tree / mesh algorithms over
    RDMA selected by size)."""

    def __init__(self, pg=None, ranks: Optional[List[int]] = None):
        """``pg``: a torch process group (None = the default group when initialised, else a
        single-rank group)."""
        self._pg = pg
        self._pc = None
        self._chan = None
        self.native_calls = 0
        self.library_calls = 0
        if dist.is_available() and dist.is_initialized():
            self.local_rank = dist.get_rank(pg)
            self.world_size = dist.get_world_size(pg)
            self.ranks = ranks or list(range(self.world_size))
        else:
            self.local_rank, self.world_size, self.ranks = 0, 1, [0]

    # ------------------------------------------------------------------ helpers
    @property
    def single(self) -> bool:
        return self.world_size == 1

    def _global(self, group_rank: int) -> int:
        if self._pg is None:
            return group_rank
        return dist.get_global_rank(self._pg, group_rank)

    @staticmethod
    def _widen(t: torch.Tensor):
        if t.dtype in (torch.bfloat16, torch.float16):
            return t.float(), t.dtype
        return t, None

    # ------------------------------------------------------------------ native path
    def _native(self, t: torch.Tensor, piece_bytes: int, summed: bool = False):
        """The peer-memory collectives for a call that moves pieces of ``piece_bytes`` per rank,
        or None when the call has to go to the library. Creating (or growing) the communicator is
        collective; every rank takes the same decision because it depends on shapes only."""
        if (self.single or not t.is_cuda or piece_bytes <= 0 or piece_bytes % 16 or
                os.environ.get("RMLX_GROUP_NATIVE", "1") == "0"):
            return None
        if summed and t.dtype not in (torch.bfloat16, torch.float32):
            return None
        if piece_bytes > (64 << 20):            # large transfers: the library's pipelined rings
            return None
        if self._pc is None or piece_bytes > self._pc.cap:
            from .collectives import PeerCollectives
            if self._pc is not None:
                self._pc.close()
            cap = 1 << 20
            while cap < piece_bytes:
                cap <<= 1
            self._pc = PeerCollectives(cap, group=self._pg, device=t.device)
        self.native_calls += 1
        return self._pc

    def enable_native_p2p(self, slot_bytes: int, device=None) -> None:
        """Collective: create the mailboxes that let ``send`` / ``recv`` / ``sendrecv`` of CUDA
        tensors up to ``slot_bytes`` run as peer stores plus counters (``parallel.p2p.PeerChannel``)
        instead of library point-to-point calls."""
        if self.single or self._chan is not None:
            return
        from .p2p import PeerChannel
        self._chan = PeerChannel(slot_bytes, group=self._pg, device=device)

    def _p2p(self, t: torch.Tensor):
        if self._chan is None or not t.is_cuda or t.numel() * t.element_size() > self._chan.slot_bytes:
            return None
        self.native_calls += 1
        return self._chan

    def close(self) -> None:
        """Release the native communicators (collective)."""
        if self._pc is not None:
            self._pc.close()
            self._pc = None
        if self._chan is not None:
            self._chan.close()
            self._chan = None

    # ------------------------------------------------------------------ collectives
    def allreduce(self, t: torch.Tensor, op: ReduceOp = ReduceOp.SUM) -> torch.Tensor:
        if self.single:
            return t.clone()
        if op == ReduceOp.SUM and t.numel() % self.world_size == 0:
            pc = self._native(t, t.numel() * t.element_size() // self.world_size, summed=True)
            if pc is not None:
                return pc.all_reduce(t.contiguous()).view(t.shape)
        self.library_calls += 1
        w, narrow = self._widen(t.contiguous())
        w = w.clone()
        dist.all_reduce(w, op=_OPS[op], group=self._pg)
        return w.to(narrow) if narrow is not None else w

    def allreduce_in_place(self, t: torch.Tensor, op: ReduceOp = ReduceOp.SUM) -> torch.Tensor:
        if self.single:
            return t
        if t.dtype in (torch.bfloat16, torch.float16) or not t.is_contiguous():
            t.copy_(self.allreduce(t, op))
        else:
            dist.all_reduce(t, op=_OPS[op], group=self._pg)
        return t

    def allreduce_sum(self, t: torch.Tensor) -> torch.Tensor:
        return self.allreduce(t, ReduceOp.SUM)

    def allgather(self, t: torch.Tensor, dim: int = 0) -> torch.Tensor:
        if self.single:
            return t.clone()
        if dim == 0 and t.dim() >= 1:
            pc = self._native(t, t.numel() * t.element_size())
            if pc is not None:
                return pc.all_gather(t.contiguous())
        self.library_calls += 1
        parts = [torch.empty_like(t) for _ in range(self.world_size)]
        dist.all_gather(parts, t.contiguous(), group=self._pg)
        return torch.cat(parts, dim)

    def broadcast(self, t: torch.Tensor, root: int = 0) -> torch.Tensor:
        if self.single:
            return t
        if t.is_contiguous():
            pc = self._native(t, t.numel() * t.element_size())
            if pc is not None:
                t.copy_(pc.broadcast(t, root=root))
                return t
        self.library_calls += 1
        dist.broadcast(t, src=self._global(root), group=self._pg)
        return t

    def reduce_scatter(self, t: torch.Tensor, op: ReduceOp = ReduceOp.SUM) -> torch.Tensor:
        """Input [world * n, ...] -> this rank's reduced chunk [n, ...]."""
        if self.single:
            return t.clone()
        if t.shape[0] % self.world_size:
            raise DistributedError("reduce_scatter: leading dim must divide by the world size")
        if op == ReduceOp.SUM:
            pc = self._native(t, t.numel() * t.element_size() // self.world_size, summed=True)
            if pc is not None:
                return pc.reduce_scatter(t.contiguous())
        self.library_calls += 1
        w, narrow = self._widen(t.contiguous())
        n = t.shape[0] // self.world_size
        if w.is_cuda:
            out = torch.empty((n, *w.shape[1:]), dtype=w.dtype, device=w.device)
            dist.reduce_scatter_tensor(out, w, op=_OPS[op], group=self._pg)
        else:   # gloo has no reduce_scatter: all-reduce then slice
            w = w.clone()
            dist.all_reduce(w, op=_OPS[op], group=self._pg)
            out = w[self.local_rank * n:(self.local_rank + 1) * n].clone()
        return out.to(narrow) if narrow is not None else out

    def all_to_all(self, t: torch.Tensor, send_counts: Optional[Sequence[int]] = None,
                   recv_counts: Optional[Sequence[int]] = None) -> torch.Tensor:
        """Rows of ``t`` are split by ``send_counts`` (equal split when None) and exchanged."""
        if self.single:
            return t.clone()
        t = t.contiguous()
        if send_counts is None:
            if t.shape[0] % self.world_size:
                raise DistributedError("all_to_all: rows must divide by the world size")
            pc = self._native(t, t.numel() * t.element_size() // self.world_size)
            if pc is not None:
                return pc.all_to_all(t)
            send_counts = recv_counts = [t.shape[0] // self.world_size] * self.world_size
        elif recv_counts is None:
            sc = torch.tensor(list(send_counts), dtype=torch.int64, device=t.device)
            rc = torch.empty_like(sc)
            dist.all_to_all_single(rc, sc, group=self._pg)
            recv_counts = rc.tolist()
        out = torch.empty((int(sum(recv_counts)), *t.shape[1:]), dtype=t.dtype, device=t.device)
        dist.all_to_all_single(out, t, list(recv_counts), list(send_counts), group=self._pg)
        return out

    def send(self, t: torch.Tensor, dst: int) -> None:
        if self.single:
            raise DistributedError("send on a single-rank group")
        ch = self._p2p(t)
        if ch is not None:
            return ch.send(t, dst)
        self.library_calls += 1
        dist.send(t.contiguous(), dst=self._global(dst), group=self._pg)

    def recv(self, t: torch.Tensor, src: int) -> torch.Tensor:
        if self.single:
            raise DistributedError("recv on a single-rank group")
        ch = self._p2p(t)
        if ch is not None and t.is_contiguous():
            return ch.recv(t, src)
        self.library_calls += 1
        dist.recv(t, src=self._global(src), group=self._pg)
        return t

    def sendrecv(self, send: torch.Tensor, recv: torch.Tensor, peer: int) -> torch.Tensor:
        if self.single:
            raise DistributedError("sendrecv on a single-rank group")
        ch = self._p2p(send)
        if ch is not None and recv.is_contiguous() and self._p2p(recv) is not None:
            return ch.sendrecv(send, recv, peer)
        self.library_calls += 1
        ops = [dist.P2POp(dist.isend, send.contiguous(), self._global(peer), self._pg),
               dist.P2POp(dist.irecv, recv, self._global(peer), self._pg)]
        for r in dist.batch_isend_irecv(ops):
            r.wait()
        return recv

    def shift(self, send: torch.Tensor, recv: torch.Tensor, dst: int, src: int) -> torch.Tensor:
        """Send ``send`` to ``dst`` while receiving ``recv`` from ``src`` (the step of a ring: two
        different peers, both transfers in flight together, so no ordering between ranks can
        deadlock)."""
        if self.single:
            raise DistributedError("shift on a single-rank group")
        ch = self._p2p(send)
        if ch is not None and recv.is_contiguous() and self._p2p(recv) is not None:
            ch.send(send, dst)                      # a put plus a signal: does not wait for the receiver
            return ch.recv(recv, src)
        self.library_calls += 1
        ops = [dist.P2POp(dist.isend, send.contiguous(), self._global(dst), self._pg),
               dist.P2POp(dist.irecv, recv, self._global(src), self._pg)]
        for r in dist.batch_isend_irecv(ops):
            r.wait()
        return recv

    def barrier(self) -> None:
        if not self.single:
            dist.barrier(group=self._pg)

    def split(self, color: int, key: int = 0) -> "Group":
        """Ranks with the same colour form a new group, ordered by (key, old rank)."""
        if self.single:
            return Group(self._pg, [0])
        mine = torch.tensor([color, key, self.local_rank], dtype=torch.int64)
        dev = "cuda" if dist.get_backend(self._pg) == "nccl" else "cpu"
        allv = [torch.empty(3, dtype=torch.int64, device=dev) for _ in range(self.world_size)]
        dist.all_gather(allv, mine.to(dev), group=self._pg)
        rows = [tuple(int(x) for x in v.tolist()) for v in allv]
        colours = sorted(set(c for c, _, _ in rows))
        new = None
        for c in colours:   # every rank creates every subgroup, in the same order
            members = [r for _, _, r in sorted((k, r, r) for cc, k, r in rows if cc == c)]
            pg = dist.new_group([self._global(r) for r in members])
            if c == color:
                new = Group(pg, members)
        return new
