"""Tensor-parallel communication for the decode path.

``PeerComm`` owns a symmetric region on every rank (same layout everywhere), maps every peer's
region into this process with CUDA IPC, and launches the fused kernels of
``csrc/comm/tp_decode.cu`` that push partial results straight into the peers' receive buffers over
NVLink. ``NcclComm`` offers the same interface on top of ``torch.distributed`` all-reduce; it is the
library baseline the fused path is measured against.

The reference's counterpart is the host-driven path: ``Group::allreduce_sum`` over RDMA between
command buffers (crates/rmlx-distributed/src/group.rs:648-675, crates/rmlx-nn/src/parallel.rs:619-693)
with rendezvous over TCP (crates/rmlx-distributed/src/init.rs:397-417). Here rendezvous is one
``all_gather_object`` of 64-byte IPC handles.
"""
from __future__ import annotations

import os

import ctypes
from typing import List, Optional

import torch
import torch.distributed as dist

from .. import _lib
from ..ops import decode as D
from ..ops.weights import LinearWeight

_lib.register_cuda_sigs({
    "rmlx_tp_status": ("", "i"),
    "rmlx_tp_set_stream": ("i", "i"),
    "rmlx_tp_stream_launches": ("", "q"),
    "rmlx_tp_gemv_allreduce": ("ippppipipiiiippiiiip", "i"),
    "rmlx_tp_moe_down_allreduce": ("ippppipppipiiiiiiippiiiip", "i"),
    "rmlx_tp_allreduce": ("pppiippiiqip", "i"),
    "rmlx_tp_argmax": ("piiiippppiiiip", "i"),
    "rmlx_tp_barrier": ("ppiiiip", "i"),
    "rmlx_symm_malloc": ("pq", "i"),
    "rmlx_symm_free": ("p", "i"),
    "rmlx_symm_get_handle": ("pp", "i"),
    "rmlx_symm_open_handle": ("pp", "i"),
    "rmlx_symm_close_handle": ("p", "i"),
})


def SymmetricRegion(nbytes: int, group=None):
    """Peer-mapped memory of ``nbytes`` per rank, zero-initialised, at the same offset of every
    rank's symmetric heap (``parallel.symm_heap``): ``local`` is this rank's address, ``ptrs[r]``
    the address, valid in this process, of rank r's copy. Falls back to one inter-process mapped
    allocation per call where the heap is unavailable or switched off (``RMLX_SYMM_HEAP=0``)."""
    from .symm_heap import default_heap
    heap = default_heap(group)
    if heap is not None:
        return heap.alloc(nbytes)
    return IpcRegion(nbytes, group)


class IpcRegion:
    """One device allocation per rank, of the same size, with every peer's copy mapped locally
    through the legacy inter-process memory handles."""

    def __init__(self, nbytes: int, group=None):
        lib = _lib.cuda()
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.nbytes = nbytes
        p = ctypes.c_void_p()
        _lib.check(lib.rmlx_symm_malloc(ctypes.byref(p), nbytes), "symm_malloc")
        self.local = p.value
        h = ctypes.create_string_buffer(64)
        _lib.check(lib.rmlx_symm_get_handle(ctypes.c_void_p(self.local), h), "symm_get_handle")
        handles: List[Optional[bytes]] = [None] * self.world
        dist.all_gather_object(handles, h.raw, group=group)
        self.ptrs: List[int] = []
        self._opened: List[int] = []
        for r, hb in enumerate(handles):
            if r == self.rank:
                self.ptrs.append(self.local)
                continue
            q = ctypes.c_void_p()
            buf = ctypes.create_string_buffer(hb, 64)
            _lib.check(lib.rmlx_symm_open_handle(buf, ctypes.byref(q)), "symm_open_handle")
            self.ptrs.append(q.value)
            self._opened.append(q.value)
        dist.barrier(group=group)

    def peer_array(self, byte_offset: int = 0):
        arr = (ctypes.c_void_p * self.world)()
        for r in range(self.world):
            arr[r] = self.ptrs[r] + byte_offset
        return arr

    def close(self) -> None:
        lib = _lib.cuda()
        torch.cuda.synchronize()
        dist.barrier(group=self.group)
        for q in self._opened:
            lib.rmlx_symm_close_handle(ctypes.c_void_p(q))
        self._opened = []
        if self.local:
            lib.rmlx_symm_free(ctypes.c_void_p(self.local))
            self.local = 0


class PeerComm:
    """Fused projection + all-reduce over peer memory for decode batches of up to ``max_batch``.

    Every all-reduce, whatever its kind, takes its arrival tag and its receive slot from one
    sequence number kept on the device (the last block of a call advances it), so captured and
    eager calls can be mixed freely and consecutive calls always alternate slots; the host keeps no
    slot state."""

    kind = "fused"
    SLOTS = 2

    def __init__(self, hidden: int, max_batch: int, group=None, device=None):
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.N, self.B = hidden, max_batch
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        w = self.world
        self.slot_floats = w * max_batch * hidden
        self.recv_bytes = self.SLOTS * self.slot_floats * 8      # 8-byte (value, tag) words
        # counters: [0] all-reduces completed, [1] exit ticket; then arg-max counters; then barrier word
        self.ctr_off = self.recv_bytes
        self.ctr_argmax_off = self.ctr_off + 16
        self.ctr_barrier_off = self.ctr_argmax_off + 2 * self.SLOTS * 4
        self.key_off = (self.ctr_barrier_off + 16 + 255) // 256 * 256
        self.key_bytes = self.SLOTS * max_batch * w * 8
        total = self.key_off + self.key_bytes
        self.region = SymmetricRegion(total, group)
        self._recv = self.region.peer_array(0)
        self._ctr = self.region.peer_array(self.ctr_off)
        self._ctr_argmax = self.region.peer_array(self.ctr_argmax_off)
        self._ctr_barrier = self.region.peer_array(self.ctr_barrier_off)
        keys = [self.region.ptrs[r] + self.key_off for r in range(w)]
        self._keys_dev = torch.tensor(keys, dtype=torch.int64, device=self.device)
        self._n = 0           # collective calls issued (statistics only)
        self._n_argmax = 0
        # The fused projections run on the weight-streaming kernels or on the per-row kernels
        # (both speak the same receive-area protocol). Measured on the 60-layer model, batch 1:
        # per-row 247 vs streaming 240 tok/s at 2 GPUs, 267 vs 292 at 4, so streaming is the
        # default from 4 ranks on; RMLX_TP_STREAM=0/1 overrides.
        env = os.environ.get("RMLX_TP_STREAM")
        self.stream = (self.world >= 4) if env is None else env != "0"
        _lib.cuda().rmlx_tp_set_stream(int(self.stream))
        self._barrier_epoch = 0

    # ------------------------------------------------------------------
    def calls_issued(self) -> int:
        return self._n

    def gemv_allreduce(self, x: torch.Tensor, w: LinearWeight, residual: Optional[torch.Tensor],
                       out: torch.Tensor, pdl: bool = False) -> torch.Tensor:
        """out = residual + sum over ranks of (W_r @ x_r): x is this rank's K shard, [B, K_local]."""
        b, k = x.shape
        assert b <= self.B and w.n == self.N and out.dtype == torch.bfloat16
        lib, st = _lib.cuda(), _lib.stream_ptr()
        for b0 in range(0, b, 4):
            bb = min(4, b - b0)
            self._n += 1
            xs, os_ = x[b0:b0 + bb], out[b0:b0 + bb]
            rs = None if residual is None else residual[b0:b0 + bb]
            rc = lib.rmlx_tp_gemv_allreduce(
                w.kernel_kind, w.w.data_ptr(), _lib.ptr(w.scales), _lib.ptr(w.biases), xs.data_ptr(),
                xs.stride(0), _lib.ptr(rs), 0 if rs is None else rs.stride(0), os_.data_ptr(),
                os_.stride(0), bb, self.N, k, self._recv, self._ctr, self.rank, self.world,
                self.B, int(pdl), st)
            _lib.check(rc, "tp_gemv_allreduce")
        return out

    def moe_down_allreduce(self, act: torch.Tensor, w: LinearWeight, idx: torch.Tensor,
                           wts: torch.Tensor, residual: Optional[torch.Tensor], out: torch.Tensor,
                           expert_base: int = 0, pdl: bool = False) -> torch.Tensor:
        b, top_k = idx.shape
        assert b <= self.B and w.n == self.N
        self._n += 1
        rc = _lib.cuda().rmlx_tp_moe_down_allreduce(
            w.kernel_kind, w.w.data_ptr(), _lib.ptr(w.scales), _lib.ptr(w.biases), act.data_ptr(),
            act.stride(0), idx.data_ptr(), wts.data_ptr(), _lib.ptr(residual),
            0 if residual is None else residual.stride(0), out.data_ptr(), out.stride(0), b, top_k,
            self.N, w.k, expert_base, w.experts, self._recv, self._ctr, self.rank, self.world,
            self.B, int(pdl), _lib.stream_ptr())
        _lib.check(rc, "tp_moe_down_allreduce")
        return out

    def allreduce(self, x: torch.Tensor, residual: Optional[torch.Tensor] = None,
                  out: Optional[torch.Tensor] = None, pdl: bool = False) -> torch.Tensor:
        """One-shot all-reduce of a small fp32 tensor (numel <= max_batch * hidden)."""
        assert x.dtype == torch.float32 and x.is_contiguous() and x.numel() <= self.B * self.N
        if out is None:
            out = torch.empty_like(x)
        self._n += 1
        rc = _lib.cuda().rmlx_tp_allreduce(x.data_ptr(), _lib.ptr(residual), out.data_ptr(),
                                           int(out.dtype == torch.float32), x.numel(), self._recv,
                                           self._ctr, self.rank, self.world, self.slot_floats,
                                           int(pdl), _lib.stream_ptr())
        _lib.check(rc, "tp_allreduce")
        return out

    def argmax(self, logits_local: torch.Tensor, vocab_base: int, out: torch.Tensor,
               pdl: bool = False) -> torch.Tensor:
        """Global arg-max over vocabulary shards: every rank ends with the same token ids."""
        b, v = logits_local.shape
        assert b <= self.B
        s = self._n_argmax % self.SLOTS
        self._n_argmax += 1
        rc = _lib.cuda().rmlx_tp_argmax(logits_local.data_ptr(), v, logits_local.stride(0),
                                        vocab_base, b, out.data_ptr(), self._keys_dev.data_ptr(),
                                        self._recv, self._ctr_argmax, self.rank, self.world, s,
                                        int(pdl), _lib.stream_ptr())
        _lib.check(rc, "tp_argmax")
        return out

    def barrier(self) -> None:
        self._barrier_epoch += 1
        rc = _lib.cuda().rmlx_tp_barrier(self._recv, self._ctr_barrier, self.rank, self.world, 0,
                                         self._barrier_epoch, _lib.stream_ptr())
        _lib.check(rc, "tp_barrier")

    def stream_launches(self) -> int:
        """Fused projections of this process that ran on the weight-streaming kernel."""
        return int(_lib.cuda().rmlx_tp_stream_launches())

    def status(self) -> int:
        """0, or the code of a device-side wait that gave up since the last call."""
        return int(_lib.cuda().rmlx_tp_status())

    def close(self) -> None:
        self.region.close()


class NcclComm:
    """Same interface through NCCL: local partial in fp32, ``all_reduce``, residual add."""

    kind = "nccl"

    def __init__(self, hidden: int, max_batch: int, group=None, device=None):
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.partial = torch.zeros(max_batch, hidden, dtype=torch.float32, device=self.device)
        self._n = 0

    def calls_issued(self) -> int:
        return self._n

    def gemv_allreduce(self, x, w, residual, out, pdl=False):
        self._n += 1
        p = self.partial[:x.shape[0]]
        D.rms_gemv(x, w, None, 0.0, out=p, pdl=False)
        dist.all_reduce(p, group=self.group)
        out.copy_(p + residual.float() if residual is not None else p)
        return out

    def moe_down_allreduce(self, act, w, idx, wts, residual, out, expert_base=0, pdl=False):
        self._n += 1
        p = self.partial[:idx.shape[0]]
        D.moe_down(act, w, idx, wts, residual=None, out=p, expert_base=expert_base, pdl=False)
        dist.all_reduce(p, group=self.group)
        out.copy_(p + residual.float() if residual is not None else p)
        return out

    def allreduce(self, x, residual=None, out=None, pdl=False):
        self._n += 1
        y = x.clone()
        dist.all_reduce(y, group=self.group)
        if residual is not None:
            y = y + residual.float()
        if out is None:
            return y
        out.copy_(y)
        return out

    def argmax(self, logits_local, vocab_base, out, pdl=False):
        val, idx = logits_local.max(dim=-1)
        vals = [torch.empty_like(val) for _ in range(self.world)]
        idxs = [torch.empty_like(idx) for _ in range(self.world)]
        dist.all_gather(vals, val, group=self.group)
        dist.all_gather(idxs, idx + vocab_base, group=self.group)
        v = torch.stack(vals, 0)
        i = torch.stack(idxs, 0)
        # largest value; ties go to the lowest rank, which holds the lowest vocabulary ids
        best = torch.argmax(v, dim=0)
        out.copy_(i.gather(0, best[None]).squeeze(0).to(torch.int32))
        return out

    def barrier(self):
        dist.barrier(group=self.group)

    def status(self) -> int:
        return 0

    def close(self):
        pass


def make_comm(kind: str, model, max_batch: int, group=None):
    hidden = model.cfg.hidden_size
    if kind == "fused":
        return PeerComm(hidden, max_batch, group, model.device)
    if kind == "nccl":
        return NcclComm(hidden, max_batch, group, model.device)
    raise ValueError(f"unknown comm kind {kind}")
