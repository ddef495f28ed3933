"""Point-to-point messages between ranks over the symmetric heap: ``PeerChannel.send`` stores the
tensor into a mailbox slot in the RECEIVER's memory and bumps a counter there; ``recv`` waits for
the counter on the stream (bounded) and copies the slot out. ``put`` / ``get`` are the one-sided
forms (no handshake). Everything is asynchronous on the current stream; nothing passes through the
host or a collective library.

The NVLink counterpart of the reference's RDMA connection layer: ``post_send`` / ``post_recv`` /
completion polling on a queue pair with chunking (crates/rmlx-rdma/src/connection.rs,
connection_manager.rs) and of ``Group::send`` / ``recv`` / ``sendrecv``
(crates/rmlx-distributed/src/group.rs:232-346)."""
from __future__ import annotations

import ctypes
from typing import Optional

import torch
import torch.distributed as dist

from .. import _lib
from .comm import SymmetricRegion
from .tp_gemm import _RawCuda, _align

_lib.register_cuda_sigs({
    "rmlx_p2p_put": ("ppqppip", "i"),
    "rmlx_p2p_signal": ("pip", "i"),
    "rmlx_p2p_wait": ("piip", "i"),
    "rmlx_p2p_status": ("", "i"),
})


class PeerChannel:
    """Mailboxes of ``slot_bytes`` per (receiver, sender) pair. Layout of every rank's block:
    ``world`` slots (slot s holds what rank s sent here), then per sender a 'sent' counter (bumped
    by the sender when a message has landed) and a 'consumed' counter (bumped by this rank when it
    has copied a message out, so the sender may overwrite the slot)."""

    def __init__(self, slot_bytes: int, group=None, device=None):
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.slot_bytes = _align(slot_bytes)
        self.off_flags = self.world * self.slot_bytes
        total = self.off_flags + _align(self.world * 16)
        self.region = SymmetricRegion(total, group)
        self._sent = [0] * self.world        # messages this rank has sent to r
        self._received = [0] * self.world    # messages this rank has taken from r

    # ---- addresses ------------------------------------------------------------------------
    def _slot(self, owner: int, sender: int) -> int:
        return self.region.ptrs[owner] + sender * self.slot_bytes

    def _flag(self, owner: int, peer: int, which: int) -> int:
        """which 0: 'sent' counter of messages from ``peer`` into ``owner``; 1: 'consumed' counter
        kept in ``owner``'s memory for messages ``owner`` sent to ``peer``; 2: ticket word."""
        return self.region.ptrs[owner] + self.off_flags + peer * 16 + which * 4

    # ---- one-sided ------------------------------------------------------------------------
    def put(self, dst_rank: int, t: torch.Tensor, slot: Optional[int] = None) -> None:
        """Store ``t`` into slot ``slot`` (default: this rank's) of ``dst_rank``; no handshake."""
        t = t.contiguous()
        nbytes = t.numel() * t.element_size()
        assert nbytes <= self.slot_bytes
        rc = _lib.cuda().rmlx_p2p_put(ctypes.c_void_p(self._slot(dst_rank, self.rank if slot is None else slot)),
                                      t.data_ptr(), nbytes, None, None, 0, _lib.stream_ptr())
        _lib.check(rc, "p2p_put")

    def get(self, src_rank: int, like: torch.Tensor, slot: int) -> torch.Tensor:
        """Read slot ``slot`` of ``src_rank``'s block into a tensor shaped like ``like``."""
        out = torch.empty_like(like).contiguous()
        rc = _lib.cuda().rmlx_p2p_put(out.data_ptr(), ctypes.c_void_p(self._slot(src_rank, slot)),
                                      out.numel() * out.element_size(), None, None, 0, _lib.stream_ptr())
        _lib.check(rc, "p2p_get")
        return out

    # ---- two-sided ------------------------------------------------------------------------
    def send(self, t: torch.Tensor, dst: int) -> None:
        """Message to ``dst``: waits (on the stream) until ``dst`` has consumed the previous one,
        stores the payload into its mailbox and bumps its 'sent' counter."""
        t = t.contiguous()
        nbytes = t.numel() * t.element_size()
        assert dst != self.rank and nbytes <= self.slot_bytes
        lib, st = _lib.cuda(), _lib.stream_ptr()
        n = self._sent[dst]
        if n > 0:      # the slot is free once message n-1 has been copied out
            _lib.check(lib.rmlx_p2p_wait(ctypes.c_void_p(self._flag(self.rank, dst, 1)), n, 0, st), "p2p_wait")
        rc = lib.rmlx_p2p_put(ctypes.c_void_p(self._slot(dst, self.rank)), t.data_ptr(), nbytes,
                              ctypes.c_void_p(self._flag(dst, self.rank, 0)),
                              ctypes.c_void_p(self._flag(self.rank, dst, 2)), 0, st)
        _lib.check(rc, "p2p_send")
        self._sent[dst] = n + 1

    def recv(self, out: torch.Tensor, src: int) -> torch.Tensor:
        """Wait (on the stream, bounded) for the next message from ``src``, copy it into ``out``
        and tell ``src`` its slot is free."""
        assert src != self.rank and out.is_contiguous()
        lib, st = _lib.cuda(), _lib.stream_ptr()
        n = self._received[src] + 1
        _lib.check(lib.rmlx_p2p_wait(ctypes.c_void_p(self._flag(self.rank, src, 0)), n, 0, st), "p2p_wait")
        nbytes = out.numel() * out.element_size()
        raw = torch.as_tensor(_RawCuda(self._slot(self.rank, src), nbytes), device=self.device)
        out.view(torch.uint8).view(-1).copy_(raw)
        _lib.check(lib.rmlx_p2p_signal(ctypes.c_void_p(self._flag(src, self.rank, 1)), 1, st), "p2p_signal")
        self._received[src] = n
        return out

    def sendrecv(self, send: torch.Tensor, recv: torch.Tensor, peer: int) -> torch.Tensor:
        self.send(send, peer)
        return self.recv(recv, peer)

    def status(self) -> int:
        return int(_lib.cuda().rmlx_p2p_status())

    def close(self) -> None:
        self.region.close()
