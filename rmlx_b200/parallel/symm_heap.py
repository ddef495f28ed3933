"""The symmetric heap: one peer-mapped arena per process group that every collective of this
package sub-allocates from.

Each rank owns physical segments created through the virtual-memory-management API
(``csrc/comm/vmm_heap.cu``), exported as file descriptors, passed to the peers over Unix-domain
sockets and mapped by every rank into address ranges reserved up front: one range per rank, so the
heap of rank r is contiguous in every process and grows in place. A first-fit free list with coalescing
hands out offsets; because every rank makes the same requests in the
same order, an offset names the same bytes on every rank. ``alloc`` returns a ``HeapBlock`` with
the interface of the older one-allocation-per-consumer region (``local``, ``ptrs``,
``peer_array``, ``close``), plus ``mc``: the block's address in the NVLink multicast mapping when
the heap was created with ``multicast=True`` (stores there reach every rank, ``multimem.ld_reduce``
sums over the ranks inside the switch).

This is what the reference builds from registered RDMA regions: a tiered pool of shared buffers
whose lifetime is tied to completion (crates/rmlx-alloc/src/zero_copy.rs:22-171,
crates/rmlx-rdma/src/shared_buffer.rs, mr_pool.rs) behind its allocator
(crates/rmlx-alloc/src/allocator.rs:242-385).

Lifetime: a block is returned to the arena by ``close()`` after a device synchronisation and a
barrier of the group (no rank may still be writing into it); the heap itself unbinds its multicast
objects, unmaps and releases everything in ``close()``, which also runs at interpreter exit.
"""
from __future__ import annotations

import atexit
import ctypes
import os
import socket
import tempfile
import uuid
from typing import Dict, List, Optional

import torch
import torch.distributed as dist

from .. import _lib

_lib.register_cuda_sigs({
    "rmlx_vmm_support": ("i", "i"),
    "rmlx_vmm_granularity": ("ii", "q"),
    "rmlx_vmm_create": ("iqpp", "i"),
    "rmlx_vmm_import": ("ip", "i"),
    "rmlx_vmm_release": ("q", "i"),
    "rmlx_vmm_reserve": ("qqp", "i"),
    "rmlx_vmm_address_free": ("qq", "i"),
    "rmlx_vmm_map": ("qqqi", "i"),
    "rmlx_vmm_unmap": ("qq", "i"),
    "rmlx_mc_create": ("iqpp", "i"),
    "rmlx_mc_add_device": ("qi", "i"),
    "rmlx_mc_bind": ("qqq", "i"),
    "rmlx_mc_unbind": ("qiq", "i"),
    "rmlx_vmm_memset": ("qq", "i"),
})


def _drv(rc: int, what: str) -> None:
    if rc == 0:
        return
    if rc == -1000:
        raise _lib.NativeError(f"{what}: the driver entry point is not available")
    if rc <= -2000:
        raise _lib.NativeError(f"{what}: driver error {-rc - 2000}")
    _lib.check(rc, what)


def vmm_support(device: Optional[int] = None) -> int:
    """Bit 0: shareable VMM allocations; bit 1: NVLink multicast. 0 on a box without a GPU."""
    if not torch.cuda.is_available():
        return 0
    dev = torch.cuda.current_device() if device is None else device
    rc = int(_lib.cuda().rmlx_vmm_support(dev))
    return rc if rc > 0 else 0


class _FdExchange:
    """All-to-all of file descriptors inside one box: every rank listens on a Unix-domain socket,
    connects to every peer and sends ``SCM_RIGHTS`` messages."""

    def __init__(self, group):
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.path = os.path.join(tempfile.gettempdir(), f"rmlx-heap-{uuid.uuid4().hex}-{self.rank}.sock")
        self.sock = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
        self.sock.bind(self.path)
        self.sock.listen(self.world + 4)
        paths: List[Optional[str]] = [None] * self.world
        dist.all_gather_object(paths, self.path, group=group)
        self.paths = paths

    def all_to_all(self, fd: int, roots: Optional[List[int]] = None) -> Dict[int, int]:
        """Every rank in ``roots`` (default: all) sends ``fd`` to every other rank. Returns
        {source rank: received descriptor}."""
        roots = list(range(self.world)) if roots is None else roots
        if self.rank in roots:
            for p in range(self.world):
                if p == self.rank:
                    continue
                with socket.socket(socket.AF_UNIX, socket.SOCK_STREAM) as c:
                    c.settimeout(60.0)
                    c.connect(self.paths[p])
                    socket.send_fds(c, [self.rank.to_bytes(4, "little")], [fd])
        got: Dict[int, int] = {}
        expect = len([r for r in roots if r != self.rank])
        self.sock.settimeout(60.0)
        for _ in range(expect):
            conn, _ = self.sock.accept()
            with conn:
                conn.settimeout(60.0)
                msg, fds, _, _ = socket.recv_fds(conn, 4, 1)
                got[int.from_bytes(msg, "little")] = fds[0]
        dist.barrier(group=self.group)
        return got

    def close(self) -> None:
        try:
            self.sock.close()
            os.unlink(self.path)
        except OSError:
            pass


class OffsetArena:
    """First-fit free list with coalescing over [0, capacity): deterministic, so ranks that make
    the same calls in the same order get the same offsets; ``grow`` appends a range."""

    def __init__(self):
        self.capacity = 0
        self.free: List[tuple] = []          # sorted (offset, size), never adjacent

    def grow(self, size: int) -> None:
        self.give(self.capacity, size)
        self.capacity += size

    def take(self, need: int) -> Optional[int]:
        for i, (o, n) in enumerate(self.free):
            if n >= need:
                if n == need:
                    self.free.pop(i)
                else:
                    self.free[i] = (o + need, n - need)
                return o
        return None

    def give(self, offset: int, size: int) -> None:
        fl = sorted(self.free + [(offset, size)])
        merged: List[tuple] = []
        for o, n in fl:
            if merged and merged[-1][0] + merged[-1][1] > o:
                raise ValueError("range returned twice")
            if merged and merged[-1][0] + merged[-1][1] == o:
                merged[-1] = (merged[-1][0], merged[-1][1] + n)
            else:
                merged.append((o, n))
        self.free = merged

    def free_bytes(self) -> int:
        return sum(n for _, n in self.free)


class HeapBlock:
    """A sub-allocation of the heap: the same offset on every rank."""

    def __init__(self, heap: "SymmetricHeap", offset: int, nbytes: int):
        self.heap, self.offset, self.nbytes = heap, offset, nbytes
        self.group, self.rank, self.world = heap.group, heap.rank, heap.world
        self.ptrs = [base + offset for base in heap.bases]
        self.local = self.ptrs[self.rank]
        self.mc = heap.mc_base + offset if heap.mc_base else 0

    def peer_array(self, byte_offset: int = 0):
        arr = (ctypes.c_void_p * self.world)()
        for r in range(self.world):
            arr[r] = self.ptrs[r] + byte_offset
        return arr

    def close(self) -> None:
        if self.local:
            self.heap.free(self)
            self.local = 0

    def __del__(self):
        # an unreachable block is only forgotten: freeing is a collective (barrier) and cannot
        # run from the collector; the heap reclaims everything when it is closed
        pass


class SymmetricHeap:
    def __init__(self, group=None, segment_bytes: Optional[int] = None, va_bytes: Optional[int] = None,
                 multicast: bool = False, device: Optional[torch.device] = None):
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.dev = self.device.index if self.device.index is not None else torch.cuda.current_device()
        lib = self._lib = _lib.cuda()
        support = vmm_support(self.dev)
        if not support & 1:
            raise _lib.NativeError("this device does not export VMM allocations as file descriptors")
        if multicast and not support & 2:
            raise _lib.NativeError("this device does not support NVLink multicast")
        self.multicast = multicast
        self.gran = int(lib.rmlx_vmm_granularity(self.dev, self.world if multicast else 0))
        if self.gran <= 0:
            raise _lib.NativeError(f"allocation granularity query failed ({self.gran})")
        seg = segment_bytes or int(os.environ.get("RMLX_SYMM_SEGMENT_MB", "256")) << 20
        self.segment_bytes = self._round(seg)
        self.va_bytes = self._round(va_bytes or int(os.environ.get("RMLX_SYMM_VA_GB", "16")) << 30)
        self.fdx = _FdExchange(group)
        # one address range per rank's heap (and one for the multicast view)
        self.bases: List[int] = []
        for _ in range(self.world):
            va = ctypes.c_ulonglong()
            _drv(lib.rmlx_vmm_reserve(self.va_bytes, self.gran, ctypes.byref(va)), "vmm_reserve")
            self.bases.append(va.value)
        self.mc_base = 0
        if multicast:
            va = ctypes.c_ulonglong()
            _drv(lib.rmlx_vmm_reserve(self.va_bytes, self.gran, ctypes.byref(va)), "vmm_reserve")
            self.mc_base = va.value
        self.capacity = 0
        self.arena = OffsetArena()
        self._segments: List[dict] = []
        self._live: Dict[int, HeapBlock] = {}
        self.closed = False
        self.stats = {"segments": 0, "allocs": 0, "frees": 0, "grown_bytes": 0}
        atexit.register(self.close)

    def _round(self, n: int) -> int:
        return (n + self.gran - 1) // self.gran * self.gran

    # ------------------------------------------------------------------ growth (collective)
    def _grow(self, at_least: int) -> None:
        lib = self._lib
        size = max(self.segment_bytes, self._round(at_least))
        if self.capacity + size > self.va_bytes:
            raise _lib.NativeError("symmetric heap: reserved address range exhausted "
                                   "(raise RMLX_SYMM_VA_GB)")
        h, fd = ctypes.c_ulonglong(), ctypes.c_int()
        _drv(lib.rmlx_vmm_create(self.dev, size, ctypes.byref(h), ctypes.byref(fd)), "vmm_create")
        seg = {"size": size, "offset": self.capacity, "handles": {self.rank: h.value}, "mc": 0}
        peers = self.fdx.all_to_all(fd.value)
        os.close(fd.value)
        for r, pfd in peers.items():
            ph = ctypes.c_ulonglong()
            _drv(lib.rmlx_vmm_import(pfd, ctypes.byref(ph)), "vmm_import")
            os.close(pfd)
            seg["handles"][r] = ph.value
        for r in range(self.world):
            _drv(lib.rmlx_vmm_map(self.bases[r] + self.capacity, size, seg["handles"][r], self.dev), "vmm_map")
        # fresh physical memory: the consumers rely on zeroed flags and counters
        with torch.cuda.device(self.device):
            _drv(lib.rmlx_vmm_memset(self.bases[self.rank] + self.capacity, size), "heap memset")
        if self.multicast:
            mh, mfd = ctypes.c_ulonglong(), ctypes.c_int(-1)
            if self.rank == 0:
                _drv(lib.rmlx_mc_create(self.world, size, ctypes.byref(mh), ctypes.byref(mfd)), "mc_create")
            got = self.fdx.all_to_all(mfd.value, roots=[0])
            if self.rank == 0:
                os.close(mfd.value)
            else:
                _drv(lib.rmlx_vmm_import(got[0], ctypes.byref(mh)), "mc_import")
                os.close(got[0])
            _drv(lib.rmlx_mc_add_device(mh.value, self.dev), "mc_add_device")
            dist.barrier(group=self.group)            # every device is in the object before any bind
            _drv(lib.rmlx_mc_bind(mh.value, seg["handles"][self.rank], size), "mc_bind")
            dist.barrier(group=self.group)
            _drv(lib.rmlx_vmm_map(self.mc_base + self.capacity, size, mh.value, self.dev), "mc_map")
            seg["mc"] = mh.value
        dist.barrier(group=self.group)
        self._segments.append(seg)
        self.arena.grow(size)
        self.capacity += size
        self.stats["segments"] += 1
        self.stats["grown_bytes"] += size

    # ------------------------------------------------------------------ allocation (collective)
    def alloc(self, nbytes: int) -> HeapBlock:
        """Every rank calls this with the same size, in the same order."""
        if self.closed:
            raise _lib.NativeError("symmetric heap is closed")
        need = (max(1, nbytes) + 255) // 256 * 256
        off = self._place(need)
        blk = HeapBlock(self, off, need)
        self._live[off] = blk
        # a recycled range may hold an earlier tenant's flags: hand it out zeroed, on every rank,
        # before any rank can write into it
        with torch.cuda.device(self.device):
            _drv(self._lib.rmlx_vmm_memset(blk.local, need), "heap memset")
        dist.barrier(group=self.group)
        self.stats["allocs"] += 1
        return blk

    def _place(self, need: int) -> int:
        off = self.arena.take(need)
        while off is None:
            self._grow(need)
            off = self.arena.take(need)
        return off

    def free(self, blk: HeapBlock) -> None:
        """Collective: no rank may still be using the block (device synchronisation + barrier)."""
        if self.closed or blk.offset not in self._live:
            return
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)
        del self._live[blk.offset]
        self.arena.give(blk.offset, blk.nbytes)
        self.stats["frees"] += 1

    def bytes_in_use(self) -> int:
        return sum(b.nbytes for b in self._live.values())

    # ------------------------------------------------------------------ teardown
    def close(self) -> None:
        if self.closed:
            return
        self.closed = True
        lib = self._lib
        try:
            torch.cuda.synchronize(self.device)
            if dist.is_initialized():
                dist.barrier(group=self.group)
        except Exception:
            pass
        for seg in self._segments:
            if seg["mc"]:
                lib.rmlx_vmm_unmap(self.mc_base + seg["offset"], seg["size"])
                lib.rmlx_mc_unbind(seg["mc"], self.dev, seg["size"])
                lib.rmlx_vmm_release(seg["mc"])
            for r in range(self.world):
                lib.rmlx_vmm_unmap(self.bases[r] + seg["offset"], seg["size"])
                lib.rmlx_vmm_release(seg["handles"][r])
        for va in self.bases + ([self.mc_base] if self.mc_base else []):
            lib.rmlx_vmm_address_free(va, self.va_bytes)
        self._segments = []
        self._live = {}
        self.fdx.close()


_HEAPS: Dict[int, SymmetricHeap] = {}


def default_heap(group=None, multicast: Optional[bool] = None) -> Optional[SymmetricHeap]:
    """The process group's heap, created on first use; None when the device cannot export VMM
    allocations or ``RMLX_SYMM_HEAP=0`` (the consumers then fall back to one inter-process mapped
    allocation each). ``RMLX_SYMM_MULTICAST=1`` binds the heap to NVLink multicast objects."""
    if os.environ.get("RMLX_SYMM_HEAP", "1") == "0":
        return None
    key = id(group) if group is not None else 0
    heap = _HEAPS.get(key)
    if heap is not None and not heap.closed:
        return heap
    if not vmm_support() & 1:
        return None
    if multicast is None:
        multicast = os.environ.get("RMLX_SYMM_MULTICAST", "0") == "1"
    heap = SymmetricHeap(group, multicast=multicast and bool(vmm_support() & 2))
    _HEAPS[key] = heap
    return heap


def close_heaps() -> None:
    for h in list(_HEAPS.values()):
        h.close()
    _HEAPS.clear()
