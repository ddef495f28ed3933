"""Python face of the native allocator (csrc/host/allocator.cpp).

``CachingAllocator`` mirrors the reference's ``MetalAllocator`` API
(crates/rmlx-alloc/src/allocator.rs:131-512): ``alloc`` / ``free`` / ``set_memory_limit`` /
``set_cache_limit`` / ``set_gc_limit`` / ``reset_peak_memory`` / ``clear_cache`` / ``stats`` /
``leak_detector``. ``BfcArena`` is the sub-allocator over one region
(crates/rmlx-alloc/src/bfc.rs); the peer-mapped heap (``parallel.symm_heap.SymmetricHeap``) keeps its own growable arena so
that every rank, performing the same allocation sequence, gets the same offsets in every peer's
memory. The backing store defaults to host memory (tests run without a GPU); ``device=True``
backs it with cudaMalloc.
"""
from __future__ import annotations

import ctypes
from ctypes import c_int, c_uint32, c_uint64, c_void_p
from dataclasses import dataclass
from typing import Optional

from .. import _lib

_bound = False


def _host():
    global _bound
    lib = _lib.host()
    if not _bound:
        lib.rmlx_bfc_create.restype = c_void_p
        lib.rmlx_bfc_create.argtypes = [c_uint64, c_uint64]
        lib.rmlx_bfc_destroy.argtypes = [c_void_p]
        for name in ("rmlx_bfc_alloc",):
            getattr(lib, name).restype = c_uint64
            getattr(lib, name).argtypes = [c_void_p, c_uint64]
        lib.rmlx_bfc_free.restype = c_int
        lib.rmlx_bfc_free.argtypes = [c_void_p, c_uint64]
        for name in ("rmlx_bfc_in_use", "rmlx_bfc_peak", "rmlx_bfc_largest_free", "rmlx_bfc_num_blocks"):
            getattr(lib, name).restype = c_uint64
            getattr(lib, name).argtypes = [c_void_p]
        lib.rmlx_bfc_block_size.restype = c_uint64
        lib.rmlx_bfc_block_size.argtypes = [c_void_p, c_uint64]
        lib.rmlx_alloc_create.restype = c_void_p
        lib.rmlx_alloc_create.argtypes = [c_void_p, c_void_p, c_void_p, c_uint64, c_uint64, c_uint64]
        lib.rmlx_alloc_destroy.argtypes = [c_void_p]
        lib.rmlx_alloc_malloc.restype = c_uint64
        lib.rmlx_alloc_malloc.argtypes = [c_void_p, c_uint64, ctypes.POINTER(c_uint64)]
        lib.rmlx_alloc_free.restype = c_int
        lib.rmlx_alloc_free.argtypes = [c_void_p, c_uint64]
        lib.rmlx_alloc_clear_cache.argtypes = [c_void_p]
        lib.rmlx_alloc_set_limits.argtypes = [c_void_p, c_uint64, c_uint64, c_uint64]
        lib.rmlx_alloc_reset_peak.argtypes = [c_void_p]
        lib.rmlx_alloc_outstanding.restype = c_uint64
        lib.rmlx_alloc_outstanding.argtypes = [c_void_p]
        lib.rmlx_alloc_stats.argtypes = [c_void_p, ctypes.POINTER(c_uint64)]
        lib.rmlx_crc32.restype = c_uint32
        lib.rmlx_crc32.argtypes = [ctypes.c_char_p, c_uint64, c_uint32]
        _bound = True
    return lib


class AllocError(RuntimeError):
    pass


@dataclass
class AllocStats:
    allocs: int
    frees: int
    bytes_in_use: int
    peak: int
    backing_allocs: int
    backing_bytes: int
    cache_hits: int
    cache_misses: int
    small_allocs: int
    errors_double_free: int
    errors_foreign_free: int
    gc_runs: int
    cached_bytes: int


class LeakDetector:
    """Outstanding allocations = allocs - frees (crates/rmlx-alloc/src/leak_detector.rs:6-110)."""

    def __init__(self, owner: "CachingAllocator"):
        self._o = owner

    def outstanding(self) -> int:
        return int(_host().rmlx_alloc_outstanding(self._o._h))

    def outstanding_bytes(self) -> int:
        return self._o.stats().bytes_in_use

    def has_leaks(self) -> bool:
        return self.outstanding() > 0


_ALLOC_CB = ctypes.CFUNCTYPE(c_uint64, c_uint64, c_void_p)
_FREE_CB = ctypes.CFUNCTYPE(None, c_uint64, c_uint64, c_void_p)


class CachingAllocator:
    def __init__(self, memory_limit: int = 0, cache_limit: int = 0, gc_limit: int = 2 << 30,
                 device: bool = False):
        lib = _host()
        self._cbs = None
        a = f = None
        if device:
            cu = _lib.cuda()

            def _a(nbytes, _ctx):
                p = c_void_p()
                rc = cu.rmlx_symm_malloc(ctypes.byref(p), nbytes)
                return 0 if rc else (p.value or 0)

            def _f(addr, _n, _ctx):
                cu.rmlx_symm_free(c_void_p(addr))

            from ..parallel import comm as _comm  # registers the symm_* signatures  # noqa: F401
            self._cbs = (_ALLOC_CB(_a), _FREE_CB(_f))
            a = ctypes.cast(self._cbs[0], c_void_p)
            f = ctypes.cast(self._cbs[1], c_void_p)
        self._h = lib.rmlx_alloc_create(a, f, None, memory_limit, cache_limit, gc_limit)
        self._limits = [memory_limit, cache_limit, gc_limit]

    def alloc(self, nbytes: int):
        """Returns (address, usable_size). Zero-size requests are rejected."""
        if nbytes <= 0:
            raise AllocError("zero-size allocation")
        sz = c_uint64()
        addr = _host().rmlx_alloc_malloc(self._h, nbytes, ctypes.byref(sz))
        if not addr:
            raise AllocError(f"allocation of {nbytes} bytes failed (limit or backing store)")
        return int(addr), int(sz.value)

    def free(self, addr: int) -> None:
        rc = _host().rmlx_alloc_free(self._h, addr)
        if rc == -2:
            raise AllocError(f"double free of {addr:#x}")
        if rc == -1:
            raise AllocError(f"free of a pointer this allocator does not own: {addr:#x}")

    def _apply(self):
        _host().rmlx_alloc_set_limits(self._h, *self._limits)

    def set_memory_limit(self, n: int) -> None:
        self._limits[0] = n; self._apply()

    def set_block_limit(self, n: int) -> None:  # same knob: the largest total the backing store may hold
        self.set_memory_limit(n)

    def set_cache_limit(self, n: int) -> None:
        self._limits[1] = n; self._apply()

    def set_gc_limit(self, n: int) -> None:
        self._limits[2] = n; self._apply()

    def reset_peak_memory(self) -> None:
        _host().rmlx_alloc_reset_peak(self._h)

    def clear_cache(self) -> None:
        _host().rmlx_alloc_clear_cache(self._h)

    def stats(self) -> AllocStats:
        out = (c_uint64 * 13)()
        _host().rmlx_alloc_stats(self._h, out)
        return AllocStats(*[int(x) for x in out])

    def leak_detector(self) -> LeakDetector:
        return LeakDetector(self)

    def close(self) -> None:
        if self._h:
            _host().rmlx_alloc_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class BfcArena:
    """Best-fit-with-coalescing over ``size`` bytes; ``alloc`` returns an offset."""

    def __init__(self, size: int, alignment: int = 256):
        self._h = _host().rmlx_bfc_create(size, alignment)
        self.size = size

    def alloc(self, nbytes: int) -> int:
        off = _host().rmlx_bfc_alloc(self._h, nbytes)
        if off == 0xFFFFFFFFFFFFFFFF:
            raise AllocError(f"arena cannot fit {nbytes} bytes (largest free {self.largest_free()})")
        return int(off)

    def free(self, offset: int) -> None:
        rc = _host().rmlx_bfc_free(self._h, offset)
        if rc == -2:
            raise AllocError(f"double free of offset {offset}")
        if rc == -1:
            raise AllocError(f"offset {offset} was not allocated from this arena")

    def in_use(self) -> int:
        return int(_host().rmlx_bfc_in_use(self._h))

    def peak(self) -> int:
        return int(_host().rmlx_bfc_peak(self._h))

    def largest_free(self) -> int:
        return int(_host().rmlx_bfc_largest_free(self._h))

    def num_blocks(self) -> int:
        return int(_host().rmlx_bfc_num_blocks(self._h))

    def close(self) -> None:
        if self._h:
            _host().rmlx_bfc_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def crc32(data: bytes, seed: int = 0) -> int:
    """IEEE CRC32 (same polynomial as zlib) computed by the native library."""
    return int(_host().rmlx_crc32(data, len(data), seed))


class ManagedBuffer:
    """RAII handle: the allocation goes back to its allocator when the handle is closed or dropped
    (crates/rmlx-metal/src/managed_buffer.rs:21-115)."""

    def __init__(self, allocator: "CachingAllocator", nbytes: int):
        self._alloc = allocator
        self.ptr, self.nbytes = allocator.alloc(nbytes)      # address, usable size

    def close(self) -> None:
        if self.ptr is not None:
            self._alloc.free(self.ptr)
            self.ptr = None

    def __enter__(self) -> "ManagedBuffer":
        return self

    def __exit__(self, *exc) -> None:
        self.close()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class ResidencyManager:
    """Book-keeping of which allocations must stay resident (crates/rmlx-alloc/src/residency.rs:
    54-235). Device memory on a discrete GPU is always resident, so this is the counting form: it
    tracks the set and its bytes and refuses to exceed a budget."""

    def __init__(self, budget_bytes: Optional[int] = None):
        self.budget = budget_bytes
        self._set = {}

    def add(self, key, nbytes: int) -> None:
        if key in self._set:
            return
        if self.budget is not None and self.resident_bytes + nbytes > self.budget:
            raise AllocError("residency budget exceeded")
        self._set[key] = int(nbytes)

    def remove(self, key) -> None:
        self._set.pop(key, None)

    def __contains__(self, key) -> bool:
        return key in self._set

    @property
    def resident_bytes(self) -> int:
        return sum(self._set.values())

    def __len__(self) -> int:
        return len(self._set)


class ForwardArena:
    """Bump allocator over one pre-allocated tensor, reset once per forward pass
    (crates/rmlx-core/src/arena.rs:12-55): temporaries of a step cost no allocator calls."""

    def __init__(self, nbytes: int, device="cpu", alignment: int = 256):
        import torch
        self._buf = torch.empty(int(nbytes), dtype=torch.uint8, device=device)
        self._align = alignment
        self._top = 0
        self.peak = 0

    def take(self, shape, dtype):
        import math
        import torch
        n = int(math.prod(shape)) * torch.empty((), dtype=dtype).element_size()
        start = (self._top + self._align - 1) // self._align * self._align
        if start + n > self._buf.numel():
            raise AllocError(f"arena exhausted: need {n} bytes at {start} of {self._buf.numel()}")
        self._top = start + n
        self.peak = max(self.peak, self._top)
        return self._buf[start:start + n].view(dtype).view(*shape)

    def reset(self) -> None:
        self._top = 0

    @property
    def used(self) -> int:
        return self._top
