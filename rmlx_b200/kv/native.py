"""Binding of the native serving core (csrc/host/serving.cpp) and the block manager built on it.

``NativeBlockManager`` has the interface and behaviour of ``kv.paged.BlockManager`` (which remains
as the behavioural oracle); the prefix cache and the scheduler of the same library are wrapped in
``serve.native``. The reference implements the block manager in Rust
(crates/rmlx-nn/src/paged_kv_cache.rs:36-631).

``available()`` is False only when the host library cannot be built or loaded;
``RMLX_NATIVE_SERVING=0`` makes the paged cache and the serving engine use the Python classes.
"""
from __future__ import annotations

import ctypes
import os
from array import array
from ctypes import POINTER, c_int, c_int64, c_void_p
from typing import List, Sequence

from .. import _lib

_IP = POINTER(c_int)
_LP = POINTER(c_int64)
_bound = False


def _host():
    global _bound
    lib = _lib.host()
    if not _bound:
        sig = {
            "rmlx_bm_create": (c_void_p, [c_int, c_int, c_int]),
            "rmlx_bm_destroy": (None, [c_void_p]),
            "rmlx_bm_num_free": (c_int, [c_void_p]),
            "rmlx_bm_has": (c_int, [c_void_p, c_int64]),
            "rmlx_bm_seq_len": (c_int, [c_void_p, c_int64]),
            "rmlx_bm_blocks_needed": (c_int, [c_void_p, c_int64, c_int]),
            "rmlx_bm_add_sequence": (c_int, [c_void_p, c_int64]),
            "rmlx_bm_reserve": (c_int, [c_void_p, c_int64, c_int, _IP, _IP, _IP]),
            "rmlx_bm_commit": (c_int, [c_void_p, c_int64, c_int]),
            "rmlx_bm_fork": (c_int, [c_void_p, c_int64, c_int64]),
            "rmlx_bm_adopt": (c_int, [c_void_p, c_int64, _IP, c_int, c_int]),
            "rmlx_bm_retain": (c_int, [c_void_p, c_int]),
            "rmlx_bm_release": (c_int, [c_void_p, c_int]),
            "rmlx_bm_trim": (c_int, [c_void_p, c_int64, c_int]),
            "rmlx_bm_drop_front": (c_int, [c_void_p, c_int64, c_int]),
            "rmlx_bm_free_sequence": (c_int, [c_void_p, c_int64]),
            "rmlx_bm_ref_count": (c_int, [c_void_p, c_int]),
            "rmlx_bm_table": (c_int, [c_void_p, c_int64, _IP, c_int]),
            "rmlx_pc_create": (c_void_p, [c_int, c_int]),
            "rmlx_pc_destroy": (None, [c_void_p]),
            "rmlx_pc_len": (c_int, [c_void_p]),
            "rmlx_pc_hits": (c_int64, [c_void_p]),
            "rmlx_pc_misses": (c_int64, [c_void_p]),
            "rmlx_pc_insert": (c_int, [c_void_p, _IP, c_int, _IP, c_int, _IP, c_int]),
            "rmlx_pc_lookup": (c_int, [c_void_p, _IP, c_int, _IP, c_int]),
            "rmlx_pc_evict": (c_int, [c_void_p, c_int, _IP, c_int]),
            "rmlx_pc_take_evicted": (c_int, [c_void_p, _IP, c_int]),
            "rmlx_sched_create": (c_void_p, [c_int, c_int64, c_int, c_int]),
            "rmlx_sched_destroy": (None, [c_void_p]),
            "rmlx_sched_add_request": (c_int, [c_void_p, c_int64, _IP, c_int, c_int]),
            "rmlx_sched_num_waiting": (c_int, [c_void_p]),
            "rmlx_sched_num_active": (c_int, [c_void_p]),
            "rmlx_sched_finish": (c_int, [c_void_p, c_int64, c_int64]),
            "rmlx_sched_admit_next": (c_int64, [c_void_p, c_void_p]),
            "rmlx_sched_set_cached": (c_int, [c_void_p, c_int64, c_int]),
            "rmlx_sched_plan": (c_int, [c_void_p, c_void_p, _LP, _LP, c_int]),
            "rmlx_sched_update": (c_int, [c_void_p, c_void_p, c_int64]),
            "rmlx_sched_prompt": (c_int, [c_void_p, c_int64, c_int, c_int, _IP]),
            "rmlx_sched_info": (c_int, [c_void_p, c_int64, _IP]),
            "rmlx_sched_finish_many": (c_int, [c_void_p, _LP, _LP, c_int, _LP]),
            "rmlx_sched_describe": (c_int, [c_void_p, c_void_p, _LP, c_int, _IP, _IP, c_int]),
        }
        for name, (res, args) in sig.items():
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = res, args
        _bound = True
    return lib


def available() -> bool:
    try:
        _host()
        return True
    except Exception:
        return False


def enabled() -> bool:
    """Native serving core wanted (default) and loadable."""
    return os.environ.get("RMLX_NATIVE_SERVING", "1") != "0" and available()


def _ints(values: Sequence[int]):
    """A C int array holding ``values`` (converted by the array module: an order of magnitude
    cheaper than filling a ctypes array element by element)."""
    if not len(values):
        return (c_int * 1)()
    arr = array("i", values)
    return (c_int * len(arr)).from_buffer(arr)


class NativeBlockManager:
    """``kv.paged.BlockManager`` backed by the native library."""

    def __init__(self, num_blocks: int, block_size: int = 16, reserved: int = 0):
        self._lib = _host()
        self._h = self._lib.rmlx_bm_create(num_blocks, block_size, reserved)
        if not self._h:
            raise ValueError("bad block manager arguments")
        self.num_blocks, self.block_size = num_blocks, block_size

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            self._lib.rmlx_bm_destroy(h)

    # -------------------------------------------------------------- queries
    def num_free_blocks(self) -> int:
        return self._lib.rmlx_bm_num_free(self._h)

    def blocks_needed(self, seq_id: int, new_tokens: int) -> int:
        return self._lib.rmlx_bm_blocks_needed(self._h, seq_id, new_tokens)

    def can_allocate(self, seq_id: int, new_tokens: int) -> bool:
        return self.blocks_needed(seq_id, new_tokens) <= self.num_free_blocks()

    def has_sequence(self, seq_id: int) -> bool:
        return bool(self._lib.rmlx_bm_has(self._h, seq_id))

    def num_blocks_of(self, seq_id: int) -> int:
        return max(0, self._lib.rmlx_bm_table(self._h, seq_id, None, 0))

    def block_table(self, seq_id: int) -> List[int]:
        n = self._lib.rmlx_bm_table(self._h, seq_id, None, 0)
        if n < 0:
            raise KeyError(seq_id)
        buf = (c_int * max(1, n))()
        self._lib.rmlx_bm_table(self._h, seq_id, buf, n)
        return list(buf[:n])

    def seq_len(self, seq_id: int) -> int:
        return self._lib.rmlx_bm_seq_len(self._h, seq_id)

    def ref_count(self, block: int) -> int:
        return self._lib.rmlx_bm_ref_count(self._h, block)

    # -------------------------------------------------------------- mutation
    def add_sequence(self, seq_id: int) -> None:
        if self._lib.rmlx_bm_add_sequence(self._h, seq_id) != 0:
            raise KeyError(f"sequence {seq_id} already exists")

    def reserve(self, seq_id: int, new_tokens: int) -> List[tuple]:
        src, dst, n = c_int(), c_int(), c_int()
        rc = self._lib.rmlx_bm_reserve(self._h, seq_id, new_tokens, ctypes.byref(src),
                                       ctypes.byref(dst), ctypes.byref(n))
        if rc == -3:
            from .paged import OutOfBlocks
            raise OutOfBlocks(f"need {self.blocks_needed(seq_id, new_tokens)} blocks, "
                              f"{self.num_free_blocks()} free")
        if rc != 0:
            raise ValueError("bad reserve arguments")
        return [(src.value, dst.value)] if n.value else []

    def commit(self, seq_id: int, new_tokens: int) -> None:
        if self._lib.rmlx_bm_commit(self._h, seq_id, new_tokens) != 0:
            raise KeyError(seq_id)

    def fork(self, parent: int, child: int) -> None:
        if self._lib.rmlx_bm_fork(self._h, parent, child) != 0:
            raise KeyError(f"sequence {child} already exists or {parent} is unknown")

    def adopt(self, seq_id: int, blocks: List[int], num_tokens: int) -> None:
        if self._lib.rmlx_bm_adopt(self._h, seq_id, _ints(blocks), len(blocks), num_tokens) != 0:
            raise ValueError(f"sequence {seq_id} is not empty, or the blocks are not live / too few")

    def retain(self, block: int) -> None:
        if self._lib.rmlx_bm_retain(self._h, block) != 0:
            raise ValueError(f"block {block} is not live")

    def release(self, block: int) -> None:
        if self._lib.rmlx_bm_release(self._h, block) != 0:
            raise ValueError(f"block {block} is not live")

    def trim(self, seq_id: int, num_tokens: int) -> None:
        if self._lib.rmlx_bm_trim(self._h, seq_id, num_tokens) != 0:
            raise KeyError(seq_id)

    def drop_front(self, seq_id: int, keep_tokens: int) -> int:
        n = self._lib.rmlx_bm_drop_front(self._h, seq_id, keep_tokens)
        if n == -1:
            raise KeyError(seq_id)
        if n < 0:
            raise ValueError("drop_front needs a reserved page and keep_tokens >= 0")
        return n

    def free_sequence(self, seq_id: int) -> None:
        self._lib.rmlx_bm_free_sequence(self._h, seq_id)
