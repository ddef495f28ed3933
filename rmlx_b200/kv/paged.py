"""Paged KV cache: a block manager with copy-on-write reference counts plus the device pools the
attention kernels read.

API and semantics follow crates/rmlx-nn/src/paged_kv_cache.rs:36-631 (``BlockManager``: free list,
per-sequence block tables, refcounts, ``fork``; ``PagedKvCache``: ``append``, ``get_keys/values``,
``trim`` for speculative rollback, ``free_sequence``). Differences that are deliberate: K and V live
in device pools laid out ``[layer][block, kv_head, page, head_dim]`` so one (block, kv head) page is
contiguous for the attention kernels; appends are done on the device by the RoPE+KV-write kernel
(the reference copies each token on the host); and the block table is mirrored in a device int32
tensor so a captured decode graph sees growth without re-capture.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..reference import ops as ref

PAGE = 16


class OutOfBlocks(RuntimeError):
    pass


class BlockManager:
    """Fixed pool of KV blocks with a free list, per-sequence block tables and refcounts."""

    def __init__(self, num_blocks: int, block_size: int = PAGE, reserved: int = 0):
        """``reserved`` leading blocks are never handed out (block 0 serves as the harmless
        target of idle batch rows in a shape-stable decode graph)."""
        self.num_blocks = num_blocks
        self.block_size = block_size
        self.reserved = reserved
        self.free: List[int] = list(range(num_blocks - 1, reserved - 1, -1))
        self.ref = [0] * num_blocks
        self.tables: Dict[int, List[int]] = {}
        self.lengths: Dict[int, int] = {}

    # -------------------------------------------------------------- queries
    def num_free_blocks(self) -> int:
        return len(self.free)

    def blocks_needed(self, seq_id: int, new_tokens: int) -> int:
        cur = self.lengths.get(seq_id, 0)
        have = len(self.tables.get(seq_id, ()))
        need = (cur + new_tokens + self.block_size - 1) // self.block_size
        return max(0, need - have)

    def can_allocate(self, seq_id: int, new_tokens: int) -> bool:
        return self.blocks_needed(seq_id, new_tokens) <= len(self.free)

    def block_table(self, seq_id: int) -> List[int]:
        return self.tables[seq_id]

    def has_sequence(self, seq_id: int) -> bool:
        return seq_id in self.tables

    def num_blocks_of(self, seq_id: int) -> int:
        return len(self.tables.get(seq_id, ()))

    def ref_count(self, block: int) -> int:
        return self.ref[block]

    def seq_len(self, seq_id: int) -> int:
        return self.lengths.get(seq_id, 0)

    # -------------------------------------------------------------- mutation
    def _take(self) -> int:
        if not self.free:
            raise OutOfBlocks("KV block pool exhausted")
        b = self.free.pop()
        self.ref[b] = 1
        return b

    def _drop(self, b: int) -> None:
        if b < self.reserved:                # a released front page (entry 0) holds no reference
            return
        self.ref[b] -= 1
        if self.ref[b] == 0:
            self.free.append(b)
        elif self.ref[b] < 0:
            raise RuntimeError(f"block {b} freed twice")

    def add_sequence(self, seq_id: int) -> None:
        if seq_id in self.tables:
            raise KeyError(f"sequence {seq_id} already exists")
        self.tables[seq_id] = []
        self.lengths[seq_id] = 0

    def reserve(self, seq_id: int, new_tokens: int) -> List[tuple]:
        """Make room for ``new_tokens`` more tokens. Returns the copy-on-write work to do:
        (src_block, dst_block) pairs for a shared last block that is about to be written."""
        if seq_id not in self.tables:
            self.add_sequence(seq_id)
        table, cur = self.tables[seq_id], self.lengths[seq_id]
        # a shared partial last block is copied before it is written: count that block too, so
        # that the request fails before anything has changed
        cow = bool(new_tokens > 0 and table and cur % self.block_size != 0 and self.ref[table[-1]] > 1)
        need = self.blocks_needed(seq_id, new_tokens) + (1 if cow else 0)
        if need > len(self.free):
            raise OutOfBlocks(f"need {need} blocks, {len(self.free)} free")
        copies = []
        if new_tokens > 0 and table and cur % self.block_size != 0:
            last = table[-1]
            if self.ref[last] > 1:                       # shared partial block: copy before write
                nb = self._take()
                copies.append((last, nb))
                self._drop(last)
                table[-1] = nb
        for _ in range(self.blocks_needed(seq_id, new_tokens)):
            table.append(self._take())
        return copies

    def commit(self, seq_id: int, new_tokens: int) -> None:
        self.lengths[seq_id] += new_tokens

    def fork(self, parent: int, child: int) -> None:
        """Child shares every block of the parent (copy-on-write)."""
        if child in self.tables:
            raise KeyError(f"sequence {child} already exists")
        self.tables[child] = list(self.tables[parent])
        self.lengths[child] = self.lengths[parent]
        for b in self.tables[child]:
            self.ref[b] += 1

    def adopt(self, seq_id: int, blocks: List[int], num_tokens: int) -> None:
        """An empty sequence starts from ``blocks`` that already hold the KV of its first
        ``num_tokens`` tokens (a cached prompt prefix): shared, copy-on-write like ``fork``."""
        if self.tables.get(seq_id) or self.lengths.get(seq_id, 0):
            raise ValueError(f"sequence {seq_id} is not empty")
        if num_tokens > len(blocks) * self.block_size:
            raise ValueError("more tokens than the blocks hold")
        for b in blocks:
            if self.ref[b] <= 0:
                raise ValueError(f"block {b} is not live")
            self.ref[b] += 1
        self.tables[seq_id] = list(blocks)
        self.lengths[seq_id] = num_tokens

    def retain(self, block: int) -> None:
        """One more owner of a live block (a prefix cache keeping pages past their sequence)."""
        if self.ref[block] <= 0:
            raise ValueError(f"block {block} is not live")
        self.ref[block] += 1

    def release(self, block: int) -> None:
        """Give up an ownership taken with ``retain``."""
        self._drop(block)

    def trim(self, seq_id: int, num_tokens: int) -> None:
        """Drop the last ``num_tokens`` tokens (speculative rollback)."""
        cur = self.lengths[seq_id]
        new = max(0, cur - num_tokens)
        keep = (new + self.block_size - 1) // self.block_size
        table = self.tables[seq_id]
        while len(table) > keep:
            self._drop(table.pop())
        self.lengths[seq_id] = new

    def drop_front(self, seq_id: int, keep_tokens: int) -> int:
        """Sliding-window sequences: release the pages that lie entirely before the last
        ``keep_tokens`` tokens; their table entries become 0, the reserved page. Returns how many
        pages were released (the rotating cache of crates/rmlx-nn/src/attention.rs:970, as a page
        policy)."""
        if seq_id not in self.tables:
            raise KeyError(seq_id)
        if self.reserved < 1 or keep_tokens < 0:
            raise ValueError("drop_front needs a reserved page and keep_tokens >= 0")
        table = self.tables[seq_id]
        first_needed = max(0, self.lengths[seq_id] - keep_tokens) // self.block_size
        n = 0
        for i in range(min(first_needed, len(table))):
            if table[i] >= self.reserved:
                self._drop(table[i])
                table[i] = 0
                n += 1
        return n

    def free_sequence(self, seq_id: int) -> None:
        for b in self.tables.pop(seq_id, []):
            self._drop(b)
        self.lengths.pop(seq_id, None)


def make_block_manager(num_blocks: int, block_size: int = PAGE, reserved: int = 0):
    """The block manager of the native host library when it is enabled (the default), else the
    Python one above; both have the same interface and behaviour."""
    from . import native
    if native.enabled():
        return native.NativeBlockManager(num_blocks, block_size, reserved)
    return BlockManager(num_blocks, block_size, reserved)


def quantize_kv_rows(x: torch.Tensor):
    """x [..., D] (D a multiple of 64) -> (codes uint8 [..., D], sb bf16 [..., D/64, 2]): 8-bit affine
    per group of 64. The bias is the group minimum rounded DOWN to bf16 and the scale is
    (max - stored bias) / 255 rounded UP to bf16, so neither end of the range clips; the codes are
    computed against the stored pair, as the device kernel does (csrc/kernels/kv_q8.cu)."""
    d = x.shape[-1]
    g = x.float().reshape(*x.shape[:-1], d // 64, 64)
    mn, mx = g.amin(-1), g.amax(-1)
    bits = mn.contiguous().view(torch.int32)
    # towards minus infinity: truncate a positive value's low bits, grow a negative one's magnitude
    down = torch.where(mn >= 0, bits & ~0xFFFF, (bits + 0xFFFF) & ~0xFFFF).view(torch.float32)
    bias = down.to(torch.bfloat16)
    span = (mx - bias.float()).clamp_min(0.0) / 255.0
    span = torch.where(span > 0, span, torch.ones_like(span))
    up = ((span.contiguous().view(torch.int32) + 0xFFFF) & ~0xFFFF).view(torch.float32)   # next bf16 at or above
    scale = up.to(torch.bfloat16)
    q = torch.round((g - bias.float()[..., None]) * (1.0 / scale.float()[..., None])).clamp_(0, 255)
    return q.to(torch.uint8).reshape(x.shape), torch.stack([scale, bias], -1)


def dequantize_kv_rows(q: torch.Tensor, sb: torch.Tensor) -> torch.Tensor:
    """Inverse of ``quantize_kv_rows``: fp32 [..., D]."""
    d = q.shape[-1]
    g = q.float().reshape(*q.shape[:-1], d // 64, 64)
    return (g * sb[..., 0].float()[..., None] + sb[..., 1].float()[..., None]).reshape(q.shape)


class PagedKvCache:
    """Device K/V pools for every layer plus the manager and a device mirror of block tables.

    ``kv_quant="q8"`` keeps the pools in the 8-bit affine format (codes uint8
    ``[blocks, Hkv, page, D]`` in ``k`` / ``v`` plus ``k_sb`` / ``v_sb`` bf16
    ``[blocks, Hkv, page, D/64, 2]`` of (scale, bias) per token and group of 64): half the bytes
    per token. The device kernels quantise on append and expand inside attention
    (csrc/kernels/kv_q8.cu, flash_decode.cu); the counterpart of the reference's host-side
    QuantizedKvCache (crates/rmlx-nn/src/attention.rs:4438-4680)."""

    def __init__(self, num_blocks: int, num_layers: int, kv_heads: int, head_dim: int,
                 dtype=torch.bfloat16, device="cpu", max_seqs: int = 64,
                 max_blocks_per_seq: int = 512, block_size: int = PAGE,
                 kv_quant: Optional[str] = None):
        self.manager = make_block_manager(num_blocks, block_size, reserved=1)
        self.num_layers, self.kv_heads, self.head_dim = num_layers, kv_heads, head_dim
        self.block_size = block_size
        if kv_quant not in (None, "q8"):
            raise ValueError(f"unsupported KV quantisation {kv_quant}")
        self.quantized = kv_quant == "q8"
        self.dtype = dtype
        if self.quantized:
            if head_dim % 64:
                raise ValueError("the 8-bit cache needs head_dim to be a multiple of 64")
            shape, sbs = (num_blocks, kv_heads, block_size, head_dim), (num_blocks, kv_heads, block_size, head_dim // 64, 2)
            self.k = [torch.zeros(shape, dtype=torch.uint8, device=device) for _ in range(num_layers)]
            self.v = [torch.zeros(shape, dtype=torch.uint8, device=device) for _ in range(num_layers)]
            self.k_sb = [torch.zeros(sbs, dtype=torch.bfloat16, device=device) for _ in range(num_layers)]
            self.v_sb = [torch.zeros(sbs, dtype=torch.bfloat16, device=device) for _ in range(num_layers)]
        else:
            self.k = [torch.zeros(num_blocks, kv_heads, block_size, head_dim, dtype=dtype, device=device)
                      for _ in range(num_layers)]
            self.v = [torch.zeros(num_blocks, kv_heads, block_size, head_dim, dtype=dtype, device=device)
                      for _ in range(num_layers)]
            self.k_sb = self.v_sb = None
        self.device = torch.device(device)
        self.max_blocks_per_seq = max_blocks_per_seq
        # row r of the device table belongs to the sequence bound to slot r
        self.block_table = torch.zeros(max_seqs, max_blocks_per_seq, dtype=torch.int32, device=device)
        self._host_table = torch.zeros(max_seqs, max_blocks_per_seq, dtype=torch.int32,
                                       pin_memory=self.device.type == "cuda")
        self.slot_of: Dict[int, int] = {}
        self._free_slots = list(range(max_seqs - 1, -1, -1))
        # the pinned row of a slot is the source of an asynchronous copy: the event recorded after
        # the copy is waited for before the row is written again (by a later update of the same
        # sequence, or by the next sequence that takes the slot)
        self._row_copied: Dict[int, "torch.cuda.Event"] = {}

    # -------------------------------------------------------------- sequences
    def add_sequence(self, seq_id: int) -> int:
        self.manager.add_sequence(seq_id)
        slot = self._free_slots.pop()
        self.slot_of[seq_id] = slot
        return slot

    def free_sequence(self, seq_id: int) -> None:
        self.manager.free_sequence(seq_id)
        slot = self.slot_of.pop(seq_id)
        self._row_idle(slot)
        self._host_table[slot].zero_()
        self._free_slots.append(slot)

    def fork(self, parent: int, child: int) -> int:
        self.manager.fork(parent, child)
        slot = self._free_slots.pop()
        self.slot_of[child] = slot
        self._sync_slot(child)
        return slot

    def adopt_prefix(self, seq_id: int, blocks: List[int], num_tokens: int) -> None:
        """Start an (empty, already added) sequence from cached prefix pages."""
        self.manager.adopt(seq_id, blocks, num_tokens)
        self._sync_slot(seq_id)

    def seq_len(self, seq_id: int) -> int:
        return self.manager.seq_len(seq_id)

    def _row_idle(self, slot: int) -> None:
        """Wait until the last queued copy out of the slot's pinned row has run."""
        ev = self._row_copied.pop(slot, None)
        if ev is not None:
            ev.synchronize()

    def _sync_slot(self, seq_id: int) -> None:
        slot = self.slot_of[seq_id]
        table = self.manager.block_table(seq_id)
        if len(table) > self.max_blocks_per_seq:
            raise OutOfBlocks("sequence exceeds max_blocks_per_seq")
        self._row_idle(slot)
        row = self._host_table[slot]
        row[:len(table)] = torch.tensor(table, dtype=torch.int32)
        self.block_table[slot].copy_(row, non_blocking=True)
        if self.device.type == "cuda":
            ev = torch.cuda.Event()
            ev.record(torch.cuda.current_stream(self.device))
            self._row_copied[slot] = ev

    def reserve(self, seq_id: int, new_tokens: int) -> None:
        """Ensure blocks exist for ``new_tokens`` more tokens (doing any copy-on-write) and push
        the table row to the device."""
        before = self.manager.num_blocks_of(seq_id)
        copies = self.manager.reserve(seq_id, new_tokens)
        for src, dst in copies:
            for l in range(self.num_layers):
                self.k[l][dst].copy_(self.k[l][src])
                self.v[l][dst].copy_(self.v[l][src])
                if self.quantized:
                    self.k_sb[l][dst].copy_(self.k_sb[l][src])
                    self.v_sb[l][dst].copy_(self.v_sb[l][src])
        if copies or len(self.manager.block_table(seq_id)) != before:
            self._sync_slot(seq_id)

    def commit(self, seq_id: int, new_tokens: int) -> None:
        self.manager.commit(seq_id, new_tokens)

    def trim(self, seq_id: int, num_tokens: int) -> None:
        self.manager.trim(seq_id, num_tokens)
        self._sync_slot(seq_id)

    def drop_front(self, seq_id: int, window: int) -> int:
        """A model with a sliding window of ``window`` tokens never reads older keys: give the
        pages that lie entirely before the window back to the pool (the device table points at the
        reserved zero page instead). Call it between steps; returns the pages released."""
        n = self.manager.drop_front(seq_id, window)
        if n:
            self._sync_slot(seq_id)
        return n

    # -------------------------------------------------------------- reference-style access
    def append(self, layer: int, seq_id: int, k: torch.Tensor, v: torch.Tensor, start: int) -> None:
        """Host-driven append of k, v [n, kv_heads, head_dim] at positions start.. (the reference's
        form; the native path writes through the RoPE+KV kernel instead)."""
        table = torch.tensor(self.manager.block_table(seq_id), dtype=torch.int64, device=self.device)
        bs = self.block_size
        pos = torch.arange(start, start + k.shape[0], device=self.device)
        blk, off = table[pos // bs], pos % bs
        if self.quantized:
            kq, ksb = quantize_kv_rows(k)
            vq, vsb = quantize_kv_rows(v)
            self.k[layer][blk, :, off], self.k_sb[layer][blk, :, off] = kq, ksb
            self.v[layer][blk, :, off], self.v_sb[layer][blk, :, off] = vq, vsb
            return
        self.k[layer][blk, :, off] = k.to(self.k[layer].dtype)
        self.v[layer][blk, :, off] = v.to(self.v[layer].dtype)

    def _gather(self, pool, sb, seq_id: int, length: Optional[int]) -> torch.Tensor:
        length = self.manager.seq_len(seq_id) if length is None else length
        row = torch.tensor(self.manager.block_table(seq_id), dtype=torch.int64, device=self.device)
        if not self.quantized:
            return ref.gather_paged(pool, row, length)
        nblk = (length + self.block_size - 1) // self.block_size
        idx = row[:nblk]
        full = dequantize_kv_rows(pool[idx], sb[idx]).to(self.dtype)      # [nblk, Hkv, page, D]
        return full.permute(0, 2, 1, 3).reshape(nblk * self.block_size, self.kv_heads, self.head_dim)[:length]

    def get_keys(self, layer: int, seq_id: int, length: Optional[int] = None) -> torch.Tensor:
        return self._gather(self.k[layer], None if self.k_sb is None else self.k_sb[layer], seq_id, length)

    def get_values(self, layer: int, seq_id: int, length: Optional[int] = None) -> torch.Tensor:
        return self._gather(self.v[layer], None if self.v_sb is None else self.v_sb[layer], seq_id, length)

    def sb(self, layer: int) -> dict:
        """Keyword arguments that tell the kernels about the 8-bit format (empty for bf16)."""
        if not self.quantized:
            return {}
        return {"k_sb": self.k_sb[layer], "v_sb": self.v_sb[layer]}

    def bytes_per_token(self) -> int:
        """Cache bytes one token occupies over all layers (K and V)."""
        per = self.head_dim + (self.head_dim // 64) * 4 if self.quantized else \
            self.head_dim * torch.empty(0, dtype=self.dtype).element_size()
        return 2 * self.num_layers * self.kv_heads * per
