"""Multi-head latent attention (DeepSeek): K/V are compressed to a latent ``c_kv`` of rank
``kv_lora_rank`` plus one decoupled RoPE key of ``rope_head_dim`` shared by all heads, and only
those are cached. Mirrors crates/rmlx-nn/src/mla.rs:47-730 (``MlaConfig``, ``MlaKvCache`` caching
``c_kv [seq, kv_lora_rank]`` and ``k_rope [seq, rope_head_dim]``, compress / expand / compute_q /
forward, compression-ratio helper at mla.rs:723)."""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional

import torch

from ..config import MlaConfig
from ..reference import ops as ref


class MlaKvCache:
    def __init__(self, cfg: MlaConfig, dtype=torch.bfloat16, device="cpu"):
        self.c_kv = torch.zeros(cfg.max_seq_len, cfg.kv_lora_rank, dtype=dtype, device=device)
        self.k_rope = torch.zeros(cfg.max_seq_len, cfg.rope_head_dim, dtype=dtype, device=device)
        self.seq_len = 0

    def append(self, c_kv: torch.Tensor, k_rope: torch.Tensor) -> None:
        n = c_kv.shape[0]
        self.c_kv[self.seq_len:self.seq_len + n] = c_kv.to(self.c_kv.dtype)
        self.k_rope[self.seq_len:self.seq_len + n] = k_rope.to(self.k_rope.dtype)
        self.seq_len += n

    def trim(self, n: int) -> None:
        self.seq_len = max(0, self.seq_len - n)


@dataclass
class MlaWeights:
    w_dkv: torch.Tensor          # [kv_lora_rank + rope_head_dim, hidden]   down-projection (+ rope key)
    kv_norm: torch.Tensor        # [kv_lora_rank]
    w_uk: torch.Tensor           # [heads * head_dim, kv_lora_rank]          latent -> keys
    w_uv: torch.Tensor           # [heads * v_head_dim, kv_lora_rank]        latent -> values
    w_q: Optional[torch.Tensor]  # [heads * (head_dim + rope_head_dim), hidden]  (q_lora_rank == 0)
    w_dq: Optional[torch.Tensor] = None    # [q_lora_rank, hidden]
    q_norm: Optional[torch.Tensor] = None  # [q_lora_rank]
    w_uq: Optional[torch.Tensor] = None    # [heads * (head_dim + rope_head_dim), q_lora_rank]
    w_o: Optional[torch.Tensor] = None     # [hidden, heads * v_head_dim]


def random_mla_weights(cfg: MlaConfig, seed: int = 0, std: float = 0.02, dtype=torch.float32) -> MlaWeights:
    g = torch.Generator().manual_seed(seed)
    r = lambda *s: (torch.randn(*s, generator=g) * std).to(dtype)
    h, qd = cfg.num_heads, cfg.head_dim + cfg.rope_head_dim
    w = MlaWeights(r(cfg.kv_lora_rank + cfg.rope_head_dim, cfg.hidden_size), torch.ones(cfg.kv_lora_rank, dtype=dtype),
                   r(h * cfg.head_dim, cfg.kv_lora_rank), r(h * cfg.v_head_dim, cfg.kv_lora_rank), None,
                   w_o=r(cfg.hidden_size, h * cfg.v_head_dim))
    if cfg.q_lora_rank:
        w.w_dq, w.q_norm, w.w_uq = r(cfg.q_lora_rank, cfg.hidden_size), torch.ones(cfg.q_lora_rank, dtype=dtype), r(h * qd, cfg.q_lora_rank)
    else:
        w.w_q = r(h * qd, cfg.hidden_size)
    return w


class MlaAttention:
    def __init__(self, cfg: MlaConfig, w: MlaWeights, eps: float = 1e-6):
        self.cfg, self.w, self.eps = cfg.validate(), w, eps
        self.cos, self.sin = ref.rope_tables(cfg.rope_head_dim, cfg.max_seq_len, cfg.rope_theta,
                                             device=w.w_dkv.device)
        self.scale = 1.0 / math.sqrt(cfg.head_dim + cfg.rope_head_dim)

    def compression_ratio(self, num_kv_heads: Optional[int] = None) -> float:
        """Bytes of a standard KV cache per token divided by bytes of the latent cache."""
        c = self.cfg
        std = 2 * (num_kv_heads or c.num_heads) * c.head_dim
        return std / (c.kv_lora_rank + c.rope_head_dim)

    def compress(self, x: torch.Tensor, pos: torch.Tensor):
        c = self.cfg
        ckr = x @ self.w.w_dkv.to(x.dtype).t()
        c_kv = ref.rms_norm(ckr[:, :c.kv_lora_rank], self.w.kv_norm, self.eps)
        k_rope = ref.apply_rope(ckr[:, None, c.kv_lora_rank:], pos, self.cos, self.sin).squeeze(1)
        return c_kv, k_rope

    def expand(self, c_kv: torch.Tensor):
        c = self.cfg
        k = (c_kv @ self.w.w_uk.to(c_kv.dtype).t()).view(-1, c.num_heads, c.head_dim)
        v = (c_kv @ self.w.w_uv.to(c_kv.dtype).t()).view(-1, c.num_heads, c.v_head_dim)
        return k, v

    def compute_q(self, x: torch.Tensor, pos: torch.Tensor) -> torch.Tensor:
        c, w = self.cfg, self.w
        if w.w_dq is not None:
            q = ref.rms_norm(x @ w.w_dq.to(x.dtype).t(), w.q_norm, self.eps) @ w.w_uq.to(x.dtype).t()
        else:
            q = x @ w.w_q.to(x.dtype).t()
        q = q.view(-1, c.num_heads, c.head_dim + c.rope_head_dim)
        q_rope = ref.apply_rope(q[..., c.head_dim:], pos, self.cos, self.sin)
        return torch.cat([q[..., :c.head_dim], q_rope], -1)

    def forward(self, x: torch.Tensor, cache: Optional[MlaKvCache] = None) -> torch.Tensor:
        c = self.cfg
        t = x.shape[0]
        start = cache.seq_len if cache is not None else 0
        pos = torch.arange(start, start + t, device=x.device)
        c_kv, k_rope = self.compress(x, pos)
        if cache is not None:
            cache.append(c_kv, k_rope)
            c_all, kr_all = cache.c_kv[:cache.seq_len].to(x.dtype), cache.k_rope[:cache.seq_len].to(x.dtype)
        else:
            c_all, kr_all = c_kv, k_rope
        k_nope, v = self.expand(c_all)
        k = torch.cat([k_nope, kr_all[:, None, :].expand(-1, c.num_heads, -1)], -1)
        q = self.compute_q(x, pos)
        out = ref.sdpa(q, k, v, self.scale, start)              # v_head_dim may differ from head_dim
        return out.reshape(t, -1) @ self.w.w_o.to(x.dtype).t()

    __call__ = forward


class MlaPagedCache:
    """Paged latent cache for several sequences: one row of ``kv_lora_rank + rope_head_dim`` values
    per token (latent, then the RoPE key), pages of 16 tokens, page 0 reserved; block tables and
    lengths live on the device so the decode kernel (csrc/kernels/mla_decode.cu) is shape-stable.
    A row is stored with ``ROW_PAD`` unused values behind it (``pages`` is a view without them):
    the kernel copies whole pages into shared memory, where the 16 bytes keep rows on different
    banks.
    The paged counterpart of ``MlaKvCache`` (crates/rmlx-nn/src/mla.rs:111-250)."""

    PAGE = 16
    ROW_PAD = 8

    def __init__(self, cfg: MlaConfig, num_blocks: int, max_seqs: int = 8, max_blocks_per_seq: Optional[int] = None,
                 dtype=torch.bfloat16, device="cpu"):
        self.cfg = cfg
        self.width = cfg.kv_lora_rank + cfg.rope_head_dim
        self.store = torch.zeros(num_blocks, self.PAGE, self.width + self.ROW_PAD, dtype=dtype, device=device)
        self.pages = self.store[..., :self.width]
        mb = max_blocks_per_seq or (cfg.max_seq_len + self.PAGE - 1) // self.PAGE
        self.block_table = torch.zeros(max_seqs, mb, dtype=torch.int32, device=device)
        self.seq_lens = torch.zeros(max_seqs, dtype=torch.int32, device=device)
        self._free = list(range(num_blocks - 1, 0, -1))
        self._tables = {}
        self._lens = {}
        self._slots = {}
        self._free_slots = list(range(max_seqs - 1, -1, -1))

    def add_sequence(self, seq_id: int) -> int:
        slot = self._free_slots.pop()
        self._slots[seq_id], self._tables[seq_id], self._lens[seq_id] = slot, [], 0
        return slot

    def free_sequence(self, seq_id: int) -> None:
        self._free.extend(self._tables.pop(seq_id))
        slot = self._slots.pop(seq_id)
        del self._lens[seq_id]
        self.block_table[slot].zero_()
        self.seq_lens[slot] = 0
        self._free_slots.append(slot)

    def slot_of(self, seq_id: int) -> int:
        return self._slots[seq_id]

    def seq_len(self, seq_id: int) -> int:
        return self._lens[seq_id]

    def append(self, seq_id: int, c_kv: torch.Tensor, k_rope: torch.Tensor) -> None:
        """c_kv [n, kv_lora_rank], k_rope [n, rope_head_dim]: the next n tokens of the sequence."""
        n, start = c_kv.shape[0], self._lens[seq_id]
        table, slot = self._tables[seq_id], self._slots[seq_id]
        need = (start + n + self.PAGE - 1) // self.PAGE
        if need > self.block_table.shape[1] or need - len(table) > len(self._free):
            raise RuntimeError("latent cache exhausted")
        while len(table) < need:
            table.append(self._free.pop())
        dev = self.pages.device
        self.block_table[slot, :len(table)] = torch.tensor(table, dtype=torch.int32, device=dev)
        pos = torch.arange(start, start + n, device=dev)
        blk = torch.tensor(table, dtype=torch.int64, device=dev)[pos // self.PAGE]
        rows = torch.cat([c_kv, k_rope], -1).to(self.pages.dtype)
        self.pages[blk, pos % self.PAGE] = rows
        self._lens[seq_id] = start + n
        self.seq_lens[slot] = start + n

    def gather(self, seq_id: int):
        """(c_kv [len, kv_lora_rank], k_rope [len, rope_head_dim]) of one sequence, contiguous."""
        n = self._lens[seq_id]
        blk = torch.tensor(self._tables[seq_id], dtype=torch.int64, device=self.pages.device)
        flat = self.pages[blk].reshape(-1, self.width)[:n]
        return flat[:, :self.cfg.kv_lora_rank], flat[:, self.cfg.kv_lora_rank:]

    def bytes_per_token(self) -> int:
        return (self.width + self.ROW_PAD) * self.pages.element_size()


def _mla_decode_kernel(q_abs: torch.Tensor, cache: MlaPagedCache, slots: torch.Tensor,
                       scale: float, splits: int = 0) -> torch.Tensor:
    """q_abs [B, H, LAT + ROPE] bf16 (absorbed queries) -> o_lat [B, H, LAT] bf16 on the device
    kernel; row b attends to the sequence in cache slot ``slots[b]``."""
    from .. import _lib
    _lib.register_cuda_sigs({
        "rmlx_mla_decode_paged": ("ppppppppiiiiiiifip", "i"),
        "rmlx_mla_decode_part_o_elems": ("iiii", "q"),
        "rmlx_mla_decode_part_ml_elems": ("iii", "q"),
    })
    lib = _lib.cuda()
    b, h, w = q_abs.shape
    lat = cache.cfg.kv_lora_rank
    table, lens = cache.block_table, cache.seq_lens      # the kernel indexes both by slots[b]
    slots = slots.to(torch.int32)
    if splits <= 0:
        # Up to 16 head tiles: wide blocks (eight warps, one per SM), one wave of 148. More: narrow
        # blocks (four warps, two per SM; the launcher picks them once the grid exceeds the SMs),
        # one wave of 296. At least 8 pages per split.
        tiles = b * ((h + 15) // 16)
        longest = int(table.shape[1]) * MlaPagedCache.PAGE
        slots_per_wave = 148 if tiles <= 16 else 296
        splits = max(1, min(64, slots_per_wave // tiles, longest // 128))
    out = torch.empty(b, h, lat, dtype=torch.bfloat16, device=q_abs.device)
    part_o = part_ml = None
    if splits > 1:
        part_o = torch.empty(lib.rmlx_mla_decode_part_o_elems(b, h, splits, lat), dtype=torch.float32,
                             device=q_abs.device)
        part_ml = torch.empty(lib.rmlx_mla_decode_part_ml_elems(b, h, splits), dtype=torch.float32,
                              device=q_abs.device)
    rc = lib.rmlx_mla_decode_paged(q_abs.data_ptr(), cache.store.data_ptr(), table.data_ptr(),
                                   lens.data_ptr(), slots.data_ptr(), out.data_ptr(), _lib.ptr(part_o), _lib.ptr(part_ml),
                                   b, h, lat, w - lat, cache.store.shape[2], table.shape[1], splits, scale, 0,
                                   _lib.stream_ptr())
    _lib.check(rc, "mla_decode_paged")
    return out


def mla_decode_paged(attn: MlaAttention, x: torch.Tensor, cache: MlaPagedCache, seq_ids,
                     use_kernel: Optional[bool] = None, splits: int = 0) -> torch.Tensor:
    """One decode step for ``len(seq_ids)`` sequences: x [B, hidden] (row b = the next token of
    sequence seq_ids[b]). The new token's latent is appended to the paged cache; attention runs
    in the absorbed form over the cached latents (the key up-projection folded into the query, the
    value up-projection applied to the attended latent), on the device kernel for CUDA bf16
    tensors of a supported width, else with library ops. Returns [B, hidden]."""
    c, w = attn.cfg, attn.w
    b = x.shape[0]
    dev = x.device
    pos = torch.tensor([cache.seq_len(s) for s in seq_ids], device=dev)
    c_kv, k_rope = attn.compress(x, pos)
    for i, s in enumerate(seq_ids):
        cache.append(s, c_kv[i:i + 1], k_rope[i:i + 1])
    q = attn.compute_q(x, pos)                                          # [B, H, hd + rope]
    w_uk = w.w_uk.to(x.dtype).view(c.num_heads, c.head_dim, c.kv_lora_rank)
    w_uv = w.w_uv.to(x.dtype).view(c.num_heads, c.v_head_dim, c.kv_lora_rank)
    q_lat = torch.einsum("bhd,hdl->bhl", q[..., :c.head_dim], w_uk)     # absorbed key up-projection
    q_abs = torch.cat([q_lat, q[..., c.head_dim:]], -1)
    if use_kernel is None:
        use_kernel = x.is_cuda and x.dtype == torch.bfloat16 and cache.pages.dtype == torch.bfloat16 and \
            (c.kv_lora_rank, c.rope_head_dim) in ((512, 64), (128, 64))
    if use_kernel:
        slots = torch.tensor([cache.slot_of(s) for s in seq_ids], dtype=torch.int32, device=dev)
        o_lat = _mla_decode_kernel(q_abs.contiguous(), cache, slots, attn.scale, splits)
    else:
        outs = []
        for i, s in enumerate(seq_ids):
            ck, kr = cache.gather(s)
            keys = torch.cat([ck, kr], -1).to(x.dtype)                 # [len, LAT + ROPE]
            sc = (q_abs[i].float() @ keys.float().t()) * attn.scale    # [H, len]
            outs.append((torch.softmax(sc, -1) @ ck.float()).to(x.dtype))
        o_lat = torch.stack(outs)
    o = torch.einsum("bhl,hvl->bhv", o_lat.to(x.dtype), w_uv)          # value up-projection
    return o.reshape(b, -1) @ w.w_o.to(x.dtype).t()
