"""Prompt-phase attention over the paged KV cache (csrc/kernels/flash_prefill.cu). The decode-phase
kernel is ``ops.decode.flash_decode_paged``. Counterpart of the reference's sdpa prefill kernels
(crates/rmlx-core/src/ops/sdpa.rs:1873-2855), reading pages in place."""
from __future__ import annotations

import math
from typing import Optional

import torch

from .. import _lib

_lib.register_cuda_sigs({
    "rmlx_flash_prefill_paged": ("pppppiiiiiifip", "i"),
})


def flash_prefill_paged(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                        block_row: torch.Tensor, pos0: int, scale: Optional[float] = None,
                        window: int = 0, out: Optional[torch.Tensor] = None,
                        pdl: bool = False) -> torch.Tensor:
    """q [T, Hq, D] bf16 at positions pos0..pos0+T-1 of one sequence whose pages (already holding
    keys/values 0..pos0+T-1) are listed in ``block_row`` (int32, device). Causal; ``window`` > 0
    limits each query to the last ``window`` keys."""
    _lib.require_cuda_tensor(q, k_cache, v_cache, block_row)
    t, hq, d = q.shape
    assert q.is_contiguous() and q.dtype == torch.bfloat16 and block_row.dtype == torch.int32
    assert k_cache.shape[2] == 16 and k_cache.shape[3] == d
    assert block_row.numel() * 16 >= pos0 + t
    if scale is None:
        scale = 1.0 / math.sqrt(d)
    if out is None:
        out = torch.empty_like(q)
    rc = _lib.cuda().rmlx_flash_prefill_paged(
        q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), block_row.data_ptr(), out.data_ptr(),
        t, hq, k_cache.shape[1], d, pos0, window, scale, int(pdl), _lib.stream_ptr())
    _lib.check(rc, "flash_prefill_paged")
    return out
