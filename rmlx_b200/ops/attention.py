"""Prompt-phase attention over the paged KV cache. Two kernels: the tcgen05 one
(csrc/kernels/flash_prefill_tc.cu; head_dim 128, optional sliding window) and the mma.sync one
(csrc/kernels/flash_prefill.cu; every other shape). The decode-phase kernel is
``ops.decode.flash_decode_paged``. Counterpart of the reference's sdpa prefill kernels
(crates/rmlx-core/src/ops/sdpa.rs:1873-2855), reading pages in place."""
from __future__ import annotations

import math
import os
from typing import Optional

import torch

from .. import _lib
from .gemm import GemmStatus

_lib.register_cuda_sigs({
    "rmlx_flash_prefill_paged": ("pppppiiiiiifip", "i"),
    "rmlx_flash_prefill_tc_supported": ("ii", "i"),
    "rmlx_flash_prefill_tc": ("pppppiiiiiiifipip", "i"),
})


def prefill_kernel_choice(head_dim: int, window: int) -> str:
    """Which kernel ``flash_prefill_paged`` runs for this shape: ``"tc"`` (tcgen05), or ``"mma"``.
    ``RMLX_FLASH_PREFILL=mma`` forces the mma.sync kernel."""
    if (os.environ.get("RMLX_FLASH_PREFILL", "tc") != "mma"
            and _lib.cuda().rmlx_flash_prefill_tc_supported(head_dim, window)):
        return "tc"
    return "mma"


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
    assert k_cache.is_contiguous() and v_cache.is_contiguous() and k_cache.shape == v_cache.shape
    assert block_row.numel() * 16 >= pos0 + t
    if scale is None:
        scale = 1.0 / math.sqrt(d)
    if out is None:
        out = torch.empty_like(q)
    kind = prefill_kernel_choice(d, window)
    if kind == "mma":
        rc = _lib.cuda().rmlx_flash_prefill_paged(
            q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), block_row.data_ptr(),
            out.data_ptr(), t, hq, k_cache.shape[1], d, pos0, window, scale, int(pdl),
            _lib.stream_ptr())
    else:
        rc = _lib.cuda().rmlx_flash_prefill_tc(
            q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), block_row.data_ptr(),
            out.data_ptr(), t, hq, k_cache.shape[1], d, k_cache.shape[0], pos0, int(window or 0), scale,
            int(os.environ.get("RMLX_FLASH_PREFILL_LANES", "0")),     # query tiles per CTA: 1, 2, 0 = choose
            GemmStatus.get(q.device).data_ptr(), int(pdl), _lib.stream_ptr())
    _lib.check(rc, "flash_prefill_paged")
    return out
