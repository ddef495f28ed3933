"""Tensor-core GEMM entry points (csrc/kernels/gemm_tcgen05.cu): ``y = x @ W^T (+ residual)`` with
bf16 operands and fp32 accumulation in tensor memory. ``W`` is the usual ``[N, K]`` row-major
projection weight, so both operands are K-major and no transpose is ever materialised (the
reference caches a contiguous transpose per weight, crates/rmlx-nn/src/linear.rs:98-192)."""
from __future__ import annotations

from typing import Optional

import torch

from .. import _lib


class GemmStatus:
    """Device word a kernel sets when one of its bounded pipeline waits gave up."""

    _by_device = {}

    @classmethod
    def get(cls, device) -> torch.Tensor:
        key = torch.device(device).index or 0
        t = cls._by_device.get(key)
        if t is None:
            t = torch.zeros(1, dtype=torch.int32, device=device)
            cls._by_device[key] = t
            from ..runtime.streams import ERRORS
            ERRORS.register(f"tensor-core kernels, device {key}", t)
        return t

    @classmethod
    def check(cls, device) -> None:
        t = cls._by_device.get(torch.device(device).index or 0)
        if t is not None and int(t.item()) != 0:
            code = int(t.item())
            t.zero_()
            raise _lib.NativeError(f"a tensor-core kernel gave up waiting (status {code})")


def gemm_bf16(x: torch.Tensor, w: torch.Tensor, residual: Optional[torch.Tensor] = None,
              out: Optional[torch.Tensor] = None, bn: int = 0, pdl: bool = False) -> torch.Tensor:
    """x [M, K] bf16 (row stride a multiple of 8), w [N, K] bf16 -> [M, N] bf16."""
    _lib.require_cuda_tensor(x, w)
    assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
    assert x.dim() == 2 and w.dim() == 2 and x.stride(1) == 1 and w.stride(1) == 1
    m, k = x.shape
    n = w.shape[0]
    assert w.shape[1] == k
    if out is None:
        out = torch.empty(m, n, dtype=torch.bfloat16, device=x.device)
    assert out.stride(1) == 1
    if residual is not None:
        assert residual.shape == out.shape and residual.stride() == out.stride()
    rc = _lib.cuda().rmlx_gemm_bf16(x.data_ptr(), w.data_ptr(), out.data_ptr(), _lib.ptr(residual),
                                    m, n, k, x.stride(0), w.stride(0), out.stride(0), bn,
                                    GemmStatus.get(x.device).data_ptr(), int(pdl), _lib.stream_ptr())
    _lib.check(rc, "gemm_bf16")
    return out


_lib.register_cuda_sigs({"rmlx_gemm_bf16_f32": ("pppiiiiiipip", "i")})


def gemm_bf16_f32(x: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None,
                  pdl: bool = False) -> torch.Tensor:
    """x [M, K] bf16, w [N, K] bf16 -> [M, N] fp32: the tensor-memory accumulator stored unrounded
    (router logits, where a bf16 result would create ties)."""
    _lib.require_cuda_tensor(x, w)
    assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
    assert x.dim() == 2 and w.dim() == 2 and x.stride(1) == 1 and w.stride(1) == 1
    m, k = x.shape
    n = w.shape[0]
    assert w.shape[1] == k
    if out is None:
        out = torch.empty(m, n, dtype=torch.float32, device=x.device)
    assert out.stride(1) == 1 and out.dtype == torch.float32
    rc = _lib.cuda().rmlx_gemm_bf16_f32(x.data_ptr(), w.data_ptr(), out.data_ptr(), m, n, k,
                                        x.stride(0), w.stride(0), out.stride(0),
                                        GemmStatus.get(x.device).data_ptr(), int(pdl), _lib.stream_ptr())
    _lib.check(rc, "gemm_bf16_f32")
    return out
