"""Quantised and grouped tensor-core matmuls (csrc/kernels/xgemm_tcgen05.cu).

``qmm``: y = x @ dequant(W)^T for MLX-affine Q4 weights, dequantised inside the tcgen05 main loop.
Shapes whose K is not a multiple of 512 (the scale arrays' rows then miss TMA's 16-byte stride
rule) take the two-step path: expand the weight once to bf16, then the bf16 tensor-core GEMM.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import _lib
from .gemm import GemmStatus, gemm_bf16
from .weights import LinearWeight, W_Q4

_lib.register_cuda_sigs({
    "rmlx_qgemm_supported": ("i", "i"),
    "rmlx_xgemm": ("ipppppppiiiiiiiipip", "i"),
    "rmlx_moe_scatter_rows": ("pipppppiiiip", "i"),
    "rmlx_moe_combine": ("ppppipiiiip", "i"),
})


def xgemm(x: torch.Tensor, w: LinearWeight, residual: Optional[torch.Tensor] = None,
          out: Optional[torch.Tensor] = None, offsets: Optional[torch.Tensor] = None, bn: int = 0,
          pdl: bool = False, swiglu: bool = False) -> torch.Tensor:
    """Plain (offsets None) or grouped tensor-core GEMM with bf16 or Q4 weights.
    Grouped: x rows sorted by expert, ``offsets`` int32 [E+1] on the device, w stacked [E, N, K].
    ``swiglu``: w's rows are [gate; up]; the result has N/2 columns of silu(gate) * up."""
    _lib.require_cuda_tensor(x, w.w)
    assert x.dtype == torch.bfloat16 and x.dim() == 2 and x.stride(1) == 1
    m, k = x.shape
    n = w.n
    assert k == w.k
    e = w.experts if offsets is not None else 0
    if offsets is not None:
        assert offsets.dtype == torch.int32 and offsets.numel() == e + 1
    if out is None:
        out = torch.empty(m, n // 2 if swiglu else n, dtype=torch.bfloat16, device=x.device)
    rc = _lib.cuda().rmlx_xgemm(w.kind, x.data_ptr(), w.w.data_ptr(), _lib.ptr(w.scales),
                                _lib.ptr(w.biases), out.data_ptr(), _lib.ptr(residual),
                                _lib.ptr(offsets), e, m, n, k, x.stride(0), out.stride(0), bn, int(swiglu),
                                GemmStatus.get(x.device).data_ptr(), int(pdl), _lib.stream_ptr())
    _lib.check(rc, "xgemm")
    return out


def qmm(x: torch.Tensor, w: LinearWeight, residual: Optional[torch.Tensor] = None,
        out: Optional[torch.Tensor] = None, pdl: bool = False) -> torch.Tensor:
    """x @ W^T for affine-quantised W: 4-bit weights are expanded inside the tensor-core GEMM's main
    loop; 8-bit weights, weights with fp16 scales and 4-bit shapes the fused kernel does not take are
    expanded to bf16 by the
    dequantisation kernel first and go through the bf16 tensor-core GEMM."""
    assert w.kind != 0
    if w.kind == W_Q4 and not w.scales_f16 and _lib.cuda().rmlx_qgemm_supported(w.k):
        return xgemm(x, w, residual, out, pdl=pdl)
    return gemm_bf16(x, w.dense_bf16(), residual=residual, out=out, pdl=pdl)
