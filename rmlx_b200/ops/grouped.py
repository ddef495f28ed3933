"""Grouped expert feed-forward for many tokens: rows sorted by expert go through two grouped
tensor-core GEMMs (gate|up, then down) with SwiGLU in between; ``moe_prefill_ffn`` wraps the whole
path from router output to combined result (scatter rows -> grouped gate/up -> SwiGLU -> grouped
down -> routing-weighted combine + residual). The reference's counterpart is
``ExpertGroup::grouped_forward`` + gather/scatter kernels (crates/rmlx-nn/src/expert_group.rs:308-533,
crates/rmlx-nn/src/moe.rs:1391-1508)."""
from __future__ import annotations

import os
from typing import Optional

import torch

from .. import _lib
from .quantized import xgemm
from .weights import LinearWeight, W_BF16, W_Q4, W_Q8


_lib.register_cuda_sigs({
    "rmlx_moe_grouped_q4_mma_supported": ("ii", "i"),
    "rmlx_moe_grouped_q4_mma": ("ppppippiiiiiiip", "i"),
})

# RMLX_MOE_NARROW_ROWS=n: up to n rows per expert on average the narrow-M kernels run instead of a
# 128-row tensor-core tile per expert. Off by default (0): on the 128-expert model they take 431 /
# 719 / 1138 us per layer at batch 16 / 32 / 64 against 371 / 601 / 975 for the tensor-core path. A
# block fetches its 16 weight rows with 48 bulk copies (weights, scales, biases per row) and does
# not overlap them with its arithmetic, and the copy engine spends about as long on a 128-byte
# copy as on a 2 KB one.
_NARROW_MAX_AVG_ROWS = float(os.environ.get("RMLX_MOE_NARROW_ROWS", "0"))
_NARROW_VARIANT = int(os.environ.get("RMLX_MOE_NARROW_VARIANT", "0"))


def narrow_supported(gate_up: LinearWeight, down: LinearWeight, variant: Optional[int] = None) -> bool:
    """Whether ``narrow_expert_ffn`` takes these weights (4-bit, bf16 scales, K a multiple of 512)."""
    v = _NARROW_VARIANT if variant is None else variant
    if gate_up.kind != W_Q4 or down.kind != W_Q4 or gate_up.scales_f16 or down.scales_f16:
        return False
    lib = _lib.cuda()
    return bool(lib.rmlx_moe_grouped_q4_mma_supported(gate_up.k, v)) and \
        bool(lib.rmlx_moe_grouped_q4_mma_supported(down.k, v))


def narrow_ok(gate_up: LinearWeight, down: LinearWeight, rows: int, experts: int) -> bool:
    """Whether ``moe_prefill_ffn`` sends this many sorted rows through the narrow-M kernels."""
    return 0 < rows <= _NARROW_MAX_AVG_ROWS * experts and narrow_supported(gate_up, down)


def narrow_expert_ffn(x_sorted: torch.Tensor, offsets: torch.Tensor, gate_up: LinearWeight,
                      down: LinearWeight, zero_rest: bool = False, variant: Optional[int] = None) -> torch.Tensor:
    """``grouped_expert_ffn`` for a handful of rows per expert on 4-bit weights: each (row tile,
    expert) block of csrc/kernels/qmv_mma.cu stages its weight rows once and multiplies them with
    all of the expert's rows on ``mma.sync``; experts without rows cost an early exit. The
    counterpart of the reference's gather_qmv kernels for small batches
    (crates/rmlx-core/src/ops/quantized.rs:9634)."""
    v = _NARROW_VARIANT if variant is None else variant
    lib, st = _lib.cuda(), _lib.stream_ptr()
    r = x_sorted.shape[0]
    e_local, inner = gate_up.experts, gate_up.n // 2
    off = offsets.to(torch.int32)
    assert off.numel() == e_local + 1 and x_sorted.stride(1) == 1
    act = torch.empty(r, inner, dtype=torch.bfloat16, device=x_sorted.device)
    alloc = torch.zeros if zero_rest else torch.empty
    out = alloc(r, down.n, dtype=torch.bfloat16, device=x_sorted.device)
    _lib.check(lib.rmlx_moe_grouped_q4_mma(gate_up.w.data_ptr(), gate_up.scales.data_ptr(), gate_up.biases.data_ptr(),
                                           x_sorted.data_ptr(), x_sorted.stride(0), off.data_ptr(), act.data_ptr(),
                                           act.stride(0), e_local, inner, gate_up.k, 1, v, 0, st),
               "moe_grouped_q4_mma (gate/up)")
    _lib.check(lib.rmlx_moe_grouped_q4_mma(down.w.data_ptr(), down.scales.data_ptr(), down.biases.data_ptr(),
                                           act.data_ptr(), act.stride(0), off.data_ptr(), out.data_ptr(),
                                           out.stride(0), e_local, down.n, down.k, 0, v, 0, st),
               "moe_grouped_q4_mma (down)")
    return out


def _grouped_ok(w: LinearWeight) -> bool:
    return w.n % 128 == 0 and (w.kind != W_Q4 or bool(_lib.cuda().rmlx_qgemm_supported(w.k)))


def _expanded_if_needed(w: LinearWeight) -> LinearWeight:
    if w.kind == W_BF16:
        return w
    if w.kind == W_Q4 and not w.scales_f16 and bool(_lib.cuda().rmlx_qgemm_supported(w.k)):
        return w
    dense = getattr(w, "_dense_bf16_cache", None)
    if dense is None:
        dense = LinearWeight(W_BF16, w.dense_bf16())
        w._dense_bf16_cache = dense
    return dense


def grouped_expert_ffn(x_sorted: torch.Tensor, offsets: torch.Tensor, gate_up: LinearWeight,
                       down: LinearWeight, zero_rest: bool = False) -> torch.Tensor:
    """x_sorted [R, D] bf16 (rows grouped by expert), offsets [E+1] -> [R, D]. The offsets are
    absolute row numbers of ``x_sorted``, so a rank that holds a slice of the experts passes the
    matching slice of the global offsets; ``zero_rest`` then returns zeros in the rows of the
    experts it does not hold."""
    # 8-bit weights, fp16 scales and 4-bit shapes the fused kernel does not take (K not a multiple
    # of 512, e.g. experts sliced along their inner dimension) are expanded to bf16 once and kept
    gate_up, down = _expanded_if_needed(gate_up), _expanded_if_needed(down)
    if not (_grouped_ok(gate_up) and _grouped_ok(down)):
        raise ImportError("shape not covered by the grouped tensor-core kernel")
    off = offsets.to(torch.int32)
    act = xgemm(x_sorted.contiguous(), gate_up, offsets=off, swiglu=True)   # SwiGLU in the epilogue
    out = None
    if zero_rest:
        out = torch.zeros(x_sorted.shape[0], down.n, dtype=torch.bfloat16, device=x_sorted.device)
    return xgemm(act, down, offsets=off, out=out)


def moe_prefill_ffn(x: torch.Tensor, idx: torch.Tensor, wts: torch.Tensor, offsets: torch.Tensor,
                    gate_up: LinearWeight, down: LinearWeight,
                    residual: Optional[torch.Tensor] = None, expert_base: int = 0) -> torch.Tensor:
    """x [T, D] bf16, idx/wts [T, k] from the router, offsets [E+1] int32 (device) over ALL
    experts. ``gate_up`` / ``down`` hold experts ``expert_base .. expert_base + E_local``; pairs
    routed elsewhere contribute zero (the caller sums the ranks' results)."""
    t, d = x.shape
    k = idx.shape[1]
    e = offsets.numel() - 1
    e_local = gate_up.experts
    lib, st = _lib.cuda(), _lib.stream_ptr()
    xs = torch.empty(t * k, d, dtype=torch.bfloat16, device=x.device)
    row_of_pair = torch.empty(t * k, dtype=torch.int32, device=x.device)
    cursors = torch.empty(e, dtype=torch.int32, device=x.device)
    _lib.check(lib.rmlx_moe_scatter_rows(x.data_ptr(), x.stride(0), idx.data_ptr(), offsets.data_ptr(),
                                         cursors.data_ptr(), xs.data_ptr(), row_of_pair.data_ptr(),
                                         t, k, d, e, st), "moe_scatter_rows")
    ffn = narrow_expert_ffn if narrow_ok(gate_up, down, t * k, e) else grouped_expert_ffn
    if e_local == e:
        y = ffn(xs, offsets, gate_up, down)
    else:
        y = ffn(xs, offsets[expert_base:expert_base + e_local + 1], gate_up, down, zero_rest=True)
    out = torch.empty(t, d, dtype=torch.bfloat16, device=x.device)
    _lib.check(lib.rmlx_moe_combine(y.data_ptr(), row_of_pair.data_ptr(), wts.data_ptr(),
                                    _lib.ptr(residual), 0 if residual is None else residual.stride(0),
                                    out.data_ptr(), out.stride(0), t, k, d, st), "moe_combine")
    return out
