"""Thin module wrappers over the ops: ``Linear`` / ``QuantizedLinear`` (+ AWQ / GPTQ import),
``Embedding``, ``RMSNorm``, ``LayerNorm``, ``RotaryEmbedding`` and the activation table.

Counterparts: crates/rmlx-nn/src/linear.rs:23-683, quantized_linear.rs:19-735, embedding.rs:13-130,
rms_norm.rs:39-115, layer_norm.rs:45-173, rope.rs:55-174, activations.rs:39-605. On CUDA with bf16
inputs ``Linear`` runs this package's kernels (GEMV kernels for a handful of rows, the tcgen05
GEMM otherwise; Q4 weights go through the Q4 kernels); everywhere else it is plain PyTorch.
"""
from __future__ import annotations

from typing import Callable, Dict, Optional

import torch

from ..ops.weights import LinearWeight, W_BF16
from ..reference import ops as ref

GEMV_MAX_ROWS = 8


class Linear:
    def __init__(self, weight: LinearWeight, bias: Optional[torch.Tensor] = None):
        self.weight, self.bias = weight, bias
        self._dense = None

    @property
    def in_features(self) -> int:
        return self.weight.k

    @property
    def out_features(self) -> int:
        return self.weight.n

    def dense(self, dtype) -> torch.Tensor:
        if self._dense is None or self._dense.dtype != dtype:
            self._dense = self.weight.dequantized().to(dtype)
        return self._dense

    def forward(self, x: torch.Tensor, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
        shp = x.shape
        x2 = x.reshape(-1, shp[-1])
        r2 = None if residual is None else residual.reshape(-1, self.out_features)
        if x2.is_cuda and x2.dtype == torch.bfloat16 and self.bias is None:
            from ..ops import decode as D
            if x2.shape[0] <= GEMV_MAX_ROWS:
                y = D.rms_gemv(x2.contiguous(), self.weight, None, 0.0, residual=r2)
            elif self.weight.kind == W_BF16:
                from ..ops.gemm import gemm_bf16
                y = gemm_bf16(x2.contiguous(), self.weight.w, residual=r2)
            else:
                from ..ops.quantized import qmm
                y = qmm(x2.contiguous(), self.weight, residual=r2)
        else:
            y = x2 @ self.dense(x2.dtype).t()
            if self.bias is not None:
                y = y + self.bias.to(y.dtype)
            if r2 is not None:
                y = y + r2
        return y.view(*shp[:-1], self.out_features)

    __call__ = forward


class QuantizedLinear(Linear):
    """MLX affine 4-bit, group 64 (crates/rmlx-nn/src/quantized_linear.rs:19-300)."""

    @staticmethod
    def from_dense(w: torch.Tensor, device=None) -> "QuantizedLinear":
        return QuantizedLinear(LinearWeight.from_dense(w, "q4", device=device))

    @staticmethod
    def from_awq(qweight: torch.Tensor, qzeros: torch.Tensor, scales: torch.Tensor,
                 group_size: int = 128, device=None) -> "QuantizedLinear":
        """AutoAWQ GEMM layout: qweight int32 [in, out/8], qzeros int32 [in/g, out/8], scales
        [in/g, out]; nibble order within a word 0,2,4,6,1,3,5,7. w = (q - z) * s."""
        return QuantizedLinear(LinearWeight.from_dense(awq_dequantize(qweight, qzeros, scales, group_size),
                                                       "q4", device=device))

    @staticmethod
    def from_gptq(qweight: torch.Tensor, qzeros: torch.Tensor, scales: torch.Tensor,
                  g_idx: Optional[torch.Tensor] = None, device=None) -> "QuantizedLinear":
        """GPTQ layout: qweight int32 [in/8, out], qzeros int32 [groups, out/8] (stored minus one),
        scales [groups, out], optional g_idx [in] mapping each input to its group."""
        return QuantizedLinear(LinearWeight.from_dense(gptq_dequantize(qweight, qzeros, scales, g_idx),
                                                       "q4", device=device))


_AWQ_ORDER = torch.tensor([0, 4, 1, 5, 2, 6, 3, 7])


def _unpack_int32_nibbles(t: torch.Tensor) -> torch.Tensor:
    """int32 [..., n] -> int64 [..., n, 8], nibble i at bits 4i."""
    w = t.to(torch.int64) & 0xFFFFFFFF
    return (w[..., None] >> (torch.arange(8, dtype=torch.int64, device=t.device) * 4)) & 0xF


def _native_4bit_dequant(kind: str, qweight, qzeros, scales, group_size=None, g_idx=None):
    """fp32 [out, in] on the device kernels (csrc/kernels/misc.cu) for CUDA checkpoints with fp16
    scales; None when the inputs do not qualify (the torch formulas below are the oracle)."""
    if not (qweight.is_cuda and scales.dtype == torch.float16 and qweight.dtype == torch.int32
            and qzeros.dtype == torch.int32):
        return None
    from .. import _lib
    _lib.register_cuda_sigs({"rmlx_awq_dequant": ("ppppiiip", "i"),
                             "rmlx_gptq_dequant": ("pppppiiip", "i")})
    lib, st = _lib.cuda(), _lib.stream_ptr()
    qweight, qzeros, scales = qweight.contiguous(), qzeros.contiguous(), scales.contiguous()
    if kind == "awq":
        in_f, out_f = qweight.shape[0], qweight.shape[1] * 8
        out = torch.empty(out_f, in_f, dtype=torch.float32, device=qweight.device)
        rc = lib.rmlx_awq_dequant(qweight.data_ptr(), qzeros.data_ptr(), scales.data_ptr(), out.data_ptr(),
                                  in_f, out_f, group_size, st)
    else:
        in_f, out_f = qweight.shape[0] * 8, qweight.shape[1]
        out = torch.empty(out_f, in_f, dtype=torch.float32, device=qweight.device)
        gi = None if g_idx is None else g_idx.to(torch.int32).contiguous()
        rc = lib.rmlx_gptq_dequant(qweight.data_ptr(), qzeros.data_ptr(), scales.data_ptr(), _lib.ptr(gi),
                                   out.data_ptr(), in_f, out_f, scales.shape[0], st)
    if rc == -2:
        return None
    _lib.check(rc, f"{kind}_dequant")
    return out


def awq_dequantize(qweight, qzeros, scales, group_size: int = 128) -> torch.Tensor:
    """-> fp32 [out, in] (crates/rmlx-core/src/ops/quantized.rs:707 awq_dequant_f32)."""
    native = _native_4bit_dequant("awq", qweight, qzeros, scales, group_size=group_size)
    if native is not None:
        return native
    order = _AWQ_ORDER.to(qweight.device)
    q = _unpack_int32_nibbles(qweight)[..., order].flatten(-2)        # [in, out]
    z = _unpack_int32_nibbles(qzeros)[..., order].flatten(-2)         # [in/g, out]
    g = torch.arange(q.shape[0], device=q.device) // group_size
    w = (q - z[g]).float() * scales.float()[g]
    return w.t().contiguous()


def gptq_dequantize(qweight, qzeros, scales, g_idx=None) -> torch.Tensor:
    """-> fp32 [out, in] (crates/rmlx-core/src/ops/quantized.rs:749 gptq_dequant_f32)."""
    native = _native_4bit_dequant("gptq", qweight, qzeros, scales, g_idx=g_idx)
    if native is not None:
        return native
    q = _unpack_int32_nibbles(qweight.t().contiguous()).flatten(-2).t()  # [in, out]
    z = _unpack_int32_nibbles(qzeros).flatten(-2) + 1                     # [groups, out]
    n_in = q.shape[0]
    if g_idx is None:
        g_idx = torch.arange(n_in, device=q.device) // (n_in // scales.shape[0])
    g = g_idx.long()
    return ((q - z[g]).float() * scales.float()[g]).t().contiguous()


class AwqLinear:
    """A linear layer kept in the AutoAWQ checkpoint layout (crates/rmlx-nn/src/quantized_linear.rs:350-540):
    ``forward`` multiplies with the expanded weight (expanded once, on the checkpoint's device, by the
    kernel of csrc/kernels/misc.cu for CUDA fp16 checkpoints); ``to_quantized`` re-encodes it in the
    framework's own 4-bit format, which is what the decode and prompt kernels consume."""

    def __init__(self, qweight: torch.Tensor, qzeros: torch.Tensor, scales: torch.Tensor,
                 group_size: int = 128, bias: Optional[torch.Tensor] = None):
        if qweight.shape[1] * 8 != scales.shape[1] or qzeros.shape != (scales.shape[0], qweight.shape[1]):
            raise ValueError("AwqLinear: qweight [in, out/8], qzeros [in/g, out/8], scales [in/g, out]")
        if qweight.shape[0] != scales.shape[0] * group_size:
            raise ValueError("AwqLinear: group_size does not match the scales")
        self.qweight, self.qzeros, self.scales, self.group_size, self.bias = qweight, qzeros, scales, group_size, bias
        self.in_features, self.out_features = qweight.shape[0], scales.shape[1]
        self._dense: Optional[torch.Tensor] = None

    def _expand(self) -> torch.Tensor:
        return awq_dequantize(self.qweight, self.qzeros, self.scales, self.group_size)

    def dense_weight(self) -> torch.Tensor:
        """fp32 [out, in], expanded on first use."""
        if self._dense is None:
            self._dense = self._expand()
        return self._dense

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        y = x.float() @ self.dense_weight().t()
        if self.bias is not None:
            y = y + self.bias.float()
        return y.to(x.dtype)

    __call__ = forward

    def to_quantized(self, device=None) -> "QuantizedLinear":
        return QuantizedLinear(LinearWeight.from_dense(self.dense_weight(), "q4", device=device))


class GptqLinear(AwqLinear):
    """The same for the GPTQ layout (qweight [in/8, out], qzeros stored minus one, optional
    activation-order index ``g_idx``)."""

    def __init__(self, qweight: torch.Tensor, qzeros: torch.Tensor, scales: torch.Tensor,
                 g_idx: Optional[torch.Tensor] = None, bias: Optional[torch.Tensor] = None):
        if qweight.shape[1] != scales.shape[1] or qzeros.shape != (scales.shape[0], scales.shape[1] // 8):
            raise ValueError("GptqLinear: qweight [in/8, out], qzeros [groups, out/8], scales [groups, out]")
        if g_idx is not None and g_idx.numel() != qweight.shape[0] * 8:
            raise ValueError("GptqLinear: g_idx has one entry per input feature")
        self.qweight, self.qzeros, self.scales, self.g_idx, self.bias = qweight, qzeros, scales, g_idx, bias
        self.in_features, self.out_features = qweight.shape[0] * 8, scales.shape[1]
        self.group_size = self.in_features // scales.shape[0]
        self._dense = None

    def _expand(self) -> torch.Tensor:
        return gptq_dequantize(self.qweight, self.qzeros, self.scales, self.g_idx)


class Embedding:
    def __init__(self, table: torch.Tensor):
        self.table = table

    def forward(self, ids: torch.Tensor) -> torch.Tensor:
        if self.table.is_cuda and self.table.dtype == torch.bfloat16:
            from ..ops import decode as D
            return D.embedding(self.table, ids.reshape(-1).to(torch.int32)).view(*ids.shape, -1)
        return self.table[ids.long()]

    __call__ = forward


class RMSNorm:
    def __init__(self, weight: Optional[torch.Tensor], eps: float = 1e-6):
        self.weight, self.eps = weight, eps

    def forward(self, x: torch.Tensor, residual: Optional[torch.Tensor] = None):
        if x.is_cuda and x.dtype == torch.bfloat16:
            from ..ops import decode as D
            return D.rms_norm(x.contiguous(), self.weight, self.eps,
                              None if residual is None else residual.contiguous())
        if residual is not None:
            x = x + residual
        return ref.rms_norm(x, self.weight, self.eps)

    __call__ = forward


RmsNorm = RMSNorm          # the reference's spelling


class LayerNorm:
    def __init__(self, weight=None, bias=None, eps: float = 1e-5):
        self.weight, self.bias, self.eps = weight, bias, eps

    def forward(self, x):
        return ref.layer_norm(x, self.weight, self.bias, self.eps)

    __call__ = forward


class RotaryEmbedding:
    """cos/sin tables ``[max_seq, head_dim/2]``, ``inv_freq[k] = base^(-2k/head_dim)``; split-half
    or traditional pairing; forward / inverse (crates/rmlx-nn/src/rope.rs:55-174)."""

    def __init__(self, head_dim: int, max_seq_len: int, base_freq: float = 1e4, scale: float = 1.0,
                 traditional: bool = False, device=None):
        self.traditional = traditional
        self.cos, self.sin = ref.rope_tables(head_dim, max_seq_len, base_freq, scale, device)

    def forward(self, x: torch.Tensor, positions: torch.Tensor, inverse: bool = False) -> torch.Tensor:
        """x [T, H, D]."""
        if x.is_cuda and x.dtype == torch.bfloat16:
            from ..ops import decode as D
            return D.rope(x.contiguous(), positions.to(torch.int32), self.cos, self.sin,
                          self.traditional, inverse)
        return ref.apply_rope(x, positions.long(), self.cos, self.sin, self.traditional, inverse)

    __call__ = forward


def _gelu_fast(x):
    return x * torch.sigmoid(1.702 * x)


ACTIVATIONS: Dict[str, Callable[[torch.Tensor], torch.Tensor]] = {
    "relu": torch.relu, "relu6": torch.nn.functional.relu6, "leaky_relu": torch.nn.functional.leaky_relu,
    "elu": torch.nn.functional.elu, "selu": torch.selu, "celu": torch.celu,
    "gelu": torch.nn.functional.gelu,
    "gelu_approx": lambda x: torch.nn.functional.gelu(x, approximate="tanh"), "gelu_fast": _gelu_fast,
    "silu": torch.nn.functional.silu, "swish": torch.nn.functional.silu, "mish": torch.nn.functional.mish,
    "sigmoid": torch.sigmoid, "tanh": torch.tanh, "softplus": torch.nn.functional.softplus,
    "softsign": torch.nn.functional.softsign, "hardswish": torch.nn.functional.hardswish,
    "hardsigmoid": torch.nn.functional.hardsigmoid, "quick_gelu": lambda x: x * torch.sigmoid(1.702 * x),
    "glu": lambda x: torch.nn.functional.glu(x, -1), "swiglu": ref.swiglu,
}


def activation(name: str) -> Callable[[torch.Tensor], torch.Tensor]:
    try:
        return ACTIVATIONS[name.lower()]
    except KeyError:
        raise ValueError(f"unknown activation {name!r}; have {sorted(ACTIVATIONS)}") from None
