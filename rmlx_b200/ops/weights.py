"""Weight containers shared by the kernels, the reference path and the loaders.

``LinearWeight`` is one [N, K] projection stored either as bf16 or in the MLX affine 4-bit or 8-bit
layout (packed ``uint32`` ``[N, K/8]`` or ``[N, K/4]`` viewed as int32, bf16 ``scales``/``biases``
``[N, K/64]``), the checkpoint triplet of crates/rmlx-nn/src/safetensors_loader.rs:420-552; the
8-bit kernels follow affine_qmv_fast_q8 / affine_qmm_q8
(crates/rmlx-core/src/ops/quantized.rs:620,2755). A leading expert dimension
turns it into a stacked expert weight ``[E, N, K]`` (crates/rmlx-nn/src/expert_group.rs:41-57).
Row and column slicing implement the tensor-parallel shards of
crates/rmlx-nn/src/parallel.rs:888-1130 (quantised shards re-slice packed words, scales and biases
together; column cuts must fall on group boundaries).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from ..reference import ops as ref

W_BF16 = 0
W_Q4 = 1
W_Q8 = 2
GROUP = 64
_BITS = {W_Q4: 4, W_Q8: 8}


@dataclass
class LinearWeight:
    kind: int
    w: torch.Tensor                       # bf16/fp32 [.., N, K]  or int32 [.., N, K/8]
    scales: Optional[torch.Tensor] = None # bf16 (or fp16) [.., N, K/64]
    biases: Optional[torch.Tensor] = None

    # ---------------------------------------------------------------- construction
    @staticmethod
    def from_dense(w: torch.Tensor, quant: Optional[str] = None, dtype=torch.bfloat16,
                   device=None) -> "LinearWeight":
        """w: fp32 [.., N, K]. quant: None | 'q4' | 'q8'."""
        device = device or w.device
        if quant in (None, "bf16", "none"):
            return LinearWeight(W_BF16, w.to(dtype).to(device).contiguous())
        if quant not in ("q4", "q8"):
            raise ValueError(f"unsupported quantisation {quant}")
        bits = 4 if quant == "q4" else 8
        lead = w.shape[:-2]
        n, k = w.shape[-2:]
        p, s, b = ref.quantize_affine(w.reshape(-1, k), bits, GROUP)
        return LinearWeight(W_Q4 if bits == 4 else W_Q8, p.view(*lead, n, k * bits // 32).to(device).contiguous(),
                            s.view(*lead, n, k // GROUP).to(device).contiguous(),
                            b.view(*lead, n, k // GROUP).to(device).contiguous())

    @staticmethod
    def random(n: int, k: int, quant: Optional[str], device, experts: int = 0, std: float = 0.02,
               generator: Optional[torch.Generator] = None, dtype=torch.bfloat16) -> "LinearWeight":
        """Random-init weight created directly on ``device`` (benchmarks: no host staging). The Q4
        form draws uniform 4-bit codes and a per-group scale/bias that span about +-3 std."""
        lead = (experts,) if experts else ()
        if quant in (None, "bf16", "none"):
            w = torch.empty(*lead, n, k, dtype=dtype, device=device)
            # normal_ in slabs to bound temporary memory on very large stacks
            flat = w.view(-1, k)
            step = max(1, (1 << 28) // k)
            for r in range(0, flat.shape[0], step):
                flat[r:r + step].normal_(0.0, std, generator=generator)
            return LinearWeight(W_BF16, w)
        bits = 8 if quant == "q8" else 4
        words = torch.empty(*lead, n, k * bits // 32, dtype=torch.int32, device=device)
        flat = words.view(-1)
        step = 1 << 28
        for r in range(0, flat.numel(), step):
            flat[r:r + step].random_(-(2 ** 31), 2 ** 31 - 1, generator=generator)
        levels = float((1 << bits) - 1)
        scales = torch.full((*lead, n, k // GROUP), 6.0 * std / levels, dtype=torch.bfloat16,
                            device=device)
        scales.mul_(torch.empty_like(scales).uniform_(0.75, 1.25, generator=generator))
        biases = (-0.5 * levels * scales.float()).to(torch.bfloat16)
        return LinearWeight(W_Q4 if bits == 4 else W_Q8, words, scales, biases)

    # ---------------------------------------------------------------- shape
    @property
    def n(self) -> int:
        return self.w.shape[-2]

    @property
    def k(self) -> int:
        return self.w.shape[-1] * (8 if self.kind == W_Q4 else 4 if self.kind == W_Q8 else 1)

    @property
    def experts(self) -> int:
        return self.w.shape[0] if self.w.dim() == 3 else 0

    @property
    def device(self):
        return self.w.device

    def nbytes(self) -> int:
        t = self.w.numel() * self.w.element_size()
        if self.scales is not None:
            t += self.scales.numel() * 2 + self.biases.numel() * 2
        return t

    # ---------------------------------------------------------------- views
    def dequantized(self) -> torch.Tensor:
        """fp32 [.., N, K] as the kernels see it (bf16-rounded or s*q+b)."""
        if self.kind == W_BF16:
            return self.w.float()
        return ref.dequantize_affine(self.w, self.scales, self.biases, _BITS[self.kind], GROUP)

    @property
    def scales_f16(self) -> bool:
        """Scales and biases are kept in fp16, the precision of half-precision MLX checkpoints (the
        decode kernels and the dequantisation kernel read either; bf16 is the default)."""
        return self.scales is not None and self.scales.dtype == torch.float16

    @property
    def kernel_kind(self) -> int:
        """Weight kind as the native launchers take it: bit 8 flags fp16 scales and biases."""
        return self.kind | (0x100 if self.scales_f16 else 0)

    @property
    def bits(self) -> int:
        """Bits per stored weight (16 for bf16)."""
        return _BITS.get(self.kind, 16)

    def dense_bf16(self) -> torch.Tensor:
        """bf16 [.., N, K] on the weight's device: the tensor itself, or (CUDA) the packed weights
        expanded by the dequantisation kernel (csrc/kernels/misc.cu)."""
        if self.kind == W_BF16:
            return self.w
        if not self.w.is_cuda:
            return self.dequantized().to(torch.bfloat16)
        from .. import _lib
        _lib.register_cuda_sigs({"rmlx_dequant_affine": ("ppppqiiip", "i")})
        out = torch.empty(*self.w.shape[:-1], self.k, dtype=torch.bfloat16, device=self.w.device)
        rows = self.w.numel() // self.w.shape[-1]
        rc = _lib.cuda().rmlx_dequant_affine(self.w.data_ptr(), self.scales.data_ptr(),
                                             self.biases.data_ptr(), out.data_ptr(), rows, self.k,
                                             self.bits, int(self.scales_f16), _lib.stream_ptr())
        _lib.check(rc, "dequant_affine")
        return out

    def to(self, device) -> "LinearWeight":
        return LinearWeight(self.kind, self.w.to(device),
                            None if self.scales is None else self.scales.to(device),
                            None if self.biases is None else self.biases.to(device))

    def rows(self, lo: int, hi: int) -> "LinearWeight":
        """Output-row slice [lo, hi) (column-parallel shard)."""
        sl = (Ellipsis, slice(lo, hi), slice(None))
        return LinearWeight(self.kind, self.w[sl].contiguous(),
                            None if self.scales is None else self.scales[sl].contiguous(),
                            None if self.biases is None else self.biases[sl].contiguous())

    def cols(self, lo: int, hi: int) -> "LinearWeight":
        """Input-column slice [lo, hi) (row-parallel shard)."""
        if self.kind == W_BF16:
            return LinearWeight(W_BF16, self.w[..., lo:hi].contiguous())
        if lo % GROUP or hi % GROUP:
            raise ValueError("quantised column shards must fall on 64-element group boundaries")
        per = 32 // _BITS[self.kind]
        return LinearWeight(self.kind, self.w[..., lo // per:hi // per].contiguous(),
                            self.scales[..., lo // GROUP:hi // GROUP].contiguous(),
                            self.biases[..., lo // GROUP:hi // GROUP].contiguous())

    def experts_slice(self, lo: int, hi: int) -> "LinearWeight":
        return LinearWeight(self.kind, self.w[lo:hi].contiguous(),
                            None if self.scales is None else self.scales[lo:hi].contiguous(),
                            None if self.biases is None else self.biases[lo:hi].contiguous())

    @staticmethod
    def stack(parts: list) -> "LinearWeight":
        """Stack per-expert [N, K] weights into [E, N, K]."""
        kind = parts[0].kind
        assert all(p.kind == kind for p in parts)
        w = torch.stack([p.w for p in parts], 0).contiguous()
        if kind == W_BF16:
            return LinearWeight(kind, w)
        return LinearWeight(kind, w, torch.stack([p.scales for p in parts], 0).contiguous(),
                            torch.stack([p.biases for p in parts], 0).contiguous())

    @staticmethod
    def cat_rows(parts: list) -> "LinearWeight":
        """Concatenate along N (merged QKV / gate_up weights, crates/rmlx-nn/src/attention.rs:3590)."""
        kind = parts[0].kind
        assert all(p.kind == kind for p in parts)
        w = torch.cat([p.w for p in parts], dim=-2).contiguous()
        if kind == W_BF16:
            return LinearWeight(kind, w)
        return LinearWeight(kind, w, torch.cat([p.scales for p in parts], dim=-2).contiguous(),
                            torch.cat([p.biases for p in parts], dim=-2).contiguous())
