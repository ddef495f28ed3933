"""Element types of the framework and of its checkpoint formats, with storage sizes
(crates/rmlx-core/src/dtype.rs:33-127): plain floats map to torch dtypes, block-quantised GGML
types carry (block elements, block bytes)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch


@dataclass(frozen=True)
class DType:
    name: str
    torch_dtype: Optional[torch.dtype]
    block_elems: int = 1
    block_bytes: int = 0

    @property
    def is_quantized(self) -> bool:
        return self.block_elems > 1

    def nbytes(self, numel: int) -> int:
        if self.block_elems > 1:
            if numel % self.block_elems:
                raise ValueError(f"{self.name}: element count must be a multiple of {self.block_elems}")
            return numel // self.block_elems * self.block_bytes
        return numel * self.block_bytes


F32 = DType("f32", torch.float32, 1, 4)
F16 = DType("f16", torch.float16, 1, 2)
BF16 = DType("bf16", torch.bfloat16, 1, 2)
U32 = DType("u32", torch.int32, 1, 4)
FP8_E4M3 = DType("fp8_e4m3", torch.float8_e4m3fn, 1, 1)
FP8_E5M2 = DType("fp8_e5m2", torch.float8_e5m2, 1, 1)
Q4_0 = DType("q4_0", None, 32, 18)      # fp16 scale + 16 bytes of nibbles
Q4_1 = DType("q4_1", None, 32, 20)      # fp16 scale + fp16 min + 16 bytes
Q8_0 = DType("q8_0", None, 32, 34)      # fp16 scale + 32 int8
Q5_0 = DType("q5_0", None, 32, 22)      # fp16 scale + 32 high bits + 16 bytes of nibbles
Q5_1 = DType("q5_1", None, 32, 24)      # fp16 scale + fp16 min + 32 high bits + 16 bytes
Q2_K = DType("q2_k", None, 256, 84)     # K-quants: 256-value super-blocks with packed sub-block scales
Q3_K = DType("q3_k", None, 256, 110)
Q4_K = DType("q4_k", None, 256, 144)
Q5_K = DType("q5_k", None, 256, 176)
Q6_K = DType("q6_k", None, 256, 210)
Q4_AFFINE_G64 = DType("q4_affine_g64", None, 64, 32 + 2 + 2)   # MLX: 64 nibbles + bf16 scale + bf16 bias

ALL = {d.name: d for d in (F32, F16, BF16, U32, FP8_E4M3, FP8_E5M2, Q4_0, Q4_1, Q5_0, Q5_1, Q8_0,
                           Q2_K, Q3_K, Q4_K, Q5_K, Q6_K, Q4_AFFINE_G64)}


def from_name(name: str) -> DType:
    try:
        return ALL[name.lower()]
    except KeyError:
        raise ValueError(f"unknown dtype {name}") from None
