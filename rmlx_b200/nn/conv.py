"""Convolution layers (thin wrappers over the framework's conv ops, as the reference's
crates/rmlx-nn/src/conv.rs:51-357 wraps its conv kernels): NLC / NHWC activations like the reference,
weights [out, kernel..., in / groups]."""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn.functional as F


class Conv1d:
    def __init__(self, weight: torch.Tensor, bias: Optional[torch.Tensor] = None, stride: int = 1,
                 padding: int = 0, dilation: int = 1, groups: int = 1):
        self.weight, self.bias = weight, bias          # [C_out, K, C_in / groups]
        self.stride, self.padding, self.dilation, self.groups = stride, padding, dilation, groups

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        """x [N, L, C_in] -> [N, L_out, C_out]."""
        y = F.conv1d(x.transpose(1, 2), self.weight.permute(0, 2, 1), self.bias, self.stride,
                     self.padding, self.dilation, self.groups)
        return y.transpose(1, 2)

    __call__ = forward


class Conv2d:
    def __init__(self, weight: torch.Tensor, bias: Optional[torch.Tensor] = None, stride=1, padding=0,
                 dilation=1, groups: int = 1):
        self.weight, self.bias = weight, bias          # [C_out, KH, KW, C_in / groups]
        self.stride, self.padding, self.dilation, self.groups = stride, padding, dilation, groups

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        """x [N, H, W, C_in] -> [N, H_out, W_out, C_out]."""
        y = F.conv2d(x.permute(0, 3, 1, 2), self.weight.permute(0, 3, 1, 2), self.bias, self.stride,
                     self.padding, self.dilation, self.groups)
        return y.permute(0, 2, 3, 1)

    __call__ = forward
