"""Convolution layers with the reference's API (crates/rmlx-nn/src/conv.rs:17-357): a config, a
layer that may exist before its weights do, weight validation on load, channels-first tensors
(``[B, C_in, W]`` / ``[B, C_in, H, W]``, weights ``[C_out, C_in / groups, K...]``). The arithmetic
is the library convolution; ``conv1d_direct`` / ``conv2d_direct`` restate it with explicit loops
over the kernel taps and are the oracle of the tests. ``channels_last=True`` takes MLX-style
``[B, W, C]`` / ``[B, H, W, C]`` activations and ``[C_out, K..., C_in / groups]`` weights instead.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple, Union

import torch
import torch.nn.functional as F

Pair = Union[int, Tuple[int, int]]


def _pair(v: Pair) -> Tuple[int, int]:
    return (v, v) if isinstance(v, int) else (int(v[0]), int(v[1]))


def conv_out_len(n: int, kernel: int, stride: int = 1, padding: int = 0, dilation: int = 1) -> int:
    """(n + 2 p - d (k - 1) - 1) // s + 1, the output extent of one axis."""
    return (n + 2 * padding - dilation * (kernel - 1) - 1) // stride + 1


@dataclass
class Conv1dConfig:
    in_channels: int
    out_channels: int
    kernel_size: int
    stride: int = 1
    padding: int = 0
    dilation: int = 1
    groups: int = 1
    has_bias: bool = False

    def validate(self) -> "Conv1dConfig":
        if min(self.in_channels, self.out_channels, self.kernel_size, self.stride, self.dilation, self.groups) < 1:
            raise ValueError("Conv1d: channels, kernel, stride, dilation and groups must be positive")
        if self.in_channels % self.groups or self.out_channels % self.groups:
            raise ValueError("Conv1d: groups must divide both channel counts")
        if self.padding < 0:
            raise ValueError("Conv1d: negative padding")
        return self


@dataclass
class Conv2dConfig:
    in_channels: int
    out_channels: int
    kernel_size: Pair
    stride: Pair = 1
    padding: Pair = 0
    dilation: Pair = 1
    groups: int = 1
    has_bias: bool = False

    def validate(self) -> "Conv2dConfig":
        ks, st, dl, pd = _pair(self.kernel_size), _pair(self.stride), _pair(self.dilation), _pair(self.padding)
        if min(self.in_channels, self.out_channels, self.groups, *ks, *st, *dl) < 1:
            raise ValueError("Conv2d: channels, kernel, stride, dilation and groups must be positive")
        if self.in_channels % self.groups or self.out_channels % self.groups:
            raise ValueError("Conv2d: groups must divide both channel counts")
        if min(pd) < 0:
            raise ValueError("Conv2d: negative padding")
        return self


class _ConvBase:
    NAME = "Conv"
    SPATIAL = 1

    def __init__(self, config, channels_last: bool = False):
        self._config = config.validate()
        self.channels_last = channels_last
        self._weight: Optional[torch.Tensor] = None
        self._bias: Optional[torch.Tensor] = None

    def _kernel(self) -> Tuple[int, ...]:
        raise NotImplementedError

    def load_weights(self, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> None:
        c = self._config
        per_group = c.in_channels // c.groups
        want = (c.out_channels, *self._kernel(), per_group) if self.channels_last else \
            (c.out_channels, per_group, *self._kernel())
        if tuple(weight.shape) != want:
            raise ValueError(f"{self.NAME}: weight shape {tuple(weight.shape)}, expected {want}")
        if bias is not None and tuple(bias.shape) != (c.out_channels,):
            raise ValueError(f"{self.NAME}: bias shape {tuple(bias.shape)}, expected ({c.out_channels},)")
        if c.has_bias and bias is None:
            raise ValueError(f"{self.NAME}: the config asks for a bias")
        self._weight, self._bias = weight, bias

    def config(self):
        return self._config

    def has_weights(self) -> bool:
        return self._weight is not None

    def weight(self) -> Optional[torch.Tensor]:
        return self._weight

    def bias(self) -> Optional[torch.Tensor]:
        return self._bias

    def _checked(self, x: torch.Tensor) -> torch.Tensor:
        if self._weight is None:
            raise ValueError(f"{self.NAME}: weights not loaded")
        if x.dim() != 2 + self.SPATIAL:
            raise ValueError(f"{self.NAME}: input must have {2 + self.SPATIAL} dimensions")
        ch = x.shape[-1] if self.channels_last else x.shape[1]
        if ch != self._config.in_channels:
            raise ValueError(f"{self.NAME}: {ch} input channels, expected {self._config.in_channels}")
        return x

    def __call__(self, x):
        return self.forward(x)


class Conv1d(_ConvBase):
    NAME, SPATIAL = "Conv1d", 1

    def __init__(self, config_or_weight, bias: Optional[torch.Tensor] = None, stride: int = 1,
                 padding: int = 0, dilation: int = 1, groups: int = 1, channels_last: bool = False):
        """``Conv1d(Conv1dConfig(...))`` makes a layer that waits for ``load_weights``;
        ``Conv1d(weight, bias, stride=..., ...)`` is ``from_arrays``."""
        if isinstance(config_or_weight, Conv1dConfig):
            super().__init__(config_or_weight, channels_last)
            return
        w = config_or_weight
        k, per = (w.shape[1], w.shape[2]) if channels_last else (w.shape[2], w.shape[1])
        super().__init__(Conv1dConfig(per * groups, w.shape[0], k, stride, padding, dilation, groups,
                                      bias is not None), channels_last)
        self.load_weights(w, bias)

    from_arrays = classmethod(lambda cls, weight, bias=None, **kw: cls(weight, bias, **kw))

    def _kernel(self):
        return (self._config.kernel_size,)

    def out_len(self, n: int) -> int:
        c = self._config
        return conv_out_len(n, c.kernel_size, c.stride, c.padding, c.dilation)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        """[B, C_in, W] -> [B, C_out, W_out] (``channels_last``: [B, W, C_in] -> [B, W_out, C_out])."""
        c, w = self._config, self._weight
        x = self._checked(x)
        if self.channels_last:
            x, w = x.transpose(1, 2), w.permute(0, 2, 1)
        y = F.conv1d(x, w, self._bias, c.stride, c.padding, c.dilation, c.groups)
        return y.transpose(1, 2) if self.channels_last else y


class Conv2d(_ConvBase):
    NAME, SPATIAL = "Conv2d", 2

    def __init__(self, config_or_weight, bias: Optional[torch.Tensor] = None, stride: Pair = 1,
                 padding: Pair = 0, dilation: Pair = 1, groups: int = 1, channels_last: bool = False):
        if isinstance(config_or_weight, Conv2dConfig):
            super().__init__(config_or_weight, channels_last)
            return
        w = config_or_weight
        ks, per = ((w.shape[1], w.shape[2]), w.shape[3]) if channels_last else ((w.shape[2], w.shape[3]), w.shape[1])
        super().__init__(Conv2dConfig(per * groups, w.shape[0], ks, stride, padding, dilation, groups,
                                      bias is not None), channels_last)
        self.load_weights(w, bias)

    from_arrays = classmethod(lambda cls, weight, bias=None, **kw: cls(weight, bias, **kw))

    def _kernel(self):
        return _pair(self._config.kernel_size)

    def out_size(self, h: int, w: int) -> Tuple[int, int]:
        c = self._config
        ks, st, pd, dl = _pair(c.kernel_size), _pair(c.stride), _pair(c.padding), _pair(c.dilation)
        return conv_out_len(h, ks[0], st[0], pd[0], dl[0]), conv_out_len(w, ks[1], st[1], pd[1], dl[1])

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        """[B, C_in, H, W] -> [B, C_out, H_out, W_out] (``channels_last``: NHWC in and out)."""
        c, w = self._config, self._weight
        x = self._checked(x)
        if self.channels_last:
            x, w = x.permute(0, 3, 1, 2), w.permute(0, 3, 1, 2)
        y = F.conv2d(x, w, self._bias, _pair(c.stride), _pair(c.padding), _pair(c.dilation), c.groups)
        return y.permute(0, 2, 3, 1) if self.channels_last else y


def conv1d_direct(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None, stride: int = 1,
                  padding: int = 0, dilation: int = 1, groups: int = 1) -> torch.Tensor:
    """The definition, tap by tap in fp32: x [B, C_in, W], w [C_out, C_in / groups, K]."""
    b, c_in, n = x.shape
    c_out, per, k = w.shape
    out_n = conv_out_len(n, k, stride, padding, dilation)
    xp = F.pad(x.float(), (padding, padding))
    y = torch.zeros(b, c_out, out_n)
    og = c_out // groups
    for g in range(groups):
        xs = xp[:, g * per:(g + 1) * per]
        ws = w[g * og:(g + 1) * og].float()
        for t in range(k):
            cols = xs[:, :, t * dilation: t * dilation + (out_n - 1) * stride + 1: stride]   # [B, per, out_n]
            y[:, g * og:(g + 1) * og] += torch.einsum("bcn,oc->bon", cols, ws[:, :, t])
    return y if bias is None else y + bias.float()[None, :, None]


def conv2d_direct(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None, stride: Pair = 1,
                  padding: Pair = 0, dilation: Pair = 1, groups: int = 1) -> torch.Tensor:
    """x [B, C_in, H, W], w [C_out, C_in / groups, KH, KW], tap by tap in fp32."""
    (sh, sw), (ph, pw), (dh, dw) = _pair(stride), _pair(padding), _pair(dilation)
    b, c_in, h, wd = x.shape
    c_out, per, kh, kw = w.shape
    oh, ow = conv_out_len(h, kh, sh, ph, dh), conv_out_len(wd, kw, sw, pw, dw)
    xp = F.pad(x.float(), (pw, pw, ph, ph))
    y = torch.zeros(b, c_out, oh, ow)
    og = c_out // groups
    for g in range(groups):
        xs = xp[:, g * per:(g + 1) * per]
        ws = w[g * og:(g + 1) * og].float()
        for i in range(kh):
            for j in range(kw):
                win = xs[:, :, i * dh: i * dh + (oh - 1) * sh + 1: sh, j * dw: j * dw + (ow - 1) * sw + 1: sw]
                y[:, g * og:(g + 1) * og] += torch.einsum("bchw,oc->bohw", win, ws[:, :, i, j])
    return y if bias is None else y + bias.float()[None, :, None, None]
