"""Tape-based reverse-mode differentiation with explicit gradient rules.

The counterpart of the reference's ``Tape`` / ``TapedValue`` / ``*Grad`` types
(crates/rmlx-core/src/vjp.rs:5-362): values are recorded on a tape together with a rule that maps
the gradient of an operation's output to the gradients of its inputs; ``backward`` walks the tape
in reverse and accumulates. Rules exist for add, mul, matmul, softmax (last axis), RMS norm (with
weight), RoPE (rotation by given cos / sin tables), mat-vec, sum and max reductions, and a
``custom`` hook. The rules are written out (no autograd inside), so they double as the oracle of
the backward formulas; ``numerical_gradient`` checks them by central differences and the tests
also compare with torch's autograd. Training is not on the serving path: LoRA (``nn/lora.py``)
differentiates through torch.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, List, Optional, Sequence, Tuple

import torch

GradFn = Callable[[torch.Tensor], Tuple[Optional[torch.Tensor], ...]]


class VjpError(RuntimeError):
    pass


@dataclass
class TapedValue:
    index: int
    value: torch.Tensor


@dataclass
class _Entry:
    inputs: Tuple[int, ...]
    grad_fn: Optional[GradFn]
    name: str


def _unbroadcast(g: torch.Tensor, shape: torch.Size) -> torch.Tensor:
    """Sum ``g`` over the axes that broadcasting added or stretched to reach its shape."""
    while g.dim() > len(shape):
        g = g.sum(0)
    for ax, n in enumerate(shape):
        if n == 1 and g.shape[ax] != 1:
            g = g.sum(ax, keepdim=True)
    return g


class Tape:
    def __init__(self):
        self._entries: List[_Entry] = []
        self._values: List[torch.Tensor] = []

    def __len__(self) -> int:
        return len(self._entries)

    # ------------------------------------------------------------------ recording
    def leaf(self, value) -> TapedValue:
        v = torch.as_tensor(value, dtype=torch.float32)
        self._entries.append(_Entry((), None, "leaf"))
        self._values.append(v)
        return TapedValue(len(self._entries) - 1, v)

    def record(self, name: str, inputs: Sequence[TapedValue], value: torch.Tensor, grad_fn: GradFn) -> TapedValue:
        for t in inputs:
            if not (0 <= t.index < len(self._entries)) or self._values[t.index] is not t.value:
                raise VjpError(f"{name}: an input does not belong to this tape")
        self._entries.append(_Entry(tuple(t.index for t in inputs), grad_fn, name))
        self._values.append(value)
        return TapedValue(len(self._entries) - 1, value)

    # ------------------------------------------------------------------ operations
    def add(self, a: TapedValue, b: TapedValue) -> TapedValue:
        sa, sb = a.value.shape, b.value.shape
        return self.record("add", (a, b), a.value + b.value,
                           lambda g: (_unbroadcast(g, sa), _unbroadcast(g, sb)))

    def mul(self, a: TapedValue, b: TapedValue) -> TapedValue:
        av, bv = a.value, b.value
        return self.record("mul", (a, b), av * bv,
                           lambda g: (_unbroadcast(g * bv, av.shape), _unbroadcast(g * av, bv.shape)))

    def matmul(self, a: TapedValue, b: TapedValue) -> TapedValue:
        """[m, k] @ [k, n]: dA = dC B^T, dB = A^T dC."""
        av, bv = a.value, b.value
        if av.dim() != 2 or bv.dim() != 2 or av.shape[1] != bv.shape[0]:
            raise VjpError(f"matmul: shapes {tuple(av.shape)} and {tuple(bv.shape)}")
        return self.record("matmul", (a, b), av @ bv, lambda g: (g @ bv.t(), av.t() @ g))

    def gemv(self, w: TapedValue, x: TapedValue) -> TapedValue:
        """[n, k] @ [k]: dW = g x^T, dx = W^T g."""
        wv, xv = w.value, x.value
        if wv.dim() != 2 or xv.dim() != 1 or wv.shape[1] != xv.shape[0]:
            raise VjpError(f"gemv: shapes {tuple(wv.shape)} and {tuple(xv.shape)}")
        return self.record("gemv", (w, x), wv @ xv, lambda g: (torch.outer(g, xv), wv.t() @ g))

    def softmax(self, x: TapedValue) -> TapedValue:
        """Over the last axis: dx = y * (g - sum(g * y))."""
        y = torch.softmax(x.value, -1)
        return self.record("softmax", (x,), y, lambda g: (y * (g - (g * y).sum(-1, keepdim=True)),))

    def rms_norm(self, x: TapedValue, weight: TapedValue, eps: float = 1e-6) -> TapedValue:
        """y = x * r * w with r = rsqrt(mean(x^2) + eps) over the last axis.
        dx = r * (g w - x r^2 mean(g w x)), dw = sum over rows of g x r."""
        xv, wv = x.value, weight.value
        r = torch.rsqrt(xv.pow(2).mean(-1, keepdim=True) + eps)

        def grad(g):
            gw = g * wv
            dx = r * (gw - xv * r * r * (gw * xv).mean(-1, keepdim=True))
            dw = (g * xv * r).reshape(-1, xv.shape[-1]).sum(0)
            return dx, dw

        return self.record("rms_norm", (x, weight), xv * r * wv, grad)

    def rope(self, x: TapedValue, cos: torch.Tensor, sin: torch.Tensor) -> TapedValue:
        """Rotation of the two halves of the last axis by fixed tables (cos, sin of shape
        [..., d / 2]): linear in x, so the gradient is the inverse rotation of g."""
        xv = x.value
        h = xv.shape[-1] // 2
        x1, x2 = xv[..., :h], xv[..., h:]
        y = torch.cat([x1 * cos - x2 * sin, x1 * sin + x2 * cos], -1)

        def grad(g):
            g1, g2 = g[..., :h], g[..., h:]
            return (torch.cat([g1 * cos + g2 * sin, -g1 * sin + g2 * cos], -1),)

        return self.record("rope", (x,), y, grad)

    def reduce_sum(self, x: TapedValue, axis: Optional[int] = None) -> TapedValue:
        xv = x.value
        if axis is None:
            return self.record("reduce_sum", (x,), xv.sum(), lambda g: (g.expand_as(xv).clone(),))
        return self.record("reduce_sum", (x,), xv.sum(axis),
                           lambda g: (g.unsqueeze(axis).expand_as(xv).clone(),))

    def reduce_max(self, x: TapedValue, axis: int = -1) -> TapedValue:
        """The gradient goes to the first maximal element along the axis."""
        xv = x.value
        vals, idx = xv.max(axis)

        def grad(g):
            out = torch.zeros_like(xv)
            out.scatter_(axis, idx.unsqueeze(axis), g.unsqueeze(axis))
            return (out,)

        return self.record("reduce_max", (x,), vals, grad)

    def custom(self, name: str, inputs: Sequence[TapedValue], value: torch.Tensor,
               grad_fn: Optional[GradFn] = None) -> TapedValue:
        """An operation of the caller's own; without a rule it can be recorded but not
        differentiated through (``backward`` raises when a gradient reaches it)."""
        return self.record(name, inputs, value, grad_fn or _unsupported(name))

    # ------------------------------------------------------------------ reverse pass
    def backward(self, output: TapedValue, seed: Optional[torch.Tensor] = None) -> List[Optional[torch.Tensor]]:
        """Gradients of ``output`` (summed against ``seed``, default ones) with respect to every
        tape entry, by index; entries the output does not depend on get None."""
        n = len(self._entries)
        if not (0 <= output.index < n) or self._values[output.index] is not output.value:
            raise VjpError("backward: the output does not belong to this tape")
        grads: List[Optional[torch.Tensor]] = [None] * n
        grads[output.index] = torch.ones_like(output.value) if seed is None else \
            torch.as_tensor(seed, dtype=torch.float32).expand_as(output.value).clone()
        for i in range(output.index, -1, -1):
            g, e = grads[i], self._entries[i]
            if g is None or e.grad_fn is None:
                continue
            ins = e.grad_fn(g)
            if len(ins) != len(e.inputs):
                raise VjpError(f"{e.name}: the rule returned {len(ins)} gradients for {len(e.inputs)} inputs")
            for j, gi in zip(e.inputs, ins):
                if gi is None:
                    continue
                if gi.shape != self._values[j].shape:
                    raise VjpError(f"{e.name}: gradient of shape {tuple(gi.shape)} for an input of shape "
                                   f"{tuple(self._values[j].shape)}")
                grads[j] = gi if grads[j] is None else grads[j] + gi
        return grads

    def grad(self, output: TapedValue, wrt: Sequence[TapedValue]) -> List[torch.Tensor]:
        """Gradients with respect to the given values (zeros where there is no dependence)."""
        all_g = self.backward(output)
        return [all_g[t.index] if all_g[t.index] is not None else torch.zeros_like(t.value) for t in wrt]


def _unsupported(name: str) -> GradFn:
    def grad_fn(_g):
        raise VjpError(f"{name}: no backward rule")
    return grad_fn


def numerical_gradient(f: Callable[..., torch.Tensor], inputs: Sequence[torch.Tensor], eps: float = 1e-3
                       ) -> List[torch.Tensor]:
    """Central differences of the scalar ``f(*inputs)`` with respect to every element of every
    input (fp64 inside, fp32 out)."""
    xs = [torch.as_tensor(x, dtype=torch.float64).clone() for x in inputs]
    out = []
    for i, x in enumerate(xs):
        g = torch.zeros_like(x)
        flat, gf = x.reshape(-1), g.reshape(-1)
        for k in range(flat.numel()):
            old = float(flat[k])
            flat[k] = old + eps
            hi = float(f(*[t.float() for t in xs]))
            flat[k] = old - eps
            lo = float(f(*[t.float() for t in xs]))
            flat[k] = old
            gf[k] = (hi - lo) / (2 * eps)
        out.append(g.float())
    return out
