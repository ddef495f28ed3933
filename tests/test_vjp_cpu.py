"""The tape's gradient rules against central differences and against torch's autograd (the shape of
the reference's phase7b VJP tests: every rule checked with ``numerical_gradient``)."""
import pytest
import torch

from rmlx_b200.utils.vjp import Tape, VjpError, numerical_gradient


def _autograd(f, *xs):
    leaves = [x.clone().requires_grad_(True) for x in xs]
    f(*leaves).backward()
    return [l.grad for l in leaves]


def test_each_rule_against_numerical_and_autograd_gradients():
    g = torch.Generator().manual_seed(0)
    r = lambda *s: torch.randn(*s, generator=g)          # noqa: E731
    a, b, row = r(3, 4), r(3, 4), r(1, 4)
    w, x, m, n = r(5, 4), r(4), r(3, 5), r(5, 2)
    nw = 1 + 0.1 * r(4)
    ang = r(3, 2)
    cos, sin = torch.cos(ang), torch.sin(ang)
    proj = r(3, 4)

    def rope_ref(x_):
        x1, x2 = x_[..., :2], x_[..., 2:]
        return torch.cat([x1 * cos - x2 * sin, x1 * sin + x2 * cos], -1)

    cases = [
        ("add (broadcast)", [a, row], lambda t, p, q: t.reduce_sum(t.mul(t.add(p, q), t.leaf(proj))),
         lambda p, q: ((p + q) * proj).sum()),
        ("mul (broadcast)", [a, row], lambda t, p, q: t.reduce_sum(t.mul(p, q)), lambda p, q: (p * q).sum()),
        ("matmul", [m, n], lambda t, p, q: t.reduce_sum(t.mul(t.matmul(p, q), t.leaf(proj[:, :2]))),
         lambda p, q: ((p @ q) * proj[:, :2]).sum()),
        ("gemv", [w, x], lambda t, p, q: t.reduce_sum(t.mul(t.gemv(p, q), t.leaf(proj[0, :1].repeat(5) + 1))),
         lambda p, q: ((p @ q) * (proj[0, :1].repeat(5) + 1)).sum()),
        ("softmax", [a], lambda t, p: t.reduce_sum(t.mul(t.softmax(p), t.leaf(proj))),
         lambda p: (torch.softmax(p, -1) * proj).sum()),
        ("rms_norm", [a, nw], lambda t, p, q: t.reduce_sum(t.mul(t.rms_norm(p, q, 1e-5), t.leaf(proj))),
         lambda p, q: (p * torch.rsqrt(p.pow(2).mean(-1, keepdim=True) + 1e-5) * q * proj).sum()),
        ("rope", [a], lambda t, p: t.reduce_sum(t.mul(t.rope(p, cos, sin), t.leaf(proj))),
         lambda p: (rope_ref(p) * proj).sum()),
        ("reduce_sum (axis)", [a], lambda t, p: t.reduce_sum(t.mul(t.reduce_sum(p, 1), t.leaf(proj[:, 0]))),
         lambda p: (p.sum(1) * proj[:, 0]).sum()),
        ("reduce_max", [a], lambda t, p: t.reduce_sum(t.mul(t.reduce_max(p, 1), t.leaf(proj[:, 0]))),
         lambda p: (p.max(1).values * proj[:, 0]).sum()),
    ]
    for name, inputs, taped, plain in cases:
        tape = Tape()
        leaves = [tape.leaf(v) for v in inputs]
        out = taped(tape, *leaves)
        assert torch.allclose(out.value, plain(*inputs), atol=1e-5), name
        got = tape.grad(out, leaves)
        for gi, ni, ai in zip(got, numerical_gradient(plain, inputs), _autograd(plain, *inputs)):
            assert torch.allclose(gi, ai, atol=1e-5), name
            assert torch.allclose(gi, ni, atol=2e-3), name


def test_a_small_network_accumulates_over_shared_inputs():
    """x feeds two branches (norm -> projection -> softmax, and a residual): gradients add up."""
    g = torch.Generator().manual_seed(1)
    x, w, nw = torch.randn(2, 6, generator=g), torch.randn(6, 6, generator=g) * 0.3, torch.ones(6)
    tgt = torch.randn(2, 6, generator=g)

    def plain(x_, w_, nw_):
        h = x_ * torch.rsqrt(x_.pow(2).mean(-1, keepdim=True) + 1e-6) * nw_
        return ((torch.softmax(h @ w_, -1) + x_) * tgt).sum()

    t = Tape()
    lx, lw, ln = t.leaf(x), t.leaf(w), t.leaf(nw)
    out = t.reduce_sum(t.mul(t.add(t.softmax(t.matmul(t.rms_norm(lx, ln), lw)), lx), t.leaf(tgt)))
    for gi, ai in zip(t.grad(out, [lx, lw, ln]), _autograd(plain, x, w, nw)):
        assert torch.allclose(gi, ai, atol=1e-5)
    all_g = t.backward(out)
    assert len(all_g) == len(t) and all_g[out.index].shape == ()


def test_errors_and_custom_operations():
    t, other = Tape(), Tape()
    a = t.leaf(torch.ones(2, 3))
    with pytest.raises(VjpError):
        t.matmul(a, t.leaf(torch.ones(2, 3)))                     # inner dimensions differ
    with pytest.raises(VjpError):
        t.add(a, other.leaf(torch.ones(2, 3)))                    # a value of another tape
    sq = t.custom("square", [a], a.value ** 2, lambda g: (2 * a.value * g,))
    assert torch.allclose(t.grad(t.reduce_sum(sq), [a])[0], 2 * torch.ones(2, 3))
    opaque = t.custom("opaque", [a], a.value.exp())
    with pytest.raises(VjpError):
        t.backward(t.reduce_sum(opaque))                          # recorded, but no backward rule
    unused = t.leaf(torch.zeros(4))
    assert torch.equal(t.grad(t.reduce_sum(sq), [unused])[0], torch.zeros(4))
    bad = t.custom("bad", [a], a.value.sum(), lambda g: (torch.ones(5),))
    with pytest.raises(VjpError):
        t.backward(bad)                                           # a rule that returns the wrong shape
