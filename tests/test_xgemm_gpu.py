"""Q4 (dequant in the tcgen05 main loop) and grouped GEMMs against fp32 PyTorch on the same
dequantised weights (oracle style: naive_matmul_with_dequant, crates/rmlx-core/src/ops/quantized.rs:10681)."""
import pytest
import torch

from rmlx_b200.ops import decode as D
from rmlx_b200.ops.gemm import GemmStatus
from rmlx_b200.ops.grouped import moe_prefill_ffn
from rmlx_b200.ops.quantized import qmm, xgemm
from rmlx_b200.ops.weights import LinearWeight
from rmlx_b200.reference import ops as ref

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _w(n, k, quant, experts=0, seed=0):
    g = torch.Generator().manual_seed(seed)
    shape = (experts, n, k) if experts else (n, k)
    return LinearWeight.from_dense(torch.randn(*shape, generator=g) * 0.05, quant, device=DEV)


def _rel(got, want, fro_bound=5e-3):
    """Maximum error over the reference's maximum; also asserts the relative Frobenius error (an
    error confined to a few columns or one K block would pass a bound scaled by the global maximum)."""
    fro = ((got.float() - want).norm() / want.norm().clamp_min(1e-12)).item()
    assert fro <= fro_bound, f"relative Frobenius error {fro} > {fro_bound}"
    return (got.float() - want).abs().max().item() / max(want.abs().max().item(), 1e-6)


@pytest.mark.parametrize("bn", [128, 256])
@pytest.mark.parametrize("m,n,k", [(128, 256, 512), (300, 1000, 1024), (2048, 4096, 4096), (64, 512, 1536)])
def test_q4_gemm(m, n, k, bn):
    w = _w(n, k, "q4")
    x = torch.randn(m, k, device=DEV).to(torch.bfloat16)
    r = torch.randn(m, n, device=DEV).to(torch.bfloat16)
    want = x.float() @ w.dequantized().t()
    got = xgemm(x, w, bn=bn)
    torch.cuda.synchronize(); GemmStatus.check(DEV)
    assert _rel(got, want) < 2e-2
    got = xgemm(x, w, residual=r, bn=bn)
    assert _rel(got, want + r.float()) < 2e-2


def test_q4_fallback_for_unaligned_k():
    w = _w(256, 192, "q4")
    x = torch.randn(40, 192, device=DEV).to(torch.bfloat16)
    assert _rel(qmm(x, w), x.float() @ w.dequantized().t()) < 2e-2


@pytest.mark.parametrize("quant", [None, "q4"])
def test_grouped_gemm_ragged_groups(quant):
    e, n, k = 8, 256, 512
    w = _w(n, k, quant, experts=e, seed=3)
    counts = torch.tensor([0, 5, 130, 0, 128, 1, 300, 0])
    off = torch.zeros(e + 1, dtype=torch.int32)
    off[1:] = torch.cumsum(counts, 0)
    x = torch.randn(int(off[-1]), k, device=DEV).to(torch.bfloat16)
    got = xgemm(x, w, offsets=off.to(DEV))
    torch.cuda.synchronize(); GemmStatus.check(DEV)
    wd = w.dequantized()
    for i in range(e):
        lo, hi = int(off[i]), int(off[i + 1])
        if hi > lo:
            assert _rel(got[lo:hi], x[lo:hi].float() @ wd[i].t()) < 2e-2, i


@pytest.mark.parametrize("quant", [None, "q4"])
def test_moe_prefill_path_matches_oracle(quant):
    torch.manual_seed(4)
    e, d, t, k = 16, 512, 200, 4
    i = 256 if quant is None else 512          # Q4 fast path needs K % 512 == 0 for the down GEMM
    gu = _w(2 * i, d, quant, experts=e, seed=5)
    dn = _w(d, i, quant, experts=e, seed=6)
    x = torch.randn(t, d, device=DEV).to(torch.bfloat16)
    logits = torch.randn(t, e, device=DEV)
    idx, wts, counts, offsets = D.topk_route(logits, k)
    out = moe_prefill_ffn(x, idx, wts, offsets, gu, dn, residual=x)
    torch.cuda.synchronize(); GemmStatus.check(DEV)
    want = x.float() + ref.moe_ffn(x.float(), idx.long(), wts, gu.dequantized(), dn.dequantized())
    assert _rel(out, want) < 3e-2


@pytest.mark.parametrize("quant", [None, "q4"])
@pytest.mark.parametrize("m,n2,k,bn", [(200, 512, 512, 0), (64, 1024, 1024, 64), (300, 1024, 512, 256)])
def test_swiglu_epilogue(dev, quant, m, n2, k, bn):
    """W = [gate; up] with n2 rows in total: the fused epilogue equals silu(x Wg^T) * (x Wu^T)."""
    torch.manual_seed(3)
    x = torch.randn(m, k, device=dev).to(torch.bfloat16)
    w = LinearWeight.from_dense(torch.randn(n2, k) * 0.05, quant, device=dev)
    got = xgemm(x, w, swiglu=True, bn=bn).float()
    h = x.float() @ w.dequantized().float().t()
    want = torch.nn.functional.silu(h[:, :n2 // 2]) * h[:, n2 // 2:]
    assert got.shape == (m, n2 // 2)
    assert (got - want).abs().max().item() / want.abs().max().item() < 1.5e-2
