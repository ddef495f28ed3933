"""tcgen05 GEMM against an fp32 PyTorch matmul of the same bf16 inputs (the oracle style of
crates/rmlx-core/tests/ops_tests.rs)."""
import pytest
import torch

from rmlx_b200.ops.gemm import GemmStatus, gemm_bf16

pytestmark = pytest.mark.gpu


def _check(m, n, k, bn=0, residual=False, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn(m, k, device="cuda", generator=g).to(torch.bfloat16)
    w = (torch.randn(n, k, device="cuda", generator=g) * 0.05).to(torch.bfloat16)
    r = torch.randn(m, n, device="cuda", generator=g).to(torch.bfloat16) if residual else None
    got = gemm_bf16(x, w, residual=r, bn=bn)
    torch.cuda.synchronize()
    GemmStatus.check(x.device)
    want = x.float() @ w.float().t()
    if residual:
        want = want + r.float()
    err = (got.float() - want).abs().max().item()
    mag = want.abs().max().item()
    assert err <= 1.5e-2 * mag, f"m{m} n{n} k{k} bn{bn}: err {err} mag {mag}"
    # an error confined to a few columns or one K block passes a bound scaled by the global
    # maximum: the relative Frobenius error must be small too (bf16 output)
    fro = ((got.float() - want).norm() / want.norm().clamp_min(1e-12)).item()
    assert fro <= 5e-3, f"m{m} n{n} k{k} bn{bn}: relative Frobenius error {fro}"


@pytest.mark.parametrize("bn", [32, 64, 128, 256])
def test_single_tile_each_width(bn):
    _check(128, 256, 64, bn)
    _check(128, 256, 256, bn)


@pytest.mark.parametrize("m,n,k", [(128, 512, 1024), (256, 4096, 4096), (2048, 4096, 4096),
                                   (512, 12288, 4096), (512, 4096, 12288)])
def test_aligned_shapes(m, n, k):
    _check(m, n, k)


@pytest.mark.parametrize("m,n,k", [(32, 4096, 4096), (1, 256, 512), (200, 1000, 520), (129, 264, 72),
                                   (77, 40, 4096)])
def test_ragged_shapes(m, n, k):
    _check(m, n, k)
    _check(m, n, k, residual=True, seed=1)


def test_many_tiles_per_cta_phases():
    # > 148 tiles so every CTA walks several tiles and both accumulators wrap their phases
    _check(4096, 4096, 512, bn=128)
    _check(8192, 4096, 256, bn=256, residual=True)
