"""Numerics of the decode-path CUDA kernels against plain PyTorch fp32 restatements of the same op
(the test style of crates/rmlx-core/tests/fused_kernel_tests.rs:91-113: CPU oracles ``cpu_rms_gemv``,
``cpu_swiglu_down``; quantised oracles as in crates/rmlx-core/src/ops/quantized.rs:10681)."""
import math

import pytest
import torch

from rmlx_b200.ops import decode as D
from rmlx_b200.ops.weights import LinearWeight
from rmlx_b200.reference import ops as ref

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True, params=["stream", "mma", "scalar"])
def q4_path(request):
    """Every test runs on the weight-streaming kernels and on both per-row Q4 implementations."""
    D.set_stream(request.param == "stream", ops="all")     # every projection on the streaming kernels
    D.set_q4_path("auto" if request.param == "stream" else request.param)
    yield request.param
    D.set_q4_path("auto")
    D.set_stream(True)
    assert D.stream_status() == 0


def _w(n, k, quant, dev, experts=0, seed=0):
    g = torch.Generator().manual_seed(seed)
    shape = (experts, n, k) if experts else (n, k)
    return LinearWeight.from_dense(torch.randn(*shape, generator=g) * 0.02, quant, device=dev)


def _close(a, b, atol=2e-2, fro=None):
    """Two bounds: the max abs error relative to the largest reference magnitude (bf16 outputs:
    2^-8 per element), and the relative Frobenius error, which an error confined to a few rows, one
    K block or the small-magnitude entries cannot hide from: 5e-3 for bf16 results, 1e-3 for fp32."""
    if fro is None:
        fro = 1e-3 if a.dtype == torch.float32 else 5e-3
    a, b = a.float().cpu(), b.float().cpu()
    assert a.shape == b.shape, (a.shape, b.shape)
    err = (a - b).abs().max().item()
    ref_mag = max(b.abs().max().item(), 1e-6)
    assert err <= atol * ref_mag, f"max err {err} vs magnitude {ref_mag}"
    rel = ((a - b).norm() / b.norm().clamp_min(1e-12)).item()
    assert rel <= fro, f"relative Frobenius error {rel} > {fro}"


@pytest.mark.parametrize("quant", [None, "q4", "q8"])
@pytest.mark.parametrize("b,n,k", [(1, 1024, 4096), (3, 72 * 128 // 8, 1024), (4, 130, 512), (6, 256, 2048), (8, 20000, 256), (1, 50, 192)])
def test_rms_gemv(dev, quant, b, n, k, q4_path):
    if quant == "q8" and q4_path != "stream":
        pytest.skip("8-bit weights run on the streaming kernels")
    torch.manual_seed(1)
    w = _w(n, k, quant, dev)
    x = torch.randn(b, k, device=dev).to(torch.bfloat16)
    nw = (1 + 0.1 * torch.randn(k, device=dev)).to(torch.bfloat16)
    res = torch.randn(b, n, device=dev).to(torch.bfloat16)
    wd = w.dequantized()
    # norm + projection
    got = D.rms_gemv(x, w, nw, 1e-6)
    want = ref.rms_norm(x.float(), nw.float(), 1e-6) @ wd.t()
    _close(got, want)
    # projection + residual, fp32 out
    got = D.rms_gemv(x, w, None, 1e-6, residual=res, out_dtype=torch.float32)
    want = x.float() @ wd.t() + res.float()
    _close(got, want)


@pytest.mark.parametrize("quant", [None, "q4", "q8"])
def test_dense_swiglu_pair(dev, quant, q4_path):
    if quant == "q8" and q4_path != "stream":
        pytest.skip("8-bit weights run on the streaming kernels")
    torch.manual_seed(2)
    b, k, i = 2, 1024, 704
    wgu = _w(2 * i, k, quant, dev, seed=3)
    wdn = _w(k, i, quant, dev, seed=4)
    x = torch.randn(b, k, device=dev).to(torch.bfloat16)
    nw = (1 + 0.1 * torch.randn(k, device=dev)).to(torch.bfloat16)
    act = D.rms_gate_up_swiglu(x, wgu, nw, 1e-6)
    gu = ref.rms_norm(x.float(), nw.float(), 1e-6) @ wgu.dequantized().t()
    want_act = ref.swiglu(gu)
    _close(act, want_act)
    # reference-style second half: raw gate_up in, silu*up fused into the staging
    if quant == "q8":
        return          # the raw-gate_up form below is a per-row kernel (bf16 / 4-bit)
    gu_bf = gu.to(torch.bfloat16)
    out = D.swiglu_down(gu_bf, wdn, residual=x)
    want = ref.swiglu(gu_bf.float()) @ wdn.dequantized().t() + x.float()
    _close(out, want)


@pytest.mark.parametrize("b", [1, 3, 5])
def test_moe_router(dev, b):
    torch.manual_seed(5)
    e, k, topk = 128, 1024, 8
    gate = (torch.randn(e, k, device=dev) * 0.05).to(torch.bfloat16)
    x = torch.randn(b, k, device=dev).to(torch.bfloat16)
    nw = (1 + 0.1 * torch.randn(k, device=dev)).to(torch.bfloat16)
    bias = torch.randn(e, device=dev) * 0.01
    idx, wts = D.moe_router(x, gate, nw, 1e-6, topk, bias)
    logits = ref.rms_norm(x.float(), nw.float(), 1e-6) @ gate.float().t()
    ridx, rw, _ = ref.topk_route(logits, topk, bias)
    # selection may legitimately differ only where two probabilities are within rounding
    same = (idx.cpu() == ridx.cpu()).float().mean().item()
    assert same > 0.9, same
    assert torch.allclose(wts.sum(-1).cpu(), torch.ones(b), atol=1e-5)
    m = idx.cpu() == ridx.cpu()
    assert torch.allclose(wts.cpu()[m], rw.cpu()[m], rtol=2e-2, atol=1e-3)


def test_topk_route_exact(dev):
    torch.manual_seed(6)
    t, e, k = 300, 128, 8
    logits = torch.randn(t, e, device=dev)
    idx, wts, counts, offsets = D.topk_route(logits, k)
    ridx, rw, rc = ref.topk_route(logits.cpu(), k)
    assert torch.equal(idx.cpu(), ridx)
    assert torch.allclose(wts.cpu(), rw, rtol=1e-4, atol=1e-6)
    assert torch.equal(counts.cpu(), rc)
    assert torch.equal(offsets.cpu(), ref.prefix_offsets(rc))
    # ties: the lowest index wins
    flat = torch.zeros(2, 16, device=dev)
    idx, _, _, _ = D.topk_route(flat, 4)
    assert idx.cpu().tolist() == [[0, 1, 2, 3]] * 2


@pytest.mark.parametrize("quant", [None, "q4", "q8"])
@pytest.mark.parametrize("b", [1, 3])
def test_moe_gate_up_down(dev, quant, b, q4_path):
    if quant == "q8" and q4_path != "stream":
        pytest.skip("8-bit weights run on the streaming kernels")
    torch.manual_seed(7)
    # Q4: 512 takes the bulk-copy tensor-core path (needs a multiple of 512); bf16: any multiple of 8
    e, d, i, topk = 16, 1024, 320 if quant is None else 512, 4
    wgu = _w(2 * i, d, quant, dev, experts=e, seed=8)
    wdn = _w(d, i, quant, dev, experts=e, seed=9)
    x = torch.randn(b, d, device=dev).to(torch.bfloat16)
    nw = (1 + 0.1 * torch.randn(d, device=dev)).to(torch.bfloat16)
    idx = torch.stack([torch.randperm(e)[:topk] for _ in range(b)]).to(torch.int32).to(dev)
    wts = torch.softmax(torch.randn(b, topk, device=dev), -1)
    act = D.moe_gate_up(x, wgu, nw, 1e-6, idx)
    xn = ref.rms_norm(x.float(), nw.float(), 1e-6)
    want_act = torch.stack([ref.swiglu(xn[t] @ wgu.dequantized()[idx[t, s]].t())
                            for t in range(b) for s in range(topk)])
    _close(act, want_act)
    out = D.moe_down(act, wdn, idx, wts, residual=x)
    want = x.float() + torch.stack([
        sum(wts[t, s] * (act[t * topk + s].float() @ wdn.dequantized()[idx[t, s]].t())
            for s in range(topk)) for t in range(b)])
    _close(out, want)
    # expert-parallel view: only experts [8, 16) are local; the rest contribute nothing
    half = LinearWeight(wdn.kind, wdn.w[8:], None if wdn.scales is None else wdn.scales[8:],
                        None if wdn.biases is None else wdn.biases[8:])
    out_hi = D.moe_down(act, half, idx, wts, residual=None, out_dtype=torch.float32, expert_base=8)
    want_hi = torch.stack([
        sum((wts[t, s] * (act[t * topk + s].float() @ wdn.dequantized()[idx[t, s]].t())
             if idx[t, s] >= 8 else torch.zeros(d, device=dev)) for s in range(topk))
        for t in range(b)])
    # fp32 result: the 4-bit path adds 16 products in fp16 pairs before widening (2^-11 per add),
    # so its floor is ~1.2e-3, not the 1e-3 of an fp32-accumulated product
    _close(out_hi, want_hi, fro=2e-3 if quant in ("q4", "q8") else None)


def _paged_setup(dev, b, hkv, hd, lens, seed=0):
    g = torch.Generator(device="cpu").manual_seed(seed)
    max_blocks = (max(lens) + 15) // 16 + 1
    nblk = 1 + sum((l + 15) // 16 for l in lens)
    kc = torch.randn(nblk, hkv, 16, hd, generator=g).to(torch.bfloat16).to(dev)
    vc = torch.randn(nblk, hkv, 16, hd, generator=g).to(torch.bfloat16).to(dev)
    bt = torch.zeros(b, max_blocks, dtype=torch.int32)
    perm = (torch.randperm(nblk - 1, generator=g) + 1).tolist()
    p = 0
    for i, l in enumerate(lens):
        n = (l + 15) // 16
        bt[i, :n] = torch.tensor(perm[p:p + n], dtype=torch.int32)
        p += n
    return kc, vc, bt.to(dev)


@pytest.mark.parametrize("hq,hkv,hd", [(64, 4, 128), (8, 1, 128), (4, 2, 64), (40, 2, 128)])
@pytest.mark.parametrize("splits", [1, 5])
def test_flash_decode_paged(dev, hq, hkv, hd, splits):
    torch.manual_seed(10)
    lens = [1, 37, 300, 1024]
    b = len(lens)
    kc, vc, bt = _paged_setup(dev, b, hkv, hd, lens)
    q = torch.randn(b, hq, hd, device=dev).to(torch.bfloat16)
    sl = torch.tensor(lens, dtype=torch.int32, device=dev)
    scale = 1 / math.sqrt(hd)
    for window in (0, 100):
        got = D.flash_decode_paged(q, kc, vc, bt, sl, scale, splits=splits, window=window)
        for i, l in enumerate(lens):
            kk = ref.gather_paged(kc, bt[i].long(), l)
            vv = ref.gather_paged(vc, bt[i].long(), l)
            want = ref.sdpa(q[i:i + 1].float(), kk.float(), vv.float(), scale, l - 1, window)
            _close(got[i:i + 1], want, atol=3e-2)
    # second call with the same scratch object: tickets must have been left at zero
    sc = D.FlashDecodeScratch(b, hq, hkv, hd, max(splits, 2), dev)
    a = D.flash_decode_paged(q, kc, vc, bt, sl, scale, scratch=sc)
    c = D.flash_decode_paged(q, kc, vc, bt, sl, scale, scratch=sc)
    assert torch.equal(a, c)


@pytest.mark.parametrize("hq,hkv,hd", [(64, 4, 128), (8, 1, 128), (4, 2, 64), (40, 2, 128)])
def test_flash_decode_cluster(dev, hq, hkv, hd, q4_path):
    """The cluster kernel (splits merged through distributed shared memory, then per-cluster
    partials merged by the last cluster) against the fp32 oracle, on short and long contexts."""
    if q4_path != "stream":
        pytest.skip("one run is enough: the kernel does not depend on the mat-vec path")
    torch.manual_seed(13)
    scale = 1 / math.sqrt(hd)
    for lens in ([5000], [1, 333], [2048, 17, 700]):
        b = len(lens)
        kc, vc, bt = _paged_setup(dev, b, hkv, hd, lens, seed=3)
        q = torch.randn(b, hq, hd, device=dev).to(torch.bfloat16)
        sl = torch.tensor(lens, dtype=torch.int32, device=dev)
        sc = D.FlashDecodeScratch(b, hq, hkv, hd, 4, dev, max_len=bt.shape[1] * 16)
        if sc.clusters == 0:
            continue
        for window in (0, 100):
            got = D.flash_decode_paged(q, kc, vc, bt, sl, scale, scratch=sc, window=window)
            for i, l in enumerate(lens):
                kk = ref.gather_paged(kc, bt[i].long(), l)
                vv = ref.gather_paged(vc, bt[i].long(), l)
                want = ref.sdpa(q[i:i + 1].float(), kk.float(), vv.float(), scale, l - 1, window)
                _close(got[i:i + 1], want, atol=3e-2)
        # tickets are left at zero: a second call gives the same bits
        a = D.flash_decode_paged(q, kc, vc, bt, sl, scale, scratch=sc)
        c = D.flash_decode_paged(q, kc, vc, bt, sl, scale, scratch=sc)
        assert torch.equal(a, c)


@pytest.mark.parametrize("traditional", [False, True])
def test_rope_kv_write(dev, traditional):
    torch.manual_seed(11)
    hq, hkv, hd, t = 8, 2, 64, 5
    cos, sin = ref.rope_tables(hd, 512, 1e6, device=dev)
    qkv = torch.randn(t, (hq + 2 * hkv) * hd, device=dev).to(torch.bfloat16)
    pos = torch.tensor([0, 17, 31, 32, 200], dtype=torch.int32, device=dev)
    nblk = 40
    kc = torch.zeros(nblk, hkv, 16, hd, dtype=torch.bfloat16, device=dev)
    vc = torch.zeros_like(kc)
    bt = torch.randint(1, nblk, (t, 16), dtype=torch.int32, device=dev)
    qo = torch.empty(t, hq, hd, dtype=torch.bfloat16, device=dev)
    D.rope_kv_write(qkv, qo, kc, vc, bt, pos, cos, sin, hq, hkv, traditional=traditional)
    q = qkv[:, :hq * hd].view(t, hq, hd)
    k = qkv[:, hq * hd:(hq + hkv) * hd].view(t, hkv, hd)
    v = qkv[:, (hq + hkv) * hd:].view(t, hkv, hd)
    _close(qo, ref.apply_rope(q.float(), pos.long(), cos, sin, traditional), atol=1e-2)
    kr = ref.apply_rope(k.float(), pos.long(), cos, sin, traditional)
    for i in range(t):
        p = int(pos[i])
        blk = int(bt[i, p // 16])
        _close(kc[blk, :, p % 16], kr[i], atol=1e-2)
        assert torch.equal(vc[blk, :, p % 16], v[i])
    # stand-alone rope and its inverse
    r = D.rope(q.contiguous(), pos, cos, sin, traditional)
    back = D.rope(r, pos, cos, sin, traditional, inverse=True)
    _close(back, q, atol=2e-2)


@pytest.mark.parametrize("traditional", [False, True])
@pytest.mark.parametrize("hd", [64, 128])
def test_q8_kv_write_and_attention(dev, hd, traditional, q4_path):
    """8-bit cache: the append kernel's codes and (scale, bias) pairs against the host quantiser
    applied to the rotated rows, the page expansion kernel, and attention over the 8-bit pages
    against fp32 attention over the dequantised cache."""
    if q4_path != "stream":
        pytest.skip("one run is enough: the kernels do not depend on the mat-vec path")
    from rmlx_b200.kv.paged import dequantize_kv_rows, quantize_kv_rows
    torch.manual_seed(21)
    hq, hkv, t = 8, 2, 6
    cos, sin = ref.rope_tables(hd, 512, 1e6, device=dev)
    qkv = (torch.randn(t, (hq + 2 * hkv) * hd, device=dev) * 2).to(torch.bfloat16)
    pos = torch.tensor([0, 17, 31, 32, 200, 201], dtype=torch.int32, device=dev)
    nblk = 100
    kq = torch.zeros(nblk, hkv, 16, hd, dtype=torch.uint8, device=dev)
    vq = torch.zeros_like(kq)
    ksb = torch.zeros(nblk, hkv, 16, hd // 64, 2, dtype=torch.bfloat16, device=dev)
    vsb = torch.zeros_like(ksb)
    bt = (torch.randperm(nblk - 1, device=dev)[:t * 16].view(t, 16) + 1).to(torch.int32)   # disjoint pages
    qo = torch.empty(t, hq, hd, dtype=torch.bfloat16, device=dev)
    D.rope_kv_write(qkv, qo, kq, vq, bt, pos, cos, sin, hq, hkv, traditional=traditional, k_sb=ksb, v_sb=vsb)
    q = qkv[:, :hq * hd].view(t, hq, hd)
    k = qkv[:, hq * hd:(hq + hkv) * hd].view(t, hkv, hd)
    v = qkv[:, (hq + hkv) * hd:].view(t, hkv, hd)
    _close(qo, ref.apply_rope(q.float(), pos.long(), cos, sin, traditional), atol=1e-2)
    kr = ref.apply_rope(k.float(), pos.long(), cos, sin, traditional)
    for i in range(t):
        p = int(pos[i])
        blk = int(bt[i, p // 16])
        for want, codes, sb in ((kr[i], kq, ksb), (v[i].float(), vq, vsb)):
            wq, wsb = quantize_kv_rows(want)
            got_sb = sb[blk, :, p % 16]
            # the rotation's fp32 rounding can move a minimum or maximum by an ulp of bf16
            assert (got_sb.float() - wsb.float()).abs().max() <= 2e-2 * wsb.float().abs().max()
            back = dequantize_kv_rows(codes[blk, :, p % 16], got_sb)
            step = got_sb[..., 0].float().repeat_interleave(64, -1).reshape(want.shape)
            assert ((back - want).abs() <= 0.55 * step + 1e-3).all()
            assert (codes[blk, :, p % 16].int() - wq.int()).abs().max() <= 2
    # page expansion
    row = bt[1].contiguous()
    pages = D.kv_dequant_pages(kq, ksb, row, 3)
    want_pages = dequantize_kv_rows(kq[row[:3].long()], ksb[row[:3].long()])
    _close(pages, want_pages, atol=1e-2)

    # attention over 8-bit pages (several lengths, splits, a window)
    lens = [1, 37, 300, 1024]
    b = len(lens)
    kc, vc, bt2 = _paged_setup(dev, b, hkv, hd, lens, seed=5)
    kq2, ksb2 = quantize_kv_rows(kc.float())
    vq2, vsb2 = quantize_kv_rows(vc.float())
    kd, vd = dequantize_kv_rows(kq2, ksb2), dequantize_kv_rows(vq2, vsb2)
    qq = torch.randn(b, hq, hd, device=dev).to(torch.bfloat16)
    sl = torch.tensor(lens, dtype=torch.int32, device=dev)
    scale = 1 / math.sqrt(hd)
    for splits in (1, 4):
        for window in (0, 100):
            got = D.flash_decode_paged(qq, kq2, vq2, bt2, sl, scale, splits=splits, window=window,
                                       k_sb=ksb2, v_sb=vsb2)
            for i, l in enumerate(lens):
                kk = ref.gather_paged(kd, bt2[i].long(), l)
                vv = ref.gather_paged(vd, bt2[i].long(), l)
                want = ref.sdpa(qq[i:i + 1].float(), kk, vv, scale, l - 1, window)
                _close(got[i:i + 1], want, atol=3e-2)


def test_small_kernels(dev):
    torch.manual_seed(12)
    table = torch.randn(1000, 256, device=dev).to(torch.bfloat16)
    ids = torch.tensor([0, 999, 5, 5], dtype=torch.int32, device=dev)
    assert torch.equal(D.embedding(table, ids), table[ids.long()])
    x = torch.randn(7, 512, device=dev).to(torch.bfloat16)
    r = torch.randn(7, 512, device=dev).to(torch.bfloat16)
    w = (1 + 0.1 * torch.randn(512, device=dev)).to(torch.bfloat16)
    _close(D.rms_norm(x, w, 1e-6), ref.rms_norm(x.float(), w.float(), 1e-6))
    s = torch.empty_like(x)
    got = D.rms_norm(x, w, 1e-6, residual=r, sum_out=s)
    hs = (x.float() + r.float()).to(torch.bfloat16)
    assert torch.equal(s, hs)
    _close(got, ref.rms_norm(hs.float(), w.float(), 1e-6))
    logits = torch.randn(3, 151936, device=dev)
    logits[1, 77] = 100.0
    logits[2, 5] = logits[2, 9] = 50.0
    am = D.argmax(logits).cpu().tolist()
    assert am[0] == int(logits[0].argmax()) and am[1] == 77 and am[2] == 5
    gu = torch.randn(9, 2 * 384, device=dev).to(torch.bfloat16)
    _close(D.silu_mul(gu), ref.swiglu(gu.float()))


@pytest.mark.parametrize("quant", [None, "q4", "q8"])
@pytest.mark.parametrize("b,traditional", [(1, False), (3, False), (2, True)])
def test_rms_qkv_rope_matches_unfused(dev, quant, b, traditional, q4_path):
    if quant == "q8" and q4_path != "stream":
        pytest.skip("8-bit weights run on the streaming kernels")
    """The fused projection + RoPE + page append equals the projection kernel followed by the
    rope/append kernel (up to the bf16 rounding of the un-rotated projection that it skips)."""
    torch.manual_seed(5)
    hq, hkv, hd, k = 8, 2, 64, 512
    w = LinearWeight.from_dense(torch.randn((hq + 2 * hkv) * hd, k) * 0.05, quant, device=dev)
    nw = (1 + 0.1 * torch.randn(k, device=dev)).to(torch.bfloat16)
    x = torch.randn(b, k, device=dev).to(torch.bfloat16)
    cos, sin = ref.rope_tables(hd, 128, 1e4, device=dev)
    pos = torch.tensor([5, 37, 70][:b], dtype=torch.int32, device=dev)
    bt = torch.arange(1, 1 + b * 8, dtype=torch.int32, device=dev).view(b, 8)
    kc1 = torch.zeros(1 + b * 8, hkv, 16, hd, device=dev, dtype=torch.bfloat16)
    vc1, kc2, vc2 = torch.zeros_like(kc1), torch.zeros_like(kc1), torch.zeros_like(kc1)
    q1 = torch.zeros(b, hq, hd, device=dev, dtype=torch.bfloat16)
    q2 = torch.zeros_like(q1)
    D.rms_qkv_rope(x, w, nw, 1e-6, q1, kc1, vc1, bt, pos, cos, sin, hq, hkv, traditional=traditional)
    qkv = D.rms_gemv(x, w, nw, 1e-6)
    D.rope_kv_write(qkv, q2, kc2, vc2, bt, pos, cos, sin, hq, hkv, traditional=traditional)
    for got, want in ((q1, q2), (kc1, kc2), (vc1, vc2)):
        assert (got.float() - want.float()).abs().max().item() < 3e-2 * max(1.0, want.float().abs().max().item())
    assert kc1.float().abs().sum() > 0 and vc1.float().abs().sum() > 0


@pytest.mark.parametrize("quant", ["q4", "q8"])
def test_fp16_scales_and_dequant_kernel(dev, quant, q4_path):
    """Scales and biases kept in fp16 (half-precision MLX checkpoints): the streaming mat-vec and the
    dequantisation kernel read them unrounded, so both match the fp32 dequantisation of the triplet."""
    if q4_path != "stream":
        pytest.skip("fp16 scales are read by the streaming kernels")
    torch.manual_seed(21)
    n, k, b = 512, 1024, 2
    w = _w(n, k, quant, dev)
    w16 = LinearWeight(w.kind, w.w, (w.scales.float() * 1.0009765625).to(torch.float16),
                       (w.biases.float() * 1.0009765625).to(torch.float16))
    assert w16.scales_f16
    wd = w16.dequantized()
    x = torch.randn(b, k, device=dev).to(torch.bfloat16)
    _close(D.rms_gemv(x, w16, out_dtype=torch.float32), x.float() @ wd.t(), fro=2e-3)
    dense = w16.dense_bf16()
    assert dense.dtype == torch.bfloat16 and torch.equal(dense.float(), wd.to(torch.bfloat16).float())
    assert torch.equal(w.dense_bf16().float(), w.dequantized().to(torch.bfloat16).float())


@pytest.mark.parametrize("lat,heads", [(128, 20), (512, 128), (512, 16)])
def test_mla_decode_over_paged_latent_cache(dev, lat, heads, q4_path):
    """Latent-attention decode kernel (absorbed queries, paged latent cache, KV splits + merge)
    against fp32 attention over the gathered latents."""
    if q4_path != "stream":
        pytest.skip("one run is enough: the kernel does not depend on the mat-vec path")
    from rmlx_b200.config import MlaConfig
    from rmlx_b200.nn.mla import MlaPagedCache, _mla_decode_kernel
    rope = 64
    cfg = MlaConfig(hidden_size=256, num_heads=heads, head_dim=64, v_head_dim=64, kv_lora_rank=lat,
                    rope_head_dim=rope, q_lora_rank=0, max_seq_len=2048)
    torch.manual_seed(31)
    lens = [1, 37, 700, 1500]
    cache = MlaPagedCache(cfg, 1 + sum((l + 15) // 16 for l in lens) + 4, max_seqs=4, device=dev)
    for s, l in enumerate(lens):
        cache.add_sequence(s)
        cache.append(s, torch.randn(l, lat, device=dev), torch.randn(l, rope, device=dev))
    q = (torch.randn(len(lens), heads, lat + rope, device=dev) * 0.5).to(torch.bfloat16)
    slots = torch.tensor([cache.slot_of(s) for s in range(len(lens))], dtype=torch.int32, device=dev)
    scale = 1.0 / math.sqrt(64 + rope)
    for splits in (1, 5, 0):
        got = _mla_decode_kernel(q, cache, slots, scale, splits)      # bf16 out: the bf16 bounds apply
        for s in range(len(lens)):
            ck, kr = cache.gather(s)
            keys = torch.cat([ck, kr], -1).float()
            sc = (q[s].float() @ keys.t()) * scale
            want = torch.softmax(sc, -1) @ ck.float()
            _close(got[s], want, atol=3e-2)
    from rmlx_b200 import _lib
    torch.cuda.synchronize()
    assert _lib.cuda().rmlx_mla_status() == 0          # no wait for staged pages ran out


def test_awq_and_gptq_dequant_kernels_are_exact(dev, q4_path):
    """AWQ / GPTQ checkpoints expanded on the device equal the torch formulas bit for bit (a small
    integer times an fp16 scale is exact in fp32); act-order group indices included."""
    if q4_path != "stream":
        pytest.skip("one run is enough")
    from rmlx_b200.nn import layers as L
    g = torch.Generator().manual_seed(5)
    in_f, out_f, group = 256, 64, 128
    qw = torch.randint(-2**31, 2**31 - 1, (in_f, out_f // 8), generator=g, dtype=torch.int64).to(torch.int32)
    qz = torch.randint(-2**31, 2**31 - 1, (in_f // group, out_f // 8), generator=g, dtype=torch.int64).to(torch.int32)
    sc = (torch.rand(in_f // group, out_f, generator=g) * 0.02 + 0.001).to(torch.float16)
    want = L.awq_dequantize(qw, qz, sc, group)                       # CPU tensors: the torch formula
    got = L.awq_dequantize(qw.to(dev), qz.to(dev), sc.to(dev), group)
    assert got.is_cuda and got.dtype == torch.float32 and torch.equal(got.cpu(), want)
    qw2 = torch.randint(-2**31, 2**31 - 1, (in_f // 8, out_f), generator=g, dtype=torch.int64).to(torch.int32)
    qz2 = torch.randint(-2**31, 2**31 - 1, (2, out_f // 8), generator=g, dtype=torch.int64).to(torch.int32)
    sc2 = (torch.rand(2, out_f, generator=g) * 0.02 + 0.001).to(torch.float16)
    for g_idx in (None, torch.randint(0, 2, (in_f,), generator=g)):
        want = L.gptq_dequantize(qw2, qz2, sc2, g_idx)
        got = L.gptq_dequantize(qw2.to(dev), qz2.to(dev), sc2.to(dev), None if g_idx is None else g_idx.to(dev))
        assert got.is_cuda and torch.equal(got.cpu(), want)
