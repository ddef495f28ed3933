#!/usr/bin/env python
"""Per-kernel timing of the decode path at the MoE-A22B layer shapes (hidden 4096, 64 q / 4 kv heads,
head_dim 128, 128 experts top-8 x 1536, vocab 151936), batch 1 unless ``--batch`` says otherwise.

Each kernel is timed with CUDA events after warm-up, rotating over enough independent weight copies
that every launch reads from HBM, not L2 (the working set of one rotation is > 126 MB). Reports
microseconds, algorithmic bytes, achieved GB/s and the fraction of the measured copy bandwidth in
``MEASURED_PEAKS.json`` (or of the 6650 GB/s fallback when that file is absent).

The analogue of the reference's fused-kernel micro benchmarks
(docs/reports/phase-f-i-benchmark-2026-03-08.md:213-218: swiglu+down, rms_norm+QKV, rms_norm+gate_up).

    python benchmarks/bench_decode_kernels.py [--weights q4|bf16] [--only NAME] [--iters 50]
"""
from __future__ import annotations

import argparse
import json
import math
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from rmlx_b200.ops import decode as D  # noqa: E402
from rmlx_b200.ops.weights import LinearWeight  # noqa: E402
from rmlx_b200.reference import ops as ref  # noqa: E402


def peak_gbs() -> tuple:
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    if os.path.exists(p):
        return json.load(open(p))["hbm_gbs"], "measured"
    return 6650.0, "fallback"


def timeit(fns, iters: int, warmup: int = 5) -> float:
    """fns: list of closures rotated so consecutive launches touch different weights."""
    for i in range(warmup):
        fns[i % len(fns)]()
    torch.cuda.synchronize()
    # The launches are captured in a CUDA graph so that the host's launch cost (tens of
    # microseconds from Python) does not hide kernels that run for a few microseconds.
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=s):
        for i in range(iters):
            fns[i % len(fns)]()
    g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    g.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / iters


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--weights", default="q4", choices=["q4", "bf16"])
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--iters", type=int, default=50)
    ap.add_argument("--only", default="")
    ap.add_argument("--ctx", type=int, default=4096)
    ap.add_argument("--splits", type=int, default=0, help="KV splits for flash decode (0 = default heuristic)")
    args = ap.parse_args()
    dev = torch.device("cuda:0")
    quant = None if args.weights == "bf16" else "q4"
    B, D_, HQ, HKV, HD, E, TOPK, I, V = args.batch, 4096, 64, 4, 128, 128, 8, 1536, 151936
    peak, how = peak_gbs()
    rows = []

    def copies_for(nbytes):
        return max(2, int(math.ceil(200e6 / max(nbytes, 1))))

    def add(name, fns, nbytes):
        if args.only and args.only not in name:
            return
        us = timeit(fns, args.iters)
        gbs = nbytes / us / 1e3
        rows.append((name, us, nbytes, gbs, gbs / peak))

    x = torch.randn(B, D_, device=dev).to(torch.bfloat16)
    nw = torch.ones(D_, device=dev, dtype=torch.bfloat16)

    def dense(name, n, k, norm, residual, out_f32=False):
        w0 = LinearWeight.random(n, k, quant, dev)
        nc = copies_for(w0.nbytes())
        ws = [w0] + [LinearWeight.random(n, k, quant, dev) for _ in range(min(nc, 16) - 1)]
        xin = torch.randn(B, k, device=dev).to(torch.bfloat16)
        res = torch.randn(B, n, device=dev).to(torch.bfloat16) if residual else None
        out = torch.empty(B, n, device=dev, dtype=torch.float32 if out_f32 else torch.bfloat16)
        nwk = torch.ones(k, device=dev, dtype=torch.bfloat16) if norm else None
        fns = [(lambda w=w: D.rms_gemv(xin, w, nwk, 1e-6, residual=res, out=out)) for w in ws]
        add(name, fns, w0.nbytes() + B * (k + n) * 2)

    dense("rms+qkv   [9216x4096]", (HQ + 2 * HKV) * HD, D_, True, False)
    dense("o_proj+res [4096x8192]", D_, HQ * HD, False, True)
    if not args.only or "lm_head" in args.only:
        dense("rms+lm_head [151936x4096]", V, D_, True, False, out_f32=True)

    # router
    gates = [(torch.randn(E, D_, device=dev) * 0.05).to(torch.bfloat16) for _ in range(8)]
    sc = D.RouterScratch(B, E, dev)
    idx = torch.zeros(B, TOPK, dtype=torch.int32, device=dev)
    wts = torch.zeros(B, TOPK, dtype=torch.float32, device=dev)
    add("router (rms+gate+topk)", [(lambda g=g: D.moe_router(x, g, nw, 1e-6, TOPK, None, sc, idx, wts))
                                   for g in gates], E * D_ * 2)

    # experts: routing spreads over all 128 experts of each copy so nothing is reused from L2
    wgu = [LinearWeight.random(2 * I, D_, quant, dev, experts=E) for _ in range(2)]
    wdn = [LinearWeight.random(D_, I, quant, dev, experts=E) for _ in range(2)]
    idxs = [torch.stack([torch.randperm(E)[:TOPK] for _ in range(B)]).to(torch.int32).to(dev)
            for _ in range(16)]
    wt = torch.softmax(torch.randn(B, TOPK, device=dev), -1)
    act = torch.zeros(B * TOPK, I, dtype=torch.bfloat16, device=dev)
    out = torch.empty(B, D_, dtype=torch.bfloat16, device=dev)
    per_e_gu = wgu[0].nbytes() // E
    per_e_dn = wdn[0].nbytes() // E
    add("moe gate_up+swiglu (8 experts)",
        [(lambda i=i: D.moe_gate_up(x, wgu[i % 2], nw, 1e-6, idxs[i], out=act)) for i in range(16)],
        B * TOPK * per_e_gu)
    add("moe down+combine+res (8 experts)",
        [(lambda i=i: D.moe_down(act, wdn[i % 2], idxs[i], wt, residual=x, out=out)) for i in range(16)],
        B * TOPK * per_e_dn)

    # attention
    ctx = args.ctx
    nblk = B * ((ctx + 15) // 16) + 1
    ncp = 12
    kcs = [torch.randn(nblk, HKV, 16, HD, device=dev).to(torch.bfloat16) for _ in range(ncp)]
    vcs = [torch.randn(nblk, HKV, 16, HD, device=dev).to(torch.bfloat16) for _ in range(ncp)]
    bt = (torch.arange(B * ((ctx + 15) // 16), dtype=torch.int32, device=dev) + 1).view(B, -1).contiguous()
    sl = torch.full((B,), ctx, dtype=torch.int32, device=dev)
    q = torch.randn(B, HQ, HD, device=dev).to(torch.bfloat16)
    ao = torch.empty_like(q)
    splits = args.splits or D.default_splits(B, HKV, 1, ctx)
    fsc = D.FlashDecodeScratch(B, HQ, HKV, HD, splits, dev)
    fcl = D.FlashDecodeScratch(B, HQ, HKV, HD, splits, dev, max_len=ctx)
    if fcl.clusters > 0:
        add(f"flash_decode ctx{ctx} clusters {fcl.clusters & 0xff}x{fcl.clusters >> 8}",
            [(lambda i=i: D.flash_decode_paged(q, kcs[i], vcs[i], bt, sl, None, None, fcl, out=ao))
             for i in range(ncp)], B * ctx * HKV * HD * 2 * 2)
    add(f"flash_decode ctx{ctx} splits{splits}",
        [(lambda i=i: D.flash_decode_paged(q, kcs[i], vcs[i], bt, sl, None, splits, fsc, out=ao))
         for i in range(ncp)], B * ctx * HKV * HD * 2 * 2)
    # the same attention over an 8-bit cache (codes + (scale, bias) per token and group of 64)
    if not args.only or "q8kv" in args.only or "flash_decode" in args.only:
        from rmlx_b200.kv.paged import quantize_kv_rows
        kq, vq = [], []
        for i in range(ncp):
            kq.append(quantize_kv_rows(kcs[i].float()))
            vq.append(quantize_kv_rows(vcs[i].float()))
        add(f"flash_decode ctx{ctx} splits{splits}, 8-bit KV (q8kv)",
            [(lambda i=i: D.flash_decode_paged(q, kq[i][0], vq[i][0], bt, sl, None, splits, fsc, out=ao,
                                               k_sb=kq[i][1], v_sb=vq[i][1])) for i in range(ncp)],
            B * ctx * HKV * (HD + 4 * HD // 64) * 2)
    # latent attention (DeepSeek-V3 widths: 128 heads, latent 512 + rope 64) over a paged latent cache
    if not args.only or "mla" in args.only:
        from rmlx_b200.config import MlaConfig
        from rmlx_b200.nn.mla import MlaPagedCache, _mla_decode_kernel
        mcfg = MlaConfig(num_heads=128, head_dim=128, v_head_dim=128, hidden_size=7168, kv_lora_rank=512,
                         q_lora_rank=0, rope_head_dim=64, max_seq_len=ctx + 16)
        caches = []
        for i in range(30):                      # 30 x 4.7 MB of latents: more than the L2
            c = MlaPagedCache(mcfg, B * ((ctx + 15) // 16) + 1, max_seqs=B, device=dev)
            for s_ in range(B):
                c.add_sequence(s_)
                c.append(s_, torch.randn(ctx, 512, device=dev), torch.randn(ctx, 64, device=dev))
            caches.append(c)
        qa = (torch.randn(B, 128, 576, device=dev) * 0.3).to(torch.bfloat16)
        slots = torch.arange(B, dtype=torch.int32, device=dev)
        add(f"mla decode ctx{ctx} 128 heads, latent 512+64" + (f", splits{args.splits}" if args.splits else ""),
            [(lambda c=c: _mla_decode_kernel(qa, c, slots, 1.0 / math.sqrt(192.0), args.splits)) for c in caches],
            B * ctx * 576 * 2)
    cos, sin = ref.rope_tables(HD, ctx + 8, 1e6, device=dev)
    qkv = torch.randn(B, (HQ + 2 * HKV) * HD, device=dev).to(torch.bfloat16)
    pos = torch.full((B,), ctx - 1, dtype=torch.int32, device=dev)
    add("rope + kv write", [lambda: D.rope_kv_write(qkv, q, kcs[0], vcs[0], bt, pos, cos, sin, HQ, HKV)],
        B * (HQ + 2 * HKV) * HD * 4)
    logits = torch.randn(B, V, device=dev)
    asc = D.ArgmaxScratch(B, dev)
    nt = torch.zeros(B, dtype=torch.int32, device=dev)
    add("argmax", [lambda: D.argmax(logits, nt, asc)], B * V * 4)

    print(f"# decode kernels, weights={args.weights}, batch={B}, q4_path={D.q4_path()}, "
          f"HBM peak {peak:.0f} GB/s ({how})")
    print(f"{'kernel':40s} {'us':>9s} {'MB':>9s} {'GB/s':>9s} {'of ' + how:>12s}")
    for name, us, nb, gbs, frac in rows:
        print(f"{name:40s} {us:9.2f} {nb / 1e6:9.2f} {gbs:9.0f} {frac:12.2f}")


if __name__ == "__main__":
    main()
