#!/usr/bin/env python
"""Prefill GEMM sweep: M in {32..8192} x (N, K) in {(4096,4096), (12288,4096), (4096,12288)}, bf16,
this package's tcgen05 kernel against torch.matmul (cuBLAS) on the same inputs.

Timing: CUDA events around a captured graph of ``iters`` launches that rotate over enough
independent weight (and activation) copies that the working set of one rotation exceeds the 126 MB
L2, after warm-up. Reports TFLOP/s and the fraction of the measured cuBLAS bf16 peak from
``MEASURED_PEAKS.json`` ("of measured"; 1590 TFLOP/s "of fallback" when the file is absent).
The counterpart of the reference's gemm benches (crates/rmlx-core/benches/gemm_bench.rs,
gemm_sweep.rs; published 24.05 TFLOPS at M=2048, K=4096, N=14336 on M3 Ultra).

    python benchmarks/bench_gemm.py [--m 512,2048] [--iters 20] [--check] [--weights q4]

``--weights q4``: the same sweep with MLX-affine Q4 weights (group 64) dequantised inside the tcgen05
main loop, against "expand to bf16 once, then cuBLAS" on the same weights (the expansion is not
timed: the baseline is charged only its GEMM); the reference's affine_qmm published 17.43 TFLOPS at
M=512 (crates/rmlx-core/benches/qmm_sweep.rs).
"""
from __future__ import annotations

import argparse
import json
import math
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from rmlx_b200.ops.gemm import GemmStatus, gemm_bf16  # noqa: E402
from rmlx_b200.ops.quantized import xgemm  # noqa: E402
from rmlx_b200.ops.weights import LinearWeight  # noqa: E402


def peak():
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    if os.path.exists(p):
        return json.load(open(p))["bf16_tflops"], "measured"
    return 1590.0, "fallback"


def graph_time(fns, iters):
    for f in fns[:3]:
        f()
    torch.cuda.synchronize()
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
    ap.add_argument("--m", default="32,64,128,256,512,2048,8192")
    ap.add_argument("--nk", default="4096x4096,12288x4096,4096x12288")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--bn", type=int, default=0)
    ap.add_argument("--check", action="store_true")
    ap.add_argument("--ours-only", action="store_true")
    ap.add_argument("--weights", default="bf16", choices=["bf16", "q4"])
    a = ap.parse_args()
    pk, how = peak()
    dev = torch.device("cuda:0")
    print(f"# {a.weights} GEMM y = x W^T, peak {pk:.0f} TFLOP/s ({how})")
    print(f"{'M':>6} {'N':>6} {'K':>6} {'ours us':>9} {'TFLOPs':>8} {'of ' + how:>12} {'cuBLAS us':>10} {'TFLOPs':>8} {'ours/cuBLAS':>12}")
    for nk in a.nk.split(","):
        n, k = (int(v) for v in nk.split("x"))
        for m in (int(v) for v in a.m.split(",")):
            bytes_one = (m * k + n * k + m * n) * 2
            copies = max(2, min(8, int(math.ceil(160e6 / bytes_one))))
            xs = [torch.randn(m, k, device=dev).to(torch.bfloat16) for _ in range(copies)]
            ws = [(torch.randn(n, k, device=dev) * 0.05).to(torch.bfloat16) for _ in range(copies)]
            out = torch.empty(m, n, device=dev, dtype=torch.bfloat16)
            if a.weights == "q4":
                qs = [LinearWeight.from_dense(w.float(), "q4", device=dev) for w in ws]
                ws = [q.dequantized().to(torch.bfloat16) for q in qs]      # what cuBLAS multiplies
                if a.check:
                    got = xgemm(xs[0], qs[0], bn=a.bn).float()
                    want = xs[0].float() @ ws[0].float().t()
                    err = (got - want).abs().max().item() / want.abs().max().item()
                    assert err < 1.5e-2, (m, n, k, err)
                ours = graph_time([(lambda x=x, q=q: xgemm(x, q, out=out, bn=a.bn)) for x, q in zip(xs, qs)], a.iters)
                GemmStatus.check(dev)
                fl = 2.0 * m * n * k
                cub = graph_time([(lambda x=x, w=w: torch.matmul(x, w.t(), out=out)) for x, w in zip(xs, ws)], a.iters)
                print(f"{m:6d} {n:6d} {k:6d} {ours:9.1f} {fl / ours / 1e6:8.1f} {fl / ours / 1e6 / pk:12.2f} "
                      f"{cub:10.1f} {fl / cub / 1e6:8.1f} {cub / ours:12.2f}")
                continue
            if a.check:
                got = gemm_bf16(xs[0], ws[0], bn=a.bn).float()
                want = xs[0].float() @ ws[0].float().t()
                err = (got - want).abs().max().item() / want.abs().max().item()
                assert err < 1.5e-2, (m, n, k, err)
            ours = graph_time([(lambda x=x, w=w: gemm_bf16(x, w, out=out, bn=a.bn)) for x, w in zip(xs, ws)], a.iters)
            GemmStatus.check(dev)
            fl = 2.0 * m * n * k
            if a.ours_only:
                print(f"{m:6d} {n:6d} {k:6d} {ours:9.1f} {fl / ours / 1e6:8.1f} {fl / ours / 1e6 / pk:12.2f}")
                continue
            cub = graph_time([(lambda x=x, w=w: torch.matmul(x, w.t(), out=out)) for x, w in zip(xs, ws)], a.iters)
            print(f"{m:6d} {n:6d} {k:6d} {ours:9.1f} {fl / ours / 1e6:8.1f} {fl / ours / 1e6 / pk:12.2f} "
                  f"{cub:10.1f} {fl / cub / 1e6:8.1f} {cub / ours:12.2f}")


if __name__ == "__main__":
    main()
