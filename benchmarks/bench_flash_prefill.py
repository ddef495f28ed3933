#!/usr/bin/env python
"""Paged causal flash attention for prompt processing: the tcgen05 kernel (one or two query tiles
per CTA) against the mma.sync kernel on the same paged cache, head_dim 128, 32 query / 8 KV heads
by default (``--heads 64 --kv-heads 4`` is the attention of the MoE-A22B-shaped model).

Timing: CUDA events around ``iters`` launches after warm-up; the K/V working set of these shapes
(a few MB to tens of MB) is L2-resident by the nature of attention, the queries and outputs stream.
Reports microseconds and TFLOP/s counting 4 * head_dim * Hq * T(T+1)/2 FLOPs (the causal half), and
the fraction of the measured cuBLAS bf16 peak from ``MEASURED_PEAKS.json`` ("of measured"; 1590
TFLOP/s "of fallback" when the file is absent). ``--check`` compares with fp32 softmax(QK^T)V.
The counterpart of the reference's sdpa prefill measurements inside its prefill benches
(crates/rmlx-nn/benches/prefill_bench.rs).

    python benchmarks/bench_flash_prefill.py [--tokens 2048,8192] [--kernels mma,tc] [--lanes 0]
"""
from __future__ import annotations

import argparse
import json
import math
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from rmlx_b200.ops.attention import flash_prefill_paged  # noqa: E402
from rmlx_b200.ops.gemm import GemmStatus  # noqa: E402
from rmlx_b200.reference import ops as ref  # noqa: E402


def peak():
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    if os.path.exists(p):
        return json.load(open(p))["bf16_tflops"], "measured"
    return 1590.0, "fallback"


def build(t, hq, hkv, hd, dev):
    torch.manual_seed(0)
    nblk = (t + 15) // 16
    kc = torch.zeros(nblk + 1, hkv, 16, hd, device=dev, dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    perm = (torch.randperm(nblk) + 1).to(torch.int32).to(dev)     # pages out of order
    k = torch.randn(t, hkv, hd, device=dev).to(torch.bfloat16)
    v = torch.randn(t, hkv, hd, device=dev).to(torch.bfloat16)
    tok = torch.arange(t, device=dev)
    kc[perm[tok // 16].long(), :, tok % 16] = k
    vc[perm[tok // 16].long(), :, tok % 16] = v
    q = torch.randn(t, hq, hd, device=dev).to(torch.bfloat16)
    return q, k, v, kc, vc, perm


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", default="512,1024,2048,4096,8192")
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--kernels", default="mma,tc")
    ap.add_argument("--lanes", default="0", help="query tiles per CTA of the tcgen05 kernel: 1, 2, 0 = its own choice")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--check", action="store_true")
    a = ap.parse_args()
    dev = torch.device("cuda:0")
    hd = 128
    pk, what = peak()
    print(f"# flash prefill, head_dim {hd}, {a.heads} query / {a.kv_heads} kv heads, peak {pk:.0f} TFLOP/s ({what})")
    for t in [int(x) for x in a.tokens.split(",")]:
        q, k, v, kc, vc, perm = build(t, a.heads, a.kv_heads, hd, dev)
        flops = 4 * hd * a.heads * (t * (t + 1) / 2)
        out = torch.empty_like(q)
        want = ref.sdpa(q.float(), k.float(), v.float(), 1.0 / math.sqrt(hd), 0, 0) if a.check else None
        for kern in a.kernels.split(","):
            for lanes in (a.lanes.split(",") if kern == "tc" else ["0"]):
                os.environ["RMLX_FLASH_PREFILL"] = kern
                os.environ["RMLX_FLASH_PREFILL_LANES"] = lanes
                for _ in range(a.warmup):
                    flash_prefill_paged(q, kc, vc, perm, 0, out=out)
                torch.cuda.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for _ in range(a.iters):
                    flash_prefill_paged(q, kc, vc, perm, 0, out=out)
                e1.record()
                torch.cuda.synchronize()
                GemmStatus.check(dev)
                us = e0.elapsed_time(e1) * 1e3 / a.iters
                tf = flops / us / 1e6
                err = f"  max_err {(out.float() - want).abs().max().item():.2e}" if a.check else ""
                name = kern if kern != "tc" else f"tc(lanes={lanes})"
                print(f"T={t:6d} {name:14s} {us:9.1f} us {tf:8.1f} TFLOP/s  {tf / pk:.2f} of {what}{err}", flush=True)


if __name__ == "__main__":
    main()
