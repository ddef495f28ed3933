#!/usr/bin/env python
"""Expert-parallel dispatch + combine: this package's peer-memory kernels against the same exchange
on NCCL all-to-alls (``parallel.ep.EpExchange``), at the MoE-A22B shapes (hidden 4096, 128 experts,
top-8), tokens per rank in {4, 32, 128, 4096}. One process per GPU:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port 29512 benchmarks/bench_ep.py [--tokens 4,32,128,4096] [--iters 20]

Times are CUDA-event times of dispatch + combine (expert compute excluded: the expert outputs are the
dispatched rows themselves), max over ranks, after warm-up. Roofline: bytes that must cross NVLink per
rank and direction (pairs to other ranks x 8 KB, both ways) over 770 GB/s. The counterpart of the
reference's ep_bench / rdma_ep_latency (crates/rmlx-nn/benches/ep_bench.rs).
"""
from __future__ import annotations

import argparse
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from rmlx_b200.ops import decode as D  # noqa: E402
from rmlx_b200.parallel.ep import EpExchange  # noqa: E402
from rmlx_b200.parallel.ep_fused import FusedEpExchange  # noqa: E402
from rmlx_b200.parallel.group import Group  # noqa: E402


def timed(fn, iters, warmup=3):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) * 1e3 / iters], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.item()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", default="4,32,128,4096")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--layer", action="store_true", help="also time the whole expert-parallel MoE layer")
    ap.add_argument("--weights", default="bf16", choices=["bf16", "q4"])
    a = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dev = torch.device("cuda", torch.cuda.current_device())
    dist.init_process_group("nccl", device_id=dev)
    hidden, E, k = 4096, 128, 8
    toks = [int(v) for v in a.tokens.split(",")]
    fused = FusedEpExchange(max(toks), hidden, k, E, device=dev, blocks=64)
    lib = EpExchange(Group(), E)
    rows = []
    for t in toks:
        torch.manual_seed(rank)
        x = torch.randn(t, hidden, device=dev).to(torch.bfloat16)
        logits = torch.randn(t, E, device=dev)
        idx, wts, counts, _ = D.topk_route(logits, k)

        def run_fused():
            slab, _ = fused.dispatch(x, idx, counts)
            return fused.combine(slab, wts, t)

        def run_lib():
            got, layout = lib.dispatch(x, idx.long())
            return lib.combine(got, wts, layout)

        a_out = run_fused().float()
        b_out = run_lib()
        err = (a_out - b_out).abs().max().item() / max(b_out.abs().max().item(), 1e-6)
        tf = timed(run_fused, a.iters)
        tn = timed(run_lib, a.iters)
        remote = t * k * (world - 1) / world
        floor = 2 * remote * hidden * 2 / 770e3
        rows.append((t, tf, tn, floor, err))
    # ---- the whole expert-parallel MoE layer: router -> dispatch -> grouped expert FFN -> combine
    layer_rows = []
    if a.layer:
        from rmlx_b200.ops.grouped import grouped_expert_ffn
        from rmlx_b200.ops.weights import LinearWeight
        from rmlx_b200.parallel.ep_fused import FusedEpMoe
        inter, el = 1536, E // world
        quant = None if a.weights == "bf16" else "q4"
        gu = LinearWeight.random(2 * inter, hidden, quant, dev, experts=el)
        dn = LinearWeight.random(hidden, inter, quant, dev, experts=el)
        router = (torch.randn(E, hidden, device=dev) * 0.05).to(torch.bfloat16)
        moe = FusedEpMoe(fused, gu, dn)
        for t in toks:
            torch.manual_seed(1000 + rank)
            x = torch.randn(t, hidden, device=dev).to(torch.bfloat16)

            def layer_fused():
                return moe.forward(x, router, k)

            def layer_lib():
                logits = torch.mm(x, router.t(), out_dtype=torch.float32)
                idx, wts, _, _ = D.topk_route(logits, k)
                got, layout = lib.dispatch(x, idx.long())
                y = grouped_expert_ffn(got, layout.offsets, gu, dn)
                return lib.combine(y, wts, layout)

            def layer_captured():
                return moe.forward_captured(x, router, k)

            fa, fb = layer_fused().float(), layer_lib()
            err = (fa - fb).abs().max().item() / max(fb.abs().max().item(), 1e-6)
            layer_rows.append((t, timed(layer_fused, a.iters), timed(layer_lib, a.iters), err,
                               timed(layer_captured, a.iters)))
    st = fused.status()
    if rank == 0 and layer_rows:
        print(f"# expert-parallel MoE layer end to end (router + exchange + grouped FFN + combine), weights={a.weights}")
        print(f"{'tokens/rank':>11s} {'fused us':>9s} {'captured us':>11s} {'nccl us':>9s} {'nccl/captured':>13s} {'max rel diff':>12s}")
        for t, tf, tn, err, tc in layer_rows:
            print(f"{t:11d} {tf:9.1f} {tc:11.1f} {tn:9.1f} {tn / tc:13.2f} {err:12.1e}")
    if rank == 0:
        print(f"# world={world} hidden={hidden} experts={E} top_k={k}; NVLink 770 GB/s/dir; status={st}")
        print(f"{'tokens/rank':>11s} {'fused us':>9s} {'nccl us':>9s} {'speedup':>8s} {'floor us':>9s} {'floor/fused':>11s} {'max rel diff':>12s}")
        for t, tf, tn, fl, err in rows:
            print(f"{t:11d} {tf:9.1f} {tn:9.1f} {tn / tf:8.2f} {fl:9.1f} {fl / tf:11.2f} {err:12.1e}")
    dist.barrier()
    fused.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
