#!/usr/bin/env python
"""Decode-sized tensor-parallel kernels in isolation: projection + all-reduce fused in one kernel
(peer stores) against the same local mat-vec alone, the stand-alone one-shot all-reduce, and NCCL's
all-reduce of the same [1, 4096] vector. Graph-captured loops (an even number of collectives per
graph), CUDA-event timed, max over ranks.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port 29514 benchmarks/bench_tp_decode_kernels.py [--weights q4|bf16]
"""
from __future__ import annotations

import argparse
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from rmlx_b200.ops import decode as D  # noqa: E402
from rmlx_b200.ops.weights import LinearWeight  # noqa: E402
from rmlx_b200.parallel.comm import PeerComm  # noqa: E402


def graph_time(fn, iters=20):
    for _ in range(4):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=s):
        for _ in range(iters):
            fn()
    g.replay()
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    g.replay()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) * 1e3 / iters], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.item()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--weights", default="q4", choices=["q4", "bf16"])
    a = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dev = torch.device("cuda", torch.cuda.current_device())
    dist.init_process_group("nccl", device_id=dev)
    quant = None if a.weights == "bf16" else "q4"
    hidden, attn, inter, E, k = 4096, 8192 // world, 1536 // world, 128, 8
    comm = PeerComm(hidden, 1, device=dev)
    x = torch.randn(1, attn, device=dev).to(torch.bfloat16)
    wo = [LinearWeight.random(hidden, attn, quant, dev) for _ in range(8)]
    res = torch.randn(1, hidden, device=dev).to(torch.bfloat16)
    out = torch.empty(1, hidden, device=dev, dtype=torch.bfloat16)
    i = [0]

    def fused_o():
        i[0] += 1
        comm.gemv_allreduce(x, wo[i[0] % 8], res, out)

    def local_o():
        i[0] += 1
        D.rms_gemv(x, wo[i[0] % 8], None, 1e-6, residual=res, out=out)

    wd = [LinearWeight.random(hidden, inter, quant, dev, experts=E) for _ in range(2)]
    act = torch.randn(k, inter, device=dev).to(torch.bfloat16)
    idxs = [torch.randperm(E)[:k].view(1, k).to(torch.int32).to(dev) for _ in range(8)]
    wts = torch.softmax(torch.randn(1, k, device=dev), -1)

    def fused_d():
        i[0] += 1
        comm.moe_down_allreduce(act, wd[i[0] % 2], idxs[i[0] % 8], wts, res, out)

    def local_d():
        i[0] += 1
        D.moe_down(act, wd[i[0] % 2], idxs[i[0] % 8], wts, residual=res, out=out)

    v = torch.randn(1, hidden, device=dev)
    vo = torch.empty(1, hidden, device=dev)

    def oneshot():
        comm.allreduce(v, out=vo)

    vb = torch.randn(1, hidden, device=dev).to(torch.bfloat16)

    def nccl():
        dist.all_reduce(vb)

    rows = [("o_proj local mat-vec only", graph_time(local_o)),
            ("o_proj + all-reduce (fused)", graph_time(fused_o)),
            ("moe down local only", graph_time(local_d)),
            ("moe down + all-reduce (fused)", graph_time(fused_d)),
            ("one-shot all-reduce [1,4096] fp32", graph_time(oneshot)),
            ("NCCL all-reduce [1,4096] bf16", graph_time(nccl))]
    if rank == 0:
        print(f"# world={world} weights={a.weights}; status={comm.status()}")
        for n, t in rows:
            print(f"{n:40s} {t:8.2f} us")
    dist.barrier()
    comm.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
