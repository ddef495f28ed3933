#!/usr/bin/env python
"""Tensor-parallel prefill GEMMs: collective fused into the tensor-core kernel (peer stores over
NVLink) against the same GEMM followed by the NCCL collective. Launch with one process per GPU:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port 29511 benchmarks/bench_tp_gemm.py [--tokens 2048,8192] [--iters 20]

Shapes are the row-parallel layers of the MoE-A22B-shaped model (hidden 4096; attention output
K = 8192/N per rank) and a column-parallel QKV projection fed by row-sharded activations. Times are
CUDA-event times per call, max over ranks, after warm-up; every call's operands exceed L2 in
aggregate over the rotation. The roofline column is the slower of FLOPs / measured GEMM peak and
NVLink bytes / 770 GB/s per direction.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from rmlx_b200.ops.weights import LinearWeight  # noqa: E402
from rmlx_b200.parallel.tp_gemm import make_gemm_comm  # noqa: E402


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
    ap.add_argument("--tokens", default="2048,8192")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--weights", default="bf16", choices=["bf16", "q4"])
    ap.add_argument("--trace", action="store_true", help="print per-phase device timestamps of one call")
    a = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dev = torch.device("cuda", torch.cuda.current_device())
    dist.init_process_group("nccl", device_id=dev)
    quant = None if a.weights == "bf16" else "q4"
    pk_path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    peak = json.load(open(pk_path))["bf16_tflops"] if os.path.exists(pk_path) else 1590.0
    ms = [int(v) for v in a.tokens.split(",")]
    hidden, attn = 4096, 8192
    fused = make_gemm_comm("fused", max(ms), hidden, max(hidden, attn), device=dev)
    nccl = make_gemm_comm("nccl", max(ms), hidden, max(hidden, attn), device=dev)
    rows = []
    for m in ms:
        # row-parallel: [m, attn/world] x [hidden, attn/world]^T, summed over ranks, + residual
        kl = attn // world
        x = torch.randn(m, kl, device=dev).to(torch.bfloat16)
        w = LinearWeight.random(hidden, kl, quant, dev)
        res = torch.randn(m, hidden, device=dev).to(torch.bfloat16)
        flops = 2.0 * m * hidden * kl
        link = 2.0 * m * hidden * 2 * (world - 1) / world       # out + back, per direction per GPU
        floor = max(flops / (peak * 1e6), link / 770e3)
        tf = timed(lambda: fused.gemm_allreduce(x, w, residual=res), a.iters)
        tn = timed(lambda: nccl.gemm_allreduce(x, w, residual=res), a.iters)
        rows.append((f"gemm+allreduce m={m} k/rank={kl}", tf, tn, floor))
        if m % (128 * world) == 0:
            # reduce-scatter: the partial tiles cross NVLink once, nothing comes back
            link_rs = m * hidden * 2 * (world - 1) / world
            floor_rs = max(flops / (peak * 1e6), link_rs / 770e3)

            def nccl_rs():
                y = nccl._mm(x, w)
                o = torch.empty(m // world, hidden, dtype=y.dtype, device=dev)
                dist.reduce_scatter_tensor(o, y)
                return o
            tf = timed(lambda: fused.gemm_reduce_scatter(x, w, residual=res), a.iters)
            tn = timed(nccl_rs, a.iters)
            rows.append((f"gemm+reduce_scatter m={m} k/rank={kl}", tf, tn, floor_rs))
        if a.trace:
            fused.enable_trace()
            fused.gemm_allreduce(x, w, residual=res)
            torch.cuda.synchronize()
            if rank == 0:
                print("trace gemm+allreduce", m, fused.trace_summary())
            fused.enable_trace(False)
        # column-parallel from row shards: [m/world, hidden] gathered, x [(9216/world), hidden]^T
        if (m // world) % 128 == 0:
            nl = 9216 // world // 128 * 128
            xs = torch.randn(m // world, hidden, device=dev).to(torch.bfloat16)
            w2 = LinearWeight.random(nl, hidden, quant, dev)
            flops = 2.0 * m * nl * hidden
            link = (m // world) * hidden * 2 * (world - 1)
            floor = max(flops / (peak * 1e6), link / 770e3)
            tf = timed(lambda: fused.allgather_gemm(xs, w2), a.iters)
            tn = timed(lambda: nccl.allgather_gemm(xs, w2), a.iters)
            rows.append((f"allgather+gemm m={m} n/rank={nl}", tf, tn, floor))
            if a.trace:
                fused.enable_trace()
                fused.allgather_gemm(xs, w2)
                torch.cuda.synchronize()
                if rank == 0:
                    print("trace allgather+gemm", m, fused.trace_summary())
                fused.enable_trace(False)
    st = fused.status()
    if rank == 0:
        print(f"# world={world} weights={a.weights} GEMM peak {peak:.0f} TFLOP/s; NVLink 770 GB/s/dir; status={st}")
        print(f"{'case':44s} {'fused us':>9s} {'gemm+nccl us':>13s} {'speedup':>8s} {'floor us':>9s} {'fused/floor':>11s}")
        for name, tf, tn, fl in rows:
            print(f"{name:44s} {tf:9.1f} {tn:13.1f} {tn / tf:8.2f} {fl:9.1f} {tf / fl:11.2f}")
    dist.barrier()
    fused.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
