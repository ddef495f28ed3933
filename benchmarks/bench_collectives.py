#!/usr/bin/env python
"""Collectives over peer memory against NCCL: all-reduce (two-shot kernel; the one-shot decode-sized
form is in bench.py's fused path), all-gather, reduce-scatter and all-to-all, 8 KB ... 64 MB (bf16).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port 29513 benchmarks/bench_collectives.py [--sizes 8192,...] [--iters 20]

With RMLX_SYMM_MULTICAST=1 (symmetric heap bound to NVLink multicast objects) two more rows per
size time the in-switch all-reduce (multimem.ld_reduce + multimem.st): staged from an ordinary
tensor, and in place on the heap buffer.

CUDA-event time per call, max over ranks, after warm-up. Bus bandwidth uses the usual factors
(all-reduce 2(N-1)/N, the others (N-1)/N of the full buffer). The counterpart of the reference's
rdma_allreduce_bench / distributed_bench (crates/rmlx-distributed/benches).
"""
from __future__ import annotations

import argparse
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from rmlx_b200.parallel.collectives import PeerCollectives  # noqa: E402


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
    ap.add_argument("--sizes", default="8192,65536,1048576,16777216,67108864")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--blocks", type=int, default=64)
    a = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dev = torch.device("cuda", torch.cuda.current_device())
    dist.init_process_group("nccl", device_id=dev)
    sizes = [int(v) for v in a.sizes.split(",")]
    pc = PeerCollectives(max(sizes), device=dev, blocks=a.blocks)
    rows = []
    for nbytes in sizes:
        n = nbytes // 2
        x = torch.randn(n, device=dev).to(torch.bfloat16)
        out = torch.empty_like(x)
        piece = torch.empty(n // world, device=dev, dtype=torch.bfloat16)
        ops = [
            ("all_reduce", lambda: pc.all_reduce(x, out), lambda: dist.all_reduce(out), 2.0 * (world - 1) / world),
            ("reduce_scatter", lambda: pc.reduce_scatter(x, piece), lambda: dist.reduce_scatter_tensor(piece, x), (world - 1) / world),
            ("all_gather", lambda: pc.all_gather(piece, out), lambda: dist.all_gather_into_tensor(out, piece), (world - 1) / world),
            ("all_to_all", lambda: pc.all_to_all(x, out), lambda: dist.all_to_all_single(out, x), (world - 1) / world),
        ]
        if pc.nvls_available and nbytes <= pc.nvls_cap:
            pc.nvls_buffer(torch.bfloat16, n).copy_(x)
            ops += [
                ("all_reduce nvls", lambda: pc.all_reduce_nvls(x, out=out), lambda: dist.all_reduce(out), 2.0 * (world - 1) / world),
                ("  in place", lambda: pc.all_reduce_nvls(numel=n, dtype=torch.bfloat16), lambda: dist.all_reduce(out), 2.0 * (world - 1) / world),
            ]
        for name, ours, lib, factor in ops:
            to, tl = timed(ours, a.iters), timed(lib, a.iters)
            rows.append((name, nbytes, to, tl, nbytes * factor / to / 1e3))
    st = pc.status()
    if rank == 0:
        print(f"# world={world} bf16; status={st}")
        print(f"{'op':16s} {'bytes':>10s} {'ours us':>9s} {'nccl us':>9s} {'nccl/ours':>10s} {'ours busbw GB/s':>16s}")
        for name, nb, to, tl, bw in rows:
            print(f"{name:16s} {nb:10d} {to:9.1f} {tl:9.1f} {tl / to:10.2f} {bw:16.1f}")
    dist.barrier()
    pc.close()
    from rmlx_b200.parallel.symm_heap import close_heaps
    close_heaps()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
