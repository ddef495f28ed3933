#!/usr/bin/env python
"""Serving-shaped numbers for the MoE-A22B-shaped model: time to first token for a 2048-token
prompt through the native prefill path, and decode throughput at batch 1 / 8 / 64 (batch 1 through
the graph-captured mat-vec engine, larger batches through the tensor-core path). The counterpart
of the reference's e2e_prefill_bench / pipeline_bench / distributed_bench
(crates/rmlx-nn/benches/e2e_prefill_bench.rs, pipeline_bench.rs, distributed_bench.rs:45-54).

    python benchmarks/bench_model_serving.py [--layers 12] [--weights q4|bf16] [--prompt 2048]
        [--batches 1,8,64] [--steps 16]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        benchmarks/bench_model_serving.py ...          # tensor parallel over N GPUs

Under a multi-rank launch the weights are sharded (heads, FFN columns, experts, vocabulary), the
row-parallel GEMMs of the tensor-core path run fused with their all-reduce over NVLink
(``--tp-gemm fused``, default) or as GEMM + NCCL (``--tp-gemm nccl``), and the mat-vec engine uses the
fused mat-vec + all-reduce kernels. Times are the maximum over ranks.

``--layers`` defaults to 12 so that the run fits a short GPU slot; every figure is printed per layer
and, labelled as such, scaled to the 60 layers of the full model (layers are identical, the LM head
is counted once). Timing: CUDA events after warm-up; the prompt's working set and the per-step
weights exceed L2, so nothing is served from cache across iterations.
"""
from __future__ import annotations

import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from rmlx_b200.config import moe_a22b_config  # noqa: E402
from rmlx_b200.models.decode_engine import CachedDecode  # noqa: E402
from rmlx_b200.models.prefill import BatchedDecode, enable_native_prefill  # noqa: E402
from rmlx_b200.models.transformer import TransformerModel  # noqa: E402
from rmlx_b200.models.weights import ParallelLayout, random_on_device  # noqa: E402


WORLD = int(os.environ.get("WORLD_SIZE", "1"))
RANK = int(os.environ.get("RANK", "0"))


def ev_time(fn, iters=1):
    """Device time per call (CUDA events), maximum over ranks."""
    if WORLD > 1:
        torch.distributed.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / iters
    if WORLD > 1:
        t = torch.tensor([ms], device="cuda")
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        ms = float(t[0])
    return ms


def say(*a):
    if RANK == 0:
        print(*a, flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=12)
    ap.add_argument("--weights", default="q4", choices=["q4", "bf16"])
    ap.add_argument("--prompt", type=int, default=2048)
    ap.add_argument("--batches", default="1,8,64")
    ap.add_argument("--steps", type=int, default=16)
    ap.add_argument("--tp-gemm", default="fused", choices=["fused", "nccl"])
    ap.add_argument("--matvec-max-batch", type=int, default=8,
                    help="largest batch that runs on the mat-vec engine (rows beyond four are chunked)")
    ap.add_argument("--kv-quant", default=None, choices=[None, "q8"])
    a = ap.parse_args()
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    batches = [int(v) for v in a.batches.split(",")]
    cfg = moe_a22b_config(a.layers, max_seq_len=a.prompt + 4 * a.steps + 64)
    quant = None if a.weights == "bf16" else "q4"
    comm = None
    if WORLD > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)

        def allreduce(t):
            t = t.contiguous()
            dist.all_reduce(t)
            return t

        def allgather(t):
            parts = [torch.empty_like(t) for _ in range(WORLD)]
            dist.all_gather(parts, t.contiguous())
            return torch.cat(parts, -1)

        # whole experts per rank (the grouped tensor-core GEMM then keeps its full inner dimension);
        # attention, the dense projections and the vocabulary are sliced
        model = TransformerModel(random_on_device(cfg, dev, quant,
                                                  ParallelLayout(RANK, WORLD, expert_parallel=True), seed=0),
                                 allreduce, allgather)
        from rmlx_b200.parallel.comm import make_comm
        from rmlx_b200.parallel.tp_gemm import make_gemm_comm
        rows = max(a.prompt, max(batches))
        attn_local = model.hq * cfg.head_dim
        i_local = max([l.w_gate_up.n // 2 for l in model.w.layers if l.w_gate_up is not None] + [0])
        model.gemm_comm = make_gemm_comm(a.tp_gemm, rows, cfg.hidden_size, max(attn_local, i_local, 64),
                                         device=dev)
        comm = make_comm("fused", model, max_batch=max(4, a.matvec_max_batch))
    else:
        model = TransformerModel(random_on_device(cfg, dev, quant))
    assert enable_native_prefill(model)
    L = a.layers
    say(f"# moe-a22b-shaped, {L} layers resident, weights={a.weights}, prompt={a.prompt}, "
        f"tensor parallel {WORLD}" + (f" (row-parallel GEMMs: {a.tp_gemm})" if WORLD > 1 else ""))

    # ---- prefill: time to first token
    blocks_per_seq = (cfg.max_seq_len + 15) // 16
    cache = model.new_cache(blocks_per_seq * (max(batches) + 3) + 2, max_seqs=max(batches) + 4,
                            max_blocks_per_seq=blocks_per_seq, kv_quant=a.kv_quant)
    g = torch.Generator().manual_seed(0)
    prompt = torch.randint(0, cfg.vocab_size, (a.prompt,), generator=g).to(dev)
    times = []
    for i in range(4):                     # first two are warm-up
        cache.add_sequence(1000 + i)
        times.append(ev_time(lambda: model.prefill(prompt, cache, 1000 + i)))
        cache.free_sequence(1000 + i)
    ttft = min(times[2:])
    head_ms = ev_time(lambda: model._native_prefill.layers.logits(torch.zeros(1, cfg.hidden_size, dtype=torch.bfloat16, device=dev)), 5)
    per_layer = (ttft - head_ms) / L
    say(f"prefill {a.prompt} tokens: {ttft:8.2f} ms ({L} layers)  {per_layer * 1e3:8.1f} us/layer  "
          f"{a.prompt / ttft * 1e3:9.0f} tok/s;  scaled to 60 layers: {per_layer * 60 + head_ms:8.2f} ms TTFT")

    # ---- decode at several batch sizes, context = the prompt
    for b in batches:
        seqs = list(range(b))
        for s in seqs:
            cache.add_sequence(s)
            cache.reserve(s, a.prompt)
            cache.commit(s, a.prompt)          # context content is irrelevant to timing (zeros)
        last = [1] * b
        if b <= a.matvec_max_batch:
            eng = CachedDecode(model, cache, max_batch=b, comm=comm)
        else:
            eng = BatchedDecode(model, cache, max_batch=b)
        eng.bind(seqs, last)
        eng.generate(3)                        # warm-up + graph capture
        eng.reserve(a.steps + 2)
        ms = ev_time(lambda: eng.step(), a.steps)
        tok_s = b / ms * 1e3
        say(f"decode batch {b:3d} ctx {a.prompt}: {ms:8.3f} ms/step ({L} layers)  {ms / L * 1e3:7.1f} us/layer  "
              f"{tok_s:9.0f} tok/s;  scaled to 60 layers: {b / (ms / L * 60) * 1e3:9.0f} tok/s")
        for s in seqs:
            cache.free_sequence(s)
    if WORLD > 1:
        torch.cuda.synchronize()
        torch.distributed.barrier()
        st = (comm.status(), model.gemm_comm.status())
        say(f"# status words (mat-vec all-reduce, GEMM collective): {st}")
        comm.close()
        model.gemm_comm.close()
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
