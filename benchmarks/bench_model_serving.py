#!/usr/bin/env python
"""Serving-shaped numbers for the MoE-A22B-shaped model on one GPU: time to first token for a
2048-token prompt through the native prefill path, and decode throughput at batch 1 / 8 / 64 (batch
1 through the graph-captured mat-vec engine, larger batches through the graph-captured tensor-core
path). The counterpart of the reference's e2e_prefill_bench / pipeline_bench
(crates/rmlx-nn/benches/e2e_prefill_bench.rs, pipeline_bench.rs).

    python benchmarks/bench_model_serving.py [--layers 12] [--weights q4|bf16] [--prompt 2048]
        [--batches 1,8,64] [--steps 16]

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
from rmlx_b200.models.weights import random_on_device  # noqa: E402


def ev_time(fn, iters=1):
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=12)
    ap.add_argument("--weights", default="q4", choices=["q4", "bf16"])
    ap.add_argument("--prompt", type=int, default=2048)
    ap.add_argument("--batches", default="1,8,64")
    ap.add_argument("--steps", type=int, default=16)
    a = ap.parse_args()
    dev = torch.device("cuda:0")
    batches = [int(v) for v in a.batches.split(",")]
    cfg = moe_a22b_config(a.layers, max_seq_len=a.prompt + 4 * a.steps + 64)
    model = TransformerModel(random_on_device(cfg, dev, None if a.weights == "bf16" else "q4"))
    assert enable_native_prefill(model)
    L = a.layers
    print(f"# moe-a22b-shaped, {L} layers resident, weights={a.weights}, prompt={a.prompt}")

    # ---- prefill: time to first token
    blocks_per_seq = (cfg.max_seq_len + 15) // 16
    cache = model.new_cache(blocks_per_seq * (max(batches) + 3) + 2, max_seqs=max(batches) + 4,
                            max_blocks_per_seq=blocks_per_seq)
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
    print(f"prefill {a.prompt} tokens: {ttft:8.2f} ms ({L} layers)  {per_layer * 1e3:8.1f} us/layer  "
          f"{a.prompt / ttft * 1e3:9.0f} tok/s;  scaled to 60 layers: {per_layer * 60 + head_ms:8.2f} ms TTFT")

    # ---- decode at several batch sizes, context = the prompt
    for b in batches:
        seqs = list(range(b))
        for s in seqs:
            cache.add_sequence(s)
            cache.reserve(s, a.prompt)
            cache.commit(s, a.prompt)          # context content is irrelevant to timing (zeros)
        last = [1] * b
        if b <= 4:
            eng = CachedDecode(model, cache, max_batch=b)
        else:
            eng = BatchedDecode(model, cache, max_batch=b)
        eng.bind(seqs, last)
        eng.generate(3)                        # warm-up + graph capture
        eng.reserve(a.steps + 2)
        ms = ev_time(lambda: eng.step(), a.steps)
        tok_s = b / ms * 1e3
        print(f"decode batch {b:3d} ctx {a.prompt}: {ms:8.3f} ms/step ({L} layers)  {ms / L * 1e3:7.1f} us/layer  "
              f"{tok_s:9.0f} tok/s;  scaled to 60 layers: {b / (ms / L * 60) * 1e3:9.0f} tok/s")
        for s in seqs:
            cache.free_sequence(s)


if __name__ == "__main__":
    main()
