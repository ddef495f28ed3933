#!/usr/bin/env python
"""Continuous batching over a handful of requests that share a system prompt: the scheduler admits
them as batch slots and KV pages allow, prompts run in chunks, the shared prefix is computed once
(prefix cache) and decode runs batched; optional sampling.

    python examples/serve_requests.py --requests 6 --max-batch 2 --temperature 0.8
"""
from __future__ import annotations

import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from rmlx_b200.config import SamplerConfig, SchedulerConfig  # noqa: E402
from rmlx_b200.models.transformer import TransformerModel  # noqa: E402
from rmlx_b200.models.weights import from_state_dict, random_state_dict  # noqa: E402
from rmlx_b200.serve.engine import ServingEngine  # noqa: E402
from rmlx_b200.utils.precision_guard import PrecisionGuard  # noqa: E402

from generate import small_moe  # noqa: E402


def main(argv=None) -> dict:
    ap = argparse.ArgumentParser()
    ap.add_argument("--requests", type=int, default=6)
    ap.add_argument("--max-batch", type=int, default=2)
    ap.add_argument("--max-new", type=int, default=8)
    ap.add_argument("--temperature", type=float, default=0.0)
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    a = ap.parse_args(argv)
    dev = torch.device(a.device)
    cfg = small_moe()
    on_gpu = dev.type == "cuda"
    model = TransformerModel(from_state_dict(cfg, random_state_dict(cfg, 0), device=dev,
                                             quant="q4" if on_gpu else None,
                                             dtype=torch.bfloat16 if on_gpu else torch.float32))
    eng = ServingEngine(model, num_blocks=128,
                        scheduler_cfg=SchedulerConfig(max_batch_size=a.max_batch, max_prefill_chunk=64),
                        sampler_cfg=SamplerConfig(temperature=a.temperature, top_k=40, seed=0),
                        use_prefix_cache=True, precision_guard=PrecisionGuard(), guard_every=4)
    warm = eng.warm_up()        # kernels loaded, one graph per batch bucket captured, pages given back
    print(f"warm-up: {warm.kernels_s * 1e3:.0f} ms")
    g = torch.Generator().manual_seed(0)
    system = torch.randint(0, cfg.vocab_size, (48,), generator=g).tolist()
    ids = [eng.submit(system + torch.randint(0, cfg.vocab_size, (5 + i,), generator=g).tolist(), a.max_new)
           for i in range(a.requests)]
    outs = eng.run_until_done()
    for i in ids:
        print(f"request {i}: {outs[i]}")
    print(f"prompt tokens run: {eng.prefill_tokens} (prefix cache hits: {eng.prefix.hits}, "
          f"pages kept: {len(eng.prefix)}); logit monitor: {eng.guard.checks} checks, "
          f"{eng.guard_warnings} warnings, {eng.guard_fallbacks} fallback verdicts")
    return outs


if __name__ == "__main__":
    main()
