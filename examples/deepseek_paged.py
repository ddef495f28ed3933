#!/usr/bin/env python
"""Latent attention with a paged latent cache: two prompts of different length are prefilled into
pages, then decoded together, one token per sequence per step. On a GPU with bf16 weights and the
published latent width (kv_lora_rank 512, rope_head_dim 64) the decode attention runs on the
latent-attention kernel; on CPU (as here by default) on library ops, with the same results.

    python examples/deepseek_paged.py --steps 6
"""
from __future__ import annotations

import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from rmlx_b200.models.deepseek import DeepSeekV3Model, deepseek_tiny  # noqa: E402


def main(argv=None) -> list:
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=6)
    ap.add_argument("--device", default="cpu")
    a = ap.parse_args(argv)
    cfg = deepseek_tiny()
    model = DeepSeekV3Model(cfg, seed=3, device=a.device)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).to(a.device) for n in (11, 4)]
    cache = model.new_paged_cache(num_blocks=16, max_seqs=4)
    tok = torch.stack([model.prefill_paged(p, cache, s)[0].argmax() for s, p in enumerate(prompts)])
    out = [[], []]
    for _ in range(a.steps):
        for s in range(2):
            out[s].append(int(tok[s]))
        tok = model.decode_paged(tok, cache, [0, 1]).argmax(-1)
    per_token = cache[0].bytes_per_token()
    full = 2 * cfg.num_heads * cfg.head_dim * cache[0].pages.element_size()
    print(f"generated {out}; latent cache: {per_token} bytes per token and layer "
          f"(an uncompressed K/V cache of this model: {full})")
    return out


if __name__ == "__main__":
    main()
