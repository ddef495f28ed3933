#!/usr/bin/env python
"""Generate tokens from a model: random weights of a small MoE decoder by default, or an MLX-style
safetensors directory (``--model-dir``; packed Q4 triplets are used as they are).

On a GPU the prompt runs through the tensor-core prefill and every new token is one replay of the
captured decode graph; on CPU the library-kernel forward runs the same model.

    python examples/generate.py --steps 16
    python examples/generate.py --model-dir /path/to/model --prompt 1,2,3 --steps 32
"""
from __future__ import annotations

import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from rmlx_b200.config import FeedForwardType, MoeConfig, TransformerConfig  # noqa: E402
from rmlx_b200.models.transformer import TransformerModel  # noqa: E402
from rmlx_b200.models.weights import from_state_dict, random_state_dict  # noqa: E402


def small_moe() -> TransformerConfig:
    moe = MoeConfig(num_experts=8, num_experts_per_token=2, hidden_dim=512, intermediate_dim=512)
    return TransformerConfig(hidden_size=512, num_heads=4, num_kv_heads=2, head_dim=128, num_layers=2,
                             vocab_size=1024, max_seq_len=1024, rope_theta=1e6,
                             ff_type=FeedForwardType.moe_(moe), name="example-moe").validate()


def main(argv=None) -> list:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model-dir", default=None)
    ap.add_argument("--prompt", default="1,2,3,4,5,6,7,8")
    ap.add_argument("--steps", type=int, default=16)
    ap.add_argument("--quant", default="q4", choices=["q4", "none"])
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    a = ap.parse_args(argv)
    dev = torch.device(a.device)
    if a.model_dir:
        from rmlx_b200.loader.safetensors_loader import load_model
        weights, _ = load_model(a.model_dir, device=dev)
    else:
        cfg = small_moe()
        quant = None if (a.quant == "none" or dev.type == "cpu") else a.quant
        dtype = torch.bfloat16 if dev.type == "cuda" else torch.float32
        weights = from_state_dict(cfg, random_state_dict(cfg, 0), device=dev, quant=quant, dtype=dtype)
    model = TransformerModel(weights)
    prompt = torch.tensor([int(t) for t in a.prompt.split(",")], device=dev)
    if dev.type == "cuda":
        from rmlx_b200.models.decode_engine import CachedDecode
        from rmlx_b200.models.prefill import enable_native_prefill
        enable_native_prefill(model)
        cache = model.new_cache((prompt.numel() + a.steps + 15) // 16 + 2, max_seqs=1)
        cache.add_sequence(0)
        logits = model.prefill(prompt, cache, 0)
        first = int(logits[0].argmax())
        eng = CachedDecode(model, cache, max_batch=1)
        eng.bind([0], [first])
        toks = [first] + (eng.generate(a.steps - 1)[0].tolist() if a.steps > 1 else [])
    else:
        toks = model.generate_greedy(prompt, a.steps)
    print("tokens:", toks)
    return toks


if __name__ == "__main__":
    main()
