#!/usr/bin/env python
"""Draft-and-verify generation: a one-layer draft proposes tokens, the target checks them in one
forward per round; the result equals the target's own greedy continuation.

    python examples/speculative.py --k 4 --steps 24
"""
from __future__ import annotations

import argparse
import dataclasses
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from rmlx_b200.config import tiny_dense_config  # noqa: E402
from rmlx_b200.models.transformer import TransformerModel  # noqa: E402
from rmlx_b200.models.weights import from_state_dict, random_state_dict  # noqa: E402
from rmlx_b200.serve.speculative import SpeculativeDecoder  # noqa: E402


def main(argv=None) -> list:
    ap = argparse.ArgumentParser()
    ap.add_argument("--k", type=int, default=4)
    ap.add_argument("--steps", type=int, default=24)
    a = ap.parse_args(argv)
    cfg = tiny_dense_config()
    sd = random_state_dict(cfg, 0)
    target = TransformerModel(from_state_dict(cfg, sd, dtype=torch.float32))
    # the draft: the target's first layer only, same embedding and head
    dcfg = dataclasses.replace(cfg, num_layers=1).validate()
    draft = TransformerModel(from_state_dict(dcfg, sd, dtype=torch.float32))
    prompt = list(range(3, 20))
    spec = SpeculativeDecoder(target, draft, k=a.k)
    out = spec.generate(prompt, a.steps)
    want = target.generate_greedy(torch.tensor(prompt), a.steps)
    print("tokens:", out)
    print(f"identical to plain greedy decoding: {out == want}; rounds {spec.stats.rounds}, "
          f"acceptance {spec.stats.acceptance_rate:.2f}, tokens per target forward "
          f"{spec.stats.tokens_per_round:.2f}")
    return out


if __name__ == "__main__":
    main()
