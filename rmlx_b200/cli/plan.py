"""``rmlx plan``: what a model costs on B200s before anything is loaded.

For a model preset, a weight format, a tensor-parallel degree, a batch and a context length it
prints (and returns) per GPU: weight bytes, KV-cache bytes per token, how many cached tokens fit
beside the weights in the memory budget (default 0.90 of 180 GB), the scratch of a prompt chunk
(``PrefillPlan``), and how the decode projections would be cut by the streaming planner (blocks,
shared memory per block; host arithmetic, no GPU needed). The arithmetic mirrors the loaders'
sharding rules (``models/weights.py::ParallelLayout``): attention heads and feed-forward columns are
split, KV heads are replicated when there are fewer of them than ranks, experts are either sliced
(tensor parallel) or partitioned whole (``--expert-parallel``), the LM head is vocabulary-parallel,
the embedding is replicated.
"""
from __future__ import annotations

import argparse
import json
from typing import Dict, Optional, Sequence

from ..config import TransformerConfig, moe_a22b_config
from ..models.prefill_plan import PrefillPlan
from ..models.weights import ParallelLayout

HBM_BYTES = 180 * 10**9
BITS = {"bf16": 16.0, "q8": 8.0 + 2 * 16 / 64, "q4": 4.0 + 2 * 16 / 64}     # affine formats: scale + bias per 64


def presets() -> Dict[str, TransformerConfig]:
    from ..models import mixtral, qwen
    return {"moe-a22b": moe_a22b_config(60), "qwen2-7b": qwen.qwen2_7b(), "mixtral-8x7b": mixtral.mixtral_8x7b()}


def weight_bytes_per_gpu(cfg: TransformerConfig, weights: str, tp: int, expert_parallel: bool = False) -> Dict[str, int]:
    """Bytes of one rank's shard, by part. Projections are in the chosen format; norms, router
    and embedding stay bf16."""
    layout = ParallelLayout(0, tp, expert_parallel)
    hq, _, hkv, _ = layout.heads(cfg)
    d, hd, bits = cfg.hidden_size, cfg.head_dim, BITS[weights]
    lin = lambda n, k: int(n * k * bits / 8)                         # noqa: E731
    attn = lin((hq + 2 * hkv) * hd, d) + lin(d, hq * hd)
    norms = 2 * d * 2
    moe = cfg.ff_type.moe if cfg.ff_type.kind == "moe" else None
    dense_layers = cfg.first_dense_layers if moe is not None else cfg.num_layers
    moe_layers = cfg.num_layers - dense_layers
    ffn_dense = 0
    if dense_layers:
        inter = (cfg.dense_intermediate_dim or cfg.ff_type.intermediate_dim) // tp
        ffn_dense = lin(2 * inter, d) + lin(d, inter)
    ffn_moe = router = 0
    if moe is not None:
        if expert_parallel:
            e_local, inter = moe.num_experts // tp, moe.intermediate_dim
        else:
            e_local, inter = moe.num_experts, moe.intermediate_dim // tp
        ffn_moe = e_local * (lin(2 * inter, d) + lin(d, inter))
        router = moe.num_experts * d * 2
    embed = cfg.vocab_size * d * 2
    lm_head = 0 if cfg.tie_embeddings else lin(cfg.vocab_size // tp, d)
    parts = {
        "attention": cfg.num_layers * attn,
        "feed_forward": dense_layers * ffn_dense + moe_layers * (ffn_moe + router),
        "norms": cfg.num_layers * norms + d * 2,
        "embedding": embed,
        "lm_head": lm_head,
    }
    parts["total"] = sum(parts.values())
    return parts


def kv_bytes_per_token_per_gpu(cfg: TransformerConfig, tp: int, kv_quant: Optional[str] = None) -> int:
    """All layers, K and V, this rank's KV heads. The 8-bit format stores one byte per value plus a
    bf16 scale and bias per 64 values."""
    _, _, hkv, _ = ParallelLayout(0, tp).heads(cfg)
    per_value = 1.0 + 4.0 / 64 if kv_quant == "q8" else 2.0
    return int(cfg.num_layers * 2 * hkv * cfg.head_dim * per_value)


def decode_roofline(cfg: TransformerConfig, weights: str, tp: int, ctx: int, batch: int = 1,
                    hbm_gbs: Optional[float] = None) -> Dict[str, float]:
    """Bytes one decode step must read per GPU (each active weight once, the cached keys and
    values of ``ctx`` tokens per sequence, the LM head) over the copy bandwidth: the floor the
    measured step time is reported against. ``hbm_gbs`` defaults to the pool's measured figure
    (``MEASURED_PEAKS.json`` beside the package) or 6650 GB/s."""
    if hbm_gbs is None:
        import os
        path = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))),
                            "MEASURED_PEAKS.json")
        hbm_gbs = json.load(open(path))["hbm_gbs"] if os.path.exists(path) else 6650.0
    layout = ParallelLayout(0, tp)
    hq, _, hkv, _ = layout.heads(cfg)
    d, hd, bits = cfg.hidden_size, cfg.head_dim, BITS[weights]
    lin = lambda n, k: n * k * bits / 8                              # noqa: E731
    layer = lin((hq + 2 * hkv) * hd, d) + lin(d, hq * hd) + batch * ctx * 2 * hkv * hd * 2
    if cfg.ff_type.kind == "moe":
        m = cfg.ff_type.moe
        inter = m.intermediate_dim // tp
        active = min(m.num_experts, batch * m.num_experts_per_token)   # distinct experts at most
        layer += active * (lin(2 * inter, d) + lin(d, inter)) + m.num_experts * d * 2
    else:
        inter = cfg.ff_type.intermediate_dim // tp
        layer += lin(2 * inter, d) + lin(d, inter)
    head = lin(cfg.vocab_size // tp, d)
    step = cfg.num_layers * layer + head
    us = step / (hbm_gbs * 1e3)
    return {"bytes_per_layer": layer, "us_per_layer": layer / (hbm_gbs * 1e3), "us_per_step": us,
            "tokens_per_s": batch * 1e6 / us, "hbm_gbs": hbm_gbs}


def decode_stream_plans(cfg: TransformerConfig, weights: str, tp: int, batch: int = 1) -> Dict[str, dict]:
    """Blocks and shared memory of the decode projections on the streaming kernels (None where
    the library cannot be loaded)."""
    try:
        from ..ops.decode import stream_plan
    except Exception:                                                 # noqa: BLE001
        return {}
    kind = {"bf16": 0, "q4": 1, "q8": 2}[weights]
    hq, _, hkv, _ = ParallelLayout(0, tp).heads(cfg)
    d, hd = cfg.hidden_size, cfg.head_dim
    ops = {"qkv": (0, (hq + 2 * hkv) * hd, d, 1), "o_proj": (0, d, hq * hd, 1),
           "lm_head": (0, cfg.vocab_size // tp, d, 1)}
    if cfg.ff_type.kind == "moe":
        m = cfg.ff_type.moe
        ops["expert_down"] = (2, d, m.intermediate_dim // tp, m.num_experts_per_token)
    else:
        inter = cfg.ff_type.intermediate_dim // tp
        ops["gate_up"] = (1, inter, d, 1)
        ops["down"] = (0, d, inter, 1)
    out = {}
    for name, (op, n, k, top_k) in ops.items():
        try:
            p = stream_plan(kind, op, 1 if op == 2 else batch, n, k, top_k, 148)
        except Exception:                                             # noqa: BLE001
            return {}
        out[name] = {"supported": p["ok"], "blocks": p["grid"], "smem_per_block": p["smem"],
                     "stage_bytes": p["stage_bytes"], "ring_stages": p["ns"]}
    return out


def plan_deepseek(weights: str = "q4", ranks: int = 8, batch: int = 1, ctx: int = 4096,
                  budget_fraction: float = 0.90, cfg=None) -> dict:
    """DeepSeek-V3 (latent attention, 256 routed experts + a shared one, first layer dense): the
    routed experts are partitioned over ``ranks`` GPUs, attention, the shared expert and the dense
    layer are replicated (how ``models/deepseek.py`` with an expert-parallel exchange lays it out).
    The cache holds one latent row of kv_lora_rank + rope_head_dim (+ 8 padding) values per token
    and layer, whatever the number of heads."""
    from ..models.deepseek import deepseek_v3
    c = cfg or deepseek_v3()
    bits = BITS[weights]
    lin = lambda n, k: int(n * k * bits / 8)                         # noqa: E731
    d, h = c.hidden_size, c.num_heads
    qk = c.head_dim + c.rope_head_dim
    q = lin(c.q_lora_rank, d) + lin(h * qk, c.q_lora_rank) if c.q_lora_rank else lin(h * qk, d)
    attn = q + lin(c.kv_lora_rank + c.rope_head_dim, d) + lin(h * (c.head_dim + c.v_head_dim), c.kv_lora_rank) \
        + lin(d, h * c.v_head_dim)
    expert = lin(2 * c.moe_intermediate, d) + lin(d, c.moe_intermediate)
    moe_layers = c.num_layers - c.first_dense_layers
    dense = c.first_dense_layers * (lin(2 * c.dense_intermediate, d) + lin(d, c.dense_intermediate))
    parts = {
        "attention": c.num_layers * attn,
        "routed_experts": moe_layers * (c.num_experts // ranks) * expert,
        "shared_experts_and_router": moe_layers * (c.num_shared_experts * expert + c.num_experts * d * 2),
        "dense_layers": dense,
        "norms": c.num_layers * (2 * d + c.kv_lora_rank + c.q_lora_rank) * 2,
        "embedding": c.vocab_size * d * 2,
        "lm_head": lin(c.vocab_size, d),
    }
    parts["total"] = sum(parts.values())
    latent_row = (c.kv_lora_rank + c.rope_head_dim + 8) * 2
    kv_tok = c.num_layers * latent_row
    full_kv_tok = c.num_layers * h * (qk + c.v_head_dim) * 2
    budget = int(HBM_BYTES * budget_fraction)
    need = batch * ctx * kv_tok
    return {
        "model": "deepseek-v3", "weights": weights, "tp": ranks, "expert_parallel": True, "batch": batch,
        "ctx": ctx, "kv_quant": "latent bf16", "weight_bytes_per_gpu": parts,
        "kv_bytes_per_token_per_gpu": kv_tok, "uncompressed_kv_bytes_per_token": full_kv_tok,
        "kv_compression": round(full_kv_tok / kv_tok, 1),
        "prefill_chunk": 0, "prefill_scratch_bytes": 0, "budget_bytes_per_gpu": budget,
        "kv_bytes_needed": need, "kv_tokens_that_fit": max(0, (budget - parts["total"]) // kv_tok),
        "fits": parts["total"] + need <= budget, "decode_stream_plans": {},
    }


def plan(model: str = "moe-a22b", weights: str = "q4", tp: int = 1, batch: int = 1, ctx: int = 4096,
         kv_quant: Optional[str] = None, expert_parallel: bool = False, prefill_chunk: int = 2048,
         budget_fraction: float = 0.90, cfg: Optional[TransformerConfig] = None) -> dict:
    if model == "deepseek-v3" and cfg is None:
        return plan_deepseek(weights, tp, batch, ctx, budget_fraction)
    cfg = cfg or presets()[model]
    w = weight_bytes_per_gpu(cfg, weights, tp, expert_parallel)
    kv_tok = kv_bytes_per_token_per_gpu(cfg, tp, kv_quant)
    budget = int(HBM_BYTES * budget_fraction)
    scratch = PrefillPlan(cfg, prefill_chunk, ParallelLayout(0, tp, expert_parallel)).scratch_bytes
    scratch = scratch() if callable(scratch) else scratch
    free_for_kv = budget - w["total"] - scratch
    kv_needed = batch * ctx * kv_tok
    return {
        "model": cfg.name, "weights": weights, "tp": tp, "expert_parallel": expert_parallel,
        "batch": batch, "ctx": ctx, "kv_quant": kv_quant or "bf16",
        "weight_bytes_per_gpu": w, "kv_bytes_per_token_per_gpu": kv_tok,
        "prefill_chunk": prefill_chunk, "prefill_scratch_bytes": int(scratch),
        "budget_bytes_per_gpu": budget,
        "kv_bytes_needed": kv_needed,
        "kv_tokens_that_fit": max(0, free_for_kv // kv_tok),
        "fits": w["total"] + scratch + kv_needed <= budget,
        "decode_roofline": decode_roofline(cfg, weights, tp, ctx, batch),
        # batches above 8 rows decode on the tensor-core path, not on the streaming mat-vecs
        "decode_stream_plans": decode_stream_plans(cfg, weights, tp, batch) if batch <= 8 else {},
    }


def _gb(n: int) -> str:
    return f"{n / 1e9:8.2f} GB"


def render(p: dict) -> str:
    w = p["weight_bytes_per_gpu"]
    if p["model"] == "deepseek-v3":
        return "\n".join([
            f"deepseek-v3: {p['weights']} weights, routed experts over {p['tp']} GPUs, batch {p['batch']}, context {p['ctx']}",
            f"  weights per GPU      {_gb(w['total'])}  (routed experts {_gb(w['routed_experts']).strip()}, attention "
            f"{_gb(w['attention']).strip()}, shared experts + router {_gb(w['shared_experts_and_router']).strip()}, "
            f"dense layer {_gb(w['dense_layers']).strip()}, embedding {_gb(w['embedding']).strip()}, LM head {_gb(w['lm_head']).strip()})",
            f"  latent cache per token {p['kv_bytes_per_token_per_gpu']} B ({p['kv_compression']}x smaller than per-head keys and values: "
            f"{p['uncompressed_kv_bytes_per_token']} B); needed {_gb(p['kv_bytes_needed']).strip()}",
            f"  budget per GPU       {_gb(p['budget_bytes_per_gpu'])}  -> {'fits' if p['fits'] else 'DOES NOT FIT'}; "
            f"room for {p['kv_tokens_that_fit']:,} cached tokens per GPU"])
    lines = [f"{p['model']}: {p['weights']} weights, TP={p['tp']}"
             f"{' (experts partitioned)' if p['expert_parallel'] else ''}, batch {p['batch']}, context {p['ctx']}, "
             f"KV {p['kv_quant']}",
             f"  weights per GPU      {_gb(w['total'])}  (attention {_gb(w['attention']).strip()}, feed-forward "
             f"{_gb(w['feed_forward']).strip()}, embedding {_gb(w['embedding']).strip()}, LM head {_gb(w['lm_head']).strip()})",
             f"  KV per token per GPU {p['kv_bytes_per_token_per_gpu']:8d} B   needed for this batch and context {_gb(p['kv_bytes_needed']).strip()}",
             f"  prompt chunk {p['prefill_chunk']}: scratch {_gb(p['prefill_scratch_bytes']).strip()}",
             f"  budget per GPU       {_gb(p['budget_bytes_per_gpu'])}  -> {'fits' if p['fits'] else 'DOES NOT FIT'}; "
             f"room for {p['kv_tokens_that_fit']:,} cached tokens per GPU"]
    r = p["decode_roofline"]
    lines.append(f"  decode floor (bytes over {r['hbm_gbs']:.0f} GB/s): {r['bytes_per_layer'] / 1e6:.1f} MB and "
                 f"{r['us_per_layer']:.1f} us per layer, {r['tokens_per_s']:.0f} tokens/s")
    if p["batch"] > 8:
        lines.append("  decode: batches above 8 rows run on the tensor-core path (GEMM tiles), no streaming plan")
    for name, sp in p["decode_stream_plans"].items():
        lines.append(f"  decode {name:12s} {'streaming' if sp['supported'] else 'per-row kernels'}: {sp['blocks']:3d} blocks, "
                     f"{sp['smem_per_block'] / 1024:5.1f} KB shared memory, {sp['ring_stages']} x {sp['stage_bytes'] // 1024} KB ring")
    return "\n".join(lines)


def main(argv: Optional[Sequence[str]] = None) -> int:
    ap = argparse.ArgumentParser(prog="rmlx plan", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", default="moe-a22b", choices=sorted(presets()) + ["deepseek-v3"])
    ap.add_argument("--weights", default="q4", choices=sorted(BITS))
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--expert-parallel", action="store_true")
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--ctx", type=int, default=4096)
    ap.add_argument("--kv-quant", default=None, choices=[None, "q8"])
    ap.add_argument("--prefill-chunk", type=int, default=2048)
    ap.add_argument("--budget", type=float, default=0.90, help="fraction of 180 GB that may be used")
    ap.add_argument("--json", action="store_true")
    a = ap.parse_args(argv)
    p = plan(a.model, a.weights, a.tp, a.batch, a.ctx, a.kv_quant, a.expert_parallel, a.prefill_chunk, a.budget)
    print(json.dumps(p) if a.json else render(p))
    return 0 if p["fits"] else 1


if __name__ == "__main__":
    raise SystemExit(main())
