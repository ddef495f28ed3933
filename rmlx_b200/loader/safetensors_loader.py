"""Hugging-Face safetensors checkpoints, single-file or sharded, including MLX-style affine
quantised ones.

What is understood (same as crates/rmlx-nn/src/safetensors_loader.rs:113-628):
  * ``model.safetensors`` or ``model.safetensors.index.json`` + shards,
  * ``config.json`` with an optional ``"quantization": {"bits": 4, "group_size": 64}`` block,
  * quantised linears stored as a triplet ``<p>.weight`` (uint32 ``[out, in*bits/32]``),
    ``<p>.scales``, ``<p>.biases`` (one value per group of ``group_size`` inputs),
  * HF tensor names, mapped to internal names by ``hf_name_to_internal``.

The packed words are used as they are (the kernels read the MLX little-endian nibble order
directly); shards for tensor / expert parallel ranks are cut from the packed form
(crates/rmlx-nn/src/parallel.rs:888-1130). ``save_checkpoint`` writes the same layout (the
reference only loads; writing is needed to make self-contained tests and random-init checkpoints).
"""
from __future__ import annotations

import json
import os
from typing import Dict, List, Optional, Tuple

import torch

from ..config import FeedForwardType, MoeConfig, QuantConfig, TransformerConfig
from ..models.weights import LayerWeights, ModelWeights, ParallelLayout, _split, is_moe_layer
from ..ops.weights import GROUP, LinearWeight, W_BF16, W_Q4, W_Q8


def hf_name_to_internal(name: str) -> str:
    """``model.layers.0.self_attn.q_proj.weight`` -> ``layers.0.attention.q_proj.weight``."""
    n = name[len("model."):] if name.startswith("model.") else name
    for a, b in (("self_attn.", "attention."), ("mlp.gate_proj.", "feed_forward.gate_proj."),
                 ("mlp.up_proj.", "feed_forward.up_proj."), ("mlp.down_proj.", "feed_forward.down_proj."),
                 ("input_layernorm.", "attention_norm."), ("post_attention_layernorm.", "ffn_norm."),
                 ("embed_tokens.", "embedding.")):
        n = n.replace(a, b)
    return n


def read_config(model_dir: str) -> Tuple[TransformerConfig, Optional[QuantConfig]]:
    with open(os.path.join(model_dir, "config.json")) as f:
        c = json.load(f)
    heads = c["num_attention_heads"]
    hd = c.get("head_dim", c["hidden_size"] // heads)
    if c.get("num_experts") or c.get("num_local_experts"):
        e = c.get("num_experts") or c["num_local_experts"]
        moe = MoeConfig(num_experts=e, num_experts_per_token=c["num_experts_per_tok"],
                        hidden_dim=c["hidden_size"],
                        intermediate_dim=c.get("moe_intermediate_size", c["intermediate_size"]))
        ff = FeedForwardType.moe_(moe)
    else:
        ff = FeedForwardType.gated(c["intermediate_size"])
    cfg = TransformerConfig(
        hidden_size=c["hidden_size"], num_heads=heads, num_kv_heads=c.get("num_key_value_heads", heads),
        head_dim=hd, num_layers=c["num_hidden_layers"], vocab_size=c["vocab_size"],
        max_seq_len=c.get("max_position_embeddings", 4096), rope_theta=float(c.get("rope_theta", 1e4)),
        rms_norm_eps=float(c.get("rms_norm_eps", 1e-6)), ff_type=ff,
        sliding_window=int(c.get("sliding_window") or 0),
        tie_embeddings=bool(c.get("tie_word_embeddings", False)),
        name=c.get("model_type", "transformer")).validate()
    q = c.get("quantization")
    quant = QuantConfig(int(q["bits"]), int(q["group_size"])).validate() if q else None
    return cfg, quant


def _file_loader():
    """``load_file`` of the native memory-mapped reader when the host library is available
    (``RMLX_NATIVE_LOADER=0`` opts out), else the one of the ``safetensors`` package."""
    from . import native_st
    if os.environ.get("RMLX_NATIVE_LOADER", "1") != "0" and native_st.available():
        return native_st.load_file
    from safetensors.torch import load_file
    return load_file


def load_tensors(model_dir: str) -> Dict[str, torch.Tensor]:
    """All tensors of a single-file or sharded checkpoint (CPU). With the native reader they are
    views of the mapped files: nothing is read until a tensor is converted or copied to a device."""
    load_file = _file_loader()
    idx = os.path.join(model_dir, "model.safetensors.index.json")
    out: Dict[str, torch.Tensor] = {}
    if os.path.exists(idx):
        with open(idx) as f:
            files = sorted(set(json.load(f)["weight_map"].values()))
    else:
        files = [f for f in sorted(os.listdir(model_dir)) if f.endswith(".safetensors")]
    if not files:
        raise FileNotFoundError(f"no .safetensors files in {model_dir}")
    for fn in files:
        out.update(load_file(os.path.join(model_dir, fn)))
    return out


def detect_triplets(tensors: Dict[str, torch.Tensor]) -> List[str]:
    """Prefixes ``p`` for which ``p.weight`` (32-bit words), ``p.scales`` and ``p.biases`` exist."""
    out = []
    for k, v in tensors.items():
        if k.endswith(".weight") and v.dtype in (torch.int32, torch.uint32):
            p = k[:-len(".weight")]
            if p + ".scales" in tensors and p + ".biases" in tensors:
                out.append(p)
    return out


class _Source:
    """Uniform access to a projection by HF prefix, dense or quantised."""

    def __init__(self, tensors, quant: Optional[QuantConfig], dtype):
        self.t, self.q, self.dtype = tensors, quant, dtype
        self.triplets = set(detect_triplets(tensors))
        if self.triplets and (quant is None or quant.bits not in (4, 8) or quant.group_size != GROUP):
            raise ValueError("quantised checkpoint: bits 4 or 8 with group_size 64 is what the kernels "
                             "support (config.json 'quantization' block missing or different)")

    def linear(self, prefix: str) -> LinearWeight:
        if prefix in self.triplets:
            w = self.t[prefix + ".weight"]
            if w.dtype == torch.uint32:
                w = w.view(torch.int32)
            sc, bi = self.t[prefix + ".scales"], self.t[prefix + ".biases"]
            # bits from the shapes (a checkpoint may mix widths): words per row * 32 / (groups * 64)
            bits = w.shape[-1] * 32 // (sc.shape[-1] * GROUP)
            if bits not in (4, 8):
                raise ValueError(f"{prefix}: {bits}-bit weights are not supported (4 or 8)")
            # scales and biases stay at checkpoint precision: fp16 is kept as fp16 (casting it to
            # bf16 would drop three mantissa bits of every group's scale and bias); wider types
            # go to bf16
            if sc.dtype != torch.float16:
                sc, bi = sc.to(torch.bfloat16), bi.to(torch.bfloat16)
            return LinearWeight(W_Q4 if bits == 4 else W_Q8, w.contiguous(), sc.contiguous(), bi.contiguous())
        return LinearWeight(W_BF16, self.t[prefix + ".weight"].to(self.dtype))

    def vec(self, name: str) -> torch.Tensor:
        return self.t[name].to(self.dtype)


def build_weights(cfg: TransformerConfig, tensors: Dict[str, torch.Tensor],
                  quant: Optional[QuantConfig] = None, device="cpu", dtype=torch.bfloat16,
                  layout: Optional[ParallelLayout] = None, shard_lm_head: bool = True) -> ModelWeights:
    """Runtime weight set of one rank from checkpoint tensors (HF names)."""
    layout = layout or ParallelLayout()
    src = _Source(tensors, quant, dtype)
    hq, q0, hkv, kv0 = layout.heads(cfg)
    hd, w, r = cfg.head_dim, layout.world, layout.rank
    layers = []
    for i in range(cfg.num_layers):
        p = f"model.layers.{i}."
        q = src.linear(p + "self_attn.q_proj").rows(q0 * hd, (q0 + hq) * hd)
        k = src.linear(p + "self_attn.k_proj").rows(kv0 * hd, (kv0 + hkv) * hd)
        v = src.linear(p + "self_attn.v_proj").rows(kv0 * hd, (kv0 + hkv) * hd)
        o = src.linear(p + "self_attn.o_proj").cols(q0 * hd, (q0 + hq) * hd)
        lw = LayerWeights(norm1=src.vec(p + "input_layernorm.weight").to(device),
                          wqkv=LinearWeight.cat_rows([q, k, v]).to(device), wo=o.to(device),
                          norm2=src.vec(p + "post_attention_layernorm.weight").to(device))
        if is_moe_layer(cfg, i):
            m = cfg.ff_type.moe
            lw.router = src.vec(p + "mlp.gate.weight").to(device)
            if layout.expert_parallel:
                (e0, e1), (i0, i1) = _split(m.num_experts, w, r), (0, m.intermediate_dim)
            else:
                (e0, e1), (i0, i1) = (0, m.num_experts), _split(m.intermediate_dim, w, r)
            gu, dn = [], []
            for e in range(e0, e1):
                qn = p + f"mlp.experts.{e}."
                gu.append(LinearWeight.cat_rows([src.linear(qn + "gate_proj").rows(i0, i1),
                                                 src.linear(qn + "up_proj").rows(i0, i1)]))
                dn.append(src.linear(qn + "down_proj").cols(i0, i1))
            lw.experts_gate_up = LinearWeight.stack(gu).to(device)
            lw.experts_down = LinearWeight.stack(dn).to(device)
            lw.expert_base = e0
        else:
            g = src.linear(p + "mlp.gate_proj")
            i0, i1 = _split(g.n, w, r)
            lw.w_gate_up = LinearWeight.cat_rows([g.rows(i0, i1),
                                                  src.linear(p + "mlp.up_proj").rows(i0, i1)]).to(device)
            lw.w_down = src.linear(p + "mlp.down_proj").cols(i0, i1).to(device)
        layers.append(lw)
    emb_prefix = "model.embed_tokens"
    if emb_prefix in src.triplets:   # quantised embedding table: gather needs dense rows
        embed = src.linear(emb_prefix).dequantized().to(dtype)
    else:
        embed = src.vec(emb_prefix + ".weight")
    head = src.linear(emb_prefix if cfg.tie_embeddings else "lm_head")
    v0, v1 = _split(cfg.vocab_size, w, r) if (shard_lm_head and w > 1) else (0, cfg.vocab_size)
    return ModelWeights(cfg=cfg, layout=layout, embed=embed.to(device), layers=layers,
                        final_norm=src.vec("model.norm.weight").to(device),
                        lm_head=head.rows(v0, v1).to(device), vocab_base=v0)


def load_model(model_dir: str, device="cpu", dtype=torch.bfloat16,
               layout: Optional[ParallelLayout] = None):
    """``(TransformerModel-ready ModelWeights, config)`` for one rank from a checkpoint folder."""
    cfg, quant = read_config(model_dir)
    return build_weights(cfg, load_tensors(model_dir), quant, device, dtype, layout), cfg


def save_checkpoint(model_dir: str, cfg: TransformerConfig, state_dict: Dict[str, torch.Tensor],
                    quant: Optional[QuantConfig] = None, shards: int = 1) -> None:
    """Write ``state_dict`` (fp32, HF names) as a checkpoint folder; with ``quant`` every 2-D
    projection except the router and the norms is stored as an MLX affine triplet."""
    from safetensors.torch import save_file
    from ..reference import ops as ref
    os.makedirs(model_dir, exist_ok=True)
    out: Dict[str, torch.Tensor] = {}
    for k, v in state_dict.items():
        is_proj = v.dim() == 2 and k.endswith("_proj.weight") or k == "lm_head.weight"
        if quant is not None and is_proj and v.shape[1] % quant.group_size == 0:
            p, s, b = ref.quantize_affine(v, quant.bits, quant.group_size)
            out[k] = p.contiguous()
            out[k[:-len("weight")] + "scales"] = s.contiguous()
            out[k[:-len("weight")] + "biases"] = b.contiguous()
        else:
            out[k] = v.to(torch.bfloat16).contiguous()
    names = sorted(out)
    if shards <= 1:
        save_file(out, os.path.join(model_dir, "model.safetensors"))
    else:
        weight_map = {}
        per = (len(names) + shards - 1) // shards
        for s in range(shards):
            part = {n: out[n] for n in names[s * per:(s + 1) * per]}
            fn = f"model-{s + 1:05d}-of-{shards:05d}.safetensors"
            save_file(part, os.path.join(model_dir, fn))
            weight_map.update({n: fn for n in part})
        with open(os.path.join(model_dir, "model.safetensors.index.json"), "w") as f:
            json.dump({"metadata": {}, "weight_map": weight_map}, f)
    c = {"model_type": cfg.name, "hidden_size": cfg.hidden_size, "num_attention_heads": cfg.num_heads,
         "num_key_value_heads": cfg.num_kv_heads, "head_dim": cfg.head_dim,
         "num_hidden_layers": cfg.num_layers, "vocab_size": cfg.vocab_size,
         "max_position_embeddings": cfg.max_seq_len, "rope_theta": cfg.rope_theta,
         "rms_norm_eps": cfg.rms_norm_eps, "tie_word_embeddings": cfg.tie_embeddings,
         "sliding_window": cfg.sliding_window or None}
    if cfg.ff_type.kind == "moe":
        m = cfg.ff_type.moe
        c.update({"num_experts": m.num_experts, "num_experts_per_tok": m.num_experts_per_token,
                  "moe_intermediate_size": m.intermediate_dim, "intermediate_size": m.intermediate_dim})
    else:
        c["intermediate_size"] = cfg.ff_type.intermediate_dim
    if quant is not None:
        c["quantization"] = {"bits": quant.bits, "group_size": quant.group_size}
    with open(os.path.join(model_dir, "config.json"), "w") as f:
        json.dump(c, f, indent=1)
