"""Model weight sets: random initialisation, construction from a Hugging-Face-style state dict,
load-time merging (QKV, gate/up), expert stacking, quantisation and tensor/expert-parallel
sharding.

Sharding follows crates/rmlx-nn/src/attention.rs:2598-2747 (query heads split by columns, output
projection by rows), crates/rmlx-nn/src/transformer.rs:695-885 (gate/up column split, down row
split) and crates/rmlx-nn/src/transformer.rs:4752-4780 (norms and embedding replicated). When there
are fewer KV heads than ranks, each rank keeps the one KV head its query heads use. Experts are
either sliced along the intermediate dimension on every rank (tensor parallel) or partitioned
contiguously, ``experts_per_rank = E / world`` (expert parallel,
crates/rmlx-distributed/src/moe_exchange.rs:578-581). The LM head is split by vocabulary rows.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional

import torch

from ..config import TransformerConfig
from ..ops.weights import LinearWeight


@dataclass
class ParallelLayout:
    """Where this rank sits. ``tp`` shards attention + FFN; ``ep`` > 1 partitions experts instead
    of slicing them (attention stays tensor-parallel over the same ranks)."""
    rank: int = 0
    world: int = 1
    expert_parallel: bool = False

    def heads(self, cfg: TransformerConfig):
        w, r = self.world, self.rank
        assert cfg.num_heads % w == 0, "num_heads must divide by the tensor-parallel size"
        hq = cfg.num_heads // w
        if cfg.num_kv_heads >= w:
            assert cfg.num_kv_heads % w == 0
            hkv = cfg.num_kv_heads // w
            kv0 = r * hkv
        else:
            assert w % cfg.num_kv_heads == 0, "ranks must be a multiple of kv heads to replicate"
            hkv = 1
            kv0 = (r * cfg.num_kv_heads) // w
        return hq, r * hq, hkv, kv0


@dataclass
class LayerWeights:
    norm1: torch.Tensor
    wqkv: LinearWeight
    wo: LinearWeight
    norm2: torch.Tensor
    w_gate_up: Optional[LinearWeight] = None
    w_down: Optional[LinearWeight] = None
    router: Optional[torch.Tensor] = None
    expert_bias: Optional[torch.Tensor] = None
    experts_gate_up: Optional[LinearWeight] = None   # [E_local, 2*I_local, D]
    experts_down: Optional[LinearWeight] = None      # [E_local, D, I_local]
    expert_base: int = 0
    shared_gate_up: Optional[LinearWeight] = None
    shared_down: Optional[LinearWeight] = None


@dataclass
class ModelWeights:
    cfg: TransformerConfig
    layout: ParallelLayout
    embed: torch.Tensor
    layers: List[LayerWeights]
    final_norm: torch.Tensor
    lm_head: LinearWeight            # [V_local, D]
    vocab_base: int = 0

    def nbytes(self) -> int:
        t = self.embed.numel() * self.embed.element_size() + self.lm_head.nbytes()
        for l in self.layers:
            for w in (l.wqkv, l.wo, l.w_gate_up, l.w_down, l.experts_gate_up, l.experts_down,
                      l.shared_gate_up, l.shared_down):
                if w is not None:
                    t += w.nbytes()
        return t


def is_moe_layer(cfg: TransformerConfig, i: int) -> bool:
    return cfg.ff_type.kind == "moe" and i >= cfg.first_dense_layers


def random_state_dict(cfg: TransformerConfig, seed: int = 0, std: float = 0.02) -> Dict[str, torch.Tensor]:
    """fp32 CPU weights ~ N(0, std) with Hugging-Face-style names (norm weights are ones)."""
    g = torch.Generator().manual_seed(seed)
    d, hd = cfg.hidden_size, cfg.head_dim
    sd: Dict[str, torch.Tensor] = {}

    def rnd(*shape):
        return torch.randn(*shape, generator=g) * std

    sd["model.embed_tokens.weight"] = rnd(cfg.vocab_size, d)
    for i in range(cfg.num_layers):
        p = f"model.layers.{i}."
        sd[p + "input_layernorm.weight"] = torch.ones(d) + rnd(d)
        sd[p + "self_attn.q_proj.weight"] = rnd(cfg.num_heads * hd, d)
        sd[p + "self_attn.k_proj.weight"] = rnd(cfg.num_kv_heads * hd, d)
        sd[p + "self_attn.v_proj.weight"] = rnd(cfg.num_kv_heads * hd, d)
        sd[p + "self_attn.o_proj.weight"] = rnd(d, cfg.num_heads * hd)
        sd[p + "post_attention_layernorm.weight"] = torch.ones(d) + rnd(d)
        if is_moe_layer(cfg, i):
            m = cfg.ff_type.moe
            sd[p + "mlp.gate.weight"] = rnd(m.num_experts, d) * (1.0 / std) * 0.05
            for e in range(m.num_experts):
                q = p + f"mlp.experts.{e}."
                sd[q + "gate_proj.weight"] = rnd(m.intermediate_dim, d)
                sd[q + "up_proj.weight"] = rnd(m.intermediate_dim, d)
                sd[q + "down_proj.weight"] = rnd(d, m.intermediate_dim)
            if m.num_shared_experts:
                si = m.shared_intermediate_dim * m.num_shared_experts
                sd[p + "mlp.shared_expert.gate_proj.weight"] = rnd(si, d)
                sd[p + "mlp.shared_expert.up_proj.weight"] = rnd(si, d)
                sd[p + "mlp.shared_expert.down_proj.weight"] = rnd(d, si)
        else:
            inter = cfg.dense_intermediate_dim if (cfg.ff_type.kind == "moe") else cfg.ff_type.intermediate_dim
            sd[p + "mlp.gate_proj.weight"] = rnd(inter, d)
            sd[p + "mlp.up_proj.weight"] = rnd(inter, d)
            sd[p + "mlp.down_proj.weight"] = rnd(d, inter)
    sd["model.norm.weight"] = torch.ones(d) + rnd(d)
    if not cfg.tie_embeddings:
        sd["lm_head.weight"] = rnd(cfg.vocab_size, d)
    return sd


def _split(n: int, world: int, rank: int):
    assert n % world == 0, f"{n} does not divide by {world}"
    s = n // world
    return rank * s, (rank + 1) * s


def from_state_dict(cfg: TransformerConfig, sd: Dict[str, torch.Tensor], device="cpu",
                    dtype=torch.bfloat16, quant: Optional[str] = None,
                    layout: Optional[ParallelLayout] = None, shard_lm_head: bool = True
                    ) -> ModelWeights:
    """Build the runtime weight set for one rank from full (unsharded) fp32 tensors."""
    layout = layout or ParallelLayout()
    hq, q0, hkv, kv0 = layout.heads(cfg)
    hd, d = cfg.head_dim, cfg.hidden_size
    w, r = layout.world, layout.rank
    # Towards a GPU the layers go through the compute / transfer pipeline: layer i's slicing,
    # packing and quantisation run on the host while layer i-1's tensors cross to the device on a
    # second stream (parallel.pipeline.LayerPipeline; pinned staging makes the copies asynchronous).
    final_device = torch.device(device)
    piped = final_device.type == "cuda"
    device = "cpu" if piped else device

    def lin(t: torch.Tensor) -> LinearWeight:
        return LinearWeight.from_dense(t, quant, dtype, device)

    def vec(t: torch.Tensor) -> torch.Tensor:
        return t.to(dtype).to(device).contiguous()

    def ship(t):
        """Host tensor (or weight container) -> the target device, asynchronously."""
        if t is None or isinstance(t, int):
            return t
        if isinstance(t, LinearWeight):
            return LinearWeight(t.kind, ship(t.w), ship(t.scales), ship(t.biases))
        return t.pin_memory().to(final_device, non_blocking=True)

    def ship_layer(_i: int, lw: "LayerWeights") -> "LayerWeights":
        for f in lw.__dataclass_fields__:
            setattr(lw, f, ship(getattr(lw, f)))
        return lw

    def host_layer(i: int) -> "LayerWeights":
        p = f"model.layers.{i}."
        q = sd[p + "self_attn.q_proj.weight"][q0 * hd:(q0 + hq) * hd]
        k = sd[p + "self_attn.k_proj.weight"][kv0 * hd:(kv0 + hkv) * hd]
        v = sd[p + "self_attn.v_proj.weight"][kv0 * hd:(kv0 + hkv) * hd]
        o = sd[p + "self_attn.o_proj.weight"][:, q0 * hd:(q0 + hq) * hd]
        lw = LayerWeights(norm1=vec(sd[p + "input_layernorm.weight"]),
                          wqkv=lin(torch.cat([q, k, v], 0)), wo=lin(o.contiguous()),
                          norm2=vec(sd[p + "post_attention_layernorm.weight"]))
        if is_moe_layer(cfg, i):
            m = cfg.ff_type.moe
            lw.router = vec(sd[p + "mlp.gate.weight"])
            if layout.expert_parallel:
                e0, e1 = _split(m.num_experts, w, r)
                i0, i1 = 0, m.intermediate_dim
            else:
                e0, e1 = 0, m.num_experts
                i0, i1 = _split(m.intermediate_dim, w, r)
            gu, dn = [], []
            for e in range(e0, e1):
                qn = p + f"mlp.experts.{e}."
                gu.append(torch.cat([sd[qn + "gate_proj.weight"][i0:i1],
                                     sd[qn + "up_proj.weight"][i0:i1]], 0))
                dn.append(sd[qn + "down_proj.weight"][:, i0:i1])
            lw.experts_gate_up = lin(torch.stack(gu, 0))
            lw.experts_down = lin(torch.stack(dn, 0).contiguous())
            lw.expert_base = e0
            if m.num_shared_experts:
                si = m.shared_intermediate_dim * m.num_shared_experts
                s0, s1 = _split(si, w, r)
                lw.shared_gate_up = lin(torch.cat([sd[p + "mlp.shared_expert.gate_proj.weight"][s0:s1],
                                                   sd[p + "mlp.shared_expert.up_proj.weight"][s0:s1]], 0))
                lw.shared_down = lin(sd[p + "mlp.shared_expert.down_proj.weight"][:, s0:s1].contiguous())
        else:
            inter = sd[p + "mlp.gate_proj.weight"].shape[0]
            i0, i1 = _split(inter, w, r)
            lw.w_gate_up = lin(torch.cat([sd[p + "mlp.gate_proj.weight"][i0:i1],
                                          sd[p + "mlp.up_proj.weight"][i0:i1]], 0))
            lw.w_down = lin(sd[p + "mlp.down_proj.weight"][:, i0:i1].contiguous())
        return lw

    if piped:
        from ..parallel.pipeline import LayerPipeline, PipelineConfig
        pipe = LayerPipeline(PipelineConfig(num_layers=cfg.num_layers), device=final_device)
        layers = pipe.run(host_layer, ship_layer)
    else:
        layers = [host_layer(i) for i in range(cfg.num_layers)]
    head = sd["model.embed_tokens.weight"] if cfg.tie_embeddings else sd["lm_head.weight"]
    v0, v1 = _split(cfg.vocab_size, w, r) if (shard_lm_head and w > 1) else (0, cfg.vocab_size)
    fin = ship if piped else (lambda t: t)
    out = ModelWeights(cfg=cfg, layout=layout, embed=fin(vec(sd["model.embed_tokens.weight"])),
                       layers=layers, final_norm=fin(vec(sd["model.norm.weight"])),
                       lm_head=fin(lin(head[v0:v1].contiguous())), vocab_base=v0)
    if piped:
        torch.cuda.synchronize(final_device)
    return out


def random_on_device(cfg: TransformerConfig, device, quant: Optional[str] = None,
                     layout: Optional[ParallelLayout] = None, seed: int = 0, std: float = 0.02,
                     shard_lm_head: bool = True) -> ModelWeights:
    """Random-init weights created shard-by-shard directly on ``device`` (no host copy), for models
    too large to stage on the host. Shapes are exactly those of ``from_state_dict``."""
    layout = layout or ParallelLayout()
    hq, _, hkv, _ = layout.heads(cfg)
    hd, d = cfg.head_dim, cfg.hidden_size
    w, r = layout.world, layout.rank
    g = torch.Generator(device=device).manual_seed(seed * 1000 + r)
    g_rep = torch.Generator(device=device).manual_seed(seed * 1000 + 499)  # replicated tensors

    def lin(n, k, experts=0):
        return LinearWeight.random(n, k, quant, device, experts=experts, std=std, generator=g)

    def norm():
        return (torch.ones(d, device=device) + torch.randn(d, device=device, generator=g_rep) * std
                ).to(torch.bfloat16)

    layers = []
    for i in range(cfg.num_layers):
        lw = LayerWeights(norm1=norm(), wqkv=lin((hq + 2 * hkv) * hd, d), wo=lin(d, hq * hd),
                          norm2=norm())
        if is_moe_layer(cfg, i):
            m = cfg.ff_type.moe
            # router weights are identical on every rank (same generator seed, rank-independent)
            gr = torch.Generator(device=device).manual_seed(seed * 1000 + 977 + i)
            lw.router = (torch.randn(m.num_experts, d, device=device, generator=gr) * 0.05
                         ).to(torch.bfloat16)
            if layout.expert_parallel:
                e_local, i_local = m.num_experts // w, m.intermediate_dim
                lw.expert_base = r * e_local
            else:
                e_local, i_local = m.num_experts, m.intermediate_dim // w
            lw.experts_gate_up = lin(2 * i_local, d, experts=e_local)
            lw.experts_down = lin(d, i_local, experts=e_local)
            if m.num_shared_experts:
                si = m.shared_intermediate_dim * m.num_shared_experts // w
                lw.shared_gate_up = lin(2 * si, d)
                lw.shared_down = lin(d, si)
        else:
            inter = (cfg.dense_intermediate_dim if cfg.ff_type.kind == "moe"
                     else cfg.ff_type.intermediate_dim) // w
            lw.w_gate_up = lin(2 * inter, d)
            lw.w_down = lin(d, inter)
        layers.append(lw)
    ge = torch.Generator(device=device).manual_seed(seed * 1000 + 991)
    embed = torch.empty(cfg.vocab_size, d, dtype=torch.bfloat16, device=device)
    embed.normal_(0.0, std, generator=ge)
    v_local = cfg.vocab_size // w if (shard_lm_head and w > 1) else cfg.vocab_size
    return ModelWeights(cfg=cfg, layout=layout, embed=embed, layers=layers, final_norm=norm(),
                        lm_head=lin(v_local, d),
                        vocab_base=r * v_local if (shard_lm_head and w > 1) else 0)
