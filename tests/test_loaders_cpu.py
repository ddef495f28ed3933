"""Checkpoint loaders: MLX-style quantised safetensors (triplets, shards, config.json) and GGUF
(the cases of crates/rmlx-nn/src/safetensors_loader.rs tests and crates/rmlx-core/src/formats/gguf.rs)."""
import numpy as np
import torch

from rmlx_b200.config import FeedForwardType, MoeConfig, QuantConfig, TransformerConfig
from rmlx_b200.loader import gguf
from rmlx_b200.loader.safetensors_loader import (build_weights, detect_triplets, hf_name_to_internal,
                                                 load_model, load_tensors, read_config, save_checkpoint)
from rmlx_b200.models.transformer import TransformerModel
from rmlx_b200.models.weights import ParallelLayout, from_state_dict, random_state_dict
from rmlx_b200.ops.weights import W_Q4
from rmlx_b200.reference import ops as ref


def _cfg():
    moe = MoeConfig(num_experts=4, num_experts_per_token=2, hidden_dim=128, intermediate_dim=128)
    return TransformerConfig(hidden_size=128, num_heads=4, num_kv_heads=2, head_dim=32, num_layers=2,
                             vocab_size=256, max_seq_len=64, ff_type=FeedForwardType.moe_(moe)).validate()


def test_name_mapping():
    assert hf_name_to_internal("model.layers.0.self_attn.q_proj.weight") == "layers.0.attention.q_proj.weight"
    assert hf_name_to_internal("model.layers.3.mlp.down_proj.weight") == "layers.3.feed_forward.down_proj.weight"
    assert hf_name_to_internal("model.embed_tokens.weight") == "embedding.weight"
    assert gguf.gguf_name_to_hf("blk.2.attn_q.weight") == "model.layers.2.self_attn.q_proj.weight"
    assert gguf.gguf_name_to_hf("blk.0.ffn_gate_inp.weight") == "model.layers.0.mlp.gate.weight"


def test_quantised_sharded_checkpoint_roundtrip(tmp_path):
    cfg = _cfg()
    sd = random_state_dict(cfg, 0)
    d = str(tmp_path / "ckpt")
    save_checkpoint(d, cfg, sd, QuantConfig(4, 64), shards=3)
    cfg2, q = read_config(d)
    assert q.bits == 4 and q.group_size == 64 and cfg2.num_layers == 2 and cfg2.ff_type.kind == "moe"
    tensors = load_tensors(d)
    trip = detect_triplets(tensors)
    assert "model.layers.0.self_attn.q_proj" in trip and "model.layers.1.mlp.experts.3.down_proj" in trip
    assert "model.layers.0.mlp.gate" not in trip          # router stays dense
    w, _ = load_model(d, dtype=torch.float32)
    want = from_state_dict(cfg, sd, dtype=torch.float32, quant="q4")
    assert w.layers[0].wqkv.kind == W_Q4
    assert torch.equal(w.layers[0].wqkv.w, want.layers[0].wqkv.w)
    assert torch.equal(w.layers[1].experts_down.w, want.layers[1].experts_down.w)
    assert torch.equal(w.layers[1].experts_gate_up.scales, want.layers[1].experts_gate_up.scales)
    # tensor-parallel shard cut from the packed form == shard of the dense weights, quantised
    w1 = build_weights(cfg2, tensors, q, dtype=torch.float32, layout=ParallelLayout(1, 2))
    want1 = from_state_dict(cfg, sd, dtype=torch.float32, quant="q4", layout=ParallelLayout(1, 2))
    assert torch.equal(w1.layers[0].wo.w, want1.layers[0].wo.w)
    assert torch.equal(w1.layers[0].experts_down.w, want1.layers[0].experts_down.w)
    assert torch.equal(w1.lm_head.w, want1.lm_head.w) and w1.vocab_base == 128
    # and the loaded model runs
    m = TransformerModel(w)
    lg = m.forward(torch.arange(8))
    assert lg.shape == (8, 256) and torch.isfinite(lg).all()


def test_dense_checkpoint_single_file(tmp_path):
    cfg = _cfg()
    sd = random_state_dict(cfg, 1)
    d = str(tmp_path / "dense")
    save_checkpoint(d, cfg, sd)
    w, cfg2 = load_model(d, dtype=torch.float32)
    a = TransformerModel(w).forward(torch.arange(6))
    sd_bf = {k: v.to(torch.bfloat16).float() for k, v in sd.items()}
    b = TransformerModel(from_state_dict(cfg, sd_bf, dtype=torch.float32)).forward(torch.arange(6))
    assert torch.allclose(a, b, atol=1e-5)


def test_gguf_roundtrip_and_block_formats(tmp_path):
    rng = np.random.default_rng(0)
    a = rng.standard_normal((8, 64)).astype(np.float32)
    b = rng.standard_normal((4, 32)).astype(np.float32)
    p = str(tmp_path / "t.gguf")
    gguf.write_gguf(p, {"general.architecture": "llama", "llama.block_count": 2, "x.f": 1.5},
                    {"blk.0.attn_q.weight": (a, "Q8_0"), "blk.0.attn_k.weight": (b, "F16"),
                     "token_embd.weight": (a, "Q4_0"), "output_norm.weight": (b[0], "F32")})
    g = gguf.read_gguf(p)
    assert g.version == 3 and g.metadata["general.architecture"] == "llama"
    assert g.metadata["llama.block_count"] == 2 and abs(g.metadata["x.f"] - 1.5) < 1e-6
    assert g.tensors["blk.0.attn_q.weight"].shape == (8, 64)
    assert g.tensors["blk.0.attn_q.weight"].type_name == "Q8_0"
    assert np.abs(g.tensor_f32("blk.0.attn_q.weight") - a).max() < 0.03
    assert np.abs(g.tensor_f32("blk.0.attn_k.weight") - b).max() < 2e-3
    assert np.abs(g.tensor_f32("token_embd.weight") - a).max() < 0.5
    assert np.array_equal(g.tensor_f32("output_norm.weight"), b[0])
    sd, meta = gguf.load_state_dict(p)
    assert set(sd) == {"model.layers.0.self_attn.q_proj.weight", "model.layers.0.self_attn.k_proj.weight",
                       "model.embed_tokens.weight", "model.norm.weight"}


def test_gguf_k_quants_against_scalar_reference():
    rng = np.random.default_rng(1)
    # Q4_K: build one block by hand and check a few elements with the scalar formula
    blk = rng.integers(0, 256, 144, dtype=np.uint8)
    blk[0:2] = np.array([0.5], np.float16).view(np.uint8)
    blk[2:4] = np.array([0.25], np.float16).view(np.uint8)
    out = gguf.dequantize(blk, 12)
    sc = blk[4:16]

    def scale_min(j):
        if j < 4:
            return sc[j] & 63, sc[j + 4] & 63
        return (sc[j + 4] & 0xF) | ((sc[j - 4] >> 6) << 4), (sc[j + 4] >> 4) | ((sc[j] >> 6) << 4)

    qs = blk[16:]
    for j in range(4):
        s0, m0 = scale_min(2 * j)
        s1, m1 = scale_min(2 * j + 1)
        for l in (0, 7, 31):
            assert abs(out[64 * j + l] - (0.5 * s0 * (qs[32 * j + l] & 0xF) - 0.25 * m0)) < 1e-4
            assert abs(out[64 * j + 32 + l] - (0.5 * s1 * (qs[32 * j + l] >> 4) - 0.25 * m1)) < 1e-4
    # Q6_K
    blk = rng.integers(0, 256, 210, dtype=np.uint8)
    blk[208:210] = np.array([0.125], np.float16).view(np.uint8)
    out = gguf.dequantize(blk, 14)
    ql, qh, s8 = blk[:128], blk[128:192], blk[192:208].view(np.int8)
    l = 5
    q1 = int((ql[l] & 0xF) | ((qh[l] & 3) << 4)) - 32
    assert abs(out[l] - 0.125 * s8[0] * q1) < 1e-4
    q4 = int((ql[64 + l + 32] >> 4) | (((qh[32 + l] >> 6) & 3) << 4)) - 32
    assert abs(out[128 + 96 + l] - 0.125 * s8[8 + 6] * q4) < 1e-4


def test_affine_quantisation_oracle():
    w = torch.randn(16, 128) * 0.02
    p, s, b = ref.quantize_affine(w)
    assert p.shape == (16, 16) and s.shape == (16, 2) and p.dtype == torch.int32
    d = ref.dequantize_affine(p, s, b)
    assert (d - w).abs().max() <= s.float().max() * 0.51 + 1e-3
    # element i of a word sits at bit 4*i
    word = int(p[0, 0]) & 0xFFFFFFFF
    q0 = round(float((w[0, 0] - b[0, 0].float()) / s[0, 0].float()))
    assert (word & 0xF) == max(0, min(15, q0))


def test_q8_triplets_and_fp16_scales_keep_checkpoint_precision(tmp_path):
    """An 8-bit group-64 checkpoint loads as the 8-bit weight kind (bits inferred from the shapes),
    and fp16 scales / biases stay fp16: the dequantised weights equal the fp32 dequantisation of the
    stored triplet exactly, which a cast to bf16 would not give."""
    import torch
    from safetensors.torch import save_file
    from rmlx_b200.config import QuantConfig
    from rmlx_b200.loader.safetensors_loader import _Source
    from rmlx_b200.ops.weights import W_Q4, W_Q8
    from rmlx_b200.reference import ops as ref
    torch.manual_seed(0)
    w = torch.randn(32, 128) * 0.05
    tensors = {}
    for name, bits in (("a", 4), ("b", 8)):
        p, s, b = ref.quantize_affine(w, bits, 64)
        # an MLX checkpoint in half precision: scales and biases are fp16 with full fp16 mantissas
        s16 = (s.float() * 1.0009765625).to(torch.float16)
        b16 = (b.float() * 1.0009765625).to(torch.float16)
        tensors[f"{name}.weight"], tensors[f"{name}.scales"], tensors[f"{name}.biases"] = p, s16, b16
    src = _Source(tensors, QuantConfig(4, 64), torch.bfloat16)
    la, lb = src.linear("a"), src.linear("b")
    assert la.kind == W_Q4 and lb.kind == W_Q8 and la.k == 128 and lb.k == 128
    for lw, name, bits in ((la, "a", 4), (lb, "b", 8)):
        assert lw.scales.dtype == torch.float16 and lw.scales_f16 and lw.kernel_kind == lw.kind | 0x100
        want = ref.dequantize_affine(tensors[f"{name}.weight"], tensors[f"{name}.scales"].float(),
                                     tensors[f"{name}.biases"].float(), bits, 64)
        assert torch.equal(lw.dequantized(), want)
        lossy = ref.dequantize_affine(tensors[f"{name}.weight"], tensors[f"{name}.scales"].to(torch.bfloat16),
                                      tensors[f"{name}.biases"].to(torch.bfloat16), bits, 64)
        assert not torch.equal(lossy, want)          # what the cast to bf16 used to lose
    # 8-bit quantisation is ~16x finer than 4-bit
    e4 = (la.dequantized() - w).abs().max().item()
    e8 = (lb.dequantized() - w).abs().max().item()
    assert e8 < e4 / 8
    # column shards re-slice the packed words of either width
    assert lb.cols(64, 128).k == 64 and torch.equal(lb.cols(64, 128).dequantized(), lb.dequantized()[:, 64:])
