"""nn layers and model presets on CPU (the shape of crates/rmlx-nn/tests/nn_tests.rs): linears and
their quantised imports, tensor-parallel linears, the KV cache family, sliding windows, latent
attention, LoRA with a numerical-gradient check, model presets."""
import pytest
import torch

from rmlx_b200.config import AttentionConfig
from rmlx_b200.models import deepseek, mixtral, qwen
from rmlx_b200.models.transformer import TransformerModel
from rmlx_b200.models.weights import from_state_dict, random_state_dict
from rmlx_b200.nn import layers as L
from rmlx_b200.nn.attention import (Attention, BatchKvCache, LayerKvCache, QuantizedKvCache,
                                    RotatingKvCache, sliding_window_mask)
from rmlx_b200.nn.lora import LoraConfig, LoraLayer, LoraModel, LoraTrainer, numerical_gradient
from rmlx_b200.nn.mla import MlaAttention, MlaKvCache, random_mla_weights
from rmlx_b200.nn.parallel import shard_column, shard_column_segments, shard_row
from rmlx_b200.ops.weights import LinearWeight


def test_linear_and_quantised_imports():
    torch.manual_seed(0)
    w = torch.randn(24, 128) * 0.05
    x = torch.randn(3, 128)
    lin = L.Linear(LinearWeight.from_dense(w, None, torch.float32), bias=torch.ones(24))
    assert torch.allclose(lin(x), x @ w.t() + 1, atol=1e-5)
    q = L.QuantizedLinear.from_dense(w)
    assert (q(x) - x @ w.t()).abs().max() < 0.3
    # AWQ layout round trip: pack a known integer matrix
    n_in, n_out, g = 128, 16, 64
    qv = torch.randint(0, 16, (n_in, n_out))
    zv = torch.randint(0, 16, (n_in // g, n_out))
    sc = torch.rand(n_in // g, n_out) * 0.1 + 0.01
    order = [0, 4, 1, 5, 2, 6, 3, 7]

    def pack_awq(m):   # [rows, cols] -> int32 [rows, cols/8]; logical column j sits in nibble order[j]
        m = m.view(m.shape[0], -1, 8)
        out = torch.zeros(m.shape[0], m.shape[1], dtype=torch.int64)
        for j in range(8):
            out |= m[:, :, j].to(torch.int64) << (4 * order[j])
        return torch.where(out >= 2 ** 31, out - 2 ** 32, out).to(torch.int32)

    wq = L.awq_dequantize(pack_awq(qv), pack_awq(zv), sc, g)
    want = ((qv - zv.repeat_interleave(g, 0)).float() * sc.repeat_interleave(g, 0)).t()
    assert torch.allclose(wq, want, atol=1e-6)
    # GPTQ layout: qweight [in/8, out], zeros stored minus one, g_idx permutes groups
    def pack_rows(m):   # [in, out] -> [in/8, out]
        m = m.view(-1, 8, m.shape[1])
        out = torch.zeros(m.shape[0], m.shape[2], dtype=torch.int64)
        for j in range(8):
            out |= m[:, j, :].to(torch.int64) << (4 * j)
        return torch.where(out >= 2 ** 31, out - 2 ** 32, out).to(torch.int32)

    def pack_cols(m):   # [g, out] -> [g, out/8]
        m = m.view(m.shape[0], -1, 8)
        out = torch.zeros(m.shape[0], m.shape[1], dtype=torch.int64)
        for j in range(8):
            out |= m[:, :, j].to(torch.int64) << (4 * j)
        return torch.where(out >= 2 ** 31, out - 2 ** 32, out).to(torch.int32)

    zg = torch.randint(1, 16, (2, n_out))
    g_idx = torch.randint(0, 2, (n_in,))
    wg = L.gptq_dequantize(pack_rows(qv), pack_cols(zg - 1), sc, g_idx)
    want = ((qv - zg[g_idx]).float() * sc[g_idx]).t()
    assert torch.allclose(wg, want, atol=1e-6)
    assert L.activation("gelu_fast")(torch.tensor([1.0])).item() > 0.8
    assert len(L.ACTIVATIONS) >= 17


def test_tensor_parallel_shards_recompose():
    w = LinearWeight.from_dense(torch.randn(32, 128) * 0.05, "q4", torch.float32)
    x = torch.randn(2, 128)
    full = x @ w.dequantized().t()
    cols = torch.cat([x @ shard_column(w, r, 2).dequantized().t() for r in range(2)], -1)
    assert torch.allclose(cols, full, atol=1e-6)
    rows = sum(x[:, r * 64:(r + 1) * 64] @ shard_row(w, r, 2).dequantized().t() for r in range(2))
    assert torch.allclose(rows, full, atol=1e-5)
    seg = shard_column_segments(w, [16, 8, 8], 1, 2)            # merged Q|K|V, second rank
    want = torch.cat([w.dequantized()[8:16], w.dequantized()[20:24], w.dequantized()[28:32]])
    assert torch.equal(seg.dequantized(), want)


def test_kv_cache_family():
    k = torch.randn(10, 2, 64); v = torch.randn(10, 2, 64)
    c = LayerKvCache.preallocated(2, 64, 16, torch.float32)
    c.append(k[:6], v[:6]); c.append(k[6:], v[6:])
    assert c.seq_len == 10 and torch.equal(c.keys(), k) and torch.equal(c.values(), v)
    c.trim(3); assert c.seq_len == 7 and c.keys().shape[0] == 7
    r = RotatingKvCache(2, 64, max_size=6, keep=2, dtype=torch.float32)
    r.append(k, v)
    assert r.positions().tolist() == [0, 1, 6, 7, 8, 9]
    assert torch.equal(r.keys(), k[[0, 1, 6, 7, 8, 9]])
    b = BatchKvCache(lambda: LayerKvCache(2, 64, 16, torch.float32)); b.extend(3)
    b[1].append(k[:4], v[:4]); assert b.offsets() == [0, 4, 0]
    b.filter([1]); assert len(b) == 1 and b.offsets() == [4]
    for bits, tol in ((8, 0.02), (4, 0.3)):
        q = QuantizedKvCache(2, 64, 16, bits=bits)
        q.append(k, v)
        assert (q.keys() - k).abs().max() < tol * k.abs().max()
    assert QuantizedKvCache(2, 64, 16, bits=4).nbytes_per_token() < 2 * 2 * 64 * 2 / 2.5
    m = sliding_window_mask(3, 6, window=2, offset=3)
    assert (m == 0).nonzero().tolist() == [[0, 2], [0, 3], [1, 3], [1, 4], [2, 4], [2, 5]]


def test_attention_cached_equals_full_and_window():
    torch.manual_seed(1)
    cfg = AttentionConfig(4, 2, 32, 64, 1e4)
    wqkv = LinearWeight.from_dense(torch.randn((4 + 4) * 32, 64) * 0.1, None, torch.float32)
    wo = LinearWeight.from_dense(torch.randn(64, 128) * 0.1, None, torch.float32)
    x = torch.randn(9, 64)
    for window in (0, 4):
        att = Attention(cfg, wqkv, wo, window=window)
        full = att(x)
        c = LayerKvCache(2, 32, 16, torch.float32)
        inc = torch.cat([att(x[:5], c), att(x[5:7], c), att(x[7:], c)])
        assert torch.allclose(inc, full, atol=1e-5)
        if window:
            rc = RotatingKvCache(2, 32, max_size=4, keep=0, dtype=torch.float32)
            rot = torch.cat([att(x[i:i + 1], rc) for i in range(9)])
            assert torch.allclose(rot, full, atol=1e-5)      # the ring holds exactly the window


def test_mla_cached_equals_full_and_compression():
    cfg = deepseek.deepseek_tiny().mla()
    att = MlaAttention(cfg, random_mla_weights(cfg, 0, 0.1))
    x = torch.randn(7, cfg.hidden_size)
    full = att(x)
    c = MlaKvCache(cfg, torch.float32)
    inc = torch.cat([att(x[:4], c), att(x[4:5], c), att(x[5:], c)])
    assert torch.allclose(inc, full, atol=1e-5)
    assert c.c_kv.shape[1] == cfg.kv_lora_rank and c.seq_len == 7
    assert abs(att.compression_ratio() - 2 * 4 * 16 / (32 + 8)) < 1e-9


def test_lora_trains_and_gradients_match_numeric():
    torch.manual_seed(2)
    base = torch.randn(6, 10) * 0.1
    layer = LoraLayer(base, LoraConfig(rank=2, alpha=4.0))
    x, target = torch.randn(5, 10), torch.randn(5, 6)
    assert torch.allclose(layer(x), x @ base.t())               # B starts at zero
    tr = LoraTrainer(LoraModel({"l": layer}), lr=0.05)
    losses = [tr.train_step(lambda: layer(x), target) for _ in range(60)]
    assert losses[-1] < 0.7 * losses[0]
    assert torch.allclose(x @ layer.merged_weight().t(), layer(x), atol=1e-5)
    layer.b.grad = None
    LoraTrainer.mse_loss(layer(x), target).backward()
    b0 = layer.b.detach().clone()

    def f(b):
        return LoraTrainer.mse_loss(x @ base.t() + x @ layer.a.detach().t() @ b.t() * layer.cfg.scaling, target)
    num = numerical_gradient(f, b0)
    assert torch.allclose(layer.b.grad, num, atol=2e-3)


def test_model_presets():
    c = qwen.qwen2_7b()
    assert (c.hidden_size, c.num_heads, c.num_kv_heads, c.num_layers, c.vocab_size) == (3584, 28, 4, 28, 152064)
    m = mixtral.mixtral_8x7b()
    assert m.sliding_window == 4096 and m.ff_type.moe.num_experts == 8 and m.ff_type.moe.num_experts_per_token == 2
    d = deepseek.deepseek_v3()
    assert d.num_experts == 256 and d.kv_lora_rank == 512 and d.first_dense_layers == 1
    for cfg in (qwen.qwen2_tiny(), mixtral.mixtral_tiny()):
        model = TransformerModel(from_state_dict(cfg, random_state_dict(cfg, 0), dtype=torch.float32))
        toks = model.generate_greedy(torch.arange(12) % cfg.vocab_size, 5)
        full = model.forward(torch.cat([torch.arange(12) % cfg.vocab_size, torch.tensor(toks[:-1])]))
        assert [int(full[11 + i].argmax()) for i in range(5)] == toks
    # the architecture classes: constructors check the architecture, accessors as in the reference
    qm = qwen.Qwen2Model.from_config()
    assert qm.num_layers() == 2 and qm.config() is qm.cfg and qm.inner() is qm
    assert qm.generate_greedy(torch.arange(6), 3) == TransformerModel(qm.w).generate_greedy(torch.arange(6), 3)
    with pytest.raises(ValueError):
        qwen.Qwen2Model.from_config(mixtral.mixtral_tiny())
    mm = mixtral.MixtralModel.from_config()
    assert mm.sliding_window_size() == 8 and mm.config().num_experts == 4 and mm.layer(1) is mm.w.layers[1]
    assert mm.layer(2) is None and mm.num_layers() == 2
    full = mixtral.mixtral_8x7b_full()
    assert (full.sliding_window_size, full.num_experts, full.num_experts_per_token) == (4096, 8, 2)
    with pytest.raises(ValueError):
        mixtral.MixtralConfig(full.base, 4096, 8, 3).validate()       # disagrees with the base config
    with pytest.raises(ValueError):
        mixtral.MixtralModel.from_config(qwen.qwen2_tiny())
    ds = deepseek.DeepSeekV3Model(deepseek.deepseek_tiny(), std=0.1)
    ids = torch.arange(9) % 256
    full = ds.forward(ids)
    cache = ds.new_cache()
    inc = torch.cat([ds.forward(ids[:5], cache), ds.forward(ids[5:], cache)])
    assert full.shape == (9, 256) and torch.allclose(inc, full, atol=1e-4)


def test_mla_absorbed_decode_over_paged_latent_cache():
    """The absorbed decode step over the paged latent cache equals the reference forward with the
    contiguous cache (prompt of 20 tokens, then three single-token steps, two sequences)."""
    from rmlx_b200.config import MlaConfig
    from rmlx_b200.nn.mla import (MlaAttention, MlaKvCache, MlaPagedCache, mla_decode_paged,
                                  random_mla_weights)
    cfg = MlaConfig(hidden_size=256, num_heads=4, head_dim=32, v_head_dim=32, kv_lora_rank=128,
                    rope_head_dim=64, q_lora_rank=0, max_seq_len=128)
    attn = MlaAttention(cfg, random_mla_weights(cfg, 0, std=0.05))
    torch.manual_seed(0)
    xs = {3: torch.randn(24, 256), 9: torch.randn(12, 256)}
    prompts = {3: 20, 9: 5}
    refs = {s: MlaKvCache(cfg, dtype=torch.float32) for s in xs}
    pc = MlaPagedCache(cfg, 16, dtype=torch.float32)
    for s, x in xs.items():
        n = prompts[s]
        attn.forward(x[:n], refs[s])
        pc.add_sequence(s)
        pc.append(s, *attn.compress(x[:n], torch.arange(n)))
    for step in range(3):
        rows = torch.stack([xs[s][prompts[s] + step] for s in (3, 9)])
        want = torch.cat([attn.forward(xs[s][prompts[s] + step][None], refs[s]) for s in (3, 9)])
        got = mla_decode_paged(attn, rows, pc, [3, 9])
        assert (got - want).abs().max() < 1e-5
    assert pc.seq_len(3) == 23 and pc.seq_len(9) == 8 and pc.bytes_per_token() == (128 + 64 + 8) * 4
    ck, kr = pc.gather(9)
    assert torch.allclose(ck, refs[9].c_kv[:8]) and torch.allclose(kr, refs[9].k_rope[:8])
    pc.free_sequence(3)
    pc.add_sequence(11)                         # the slot and the pages are reusable
    pc.append(11, *attn.compress(xs[9][:3], torch.arange(3)))
    assert pc.seq_len(11) == 3


def test_sliding_window_attention_layer_and_dynamic_context():
    """The layer-level sliding-window attention: same result as the plain layer with that window,
    incremental decoding over a rotating cache of the window's size equals the full pass, config
    checks; the pre-allocated intermediates hand out views, never copies."""
    from rmlx_b200.models.prefill_plan import DynamicExecContext
    from rmlx_b200.nn.attention import SlidingWindowAttention, SlidingWindowAttentionConfig, sliding_window_mask
    from rmlx_b200.ops.weights import LinearWeight
    g = torch.Generator().manual_seed(4)
    base = AttentionConfig(num_heads=4, num_kv_heads=2, head_dim=8, max_seq_len=64)
    d = 32
    wq, wk, wv = torch.randn(32, d, generator=g) * 0.2, torch.randn(16, d, generator=g) * 0.2, torch.randn(16, d, generator=g) * 0.2
    wo = torch.randn(d, 32, generator=g) * 0.2
    cfg = SlidingWindowAttentionConfig(base, window_size=5)
    layer = SlidingWindowAttention.from_projections(cfg, wq, wk, wv, wo)
    assert layer.window_size() == 5 and layer.base_config() is base
    plain = Attention(base, LinearWeight.from_dense(torch.cat([wq, wk, wv], 0), None, dtype=torch.float32),
                      LinearWeight.from_dense(wo, None, dtype=torch.float32), window=5)
    layer.qkv, layer.o = plain.qkv, plain.o                      # same fp32 weights for an exact comparison
    x = torch.randn(12, d, generator=g)
    full = layer(x)
    assert torch.allclose(full, plain(x), atol=1e-6)
    cache = layer.new_cache()
    assert cache.max_size == 5                                   # token by token: exactly the window
    inc = torch.cat([layer(x[i:i + 1], cache) for i in range(12)])
    assert torch.allclose(inc, full, atol=1e-5)
    cache4 = layer.new_cache(chunk=4)
    assert cache4.max_size == 8                                  # chunks of up to four tokens
    inc4 = torch.cat([layer(x[:4], cache4), layer(x[4:5], cache4), layer(x[5:9], cache4), layer(x[9:], cache4)])
    assert torch.allclose(inc4, full, atol=1e-5)
    m = layer.build_sliding_window_mask(3, 6, offset=3)
    assert torch.equal(m, sliding_window_mask(3, 6, 5, 3)) and float(m[0, 3]) == 0.0 and m[2, 0] == float("-inf")
    with pytest.raises(ValueError):
        SlidingWindowAttentionConfig(base, 0).validate()

    ctx = DynamicExecContext(16, 8, dtype=torch.float32, num_intermediates=2)
    a = ctx.get_intermediate(1, 5)
    a.fill_(3.0)
    assert a.shape == (5, 8) and float(ctx.get_intermediate(1, 16)[:5].mean()) == 3.0      # a view, not a copy
    assert (ctx.max_seq_len(), ctx.hidden_dim(), ctx.num_intermediates(), ctx.allocated_bytes()) == (16, 8, 2, 2 * 16 * 8 * 4)
    for bad in ((2, 4), (0, 17)):
        with pytest.raises(ValueError):
            ctx.get_intermediate(*bad)
