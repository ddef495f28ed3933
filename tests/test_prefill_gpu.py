"""Prompt-phase kernels: paged causal flash attention against a plain fp32 softmax(QK^T)V, and the
native prefill forward against the fp32 library-kernel forward on the same weights (the shape of the
reference's prefill parity tests, crates/rmlx-nn/tests/prefill_cb_comparison.rs)."""
import math

import pytest
import torch

from rmlx_b200.config import FeedForwardType, MoeConfig, TransformerConfig
from rmlx_b200.models.prefill import enable_native_prefill
from rmlx_b200.models.transformer import TransformerModel
from rmlx_b200.models.weights import from_state_dict, random_state_dict
from rmlx_b200.ops.attention import flash_prefill_paged, prefill_kernel_choice
from rmlx_b200.ops.gemm import GemmStatus
from rmlx_b200.reference import ops as ref

from test_decode_engine_gpu import _oracle_from

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("kernel", ["tc", "mma"])
@pytest.mark.parametrize("hd", [64, 128])
@pytest.mark.parametrize("t,pos0,window", [(200, 0, 0), (64, 0, 0), (77, 37, 0), (300, 19, 50), (1, 130, 0),
                                           (640, 100, 0), (1500, 0, 0), (1500, 0, 200), (640, 100, 64),
                                           (700, 333, 129)])
def test_flash_prefill_matches_reference(dev, hd, t, pos0, window, kernel, monkeypatch):
    """Both kernels against fp32 softmax(QK^T)V: the tcgen05 one covers head_dim 128 (several
    key steps, partial pages, a tile that starts off the diagonal, sliding windows shorter and
    longer than a step, rows whose first steps are entirely outside their window), the mma.sync
    one everything else and, forced, the same shapes."""
    monkeypatch.setenv("RMLX_FLASH_PREFILL", kernel)
    expect = "tc" if (kernel == "tc" and hd == 128) else "mma"
    assert prefill_kernel_choice(hd, window) == expect
    if kernel == "tc" and expect == "mma":
        pytest.skip("shape not covered by the tcgen05 kernel; the mma.sync case runs it")
    torch.manual_seed(0)
    hq, hkv = 8, 2
    total = pos0 + t
    nblk = (total + 15) // 16
    kc = torch.zeros(nblk + 3, hkv, 16, hd, device=dev, dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    perm = (torch.randperm(nblk) + 1).to(torch.int32)             # pages out of order, block 0 unused
    k = torch.randn(total, hkv, hd, device=dev).to(torch.bfloat16)
    v = torch.randn(total, hkv, hd, device=dev).to(torch.bfloat16)
    tok = torch.arange(total, device=dev)
    kc[perm.to(dev)[tok // 16].long(), :, tok % 16] = k
    vc[perm.to(dev)[tok // 16].long(), :, tok % 16] = v
    q = torch.randn(t, hq, hd, device=dev).to(torch.bfloat16)
    got = flash_prefill_paged(q, kc, vc, perm.to(dev), pos0, window=window).float()
    GemmStatus.check(dev)
    want = ref.sdpa(q.float(), k.float(), v.float(), 1.0 / math.sqrt(hd), pos0, window)
    assert torch.isfinite(got).all()
    assert (got - want).abs().max().item() < 2e-2


@pytest.mark.parametrize("t,pos0", [(300, 19), (640, 100), (140, 10), (1500, 0), (100, 0)])
def test_flash_prefill_tc_two_query_tiles_per_cta(dev, t, pos0, monkeypatch):
    """The two-lane form of the tcgen05 kernel (256 query rows per CTA, K/V tiles shared by the
    lanes): lanes with different step counts, an idle second lane, pages only the second lane sees."""
    monkeypatch.setenv("RMLX_FLASH_PREFILL", "tc")
    monkeypatch.setenv("RMLX_FLASH_PREFILL_LANES", "2")
    torch.manual_seed(2)
    hq, hkv, hd = 8, 2, 128
    total = pos0 + t
    nblk = (total + 15) // 16
    kc = torch.zeros(nblk + 2, hkv, 16, hd, device=dev, dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    perm = (torch.randperm(nblk) + 1).to(torch.int32).to(dev)
    tok = torch.arange(total, device=dev)
    k = torch.randn(total, hkv, hd, device=dev).to(torch.bfloat16)
    v = torch.randn(total, hkv, hd, device=dev).to(torch.bfloat16)
    kc[perm[tok // 16].long(), :, tok % 16] = k
    vc[perm[tok // 16].long(), :, tok % 16] = v
    q = torch.randn(t, hq, hd, device=dev).to(torch.bfloat16)
    got = flash_prefill_paged(q, kc, vc, perm, pos0).float()
    GemmStatus.check(dev)
    want = ref.sdpa(q.float(), k.float(), v.float(), 1.0 / math.sqrt(hd), pos0, 0)
    assert torch.isfinite(got).all()
    assert (got - want).abs().max().item() < 2e-2


def test_flash_prefill_tc_growing_scores(dev, monkeypatch):
    """Keys whose scores grow from one 128-key step to the next force the tcgen05 kernel to move its
    reference maximum and rescale the output accumulator in tensor memory several times per row."""
    monkeypatch.setenv("RMLX_FLASH_PREFILL", "tc")
    torch.manual_seed(1)
    hq, hkv, hd, t = 4, 2, 128, 900
    nblk = (t + 15) // 16
    kc = torch.zeros(nblk + 1, hkv, 16, hd, device=dev, dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    perm = (torch.randperm(nblk) + 1).to(torch.int32).to(dev)
    tok = torch.arange(t, device=dev)
    k = (torch.randn(t, hkv, hd, device=dev) * (1 + 3 * (tok // 128))[:, None, None]).to(torch.bfloat16)
    v = torch.randn(t, hkv, hd, device=dev).to(torch.bfloat16)
    kc[perm[tok // 16].long(), :, tok % 16] = k
    vc[perm[tok // 16].long(), :, tok % 16] = v
    q = torch.randn(t, hq, hd, device=dev).to(torch.bfloat16)
    got = flash_prefill_paged(q, kc, vc, perm, 0).float()
    GemmStatus.check(dev)
    want = ref.sdpa(q.float(), k.float(), v.float(), 1.0 / math.sqrt(hd), 0, 0)
    assert torch.isfinite(got).all()
    assert (got - want).abs().max().item() < 3e-2


def _moe_cfg():
    moe = MoeConfig(num_experts=8, num_experts_per_token=2, hidden_dim=512, intermediate_dim=512)
    return TransformerConfig(hidden_size=512, num_heads=4, num_kv_heads=2, head_dim=128, num_layers=2,
                             vocab_size=1024, max_seq_len=512, rope_theta=1e6,
                             ff_type=FeedForwardType.moe_(moe), name="tiny-moe-512").validate()


def _dense_cfg():
    return TransformerConfig(hidden_size=512, num_heads=8, num_kv_heads=2, head_dim=64, num_layers=2,
                             vocab_size=1024, max_seq_len=512, rope_theta=1e4,
                             ff_type=FeedForwardType.gated(1024), name="tiny-dense-512").validate()


@pytest.mark.parametrize("cfg_fn", [_dense_cfg, _moe_cfg])
@pytest.mark.parametrize("quant", [None, "q4"])
def test_native_prefill_matches_oracle(dev, cfg_fn, quant):
    cfg = cfg_fn()
    model = TransformerModel(from_state_dict(cfg, random_state_dict(cfg, 0), device=dev, quant=quant))
    assert enable_native_prefill(model, chunk=96)         # two chunks: exercises pos0 > 0
    oracle = _oracle_from(model)
    g = torch.Generator().manual_seed(1)
    prompt = torch.randint(0, cfg.vocab_size, (150,), generator=g)
    oc = oracle.new_cache(16, max_seqs=1)
    oc.add_sequence(0)
    want = oracle.forward(prompt, oc, [0], last_only=True)
    cache = model.new_cache(16, max_seqs=1)
    cache.add_sequence(0)
    got = model.prefill(prompt.to(dev), cache, 0).float().cpu()
    assert cache.seq_len(0) == 150
    rel = (got - want).abs().max().item() / want.abs().max().item()
    assert rel < 4e-2, rel
    # the KV pages the native path wrote are what the oracle cached
    kk = cache.get_keys(1, 0).float().cpu()
    assert (kk - oc.get_keys(1, 0)).abs().max().item() < 0.2
    # and decode continues from them
    from rmlx_b200.models.decode_engine import CachedDecode
    eng = CachedDecode(model, cache, max_batch=1, use_graph=False)
    tok = int(got[0].argmax())
    eng.bind([0], [tok])
    out = eng.generate(3)
    # the oracle, fed the same tokens, agrees on the first generated token's logits ranking
    lg = oracle.forward(torch.tensor([tok]), oc, [0], last_only=True)
    top5 = lg[0].topk(5).indices.tolist()
    assert int(out[0, 0]) in top5


def test_native_prefill_all_positions_and_speculative_verify(dev):
    """Every position's logits from the tensor-core forward (what speculative verification
    reads), and the draft-and-verify runner on that path reproduces the target's greedy output."""
    from rmlx_b200.serve.speculative import SpeculativeDecoder
    cfg = _dense_cfg()      # no router: a near-tie between experts would move single positions
    model = TransformerModel(from_state_dict(cfg, random_state_dict(cfg, 0), device=dev, quant=None))
    assert enable_native_prefill(model, chunk=64)
    oracle = _oracle_from(model)
    prompt = torch.randint(0, cfg.vocab_size, (70,), generator=torch.Generator().manual_seed(4))
    oc = oracle.new_cache(8, max_seqs=1)
    oc.add_sequence(0)
    want = oracle.forward(prompt, oc, [0])
    cache = model.new_cache(8, max_seqs=1)
    cache.add_sequence(0)
    got = model.prefill(prompt.to(dev), cache, 0, all_logits=True).float().cpu()
    assert got.shape == want.shape == (70, cfg.vocab_size)
    assert (got - want).abs().max().item() / want.abs().max().item() < 4e-2
    rel_fro = ((got - want).norm() / want.norm()).item()
    assert rel_fro < 2e-2, rel_fro
    # a draft equal to the target: every proposal is accepted, output = the target's greedy tokens
    dec = SpeculativeDecoder(model, model, k=3)
    out = dec.generate(prompt[:20].tolist(), 8)
    c2 = model.new_cache(8, max_seqs=1)
    c2.add_sequence(0)
    lg = model.prefill(prompt[:20].to(dev), c2, 0)
    ref_toks = []
    for _ in range(8):
        tok = int(lg[0].argmax())
        ref_toks.append(tok)
        lg = model.prefill(torch.tensor([tok], device=dev), c2, 0)
    assert out == ref_toks
    assert dec.stats.accepted == dec.stats.proposed


@pytest.mark.parametrize("cfg_fn", [_dense_cfg, _moe_cfg])
@pytest.mark.parametrize("use_graph", [False, True])
def test_batched_decode_matches_oracle(dev, cfg_fn, use_graph):
    """Six sequences of different lengths (more rows than the mat-vec kernels take) decode three
    steps through the tensor-core path; tokens and logits follow the fp32 forward."""
    from rmlx_b200.models.prefill import BatchedDecode
    cfg = cfg_fn()
    model = TransformerModel(from_state_dict(cfg, random_state_dict(cfg, 0), device=dev, quant="q4"))
    assert enable_native_prefill(model)
    oracle = _oracle_from(model)
    g = torch.Generator().manual_seed(3)
    lens = [5, 17, 32, 9, 40, 3]
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g) for n in lens]
    cache = model.new_cache(40, max_seqs=8)
    oc = oracle.new_cache(40, max_seqs=8)
    last = []
    for s, p in enumerate(prompts):
        cache.add_sequence(s)
        oc.add_sequence(s)
        lg = model.prefill(p.to(dev), cache, s)
        oracle.forward(p, oc, [s], last_only=True)
        last.append(int(lg[0].argmax()))
    eng = BatchedDecode(model, cache, max_batch=8, use_graph=use_graph)
    eng.bind(list(range(6)), last)
    toks = eng.generate(3)
    assert toks.shape == (6, 3)
    got = eng.logits[:6].float().cpu()
    # oracle: feed the engine's own tokens, compare the logits of the last step
    feed = [last] + [toks[:, i].tolist() for i in range(2)]
    for step_tokens in feed:
        want = torch.cat([oracle.forward(torch.tensor([step_tokens[s]]), oc, [s], last_only=True)
                          for s in range(6)])
    rel = (got - want).abs().max().item() / want.abs().max().item()
    assert rel < 5e-2, rel
    assert all(cache.seq_len(s) == lens[s] + 3 for s in range(6))


def test_serving_engine_large_batch_uses_tensor_core_decode(dev):
    """Six requests with max_batch 16 (beyond the 8 rows the mat-vec engine takes): prompts go
    through the native prefill, decode through the batched tensor-core step; first tokens match the
    oracle. With max_batch 8 the mat-vec engine is chosen."""
    from rmlx_b200.config import SchedulerConfig
    from rmlx_b200.models.prefill import BatchedDecode
    from rmlx_b200.serve.engine import ServingEngine
    cfg = _moe_cfg()
    model = TransformerModel(from_state_dict(cfg, random_state_dict(cfg, 0), device=dev, quant="q4"))
    oracle = _oracle_from(model)
    from rmlx_b200.models.decode_engine import CachedDecode
    small = ServingEngine(model, num_blocks=32, scheduler_cfg=SchedulerConfig(max_batch_size=8, max_prefill_chunk=64))
    assert isinstance(small._engine, CachedDecode)
    eng = ServingEngine(model, num_blocks=160, scheduler_cfg=SchedulerConfig(max_batch_size=16, max_prefill_chunk=64))
    assert isinstance(eng._engine, BatchedDecode)
    g = torch.Generator().manual_seed(11)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (12, 30, 7, 21, 16, 9)]
    ids = [eng.submit(p, 4) for p in prompts]
    out = eng.run_until_done()
    for sid, p in zip(ids, prompts):
        assert len(out[sid]) == 4
        want = oracle.generate_greedy(torch.tensor(p), 1)
        assert out[sid][0] == want[0]


@pytest.mark.parametrize("max_batch", [2, 8])
def test_serving_engine_samples_through_the_device_engines(dev, max_batch):
    """A sampler that is not greedy (temperature > 0) but can only pick the most likely token
    (top_k = 1) must reproduce the greedy run: the step's logits are read back, the sampled token
    replaces the arg-max the step fed to itself. 2 rows: mat-vec engine; 8 rows: tensor-core engine."""
    from rmlx_b200.config import SamplerConfig, SchedulerConfig
    from rmlx_b200.serve.engine import ServingEngine
    cfg = _moe_cfg()
    model = TransformerModel(from_state_dict(cfg, random_state_dict(cfg, 0), device=dev, quant="q4"))
    g = torch.Generator().manual_seed(12)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (12, 30, 7)]
    outs = []
    for scfg in (SamplerConfig(), SamplerConfig(temperature=0.7, top_k=1, seed=0)):
        eng = ServingEngine(model, num_blocks=64, sampler_cfg=scfg,
                            scheduler_cfg=SchedulerConfig(max_batch_size=max_batch, max_prefill_chunk=64))
        assert eng._engine is not None and eng.greedy == (scfg.temperature == 0.0)
        ids = [eng.submit(p, 5) for p in prompts]
        res = eng.run_until_done()
        outs.append([res[i] for i in ids])
        GemmStatus.check(dev)
    assert outs[0] == outs[1]


def test_serving_engine_warm_up_and_logit_monitor_on_device(dev):
    """``warm_up`` captures every batch bucket with throw-away requests and leaves pages, outputs
    and counters as they were; the requests served afterwards match an engine that was not warmed
    up, and the logit monitor reads the device engine's logits without a verdict."""
    from rmlx_b200.config import SchedulerConfig
    from rmlx_b200.serve.engine import ServingEngine
    from rmlx_b200.utils.precision_guard import PrecisionGuard
    cfg = _moe_cfg()
    model = TransformerModel(from_state_dict(cfg, random_state_dict(cfg, 0), device=dev, quant="q4"))
    g = torch.Generator().manual_seed(13)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (12, 30, 7)]
    scfg = SchedulerConfig(max_batch_size=4, max_prefill_chunk=64)
    cold = ServingEngine(model, num_blocks=64, scheduler_cfg=scfg)
    ids = [cold.submit(p, 6) for p in prompts]
    want = cold.run_until_done()
    eng = ServingEngine(model, num_blocks=64, scheduler_cfg=scfg, precision_guard=PrecisionGuard(), guard_every=2)
    free = eng.cache.manager.num_free_blocks()
    res = eng.warm_up()
    assert res.ran and len(eng._engine.graphs) == len(eng._engine.buckets)      # one graph per bucket
    assert eng.outputs == {} and eng.cache.manager.num_free_blocks() == free and eng.guard.checks == 0
    assert not eng.warm_up().ran
    ids2 = [eng.submit(p, 6) for p in prompts]
    got = eng.run_until_done()
    # (the warmed-up engine's rows were bound to other sequences before: an idle row whose block
    # table still named one of their pages would write into a page that a live sequence owns now)
    assert [got[i] for i in ids2] == [want[i] for i in ids]
    assert int(eng._engine.block_table[len(eng._engine.seq_ids):].abs().sum()) == 0
    assert eng.guard.checks >= 3 and eng.guard_fallbacks == 0 and eng.guard.nan_events == 0
    GemmStatus.check(dev)
