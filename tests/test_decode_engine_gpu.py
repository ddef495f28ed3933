"""End-to-end: the graph-captured native decode step against the fp32 library-kernel forward on the
same (bf16-rounded or Q4-dequantised) weights — the shape of crates/rmlx-nn/tests/e2e_generate.rs
(tiny random-weight transformer, multi-step greedy decode with a KV cache)."""
import pytest
import torch

from rmlx_b200.config import FeedForwardType, MoeConfig, TransformerConfig, tiny_dense_config
from rmlx_b200.models.decode_engine import CachedDecode
from rmlx_b200.models.transformer import TransformerModel
from rmlx_b200.models.weights import from_state_dict, random_state_dict

pytestmark = pytest.mark.gpu


def tiny_moe_config():
    moe = MoeConfig(num_experts=16, num_experts_per_token=4, hidden_dim=256, intermediate_dim=128)
    return TransformerConfig(hidden_size=256, num_heads=8, num_kv_heads=2, head_dim=64, num_layers=2,
                             vocab_size=1024, max_seq_len=256, rope_theta=1e6,
                             ff_type=FeedForwardType.moe_(moe), name="tiny-moe").validate()


def _oracle_from(gpu_weights_model: TransformerModel) -> TransformerModel:
    """fp32 CPU model whose weights are exactly what the kernels see."""
    import copy
    from rmlx_b200.ops.weights import LinearWeight, W_BF16
    w = copy.copy(gpu_weights_model.w)

    def deq(lw):
        return None if lw is None else LinearWeight(W_BF16, lw.dequantized().float().cpu())

    layers = []
    for l in w.layers:
        n = copy.copy(l)
        for name in ("wqkv", "wo", "w_gate_up", "w_down", "experts_gate_up", "experts_down",
                     "shared_gate_up", "shared_down"):
            setattr(n, name, deq(getattr(l, name)))
        n.norm1, n.norm2 = l.norm1.float().cpu(), l.norm2.float().cpu()
        n.router = None if l.router is None else l.router.float().cpu()
        layers.append(n)
    w.layers = layers
    w.embed = w.embed.float().cpu()
    w.final_norm = w.final_norm.float().cpu()
    w.lm_head = deq(w.lm_head)
    return TransformerModel(w)


@pytest.mark.parametrize("cfg_fn", [tiny_dense_config, tiny_moe_config])
@pytest.mark.parametrize("quant", [None, "q4", "q8"])
@pytest.mark.parametrize("use_graph", [False, True])
def test_decode_matches_oracle(dev, cfg_fn, quant, use_graph):
    cfg = cfg_fn()
    if quant in ("q4", "q8") and cfg.ff_type.kind == "gated":
        # group-64 quantisation needs the FFN width to be a multiple of 64 (688 is not)
        cfg = cfg.replace(ff_type=FeedForwardType.gated(704))
    sd = random_state_dict(cfg, 0)
    model = TransformerModel(from_state_dict(cfg, sd, device=dev, quant=quant))
    oracle = _oracle_from(model)
    g = torch.Generator().manual_seed(0)
    prompt = torch.randint(0, cfg.vocab_size, (16,), generator=g)
    steps = 8

    # oracle: prefill + per-step logits
    oc = oracle.new_cache(8, max_seqs=1)
    oc.add_sequence(0)
    lg = oracle.forward(prompt, oc, [0], last_only=True)
    want_logits, toks = [], []
    tok = int(lg[0].argmax())
    for _ in range(steps):
        toks.append(tok)
        lg = oracle.forward(torch.tensor([tok]), oc, [0], last_only=True)
        want_logits.append(lg[0].clone())
        tok = int(lg[0].argmax())

    # native: prefill through the library path on the GPU, decode through the kernels;
    # feed the oracle's tokens so one near-tie cannot derail the comparison
    cache = model.new_cache(8, max_seqs=2)
    cache.add_sequence(0)
    model.forward(prompt.to(dev), cache, [0], last_only=True)
    eng = CachedDecode(model, cache, max_batch=2, use_graph=use_graph)
    eng.bind([0], [toks[0]])
    eng.reserve(steps + 1)
    agree = 0
    for i in range(steps):
        eng.tokens[0] = toks[i]
        eng.step()
        torch.cuda.synchronize()
        got = eng.logits[0].cpu()
        err = (got - want_logits[i]).abs().max().item()
        mag = want_logits[i].abs().max().item()
        assert err <= 5e-2 * mag + 2e-2, f"step {i}: err {err} mag {mag}"
        agree += int(got.argmax()) == int(want_logits[i].argmax())
    assert agree >= steps - 1
    assert eng.launches_per_step > 0
    assert cache.seq_len(0) == 16 + steps


def test_batched_decode_rows_independent(dev):
    cfg = tiny_moe_config()
    sd = random_state_dict(cfg, 1)
    model = TransformerModel(from_state_dict(cfg, sd, device=dev))
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g) for n in (5, 33, 16)]
    cache = model.new_cache(32, max_seqs=4)
    last = []
    for s, p in enumerate(prompts):
        cache.add_sequence(s)
        lg = model.forward(p.to(dev), cache, [s], last_only=True)
        last.append(int(lg[0].argmax()))
    eng = CachedDecode(model, cache, max_batch=3, use_graph=True, splits=2)
    eng.bind([0, 1, 2], last)
    out = eng.generate(6)
    # each row alone gives the same tokens
    for s, p in enumerate(prompts):
        c1 = model.new_cache(8, max_seqs=1)
        c1.add_sequence(0)
        lg = model.forward(p.to(dev), c1, [0], last_only=True)
        e1 = CachedDecode(model, c1, max_batch=1, use_graph=False, splits=2)
        e1.bind([0], [int(lg[0].argmax())])
        o1 = e1.generate(6)
        assert out[s].tolist() == o1[0].tolist()


def test_decode_engine_ten_rows_in_chunks(dev):
    """More rows than one mat-vec launch takes (10 > 4): every kernel runs in row chunks inside the
    same captured step; tokens follow the fp32 forward for each sequence."""
    cfg = tiny_moe_config()
    model = TransformerModel(from_state_dict(cfg, random_state_dict(cfg, 0), device=dev, quant="q4"))
    oracle = _oracle_from(model)
    g = torch.Generator().manual_seed(4)
    lens = [3, 9, 17, 5, 12, 7, 20, 4, 6, 11]
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g) for n in lens]
    cache = model.new_cache(40, max_seqs=12)
    oc = oracle.new_cache(40, max_seqs=12)
    last = []
    for s, p in enumerate(prompts):
        cache.add_sequence(s)
        oc.add_sequence(s)
        lg = model.forward(p.to(dev), cache, [s], last_only=True)
        oracle.forward(p, oc, [s], last_only=True)
        last.append(int(lg[0].argmax()))
    eng = CachedDecode(model, cache, max_batch=12, use_graph=True)
    eng.bind(list(range(10)), last)
    toks = eng.generate(2)
    assert toks.shape == (10, 2)
    got = eng.logits[:10].float().cpu()
    for feed in (last, toks[:, 0].tolist()):
        want = torch.cat([oracle.forward(torch.tensor([feed[s]]), oc, [s], last_only=True) for s in range(10)])
    rel = (got - want).abs().max().item() / want.abs().max().item()
    assert rel < 5e-2, rel


@pytest.mark.parametrize("quant", [None, "q4", "q8"])
@pytest.mark.parametrize("use_graph", [False, True])
@pytest.mark.parametrize("ctx", [16, 150])
def test_step_kernel_matches_oracle(dev, quant, use_graph, ctx):
    """The persistent one-kernel decode step (batch 1, routed-expert layers) against the fp32
    oracle on the same weights, and against the chain-of-kernels engine."""
    from rmlx_b200.models.step_kernel import DecodeStepKernel
    cfg = tiny_moe_config()
    model = TransformerModel(from_state_dict(cfg, random_state_dict(cfg, 2), device=dev, quant=quant))
    oracle = _oracle_from(model)
    g = torch.Generator().manual_seed(5)
    prompt = torch.randint(0, cfg.vocab_size, (ctx,), generator=g)
    steps = 6
    oc = oracle.new_cache(16, max_seqs=1)
    oc.add_sequence(0)
    lg = oracle.forward(prompt, oc, [0], last_only=True)
    want_logits, toks = [], []
    tok = int(lg[0].argmax())
    for _ in range(steps):
        toks.append(tok)
        lg = oracle.forward(torch.tensor([tok]), oc, [0], last_only=True)
        want_logits.append(lg[0].clone())
        tok = int(lg[0].argmax())
    engines = []
    for sk in (True, False):
        cache = model.new_cache(16, max_seqs=1)
        cache.add_sequence(0)
        model.forward(prompt.to(dev), cache, [0], last_only=True)
        eng = CachedDecode(model, cache, max_batch=1, use_graph=use_graph, step_kernel=sk)
        assert (eng.step_kernel is not None) == sk
        eng.bind([0], [toks[0]])
        eng.reserve(steps + 1)
        engines.append(eng)
    for i in range(steps):
        outs = []
        for eng in engines:
            eng.tokens[0] = toks[i]
            eng.step()
            torch.cuda.synchronize()
            outs.append(eng.logits[0].cpu().clone())
        st = DecodeStepKernel.status()
        assert st == 0, hex(st)
        mag = want_logits[i].abs().max().item()
        for got in outs:
            err = (got - want_logits[i]).abs().max().item()
            assert err <= 5e-2 * mag + 2e-2, f"step {i}: err {err} mag {mag}"
        assert (outs[0] - outs[1]).abs().max().item() <= 3e-2 * mag + 1e-2
    assert engines[0].cache.seq_len(0) == ctx + steps


def test_one_graph_per_batch_bucket(dev):
    """An engine sized for 8 rows runs the smallest bucket that holds the bound rows, keeps one
    captured graph per bucket, and gives the same tokens whichever bucket ran."""
    cfg = tiny_moe_config()
    model = TransformerModel(from_state_dict(cfg, random_state_dict(cfg, 0), device=dev, quant="q4"))
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g) for n in (9, 14, 5)]

    def run(max_batch, seqs):
        cache = model.new_cache(8 * max(2, len(prompts)), max_seqs=4)
        last = []
        for s in seqs:
            cache.add_sequence(s)
            last.append(int(model.forward(prompts[s].to(dev), cache, [s], last_only=True)[0].argmax()))
        eng = CachedDecode(model, cache, max_batch=max_batch)
        eng.bind(seqs, last)
        return eng, eng.generate(4)

    eng1, t1 = run(1, [0])
    eng8, t8 = run(8, [0])
    assert eng8.buckets == (1, 2, 4, 8) and eng8.bucket() == 1
    assert torch.equal(t1, t8)
    assert len(eng8.graphs) == 1 and eng8.graphs.captures == 1 and eng8.graphs.hits >= 3
    # three rows: the 4-row bucket; a second graph appears, the first stays
    eng8b, t3 = run(8, [0, 1, 2])
    assert eng8b.bucket() == 4 and torch.equal(t3[0], t1[0])
    eng8b.bind([1], [int(t3[1, -1])])
    eng8b.reserve(2)
    eng8b.step()
    assert len(eng8b.graphs) == 2


def test_debug_serialize_runs_launch_by_launch(dev):
    """Debug-serialize mode: the step runs un-captured, every launch is followed by a device
    synchronisation and a read of the status words, and the result is unchanged."""
    from rmlx_b200 import _lib
    cfg = tiny_moe_config()
    model = TransformerModel(from_state_dict(cfg, random_state_dict(cfg, 0), device=dev, quant=None))
    prompt = torch.randint(0, cfg.vocab_size, (11,), generator=torch.Generator().manual_seed(1))

    def run(serialize):
        cache = model.new_cache(8, max_seqs=1)
        cache.add_sequence(0)
        last = int(model.forward(prompt.to(dev), cache, [0], last_only=True)[0].argmax())
        eng = CachedDecode(model, cache, max_batch=1)
        eng.serialize = serialize
        eng.bind([0], [last])
        return eng, eng.generate(3)

    _, want = run(False)
    _lib.set_debug_serialize(True)
    try:
        _lib.serial_trace()
        eng, got = run(True)
        trace = _lib.serial_trace()
    finally:
        _lib.set_debug_serialize(False)
    assert torch.equal(got, want)
    assert len(eng.graphs) == 0
    assert len(trace) >= 3 * eng.launches_per_step and "decode_advance" in trace


def test_moe_overlap_schedules_on_two_streams(dev):
    """Shared-expert and token-batch overlap on real streams: the hazard tracker inserts the event
    waits, the result equals the plain forward."""
    from rmlx_b200.config import MoeConfig
    from rmlx_b200.nn.moe import ExpertGroup, MoeLayer
    from rmlx_b200.ops.weights import LinearWeight
    torch.manual_seed(0)
    mc = MoeConfig(num_experts=4, num_experts_per_token=2, hidden_dim=64, intermediate_dim=128)
    mk = lambda *s: LinearWeight.from_dense(torch.randn(*s) * 0.1, None, dtype=torch.bfloat16, device=dev)
    layer = MoeLayer(mc, (torch.randn(4, 64) * 0.3).to(dev), ExpertGroup(mk(4, 256, 64), mk(4, 64, 128)))
    layer.with_shared_expert(mk(256, 64), mk(64, 128))
    x = torch.randn(48, 64, device=dev, dtype=torch.bfloat16)
    want = layer.forward(x).float()
    for mode in ("sbo", "tbo"):
        got = layer.with_overlap(mode).forward_overlapped(x).float()
        torch.cuda.synchronize()
        assert (got - want).abs().max() <= 2e-2 * want.abs().max()
        sm = layer._pipeline._streams
        assert sm.waits_inserted >= 2            # x -> side stream, side stream -> sum


@pytest.mark.parametrize("use_graph", [False, True])
def test_decode_with_8bit_kv_cache(dev, use_graph):
    """The decode engine over an 8-bit cache (quantising append + in-kernel page expansion) against
    the fp32 forward over a cache quantised the same way; prompt through the native prefill."""
    cfg = tiny_moe_config()
    model = TransformerModel(from_state_dict(cfg, random_state_dict(cfg, 0), device=dev, quant=None))
    oracle = _oracle_from(model)
    prompt = torch.randint(0, cfg.vocab_size, (40,), generator=torch.Generator().manual_seed(6))
    steps = 6
    oc = oracle.new_cache(8, max_seqs=1, kv_quant="q8")
    oc.add_sequence(0)
    lg = oracle.forward(prompt, oc, [0], last_only=True)
    want_logits, toks = [], []
    tok = int(lg[0].argmax())
    for _ in range(steps):
        toks.append(tok)
        lg = oracle.forward(torch.tensor([tok]), oc, [0], last_only=True)
        want_logits.append(lg[0].clone())
        tok = int(lg[0].argmax())
    cache = model.new_cache(8, max_seqs=2, kv_quant="q8")
    assert cache.quantized and cache.k[0].dtype == torch.uint8
    cache.add_sequence(0)
    model.prefill(prompt.to(dev), cache, 0)
    # what the prompt path wrote decodes to what the oracle cached
    assert (cache.get_keys(1, 0).float().cpu() - oc.get_keys(1, 0, 40).float()).abs().max() < 0.25
    eng = CachedDecode(model, cache, max_batch=2, use_graph=use_graph)
    assert not eng.fuse_rope and eng.step_kernel is None
    eng.bind([0], [toks[0]])
    eng.reserve(steps + 1)
    for i in range(steps):
        eng.step()
        torch.cuda.synchronize()
        got = eng.logits[0].float().cpu()
        rel = (got - want_logits[i]).abs().max().item() / want_logits[i].abs().max().item()
        assert rel < 6e-2, (i, rel)
        if i + 1 < steps:
            eng.set_next_tokens([toks[i + 1]])
