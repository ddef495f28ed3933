"""Scheduler, sampler, prefix cache and the serving loop on CPU (the logic tests of
crates/rmlx-nn/src/scheduler.rs, sampler.rs:543-640 and prefix_cache.rs)."""
import pytest
import torch

from rmlx_b200.config import SamplerConfig, SchedulerConfig, tiny_dense_config
from rmlx_b200.kv.paged import BlockManager, OutOfBlocks
from rmlx_b200.models.transformer import TransformerModel
from rmlx_b200.models.weights import from_state_dict, random_state_dict
from rmlx_b200.serve.engine import ServingEngine
from rmlx_b200.serve.prefix_cache import PrefixCache
from rmlx_b200.serve.sampler import Sampler
from rmlx_b200.serve.scheduler import GenerationRequest, Scheduler


def test_block_manager_cow_fork_trim():
    bm = BlockManager(8, 4)
    bm.reserve(1, 6); bm.commit(1, 6)
    assert len(bm.block_table(1)) == 2 and bm.num_free_blocks() == 6
    bm.fork(1, 2)
    assert bm.block_table(2) == bm.block_table(1)
    copies = bm.reserve(2, 1)                       # shared partial last block: copy on write
    assert len(copies) == 1 and copies[0][0] == bm.block_table(1)[1]
    assert bm.block_table(2)[1] != bm.block_table(1)[1] and bm.block_table(2)[0] == bm.block_table(1)[0]
    bm.commit(2, 1)
    bm.trim(2, 3)                                   # 7 -> 4 tokens: second block released
    assert bm.seq_len(2) == 4 and len(bm.block_table(2)) == 1
    bm.free_sequence(1); bm.free_sequence(2)
    assert bm.num_free_blocks() == 8
    try:
        bm.reserve(3, 100)
        assert False
    except OutOfBlocks:
        pass


def test_scheduler_admission_chunked_prefill_and_eviction():
    bm = BlockManager(16, 4)
    s = Scheduler(SchedulerConfig(max_batch_size=2, eos_token_id=99, block_size=4, max_prefill_chunk=8))
    s.add_request(GenerationRequest(0, list(range(20)), 3))
    s.add_request(GenerationRequest(1, list(range(5)), 2))
    s.add_request(GenerationRequest(2, [1, 2, 3], 2))
    o = s.schedule(bm)
    assert [m.seq_id for m in o.prefill_seqs] == [0] and o.prefill_chunk_range == (0, 8)
    assert s.num_active() == 2 and s.num_waiting() == 1
    o = s.schedule(bm)
    assert o.prefill_chunk_range == (8, 16) and o.prefill_seqs[0].is_chunked_prefill()
    o = s.schedule(bm)
    assert o.prefill_chunk_range == (16, 20)
    o = s.schedule(bm)                              # seq 1 prefills now, seq 0 decodes
    assert [m.seq_id for m in o.prefill_seqs] == [1] and [m.seq_id for m in o.decode_seqs] == [0]
    s.update_sequence(0, bm, 5)
    o = s.schedule(bm, {0: 99})                     # EOS: evicted, waiting request admitted
    assert o.evicted_seq_ids == [0] and s.num_waiting() == 0 and 2 in s.active


def test_sampler_pipeline_and_speculative():
    logits = torch.tensor([1.0, 3.0, 2.0, -1.0])
    assert Sampler().sample_token(logits) == 1
    s = Sampler(SamplerConfig(temperature=1.0, top_k=2, seed=0))
    p = s.probabilities(logits)
    assert p[0] == 0 and p[3] == 0 and abs(float(p.sum()) - 1) < 1e-6
    s = Sampler(SamplerConfig(temperature=1.0, top_p=0.5, seed=0))
    p = s.probabilities(logits)
    assert int((p > 0).sum()) == 1 and p[1] == 1
    s = Sampler(SamplerConfig(repetition_penalty=2.0))
    assert s.sample_token(logits, history=[1]) == 2          # 3.0 / 2 < 2.0
    draws = [Sampler(SamplerConfig(temperature=1.0, seed=i)).sample_token(logits) for i in range(50)]
    assert set(draws) <= {0, 1, 2, 3} and len(set(draws)) > 1
    tl = torch.eye(4)[[1, 2, 0, 3]] * 5
    r = Sampler.greedy_verify([1, 2, 3], tl)
    assert r.num_accepted == 2 and r.accepted_tokens == [1, 2] and r.correction_token == 0
    r = Sampler.greedy_verify([1, 2, 0], tl)
    assert r.num_accepted == 3 and r.correction_token == 3    # bonus token
    s = Sampler(SamplerConfig(temperature=1.0, seed=1))
    tp = torch.tensor([[0.0, 1.0, 0.0], [0.5, 0.5, 0.0]])
    dp = torch.tensor([[0.0, 1.0, 0.0], [0.0, 0.0, 1.0]])
    r = s.rejection_sample([1, 2], dp, tp)
    assert r.num_accepted == 1 and r.correction_token in (0, 1)


def test_prefix_cache():
    pc = PrefixCache(block_size=4)
    toks = list(range(10))
    assert pc.insert(toks, [7, 8]) == 2               # two full blocks; the ragged tail is not cached
    assert pc.lookup(toks) == (8, [7, 8])
    assert pc.lookup([0, 1, 2, 3, 9, 9, 9, 9]) == (4, [7])
    assert pc.lookup([5, 5, 5, 5]) == (0, [])
    pc.insert([0, 1, 2, 3, 9, 9, 9, 9], [7, 11])
    assert len(pc) == 3
    pc.lookup(toks)                                   # touch the [7, 8] branch
    assert pc.evict(1) == [11]
    assert pc.hits >= 2 and pc.misses == 1


def test_serving_engine_matches_single_sequence_generation():
    cfg = tiny_dense_config()
    model = TransformerModel(from_state_dict(cfg, random_state_dict(cfg, 0), dtype=torch.float32))
    g = torch.Generator().manual_seed(2)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (5, 19, 9)]
    eng = ServingEngine(model, num_blocks=24,
                        scheduler_cfg=SchedulerConfig(max_batch_size=2, max_prefill_chunk=8))
    ids = [eng.submit(p, 4) for p in prompts]
    outs = eng.run_until_done()
    for sid, p in zip(ids, prompts):
        want = model.generate_greedy(torch.tensor(p), 4)
        assert outs[sid][:4] == want, (sid, outs[sid], want)
    assert eng.cache.manager.num_free_blocks() == 23   # everything returned (block 0 is reserved)


def test_block_manager_adopt_retain_release():
    bm = BlockManager(8, 4)
    bm.reserve(1, 8); bm.commit(1, 8)
    shared = list(bm.block_table(1))
    bm.retain(shared[0])                               # a cache keeps the first page
    bm.add_sequence(2)
    bm.adopt(2, shared, 8)
    assert bm.seq_len(2) == 8 and bm.block_table(2) == shared
    bm.free_sequence(1)
    assert bm.num_free_blocks() == 6                   # still owned by sequence 2 (and the cache)
    bm.reserve(2, 1); bm.commit(2, 1)                  # full shared pages: a new page, no copy
    assert len(bm.block_table(2)) == 3
    bm.free_sequence(2)
    assert bm.num_free_blocks() == 7                   # the retained page survives its sequences
    bm.release(shared[0])
    assert bm.num_free_blocks() == 8
    try:
        bm.retain(shared[0])
        assert False
    except ValueError:
        pass


def test_serving_engine_prefix_cache_reuses_prompt_pages():
    """Requests that share a prompt prefix skip its prefill, produce the same tokens as without the
    cache, and cached pages are given back when blocks run short or on request."""
    cfg = tiny_dense_config()
    model = TransformerModel(from_state_dict(cfg, random_state_dict(cfg, 0), dtype=torch.float32))
    g = torch.Generator().manual_seed(5)
    common = torch.randint(0, cfg.vocab_size, (40,), generator=g).tolist()
    prompts = [common + torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (3, 7, 0)]
    scfg = SchedulerConfig(max_batch_size=1, max_prefill_chunk=16)      # one at a time: later ones hit

    plain = ServingEngine(model, num_blocks=24, scheduler_cfg=scfg)
    ids = [plain.submit(p, 3) for p in prompts]
    want = plain.run_until_done()

    eng = ServingEngine(model, num_blocks=24, scheduler_cfg=scfg, use_prefix_cache=True)
    ids2 = [eng.submit(p, 3) for p in prompts]
    got = eng.run_until_done()
    for a, b in zip(ids, ids2):
        assert got[b] == want[a]
    # 40 common tokens = two full 16-token pages shared by the second and third request; the third
    # prompt is exactly the common part, so its last page (tokens 32..39) is partial and runs again
    assert eng.prefix.hits == 2
    assert eng.prefill_tokens == plain.prefill_tokens - 2 * 32
    held = len(eng.prefix)
    assert held >= 2 and eng.cache.manager.num_free_blocks() == 23 - held
    assert eng.reclaim(100) == held
    assert eng.cache.manager.num_free_blocks() == 23


def test_serving_engine_prefix_cache_gives_way_under_pressure():
    cfg = tiny_dense_config()
    model = TransformerModel(from_state_dict(cfg, random_state_dict(cfg, 0), dtype=torch.float32))
    g = torch.Generator().manual_seed(6)
    scfg = SchedulerConfig(max_batch_size=1, max_prefill_chunk=64)
    eng = ServingEngine(model, num_blocks=6, scheduler_cfg=scfg, use_prefix_cache=True)   # 5 usable pages
    first = torch.randint(0, cfg.vocab_size, (50,), generator=g).tolist()
    second = torch.randint(0, cfg.vocab_size, (60,), generator=g).tolist()
    a = eng.submit(first, 2)
    eng.run_until_done()
    assert len(eng.prefix) == 3                         # 48 of the 50 prompt tokens stay cached
    b = eng.submit(second, 2)                           # needs 4 pages at once: 2 free + cached ones
    outs = eng.run_until_done()
    assert outs[b] == model.generate_greedy(torch.tensor(second), 2)
    assert len(outs[a]) == 2


def test_speculative_decoder_reproduces_target_greedy():
    """Whatever the draft proposes, greedy draft-and-verify yields the target's greedy continuation:
    a perfect draft (the target itself) is accepted every time, an unrelated one almost never."""
    from rmlx_b200.serve.speculative import SpeculativeDecoder
    cfg = tiny_dense_config()
    target = TransformerModel(from_state_dict(cfg, random_state_dict(cfg, 0), dtype=torch.float32))
    other = TransformerModel(from_state_dict(cfg, random_state_dict(cfg, 7), dtype=torch.float32))
    g = torch.Generator().manual_seed(3)
    prompt = torch.randint(0, cfg.vocab_size, (21,), generator=g).tolist()
    want = target.generate_greedy(torch.tensor(prompt), 14)

    same = SpeculativeDecoder(target, target, k=4)
    assert same.generate(prompt, 14) == want
    assert same.stats.acceptance_rate == 1.0 and same.stats.rounds == 3      # 1 + 3 * (4 + 1) >= 14
    assert same.stats.tokens_per_round == 5.0

    for k in (1, 3, 5):
        spec = SpeculativeDecoder(target, other, k=k)
        assert spec.generate(prompt, 14) == want, k
        assert spec.stats.proposed == spec.stats.rounds * k
        assert spec.stats.acceptance_rate < 1.0


def test_speculative_decoder_sampling_runs_and_stops_at_eos():
    from rmlx_b200.serve.speculative import SpeculativeDecoder
    cfg = tiny_dense_config()
    target = TransformerModel(from_state_dict(cfg, random_state_dict(cfg, 0), dtype=torch.float32))
    draft = TransformerModel(from_state_dict(cfg, random_state_dict(cfg, 7), dtype=torch.float32))
    prompt = list(range(1, 12))
    spec = SpeculativeDecoder(target, draft, k=3, sampler_cfg=SamplerConfig(temperature=0.8, top_k=20, seed=1))
    out = spec.generate(prompt, 10)
    assert len(out) == 10 and all(0 <= t < cfg.vocab_size for t in out)
    # greedy with an end-of-sequence id taken from the known continuation: generation stops on it
    want = target.generate_greedy(torch.tensor(prompt), 8)
    eos = want[4]
    cut = want[:want.index(eos) + 1]
    spec = SpeculativeDecoder(target, target, k=3, eos_token_id=eos)
    assert spec.generate(prompt, 8) == cut


def test_sampler_batch_matches_per_row():
    g = torch.Generator().manual_seed(4)
    logits = torch.randn(5, 97, generator=g) * 3
    hist = [[1, 5, 5, 9], [], [96], [0, 1, 2, 3], [50]]
    for cfg in (SamplerConfig(), SamplerConfig(repetition_penalty=1.3),
                SamplerConfig(temperature=0.7), SamplerConfig(temperature=1.2, top_k=10),
                SamplerConfig(temperature=0.9, top_p=0.8),
                SamplerConfig(temperature=0.8, top_k=20, top_p=0.6, repetition_penalty=1.2)):
        s = Sampler(cfg)
        batch = s.probabilities_batch(logits, hist)
        rows = torch.stack([s.probabilities(logits[i], hist[i]) for i in range(5)])
        assert torch.allclose(batch, rows, atol=1e-6), cfg
        assert torch.allclose(batch.sum(-1), torch.ones(5), atol=1e-5)
        if cfg.temperature == 0.0:
            assert s.sample_batch(logits, hist) == [s.sample_token(logits[i], hist[i]) for i in range(5)]
    # draws follow the distribution: with top_k = 2 only the two best tokens of each row ever appear
    s = Sampler(SamplerConfig(temperature=1.0, top_k=2, seed=3))
    best2 = [set(logits[i].topk(2).indices.tolist()) for i in range(5)]
    seen = [set() for _ in range(5)]
    for _ in range(40):
        for i, t in enumerate(s.sample_batch(logits)):
            assert t in best2[i]
            seen[i].add(t)
    assert any(len(v) == 2 for v in seen)
    # the same seed gives the same draws
    a, b = Sampler(SamplerConfig(temperature=1.0, seed=11)), Sampler(SamplerConfig(temperature=1.0, seed=11))
    assert [a.sample_batch(logits) for _ in range(3)] == [b.sample_batch(logits) for _ in range(3)]


def test_q8_kv_cache_on_the_host_path():
    """The 8-bit paged cache through the host-driven append / gather: error within half a code
    step per group, copy-on-write carries the scales, and a tiny model generates the same tokens
    as with the bf16 cache."""
    from rmlx_b200.kv.paged import PagedKvCache, dequantize_kv_rows, quantize_kv_rows
    torch.manual_seed(0)
    x = torch.randn(5, 2, 128) * 3
    q, sb = quantize_kv_rows(x)
    assert q.dtype == torch.uint8 and sb.shape == (5, 2, 2, 2)
    back = dequantize_kv_rows(q, sb)
    step = sb[..., 0].float().repeat_interleave(64, -1).reshape(x.shape)
    assert ((back - x).abs() <= 0.51 * step + 1e-6).all()

    c = PagedKvCache(8, 1, 2, 128, dtype=torch.float32, max_seqs=4, max_blocks_per_seq=4, kv_quant="q8")
    assert c.quantized and c.bytes_per_token() == 2 * 2 * (128 + 8)
    c.add_sequence(0)
    c.reserve(0, 20)
    k, v = torch.randn(20, 2, 128), torch.randn(20, 2, 128)
    c.append(0, 0, k, v, 0)
    c.commit(0, 20)
    assert (c.get_keys(0, 0) - k).abs().max() < 0.03 and (c.get_values(0, 0) - v).abs().max() < 0.03
    c.fork(0, 1)
    c.reserve(1, 1)                            # shared partial last block: copied with its scales
    assert c.manager.block_table(1)[-1] != c.manager.block_table(0)[-1]
    assert torch.equal(c.get_keys(0, 1, 20), c.get_keys(0, 0, 20))
    with pytest.raises(ValueError):
        PagedKvCache(4, 1, 2, 96, kv_quant="q8")

    from rmlx_b200.config import tiny_dense_config
    from rmlx_b200.models.transformer import TransformerModel
    from rmlx_b200.models.weights import from_state_dict, random_state_dict
    cfg = tiny_dense_config()
    model = TransformerModel(from_state_dict(cfg, random_state_dict(cfg, 0), dtype=torch.float32))
    prompt = torch.randint(0, cfg.vocab_size, (12,), generator=torch.Generator().manual_seed(2))
    plain = model.generate_greedy(prompt, 6)
    cq = model.new_cache(4, max_seqs=1, kv_quant="q8")
    assert model.generate_greedy(prompt, 6, cache=cq) == plain


def test_serving_engine_warm_up_leaves_no_trace_and_runs_once():
    """``warm_up`` runs throw-away requests through the prompt and decode paths, gives every page
    back, keeps its tokens out of the outputs and counters, and does nothing the second time."""
    cfg = tiny_dense_config()
    model = TransformerModel(from_state_dict(cfg, random_state_dict(cfg, 0), dtype=torch.float32))
    eng = ServingEngine(model, num_blocks=24, use_prefix_cache=True,
                        scheduler_cfg=SchedulerConfig(max_batch_size=2, max_prefill_chunk=8))
    first = eng.warm_up()
    assert first.ran and first.kernels_s > 0
    assert eng.outputs == {} and eng.prefill_tokens == 0 and len(eng.prefix) == 0
    assert eng.cache.manager.num_free_blocks() == 23
    again = eng.warm_up()
    assert not again.ran and again.kernels_s == first.kernels_s
    prompt = [3, 1, 4, 1, 5, 9, 2, 6]
    sid = eng.submit(prompt, 4)
    assert eng.run_until_done()[sid][:4] == model.generate_greedy(torch.tensor(prompt), 4)


def test_serving_engine_precision_guard_counts_bad_logits():
    """The logit monitor sees every ``guard_every``-th decode step and each completed prompt; a
    non-finite row is counted as a fallback verdict with the step it came from."""
    from rmlx_b200.utils.precision_guard import GuardAction, PrecisionGuard
    cfg = tiny_dense_config()
    model = TransformerModel(from_state_dict(cfg, random_state_dict(cfg, 0), dtype=torch.float32))
    guard = PrecisionGuard()
    eng = ServingEngine(model, num_blocks=24, precision_guard=guard, guard_every=2,
                        scheduler_cfg=SchedulerConfig(max_batch_size=2, max_prefill_chunk=8))
    sid = eng.submit([5, 6, 7], 9)
    eng.run_until_done()
    # one prompt + decode steps 2, 4, 6, 8 (the first of the 9 tokens came from the prompt)
    assert guard.checks == 5 and eng.guard_fallbacks == 0 and guard.nan_events == 0
    assert len(eng.outputs[sid]) == 9

    real = model.forward
    def poisoned(*a, **k):
        out = real(*a, **k).clone()
        out[0, 0] = float("nan")
        return out
    model.forward = poisoned
    try:
        eng2 = ServingEngine(model, num_blocks=24, precision_guard=PrecisionGuard(), guard_every=1,
                             scheduler_cfg=SchedulerConfig(max_batch_size=2, max_prefill_chunk=8))
        eng2.submit([5, 6, 7], 3)
        eng2.run_until_done()
    finally:
        model.forward = real
    # the prompt's logits (decode step 0: the library prompt path runs the same forward) and both decode steps
    assert eng2.guard_fallbacks == 3 and eng2.guard.nan_events == 3
    assert eng2.guard_events == [(s, GuardAction.FALLBACK) for s in (0, 1, 2)]
