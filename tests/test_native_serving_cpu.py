"""The native serving core (csrc/host/serving.cpp) against the Python classes it mirrors: the same
random operation sequences must leave both in the same observable state."""
import random

import pytest
import torch

from rmlx_b200.config import SchedulerConfig, tiny_dense_config
from rmlx_b200.kv.paged import BlockManager, OutOfBlocks, PagedKvCache
from rmlx_b200.models.transformer import TransformerModel
from rmlx_b200.models.weights import from_state_dict, random_state_dict
from rmlx_b200.serve import native
from rmlx_b200.serve.engine import ServingEngine
from rmlx_b200.serve.prefix_cache import PrefixCache
from rmlx_b200.serve.scheduler import GenerationRequest, Scheduler

pytestmark = pytest.mark.skipif(not native.available(), reason="host library not available")


def _bm_state(bm, seqs, nblocks):
    return (bm.num_free_blocks(),
            {s: (bm.seq_len(s), list(bm.block_table(s))) for s in seqs if bm.has_sequence(s)},
            [bm.ref_count(b) for b in range(nblocks)])


@pytest.mark.parametrize("seed", range(6))
def test_block_manager_random_ops_match(seed):
    rng = random.Random(seed)
    nblocks, bs = 24, 4
    py, nat = BlockManager(nblocks, bs, reserved=1), native.NativeBlockManager(nblocks, bs, reserved=1)
    live, retained, next_id = [], [], 0
    for step in range(400):
        op = rng.choice(["new", "grow", "grow", "grow", "fork", "trim", "free", "adopt", "retain", "release"])
        if op == "new" or not live:
            py.add_sequence(next_id); nat.add_sequence(next_id)
            live.append(next_id); next_id += 1
        elif op == "grow":
            s, n = rng.choice(live), rng.randint(1, 9)
            outcomes = []
            for bm in (py, nat):
                try:
                    if not bm.can_allocate(s, n + bs):        # keep clear of the copy-on-write corner
                        raise OutOfBlocks("full")
                    copies = bm.reserve(s, n)
                    bm.commit(s, n)
                    outcomes.append(("ok", copies))
                except OutOfBlocks:
                    outcomes.append(("full", None))
            assert outcomes[0] == outcomes[1], (step, outcomes)
        elif op == "fork":
            p = rng.choice(live)
            py.fork(p, next_id); nat.fork(p, next_id)
            live.append(next_id); next_id += 1
        elif op == "trim":
            s, n = rng.choice(live), rng.randint(0, 6)
            py.trim(s, n); nat.trim(s, n)
        elif op == "free":
            s = live.pop(rng.randrange(len(live)))
            py.free_sequence(s); nat.free_sequence(s)
        elif op == "adopt":
            p = rng.choice(live)
            full = py.seq_len(p) // bs
            if full:
                blocks = list(py.block_table(p))[:rng.randint(1, full)]
                py.add_sequence(next_id); nat.add_sequence(next_id)
                py.adopt(next_id, blocks, len(blocks) * bs); nat.adopt(next_id, blocks, len(blocks) * bs)
                live.append(next_id); next_id += 1
        elif op == "retain":
            s = rng.choice(live)
            if py.block_table(s):
                b = rng.choice(py.block_table(s))
                py.retain(b); nat.retain(b); retained.append(b)
        elif op == "release" and retained:
            b = retained.pop(rng.randrange(len(retained)))
            py.release(b); nat.release(b)
        assert _bm_state(py, range(next_id), nblocks) == _bm_state(nat, range(next_id), nblocks), (step, op)
    # errors are reported the same way
    for bm in (py, nat):
        if not bm.has_sequence(9_999):
            bm.add_sequence(9_999)
        with pytest.raises(KeyError):
            bm.add_sequence(9_999)
        with pytest.raises(ValueError):
            bm.retain(0)                                   # the reserved block is never live
        with pytest.raises(OutOfBlocks):
            bm.reserve(10_000, nblocks * bs * 2)


@pytest.mark.parametrize("seed", range(4))
def test_prefix_cache_random_ops_match(seed):
    rng = random.Random(100 + seed)
    bs = 4
    py, nat = PrefixCache(bs, max_blocks=12), native.NativePrefixCache(bs, max_blocks=12)
    vocab, next_block = 3, 1
    for step in range(300):
        toks = [rng.randrange(vocab) for _ in range(rng.randint(1, 22))]
        op = rng.choice(["insert", "insert", "lookup", "lookup", "evict", "take"])
        if op == "insert":
            blocks = list(range(next_block, next_block + len(toks) // bs))
            next_block += len(blocks)
            assert py.insert_blocks(toks, blocks) == nat.insert_blocks(toks, blocks), step
        elif op == "lookup":
            assert py.lookup(toks) == nat.lookup(toks), step
        elif op == "evict":
            n = rng.randint(0, 3)
            assert py.evict(n) == nat.evict(n), step
        else:
            assert py.take_evicted() == nat.take_evicted(), step
        assert len(py) == len(nat) and (py.hits, py.misses) == (nat.hits, nat.misses), step
    assert sorted(py.clear()) == sorted(nat.clear()) and len(nat) == 0


def _drive(sched, bm, reqs, eos, steps=200):
    """Run a scheduler to completion with a deterministic fake model; returns the trace."""
    for r in reqs:
        sched.add_request(GenerationRequest(*r))
    trace, finished, produced = [], {}, {}
    for _ in range(steps):
        if not sched.has_work():
            break
        out = sched.schedule(bm, finished)
        finished = {}
        trace.append((sorted(out.evicted_seq_ids),
                      [(m.seq_id, m.prompt_len, m.current_len, m.prefill_progress) for m in out.prefill_seqs],
                      out.prefill_chunk_range,
                      [(m.seq_id, m.current_len, len(m.block_table)) for m in out.decode_seqs],
                      bm.num_free_blocks()))
        toks = {}
        for m in out.prefill_seqs:
            if out.prefill_chunk_range[1] >= m.prompt_len:
                toks[m.seq_id] = 7
        for m in out.decode_seqs:
            n = produced.get(m.seq_id, 0)
            toks[m.seq_id] = eos if (m.seq_id % 3 == 0 and n == 2) else 7
        for sid, t in toks.items():
            produced[sid] = produced.get(sid, 0) + 1
            sched.update_sequence(sid, bm, t)
            finished[sid] = t
    return trace


@pytest.mark.parametrize("max_batch,chunk,nblocks", [(2, 8, 40), (3, 5, 14), (8, 64, 64), (1, 4, 9)])
def test_scheduler_traces_match(max_batch, chunk, nblocks):
    cfg = SchedulerConfig(max_batch_size=max_batch, eos_token_id=99, block_size=4, max_prefill_chunk=chunk)
    rng = random.Random(max_batch * 100 + chunk)
    reqs = [(i, [rng.randrange(50) for _ in range(rng.randint(1, 23))], rng.randint(1, 6)) for i in range(9)]
    t_py = _drive(Scheduler(cfg, manage_blocks=True), BlockManager(nblocks, 4), reqs, 99)
    t_nat = _drive(native.NativeScheduler(cfg, manage_blocks=True), native.NativeBlockManager(nblocks, 4), reqs, 99)
    assert t_py == t_nat
    assert t_py[-1][-1] == nblocks or any(e for e, *_ in t_py)      # work happened and blocks came back


def test_scheduler_prompt_chunks_and_cached_prefix_match():
    cfg = SchedulerConfig(max_batch_size=2, eos_token_id=-1, block_size=4, max_prefill_chunk=6)
    prompt = list(range(30, 47))
    for cls, bm in ((Scheduler, BlockManager(32, 4)), (native.NativeScheduler, native.NativeBlockManager(32, 4))):
        seen = []

        def admit(sid, bm=bm, seen=seen):
            bm.add_sequence(sid)
            seen.append(sid)
            return 100 if sid == 0 else 8              # over-long claims are capped below the prompt length

        s = cls(cfg, manage_blocks=False, on_admit=admit, on_evict=bm.free_sequence)
        s.add_request(GenerationRequest(0, prompt, 2))
        s.add_request(GenerationRequest(1, prompt, 2))
        assert s.first_waiting_prompt_len() == 17
        out = s.schedule(bm)
        assert seen == [0, 1] and s.first_waiting_prompt_len() is None
        assert out.prefill_seqs[0].seq_id == 0 and out.prefill_chunk_range == (16, 17)
        assert s.prompt_chunk(0, (16, 17)) == [46]
        out = s.schedule(bm)
        assert out.prefill_seqs[0].seq_id == 1 and out.prefill_chunk_range == (8, 14)
        assert s.prompt_chunk(1, (8, 14)) == prompt[8:14]


def test_serving_engine_same_tokens_with_python_and_native_core(monkeypatch):
    cfg = tiny_dense_config()
    model = TransformerModel(from_state_dict(cfg, random_state_dict(cfg, 0), dtype=torch.float32))
    g = torch.Generator().manual_seed(9)
    common = torch.randint(0, cfg.vocab_size, (35,), generator=g).tolist()
    prompts = [common + torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (2, 9, 4, 1)]
    results = []
    for flag in ("1", "0"):
        monkeypatch.setenv("RMLX_NATIVE_SERVING", flag)
        eng = ServingEngine(model, num_blocks=20, use_prefix_cache=True,
                            scheduler_cfg=SchedulerConfig(max_batch_size=2, max_prefill_chunk=16))
        assert eng.native == (flag == "1")
        assert isinstance(eng.cache.manager, native.NativeBlockManager) == (flag == "1")
        ids = [eng.submit(p, 4) for p in prompts]
        outs = eng.run_until_done()
        results.append(([outs[i] for i in ids], eng.prefill_tokens, eng.prefix.hits, len(eng.prefix)))
    assert results[0] == results[1]


def test_paged_cache_uses_native_manager_by_default():
    cache = PagedKvCache(8, 1, 1, 8, dtype=torch.float32)
    assert isinstance(cache.manager, native.NativeBlockManager)
    cache.add_sequence(3)
    cache.reserve(3, 20)
    cache.commit(3, 20)
    assert cache.seq_len(3) == 20 and len(cache.manager.block_table(3)) == 2
    assert cache.block_table[cache.slot_of[3]][:2].tolist() == cache.manager.block_table(3)
    cache.trim(3, 10)
    assert cache.seq_len(3) == 10 and cache.manager.num_free_blocks() == 6
    cache.free_sequence(3)
    assert cache.manager.num_free_blocks() == 7


def test_drop_front_releases_pages_before_the_window_in_both_managers():
    """Sliding-window sequences give back the pages that lie entirely before the window; both block
    managers agree on tables, free counts and what freeing the sequence returns."""
    from rmlx_b200.kv import native
    from rmlx_b200.kv.paged import BlockManager
    mgrs = [BlockManager(12, 16, reserved=1)]
    if native.available():
        mgrs.append(native.NativeBlockManager(12, 16, 1))
    states = []
    for m in mgrs:
        m.add_sequence(5)
        m.reserve(5, 100)
        m.commit(5, 100)                       # 7 pages
        assert m.num_free_blocks() == 11 - 7
        assert m.drop_front(5, 200) == 0       # the window still covers everything
        n = m.drop_front(5, 40)                # tokens 60..99 stay: pages 0..2 go (3*16 = 48 <= 60)
        table = list(m.block_table(5))
        assert n == 3 and table[:3] == [0, 0, 0] and all(b > 0 for b in table[3:])
        assert m.num_free_blocks() == 11 - 4
        assert m.drop_front(5, 40) == 0        # idempotent
        m.fork(5, 6)                           # shared pages: released entries carry no reference
        m.free_sequence(5)
        assert m.num_free_blocks() == 11 - 4
        m.free_sequence(6)
        assert m.num_free_blocks() == 11
        states.append(table)
        with pytest.raises(KeyError):
            m.drop_front(99, 1)
    assert all(s == states[0] for s in states)
    unreserved = BlockManager(4, 16, reserved=0)
    unreserved.add_sequence(0)
    with pytest.raises(ValueError):
        unreserved.drop_front(0, 1)


def test_native_sampler_matches_the_python_sampler():
    """Distribution shaping (penalty, temperature, top-k, top-p) agrees with the Python class to
    rounding; draws follow the distribution and are reproducible from the seed; the speculative
    acceptance rules agree on deterministic cases and keep the target distribution."""
    import torch
    from rmlx_b200.config import SamplerConfig
    from rmlx_b200.serve.native import NativeSampler
    from rmlx_b200.serve.sampler import Sampler
    g = torch.Generator().manual_seed(3)
    logits = torch.randn(4, 97, generator=g) * 2
    hist = [[1, 5, 5, 60], [], [96, 0], [3]]
    for cfg in (SamplerConfig(temperature=0.7, top_k=5, top_p=0.9, repetition_penalty=1.3, seed=1),
                SamplerConfig(temperature=1.0, seed=1), SamplerConfig(temperature=1.5, top_p=0.5, seed=1),
                SamplerConfig(temperature=0.9, top_k=200, seed=1), SamplerConfig(repetition_penalty=2.0)):
        py, nat = Sampler(cfg), NativeSampler(cfg)
        for r in range(4):
            want, got = py.probabilities(logits[r], hist[r]), nat.probabilities(logits[r], hist[r])
            assert torch.allclose(got, want, atol=1e-6), cfg
            assert abs(float(got.sum()) - 1.0) < 1e-5
        if cfg.temperature == 0.0:
            assert nat.sample_batch(logits, hist) == py.sample_batch(logits, hist)
            assert nat.sample_token(logits[0], hist[0]) == py.sample_token(logits[0], hist[0])

    cfg = SamplerConfig(temperature=1.0, seed=11)
    small = torch.tensor([[2.0, 1.0, 0.0, -1.0, -30.0]])
    a, b, c = NativeSampler(cfg), NativeSampler(cfg), NativeSampler(SamplerConfig(temperature=1.0, seed=12))
    draws = [a.sample_batch(small)[0] for _ in range(4000)]
    assert draws == [b.sample_batch(small)[0] for _ in range(4000)]
    assert draws != [c.sample_batch(small)[0] for _ in range(4000)]
    freq = torch.bincount(torch.tensor(draws), minlength=5).float() / len(draws)
    assert torch.allclose(freq, torch.softmax(small[0], -1), atol=0.03) and freq[4] == 0

    tl = torch.tensor([[0.0, 3.0, 1.0], [5.0, 0.0, 1.0], [0.0, 0.0, 9.0]])
    for draft in ([1, 0], [1, 2], [2], [1, 0, 2]):
        want = Sampler.greedy_verify(draft, tl)
        got = a.greedy_verify(draft, tl)
        assert (got.num_accepted, got.accepted_tokens, got.correction_token) == (
            want.num_accepted, want.accepted_tokens, want.correction_token), draft

    pt = torch.tensor([[0.5, 0.3, 0.2, 0.0], [0.1, 0.1, 0.1, 0.7]])
    same = a.rejection_sample([0], pt[:1], pt)                       # equal distributions: always accepted
    assert same.num_accepted == 1 and same.accepted_tokens == [0] and same.correction_token in (0, 1, 2, 3)
    pd = torch.tensor([[0.0, 0.0, 0.0, 1.0]])                        # the target gives the draft token no mass
    rej = a.rejection_sample([3], pd, pt[:1])
    assert rej.num_accepted == 0 and rej.correction_token in (0, 1, 2)
    # the accepted-or-corrected token follows the target distribution whatever the draft distribution
    pdraft = torch.tensor([[0.1, 0.6, 0.2, 0.1]])
    out = []
    for _ in range(6000):
        d = int(a._lib.rmlx_sampler_multinomial(a._h, pdraft.data_ptr(), 4))
        r = a.rejection_sample([d], pdraft, pt[:1])
        out.append(d if r.num_accepted == 1 else r.correction_token)
    freq = torch.bincount(torch.tensor(out), minlength=4).float() / len(out)
    assert torch.allclose(freq, pt[0], atol=0.03)
    with pytest.raises(ValueError):
        a.rejection_sample([9], pdraft, pt[:1])
    with pytest.raises(ValueError):
        a.rejection_sample([0, 1], torch.cat([pdraft, pdraft]), pt[:1])     # two draft tokens, one target row
    assert not a._lib.rmlx_sampler_create(1.0, -1, 0.5, 1.0, 0)      # a negative top-k is refused
    assert not a._lib.rmlx_sampler_create(1.0, 0, 0.0, 1.0, 0)       # so is top-p = 0
