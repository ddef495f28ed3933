"""CPU plumbing checks on the tiny dense decoder (hidden 256, 4 q / 2 kv heads, head_dim 64,
SwiGLU 688, vocab 1024, weights N(0, 0.02) seed 0): a 16-token prefill followed by 8 greedy decode
steps on a paged KV cache with page size 16, alone and tensor-parallel over two gloo ranks.
Mirrors crates/rmlx-nn/tests/e2e_generate.rs:244-404 and the mock-transport multi-rank tests of
crates/rmlx-distributed/tests/tree_allreduce_tests.rs:10-121 (one OS process per simulated rank)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from rmlx_b200.config import FeedForwardType, MoeConfig, TransformerConfig, tiny_dense_config
from rmlx_b200.models.transformer import TransformerModel
from rmlx_b200.models.weights import ParallelLayout, from_state_dict, random_state_dict


def _prompt(cfg):
    g = torch.Generator().manual_seed(0)
    return torch.randint(0, cfg.vocab_size, (16,), generator=g)


def tiny_moe_config():
    moe = MoeConfig(num_experts=8, num_experts_per_token=2, hidden_dim=256, intermediate_dim=128)
    return TransformerConfig(hidden_size=256, num_heads=4, num_kv_heads=2, head_dim=64, num_layers=2,
                             vocab_size=1024, max_seq_len=256, ff_type=FeedForwardType.moe_(moe)).validate()


def test_prefill_then_cached_decode_matches_full_forward():
    cfg = tiny_dense_config()
    model = TransformerModel(from_state_dict(cfg, random_state_dict(cfg, 0), dtype=torch.float32))
    prompt = _prompt(cfg)
    toks = model.generate_greedy(prompt, 8)
    assert len(toks) == 8
    full = torch.cat([prompt, torch.tensor(toks[:-1])])
    logits = model.forward(full)
    assert logits.shape == (23, cfg.vocab_size)
    assert [int(logits[15 + i].argmax()) for i in range(8)] == toks


def test_batched_decode_equals_single():
    cfg = tiny_moe_config()
    model = TransformerModel(from_state_dict(cfg, random_state_dict(cfg, 0), dtype=torch.float32))
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, cfg.vocab_size, (8,), generator=g) for _ in range(3)]
    cache = model.new_cache(16, max_seqs=4)
    for s in range(3):
        cache.add_sequence(s)
    lg = model.forward(torch.cat(prompts), cache, [0, 1, 2], last_only=True)
    for s in range(3):
        alone = model.forward(prompts[s], last_only=True)
        assert torch.allclose(lg[s], alone[0], atol=1e-4)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _tp_worker(rank, world, port, cfg, expert_parallel, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.set_num_threads(1)
        sd = random_state_dict(cfg, 0)
        layout = ParallelLayout(rank, world, expert_parallel)
        w = from_state_dict(cfg, sd, dtype=torch.float32, layout=layout)

        def allreduce(t):
            t = t.contiguous()
            dist.all_reduce(t)
            return t

        def allgather(t):
            parts = [torch.empty_like(t) for _ in range(world)]
            dist.all_gather(parts, t.contiguous())
            return torch.cat(parts, -1)

        model = TransformerModel(w, allreduce, allgather)
        toks = model.generate_greedy(_prompt(cfg), 8)
        if rank == 0:
            q.put(toks)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("kind,ep", [("dense", False), ("moe", False), ("moe", True)])
def test_tensor_parallel_gloo_world2_matches_single(kind, ep):
    cfg = tiny_dense_config() if kind == "dense" else tiny_moe_config()
    single = TransformerModel(from_state_dict(cfg, random_state_dict(cfg, 0), dtype=torch.float32))
    want = single.generate_greedy(_prompt(cfg), 8)
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_tp_worker, args=(r, 2, port, cfg, ep, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = q.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert got == want


def test_deepseek_paged_latent_decode_matches_the_contiguous_cache():
    """Batched decode over paged latent caches (absorbed attention) generates the same tokens as
    the per-sequence forward with contiguous latent caches."""
    from rmlx_b200.models.deepseek import DeepSeekV3Model, deepseek_tiny
    m = DeepSeekV3Model(deepseek_tiny(), seed=1)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, 256, (9,), generator=g), torch.randint(0, 256, (5,), generator=g)]
    want = []
    for p in prompts:
        c = m.new_cache()
        lg = m.forward(p, c)
        toks = []
        for _ in range(4):
            toks.append(int(lg[-1].argmax()))
            lg = m.forward(torch.tensor([toks[-1]]), c)
        want.append(toks)
    pc = m.new_paged_cache(16)
    t = torch.tensor([int(m.prefill_paged(p, pc, s)[0].argmax()) for s, p in enumerate(prompts)])
    got = [[], []]
    for _ in range(4):
        got[0].append(int(t[0])); got[1].append(int(t[1]))
        t = m.decode_paged(t, pc, [0, 1]).argmax(-1)
    assert got == want


def test_sliding_window_model_keeps_generating_after_old_pages_are_released():
    """A model with a sliding window never reads keys before the window, so releasing their pages
    between steps (the rotating cache as a page policy) changes nothing."""
    from rmlx_b200.config import tiny_dense_config
    from rmlx_b200.models.transformer import TransformerModel
    from rmlx_b200.models.weights import from_state_dict, random_state_dict
    cfg = tiny_dense_config().replace(sliding_window=24)
    model = TransformerModel(from_state_dict(cfg, random_state_dict(cfg, 0), dtype=torch.float32))
    prompt = torch.randint(0, cfg.vocab_size, (70,), generator=torch.Generator().manual_seed(3))

    def run(release):
        cache = model.new_cache(12, max_seqs=1)
        cache.add_sequence(0)
        lg = model.forward(prompt, cache, [0], last_only=True)
        toks, freed = [], 0
        for _ in range(10):
            toks.append(int(lg[0].argmax()))
            if release:
                freed += cache.drop_front(0, cfg.sliding_window)
            lg = model.forward(torch.tensor([toks[-1]]), cache, [0], last_only=True)
        return toks, freed, cache.manager.num_free_blocks()

    plain, _, free_plain = run(False)
    rotated, freed, free_rot = run(True)
    assert rotated == plain
    assert freed >= 2 and free_rot == free_plain + freed
