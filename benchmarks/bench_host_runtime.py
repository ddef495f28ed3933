#!/usr/bin/env python
"""Host-side micro-benchmarks (no GPU): the native serving core against the Python classes it
mirrors, the memory-mapped safetensors reader against the ``safetensors`` package, and the native
GGML dequantisers against numpy. Wall-clock, best of ``--repeat`` runs.

    python benchmarks/bench_host_runtime.py [--requests 256] [--file-mb 512] [--repeat 3]
"""
from __future__ import annotations

import argparse
import os
import random
import sys
import tempfile
import time

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from rmlx_b200.config import SchedulerConfig  # noqa: E402
from rmlx_b200.kv.paged import BlockManager  # noqa: E402
from rmlx_b200.loader import gguf, native_st  # noqa: E402
from rmlx_b200.serve import native  # noqa: E402
from rmlx_b200.serve.prefix_cache import PrefixCache  # noqa: E402
from rmlx_b200.serve.scheduler import GenerationRequest, Scheduler  # noqa: E402


def best(fn, repeat):
    t = []
    for _ in range(repeat):
        t0 = time.perf_counter()
        r = fn()
        t.append(time.perf_counter() - t0)
    return min(t), r


def drive(sched, bm, reqs):
    """A serving loop without a model: every scheduled sequence produces one token per step."""
    for r in reqs:
        sched.add_request(GenerationRequest(*r))
    finished, steps = {}, 0
    while sched.has_work():
        out = sched.schedule(bm, finished)
        finished = {}
        for m in out.prefill_seqs:
            if out.prefill_chunk_range[1] >= m.prompt_len:
                finished[m.seq_id] = 7
        for m in out.decode_seqs:
            finished[m.seq_id] = 7
        for sid, t in finished.items():
            sched.update_sequence(sid, bm, t)
        steps += 1
    return steps


def bench_scheduler(n_requests, repeat):
    rng = random.Random(0)
    reqs = [(i, [rng.randrange(1000) for _ in range(rng.randint(64, 1024))], rng.randint(16, 128))
            for i in range(n_requests)]
    cfg = SchedulerConfig(max_batch_size=64, eos_token_id=-1, block_size=16, max_prefill_chunk=512)
    for tables in (True, False):           # the serving engine asks for no block tables in the step plan
        t_py, steps = best(lambda: drive(Scheduler(cfg, tables_in_meta=tables), BlockManager(8192, 16), reqs), repeat)
        t_nat, steps2 = best(lambda: drive(native.NativeScheduler(cfg, tables_in_meta=tables),
                                           native.NativeBlockManager(8192, 16), reqs), repeat)
        assert steps == steps2
        print(f"scheduler + block manager, {n_requests} requests, batch 64, {steps} steps, "
              f"block tables in the plan: {tables}: python {t_py / steps * 1e6:7.1f} us/step   "
              f"native {t_nat / steps * 1e6:7.1f} us/step   ({t_py / t_nat:.1f}x)")


def bench_prefix_cache(repeat):
    rng = random.Random(1)
    system = [rng.randrange(1000) for _ in range(2048)]
    prompts = [system[:rng.randrange(256, 2048)] + [rng.randrange(1000) for _ in range(256)] for _ in range(400)]

    def run(pc):
        nb = 1
        for p in prompts:
            pc.lookup(p)
            blocks = list(range(nb, nb + len(p) // 16))
            nb += len(blocks)
            pc.insert_blocks(p, blocks)
        return len(pc)

    t_py, n1 = best(lambda: run(PrefixCache(16)), repeat)
    t_nat, n2 = best(lambda: run(native.NativePrefixCache(16)), repeat)
    assert n1 == n2
    print(f"prefix cache, 400 lookups + inserts of ~1.4 k-token prompts ({n1} blocks): "
          f"python {t_py * 1e3:7.1f} ms   native {t_nat * 1e3:7.1f} ms   ({t_py / t_nat:.1f}x)")


def bench_loader(file_mb, repeat):
    from safetensors.torch import load_file, save_file
    n = file_mb * (1 << 20) // 2 // 8
    tensors = {f"model.layers.{i}.w": torch.zeros(n, dtype=torch.bfloat16) for i in range(8)}
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "m.safetensors")
        save_file(tensors, path)
        size = os.path.getsize(path) / 1e9

        def pkg():
            return sum(int(t[0]) for t in load_file(path).values())

        def nat_open():
            return sum(int(t[0]) for t in native_st.load_file(path).values())

        pinned = torch.empty(n, dtype=torch.bfloat16)

        def nat_read():
            f = native_st.SafetensorsFile(path)
            for k in f.keys():
                f.read_into(k, pinned)
            return 0

        t_pkg, _ = best(pkg, repeat)
        t_open, _ = best(nat_open, repeat)
        t_read, _ = best(nat_read, repeat)
        print(f"safetensors, {size:.2f} GB file (page cache warm): package load_file {t_pkg * 1e3:7.1f} ms   "
              f"native open + views {t_open * 1e3:7.2f} ms   native threaded copy of every tensor "
              f"{t_read * 1e3:7.1f} ms ({size / t_read:.1f} GB/s)")


def bench_dequant(repeat):
    rng = np.random.default_rng(0)
    for name in ("Q4_0", "Q8_0", "Q4_K", "Q6_K"):
        t = gguf._T[name]
        _, be, bb = gguf.GGML_TYPES[t]
        nblocks = (64 << 20) // be                      # 64 Mi weights
        raw = rng.integers(0, 256, size=nblocks * bb, dtype=np.uint8)
        for off in {"Q4_0": [0], "Q8_0": [0], "Q4_K": [0, 2], "Q6_K": [208]}[name]:   # fp16 scale fields
            hi = raw.reshape(nblocks, bb)[:, off + 1]
            hi[(hi & 0x7C) == 0x7C] &= 0xBF                                          # keep them finite
            hi &= 0xBF                                                               # and small (|d| < 2)
        t_np, _ = best(lambda: gguf.dequantize_numpy(raw, t), max(1, repeat - 1))
        t_nat, _ = best(lambda: gguf.dequantize(raw, t), repeat)
        print(f"dequantise {name}: 64 Mi weights   numpy {t_np * 1e3:7.1f} ms   native {t_nat * 1e3:7.1f} ms "
              f"({64 * 4 / 1024 / t_nat:.1f} GB/s of fp32 out, {t_np / t_nat:.1f}x)")


def bench_sampler(repeat):
    """Host-side sampling of one token per row from 151936 logits: the torch-op sampler against the
    native one (same distribution; each draws from its own seeded generator)."""
    import torch
    from rmlx_b200.config import SamplerConfig
    from rmlx_b200.serve.native import NativeSampler
    from rmlx_b200.serve.sampler import Sampler
    torch.manual_seed(0)
    for rows in (1, 8):
        logits = torch.randn(rows, 151936)
        hist = [list(range(0, 400, 3)) for _ in range(rows)]
        for name, cfg in (("top-k 40, top-p 0.9, penalty 1.1",
                           SamplerConfig(temperature=0.8, top_k=40, top_p=0.9, repetition_penalty=1.1, seed=0)),
                          ("temperature only", SamplerConfig(temperature=0.8, seed=0)),
                          ("top-p 0.9 only (flat logits: 60 % of the vocabulary is the nucleus)",
                           SamplerConfig(temperature=0.8, top_p=0.9, seed=0))):
            t = []
            for cls in (Sampler, NativeSampler):
                smp = cls(cfg)
                smp.sample_batch(logits, hist)
                t.append(best(lambda: [smp.sample_batch(logits, hist) for _ in range(5)], repeat)[0] / 5)
            print(f"sampler, {rows} row(s), {name}: torch ops {t[0] * 1e3:6.2f} ms   native {t[1] * 1e3:6.2f} ms "
                  f"({t[0] / t[1]:.1f}x)")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--requests", type=int, default=256)
    ap.add_argument("--file-mb", type=int, default=512)
    ap.add_argument("--repeat", type=int, default=3)
    a = ap.parse_args()
    print(f"# host runtime micro-benchmarks, {os.cpu_count()} CPUs")
    bench_scheduler(a.requests, a.repeat)
    bench_prefix_cache(a.repeat)
    bench_loader(a.file_mb, a.repeat)
    bench_dequant(a.repeat)
    bench_sampler(a.repeat)


if __name__ == "__main__":
    main()
