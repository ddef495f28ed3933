#!/usr/bin/env python
"""Headline benchmark: decode throughput of the 60-layer MoE-A22B-shaped model (hidden 4096,
64 q / 4 kv heads, head_dim 128, 128 experts top-8, expert width 1536, vocab 151936) at batch 1 on
a paged KV cache pre-filled to 4096 tokens, tensor-parallel over N GPUs of one node, one CUDA-graph
replay per token. Prints ONE JSON line on rank 0.

    python bench.py --gpus 1 --steps 64 --warmup 8
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29500 bench.py --gpus 8 --steps 64 --warmup 8

The headline value is the model's MLX-affine Q4 (group 64) weight variant with bf16 activations and
fp32 accumulation: the bf16 model is 298 GB and does not fit one 180 GB GPU, and the scaling run
needs the same model at every N. From N = 2 on the line also carries

  "bf16"         the same engine on bf16 weights (the configuration the target names), and
  "nccl_cublas"  the same model written in plain PyTorch (``benchmarks/baseline_torch.py``: cuBLAS
                 GEMMs, library attention, ``torch.distributed`` all-reduce, eager launches, none
                 of this package's kernels): the bar the fused path has to beat on the same box,

plus ``tp_selfcheck_max_rel_err`` (fused projection + all-reduce kernels against an fp32
``dist.all_reduce`` on a tiny shape, measured before timing). Every number is device-timed with CUDA
events over ``--windows`` windows of ``--steps`` steps (median reported, min and max beside it), max
over ranks.

The published reference figure is its fused 7-dispatch decode at 703 us per layer over a 60-layer
pipeline (README.md:92 of the reference), i.e. 23.7 tokens/s on an M3 Ultra, f16, dense model.
"""
from __future__ import annotations

import argparse
import gc
import json
import os
import subprocess
import sys
import threading
import time

REF_TOKENS_PER_S = 1e6 / (703.0 * 60.0)   # 703 us/layer x 60 layers per token


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--windows", type=int, default=10, help="timed windows of --steps steps each")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--weights", default="q4", choices=["q4", "bf16"])
    ap.add_argument("--layers", type=int, default=60)
    ap.add_argument("--ctx", type=int, default=4096, help="tokens already in the KV cache")
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--no-pdl", action="store_true")
    ap.add_argument("--arms", default="auto",
                    help="comma list of extra arms: bf16, nccl_cublas; 'auto' = both from 2 GPUs on, "
                         "'none' = headline only")
    return ap.parse_args()


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.idx, self.proc, self.lines = gpu_index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.idx)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _read(self):
        for ln in self.proc.stdout:
            self.lines.append(ln.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def reference_arm(args):
    # The reference is a Rust workspace whose GPU code is Metal Shading Language compiled with
    # Apple's toolchain for Apple GPUs; it has no Python package and no CUDA path, so there is
    # nothing pip can install or run on this machine.
    print(json.dumps({"impl": "reference",
                      "unavailable": "reference is Rust + Apple Metal (macOS-only, needs xcrun metal "
                                     "and an Apple GPU); no pip-installable or CUDA path exists"}))
    return 0


def _stats(ms_list):
    s = sorted(ms_list)
    return s[len(s) // 2], s[0], s[-1]


class Ctx:
    def __init__(self, args):
        import torch
        import torch.distributed as dist
        self.torch, self.dist = torch, dist
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(self.local)
        self.dev = torch.device("cuda", self.local)
        if self.world > 1:
            dist.init_process_group("nccl", device_id=self.dev)
        self.args = args

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def max_over_ranks(self, vals):
        if self.world == 1:
            return list(vals)
        t = self.torch.tensor(list(vals), device=self.dev, dtype=self.torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return [float(v) for v in t]

    def free(self):
        gc.collect()
        self.torch.cuda.synchronize()
        self.torch.cuda.empty_cache()


def build_ours(c: Ctx, weights: str, total_steps: int):
    torch = c.torch
    from rmlx_b200.config import moe_a22b_config
    from rmlx_b200.models.decode_engine import CachedDecode
    from rmlx_b200.models.transformer import TransformerModel
    from rmlx_b200.models.weights import ParallelLayout, random_on_device
    a = c.args
    B, ctx = a.batch, a.ctx
    cfg = moe_a22b_config(a.layers, max_seq_len=ctx + 2 * total_steps + 64)
    quant = None if weights == "bf16" else "q4"
    w = random_on_device(cfg, c.dev, quant, ParallelLayout(c.rank, c.world), seed=0)
    comm = None
    if c.world > 1:
        import torch.distributed as dist

        def allreduce(t):
            t = t.contiguous()
            dist.all_reduce(t)
            return t

        def allgather(t):
            parts = [torch.empty_like(t) for _ in range(c.world)]
            dist.all_gather(parts, t.contiguous())
            return torch.cat(parts, -1)

        model = TransformerModel(w, allreduce, allgather)
        from rmlx_b200.parallel.comm import make_comm
        comm = make_comm("fused", model, max_batch=min(B, 4))
    else:
        model = TransformerModel(w)
    bps = (cfg.max_seq_len + 15) // 16
    cache = model.new_cache(1 + B * bps, max_seqs=B, max_blocks_per_seq=bps)
    for s in range(B):      # synthetic context: K/V ~ N(0,1) for `ctx` tokens per sequence
        cache.add_sequence(s)
        cache.reserve(s, ctx)
        cache.commit(s, ctx)
    for l in range(cfg.num_layers):
        cache.k[l].normal_(0, 1)
        cache.v[l].normal_(0, 1)
    if B <= 4:
        eng = CachedDecode(model, cache, max_batch=B, use_graph=not a.no_graph, pdl=not a.no_pdl, comm=comm)
    else:   # more rows than one mat-vec launch takes: the tensor-core decode step
        from rmlx_b200.models.prefill import BatchedDecode, enable_native_prefill
        if c.world > 1:      # row-parallel GEMMs fused with their all-reduce over NVLink
            from rmlx_b200.parallel.tp_gemm import make_gemm_comm
            i_local = max([l.w_gate_up.n // 2 for l in w.layers if l.w_gate_up is not None] + [64])
            model.gemm_comm = make_gemm_comm("fused", B, cfg.hidden_size,
                                             max(model.hq * cfg.head_dim, i_local), device=c.dev)
        enable_native_prefill(model)
        eng = BatchedDecode(model, cache, max_batch=B, use_graph=not a.no_graph)
    eng.bind(list(range(B)), [1] * B)
    eng.reserve(total_steps + 1)
    torch.cuda.synchronize()
    return cfg, w, model, comm, cache, eng


def time_engine(c: Ctx, eng, steps: int, windows: int):
    """`windows` windows of `steps` steps, CUDA events, returns per-window ms per step."""
    torch = c.torch
    out = []
    for _ in range(windows):
        c.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            eng.step()
        e1.record()
        torch.cuda.synchronize()
        out.append(e0.elapsed_time(e1) / steps)
    return c.max_over_ranks(out)


def e2e_engine(c: Ctx, eng, steps: int):
    """Through the public API: every step copies the next input token(s) from pinned host memory
    to the device, runs one decode step and reads the sampled token(s) back."""
    torch = c.torch
    B = c.args.batch
    pin_in = torch.ones(B, dtype=torch.int32).pin_memory()
    pin_out = torch.zeros(B, dtype=torch.int32).pin_memory()

    def one():
        eng.tokens.copy_(pin_in, non_blocking=True)
        pin_out.copy_(eng.step(), non_blocking=True)
        torch.cuda.current_stream().synchronize()
        pin_in.copy_(pin_out)

    for _ in range(4):
        one()
    c.barrier()
    w0 = time.perf_counter()
    for _ in range(steps):
        one()
    c.barrier()
    return c.max_over_ranks([(time.perf_counter() - w0) * 1e3 / steps])[0]


def tp_selfcheck(c: Ctx):
    """Fused mat-vec + all-reduce and fused GEMM + all-reduce on tiny shapes against
    ``dist.all_reduce`` of the fp32 partial products. Returns the largest relative error."""
    torch, dist = c.torch, c.dist
    from rmlx_b200.ops.weights import LinearWeight
    from rmlx_b200.parallel.comm import PeerComm
    from rmlx_b200.parallel.tp_gemm import FusedGemmComm
    g = torch.Generator(device=c.dev).manual_seed(77 + c.rank)
    n, k = 512, 1024
    worst = 0.0
    comm = PeerComm(n, 2, device=c.dev)
    for quant in (None, "q4"):
        w = LinearWeight.from_dense((torch.randn(n, k, generator=g, device=c.dev) * 0.05).cpu(), quant, device=c.dev)
        x = torch.randn(2, k, device=c.dev, generator=g).to(torch.bfloat16)
        want = x.float() @ w.dequantized().t()
        dist.all_reduce(want)
        got = torch.empty(2, n, dtype=torch.bfloat16, device=c.dev)
        comm.gemv_allreduce(x, w, None, got)
        torch.cuda.synchronize()
        worst = max(worst, ((got.float() - want).abs().max() / want.abs().max()).item())
    if comm.status() != 0:
        worst = float("inf")
    comm.close()
    gc_ = FusedGemmComm(256, n, k, device=c.dev)
    w = LinearWeight.from_dense((torch.randn(n, k, generator=g, device=c.dev) * 0.05).cpu(), None, device=c.dev)
    x = torch.randn(256, k, device=c.dev, generator=g).to(torch.bfloat16)
    want = x.float() @ w.dequantized().t()
    dist.all_reduce(want)
    got = gc_.gemm_allreduce(x, w)
    torch.cuda.synchronize()
    worst = max(worst, ((got.float() - want).abs().max() / want.abs().max()).item())
    gc_.close()
    return c.max_over_ranks([worst])[0]


def run_baseline(c: Ctx, steps: int, warmup: int, windows: int):
    sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "benchmarks"))
    from baseline_torch import TorchMoeDecoder, time_decode
    a = c.args
    need = 2 * (a.layers * (9216 * 4096 + 4096 * 8192 + 128 * 4096 + 128 * 3 * 1536 * 4096) + 2 * 151936 * 4096)
    free, _ = c.torch.cuda.mem_get_info()
    if need / c.world > 0.92 * free:
        return {"unavailable": f"bf16 weights need {need / c.world / 2**30:.0f} GiB per GPU"}
    m = TorchMoeDecoder(layers=a.layers, hidden=4096, heads=64, kv_heads=4, head_dim=128, experts=128,
                        top_k=8, inter=1536, vocab=151936, max_len=a.ctx + (warmup + windows * steps) + 8,
                        batch=a.batch, rank=c.rank, world=c.world, device=c.dev)
    m.fill_context(a.ctx)
    ms = c.max_over_ranks(time_decode(m, a.ctx, steps, warmup, windows))
    med, lo, hi = _stats(ms)
    out = {"value": round(a.batch * 1000.0 / med, 2), "unit": "tokens/s", "ms_per_step": round(med, 4),
           "ms_per_step_min": round(lo, 4), "ms_per_step_max": round(hi, 4),
           "us_per_layer": round(med * 1e3 / a.layers, 2), "windows": len(ms), "weights": "bf16",
           "how": "plain PyTorch, eager: F.linear / matmul (cuBLAS), scaled_dot_product_attention, "
                  "topk, dist.all_reduce (NCCL); no kernel of this package"}
    del m
    return out


def main():
    args = parse()
    if args.impl == "reference":
        return reference_arm(args)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.gpus != world and world == 1 and args.gpus > 1:
        print(f"bench.py: --gpus {args.gpus} needs torchrun with {args.gpus} ranks", file=sys.stderr)
        return 2
    c = Ctx(args)
    torch = c.torch
    t_start = time.time()
    arms = {"auto": ["bf16", "nccl_cublas"] if world > 1 else [], "none": []}.get(
        args.arms, [x for x in args.arms.split(",") if x])
    total_steps = args.warmup + args.windows * args.steps + 8 + args.steps

    selfcheck = tp_selfcheck(c) if world > 1 else None

    # ---------------- headline arm ----------------
    cfg, weights, model, comm, cache, eng = build_ours(c, args.weights, total_steps)
    setup_s = time.time() - t_start
    for _ in range(max(3, args.warmup)):
        eng.step()
    c.barrier()
    sampler = ClockSampler(c.local)
    if c.rank == 0:
        sampler.start()
        time.sleep(0.3)
    ms_windows = time_engine(c, eng, args.steps, args.windows)
    clocks = sampler.stop() if c.rank == 0 else None
    e2e_ms = e2e_engine(c, eng, args.steps)
    status = comm.status() if comm is not None else 0
    launches = eng.launches_per_step
    use_graph = bool(getattr(eng, "use_graph", False))
    graphs = getattr(eng, "graphs", None)
    graph_store = "none" if not use_graph else \
        "native store (csrc/runtime/graph_exec.cu)" if getattr(graphs, "native_captures", 0) else "torch.cuda.CUDAGraph"
    graph_retries = int(getattr(graphs, "capture_failures", 0))
    graph_eager = int(getattr(graphs, "eager_fallbacks", 0))
    del graphs                       # plain numbers only from here on: the cache must die with the engine
    nbytes = weights.nbytes()
    nlayers = cfg.num_layers
    extra = {}

    def release():
        nonlocal cfg, weights, model, comm, cache, eng
        if comm is not None:
            comm.close()
        if getattr(model, "gemm_comm", None) is not None:
            model.gemm_comm.close()
        cfg = weights = model = comm = cache = eng = None
        c.free()

    # ---------------- the same engine on bf16 weights ----------------
    if "bf16" in arms and args.weights != "bf16":
        release()
        try:
            cfg, weights, model, comm, cache, eng = build_ours(c, "bf16", total_steps)
            for _ in range(max(3, args.warmup)):
                eng.step()
            ms_b = time_engine(c, eng, args.steps, max(3, args.windows // 2))
            med, lo, hi = _stats(ms_b)
            extra["bf16"] = {"value": round(args.batch * 1000.0 / med, 2), "unit": "tokens/s",
                             "ms_per_step": round(med, 4), "ms_per_step_min": round(lo, 4),
                             "ms_per_step_max": round(hi, 4), "us_per_layer": round(med * 1e3 / nlayers, 2),
                             "windows": len(ms_b), "weight_bytes_per_gpu": weights.nbytes(),
                             "comm_status": comm.status() if comm is not None else 0}
        except torch.OutOfMemoryError:
            extra["bf16"] = {"unavailable": "bf16 weights do not fit this many GPUs"}
    # ---------------- NCCL + cuBLAS PyTorch build of the same model ----------------
    if "nccl_cublas" in arms:
        release()
        try:
            extra["nccl_cublas"] = run_baseline(c, min(args.steps, 16), 3, 3)
        except torch.OutOfMemoryError:
            extra["nccl_cublas"] = {"unavailable": "bf16 weights do not fit this many GPUs"}
        c.free()

    if c.rank == 0:
        med, lo, hi = _stats(ms_windows)
        B = args.batch
        value = B * 1000.0 / med
        out = {
            "metric": "decode_tokens_per_s", "value": round(value, 2), "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": round(med, 4), "ms_per_step_min": round(lo, 4), "ms_per_step_max": round(hi, 4),
            "windows": len(ms_windows), "higher_is_better": True, "scaling": "strong",
            "vs_baseline": round(value / REF_TOKENS_PER_S, 2),
            "dtype": "q4w-bf16a" if args.weights == "q4" else "bf16", "data": "synthetic",
            "us_per_layer": round(med * 1e3 / nlayers, 2),
            "config": {"model": f"moe-a22b-shaped {nlayers}L (hidden 4096, 64q/4kv, 128 experts "
                                f"top-8 x1536, vocab 151936), random init",
                       "weights": "q4 group-64 affine (bf16 activations, fp32 accumulate)"
                       if args.weights == "q4" else "bf16",
                       "global_batch": B, "seq_len": args.ctx, "kv": "paged (page 16), ~N(0,1) context",
                       "parallelism": f"tp{world}", "cuda_graph": use_graph, "graph_store": graph_store,
                       "graph_recordings_retried": graph_retries,
                       "graph_keys_run_launch_by_launch": graph_eager,
                       "tp_reduction": "fused" if world > 1 else "none",
                       "l2": "no flush needed: each step streams the active weights of "
                             f"{nlayers} layers (>> 126 MB L2) so nothing is reused across steps",
                       "weight_bytes_per_gpu": nbytes},
            "clocks": clocks,
            "e2e": {"value": round(B * 1000.0 / e2e_ms, 2), "unit": "tokens/s",
                    "ms_per_step": round(e2e_ms, 4),
                    "h2d_bytes_per_step": 4 * B, "d2h_bytes_per_step": 4 * B},
            "gpu_launches": launches * args.steps * args.windows,
            "launches_per_step": launches,
            "comm_status": status, "setup_s": round(setup_s, 1), "impl": "ours",
            "total_s": round(time.time() - t_start, 1),
        }
        if selfcheck is not None:
            out["tp_selfcheck_max_rel_err"] = round(selfcheck, 5)
        out.update(extra)
        print(json.dumps(out))
    if world > 1:
        c.dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
