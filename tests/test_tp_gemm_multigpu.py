"""Tensor-parallel GEMMs with the collective inside the tensor-core kernel, on 2+ GPUs: results
against a plain fp32 matmul of the unsharded operands and against the GEMM + NCCL baseline; several
calls per shape so that the per-shape counters and the alternating buffers recycle."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from rmlx_b200.ops.weights import LinearWeight
        from rmlx_b200.parallel.tp_gemm import make_gemm_comm
        comm = make_gemm_comm("fused", 1024, 1024, 1024 * world, device=dev)
        base = make_gemm_comm("nccl", 1024, 1024, 1024 * world, device=dev)
        errs = []
        g = torch.Generator().manual_seed(0)           # same stream of numbers on every rank
        for quant in (None, "q4"):
            for (m, n, k) in ((512, 1024, 512 * world), (300, 512, 1024 * world), (512, 1024, 512 * world)):
                kl = k // world
                x = torch.randn(m, k, generator=g)
                wd = torch.randn(n, k, generator=g) * 0.05
                res = torch.randn(m, n, generator=g).to(torch.bfloat16)
                xs = x[:, rank * kl:(rank + 1) * kl].to(torch.bfloat16).to(dev).contiguous()
                w = LinearWeight.from_dense(wd[:, rank * kl:(rank + 1) * kl].contiguous(), quant, device=dev)
                # fp32 oracle from what every rank's kernel sees
                part = xs.float() @ w.dequantized().float().t()
                dist.all_reduce(part)
                want = part + res.to(dev).float()
                for it in range(3):
                    got = comm.gemm_allreduce(xs, w, residual=res.to(dev))
                    torch.cuda.synchronize()
                    errs.append(((got.float() - want).abs().max() / want.abs().max()).item())
                b = base.gemm_allreduce(xs, w, residual=res.to(dev))
                errs.append(((b.float() - want).abs().max() / want.abs().max()).item())
                if m % (128 * world) == 0:
                    # GEMM + reduce-scatter: the owner keeps its 128-row blocks, nothing is broadcast
                    rows = comm.owned_rows(m).to(dev)
                    for it in range(2):
                        mine = comm.gemm_reduce_scatter(xs, w, residual=res.to(dev))
                        torch.cuda.synchronize()
                        assert mine.shape == (m // world, n)
                        errs.append(((mine.float() - want[rows]).abs().max() / want.abs().max()).item())
                    bm = base.gemm_reduce_scatter(xs, w, residual=res.to(dev))
                    errs.append(((bm.float() - want[rows]).abs().max() / want.abs().max()).item())
            # all-gather + GEMM: rows sharded, weight columns sharded
            for (ms, n, k) in ((128, 512, 1024), (256, 1024, 512)):
                m = ms * world
                x = torch.randn(m, k, generator=g).to(torch.bfloat16)
                wd = torch.randn(n, k, generator=g) * 0.05
                nl = n // world
                w = LinearWeight.from_dense(wd[rank * nl:(rank + 1) * nl].contiguous(), quant, device=dev)
                want = x.to(dev).float() @ w.dequantized().float().t()
                shard = x[rank * ms:(rank + 1) * ms].to(dev).contiguous()
                for it in range(3):
                    got = comm.allgather_gemm(shard, w)
                    torch.cuda.synchronize()
                    errs.append(((got.float() - want).abs().max() / want.abs().max()).item())
                b = base.allgather_gemm(shard, w)
                errs.append(((b.float() - want).abs().max() / want.abs().max()).item())
        torch.cuda.synchronize()
        status = comm.status()
        dist.barrier()
        ret.put((rank, max(errs), status))
        comm.close()
    except Exception as e:      # report instead of leaving the parent to time out
        import traceback
        ret.put((rank, f"{e!r}\n{traceback.format_exc()}", -1))
        raise
    finally:
        dist.destroy_process_group()


def test_fused_tp_gemms_match_oracle():
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs two GPUs")
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    try:
        results = [q.get(timeout=90) for _ in range(world)]
    finally:
        for p in procs:
            p.join(timeout=30)
            if p.is_alive():
                p.kill()
    for rank, err, status in results:
        assert not isinstance(err, str), err
        assert status == 0, (rank, status)
        assert err < 2e-2, (rank, err)


def _prefill_worker(rank, world, port, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from rmlx_b200.config import FeedForwardType, TransformerConfig
        from rmlx_b200.models.prefill import enable_native_prefill
        from rmlx_b200.models.transformer import TransformerModel
        from rmlx_b200.models.weights import ParallelLayout, from_state_dict, random_state_dict
        from rmlx_b200.parallel.tp_gemm import make_gemm_comm
        cfg = TransformerConfig(hidden_size=512, num_heads=8, num_kv_heads=4, head_dim=64, num_layers=2,
                                vocab_size=1024, max_seq_len=512, rope_theta=1e4,
                                ff_type=FeedForwardType.gated(1024), name="tp-prefill").validate()
        sd = random_state_dict(cfg, 0)

        def allreduce(t):
            t = t.contiguous()
            dist.all_reduce(t)
            return t

        def allgather(t):
            parts = [torch.empty_like(t) for _ in range(world)]
            dist.all_gather(parts, t.contiguous())
            return torch.cat(parts, -1)

        model = TransformerModel(from_state_dict(cfg, sd, device=dev, layout=ParallelLayout(rank, world)),
                                 allreduce, allgather)
        model.gemm_comm = make_gemm_comm("fused", 256, 512, 512, device=dev)
        assert enable_native_prefill(model)
        g = torch.Generator().manual_seed(3)
        prompt = torch.randint(0, cfg.vocab_size, (200,), generator=g).to(dev)
        cache = model.new_cache(16, max_seqs=1)
        cache.add_sequence(0)
        got = model.prefill(prompt, cache, 0).float()
        torch.cuda.synchronize()
        status = model.gemm_comm.status()
        err = 0.0
        if rank == 0:
            full = TransformerModel(from_state_dict(cfg, sd, device=dev))
            assert enable_native_prefill(full)
            c1 = full.new_cache(16, max_seqs=1)
            c1.add_sequence(0)
            want = full.prefill(prompt, c1, 0).float()
            err = ((got - want).abs().max() / want.abs().max()).item()
        dist.barrier()
        ret.put((rank, err, status))
        model.gemm_comm.close()
    except Exception as e:      # report instead of leaving the parent to time out
        import traceback
        ret.put((rank, f"{e!r}\\n{traceback.format_exc()}", -1))
        raise
    finally:
        dist.destroy_process_group()


def test_tensor_parallel_native_prefill_matches_single_gpu():
    """Prompt processing with the row-parallel projections on the fused GEMM + all-reduce kernel:
    logits equal the single-GPU native prefill up to the rounding of the sharded sums."""
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs two GPUs")
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_prefill_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    try:
        results = [q.get(timeout=90) for _ in range(world)]
    finally:
        for p in procs:
            p.join(timeout=30)
            if p.is_alive():
                p.kill()
    for rank, err, status in results:
        assert not isinstance(err, str), err
        assert status == 0, (rank, status)
        assert err < 4e-2, (rank, err)
