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
