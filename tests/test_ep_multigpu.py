"""Expert-parallel dispatch / combine over peer memory on 2+ GPUs: the fused exchange and the whole
expert-parallel MoE block against a plain fp32 MoE over all experts (the semantics checked on CPU
ranks in tests/test_parallel_cpu.py), several calls in a row with different token counts per rank."""
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
        from rmlx_b200.parallel.ep_fused import FusedEpExchange, FusedEpMoe
        from rmlx_b200.reference import ops as ref
        E, k, d, inter = 4 * world, 2, 512, 512
        el = E // world
        g = torch.Generator().manual_seed(0)              # identical on every rank
        wgu = torch.randn(E, 2 * inter, d, generator=g) * 0.05
        wdn = torch.randn(E, d, inter, generator=g) * 0.05
        router = torch.randn(E, d, generator=g) * 0.2
        errs = []
        for quant in (None, "q4"):
            gu = LinearWeight.from_dense(wgu[rank * el:(rank + 1) * el].contiguous(), quant, device=dev)
            dn = LinearWeight.from_dense(wdn[rank * el:(rank + 1) * el].contiguous(), quant, device=dev)
            # what the kernels see, for every expert, on this rank (oracle only)
            gu_all = LinearWeight.from_dense(wgu, quant, device=dev).dequantized().float()
            dn_all = LinearWeight.from_dense(wdn, quant, device=dev).dequantized().float()
            ex = FusedEpExchange(256, d, k, E, device=dev, blocks=16)
            moe = FusedEpMoe(ex, gu, dn)
            for it, t in enumerate((96 + 16 * rank, 1, 200 - 8 * rank, 33)):
                gx = torch.Generator().manual_seed(100 * it + rank)
                x = torch.randn(t, d, generator=gx).to(torch.bfloat16).to(dev)
                res = torch.randn(t, d, generator=gx).to(torch.bfloat16).to(dev)
                got = moe.forward(x, router.to(dev).to(torch.bfloat16), k, residual=res)
                torch.cuda.synchronize()
                logits = x.float() @ router.to(dev).to(torch.bfloat16).float().t()
                idx, wts, _ = ref.topk_route(logits, k)
                want = ref.moe_ffn(x, idx, wts, gu_all, dn_all) + res.float()
                errs.append(((got.float() - want).abs().max() / want.abs().max()).item())
            # the whole layer as one CUDA-graph replay per token count (two replays each)
            rw = router.to(dev).to(torch.bfloat16)
            for it, t in enumerate((8, 64 + 8 * rank, 8)):
                for rep in range(2):
                    gx = torch.Generator().manual_seed(7000 + 100 * it + 10 * rep + rank)
                    x = torch.randn(t, d, generator=gx).to(torch.bfloat16).to(dev)
                    res = torch.randn(t, d, generator=gx).to(torch.bfloat16).to(dev)
                    # the same parameter tensor, or (second replay) a copy that the layer takes over
                    got = moe.forward_captured(x, rw if rep == 0 else rw.clone(), k, residual=res)
                    torch.cuda.synchronize()
                    logits = x.float() @ router.to(dev).to(torch.bfloat16).float().t()
                    idx, wts, _ = ref.topk_route(logits, k)
                    want = ref.moe_ffn(x, idx, wts, gu_all, dn_all) + res.float()
                    errs.append(((got.float() - want).abs().max() / want.abs().max()).item())
            assert moe.graphs.captures == 2 and moe.graphs.hits == 4
            status = ex.status()
            dist.barrier()
            ex.close()
            if status:
                break
        ret.put((rank, max(errs), status))
    except Exception as e:      # report instead of leaving the parent to time out
        import traceback
        ret.put((rank, f"{e!r}\n{traceback.format_exc()}", -1))
        raise
    finally:
        dist.destroy_process_group()


def test_fused_expert_parallel_moe_matches_oracle():
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
        assert err < 3e-2, (rank, err)
