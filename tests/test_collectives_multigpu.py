"""Peer-memory collectives on 2+ GPUs against torch.distributed (NCCL) on the same tensors; several
rounds per operation so that the alternating receive areas and the growing counters recycle."""
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
        from rmlx_b200.parallel.collectives import PeerCollectives
        pc = PeerCollectives(1 << 20, device=dev, blocks=8)
        bad = []
        g = torch.Generator(device=dev).manual_seed(7 + rank)
        for rnd in range(3):
            for dtype in (torch.bfloat16, torch.float32):
                n = 1024 * (rnd + 1)
                x = torch.randn(world * n, 8, device=dev, generator=g).to(dtype)
                # all-reduce
                want = x.clone(); dist.all_reduce(want)
                got = pc.all_reduce(x)
                tol = 2e-2 if dtype == torch.bfloat16 else 1e-5
                if not torch.allclose(got.float(), want.float(), rtol=tol, atol=tol):
                    bad.append(("all_reduce", rnd, str(dtype)))
                # reduce-scatter
                want_rs = torch.empty(n, 8, device=dev, dtype=dtype)
                dist.reduce_scatter_tensor(want_rs, x)
                if not torch.allclose(pc.reduce_scatter(x).float(), want_rs.float(), rtol=tol, atol=tol):
                    bad.append(("reduce_scatter", rnd, str(dtype)))
                # all-gather
                want_ag = torch.empty(world * n, 8, device=dev, dtype=dtype)
                dist.all_gather_into_tensor(want_ag, x[:n].contiguous())
                if not torch.equal(pc.all_gather(x[:n]), want_ag):
                    bad.append(("all_gather", rnd, str(dtype)))
                # all-to-all
                want_a2a = torch.empty_like(x)
                dist.all_to_all_single(want_a2a, x)
                if not torch.equal(pc.all_to_all(x), want_a2a):
                    bad.append(("all_to_all", rnd, str(dtype)))
                # broadcast from the last rank
                want_b = x.clone(); dist.broadcast(want_b, world - 1)
                if not torch.equal(pc.broadcast(x, root=world - 1), want_b):
                    bad.append(("broadcast", rnd, str(dtype)))
        # the Group API takes the same kernels for CUDA tensors that fit them, the library otherwise
        from rmlx_b200.parallel.group import Group
        grp = Group()
        x = torch.randn(world * 512, 16, device=dev, generator=g).to(torch.bfloat16)
        want = x.clone(); dist.all_reduce(want)
        if not torch.allclose(grp.allreduce(x).float(), want.float(), rtol=2e-2, atol=2e-2):
            bad.append(("group.allreduce",))
        want_ag = torch.empty(world * x.shape[0], 16, device=dev, dtype=x.dtype)
        dist.all_gather_into_tensor(want_ag, x)
        if not torch.equal(grp.allgather(x), want_ag):
            bad.append(("group.allgather",))
        want_rs = torch.empty(512, 16, device=dev, dtype=x.dtype)
        dist.reduce_scatter_tensor(want_rs, x)
        if not torch.allclose(grp.reduce_scatter(x).float(), want_rs.float(), rtol=2e-2, atol=2e-2):
            bad.append(("group.reduce_scatter",))
        want_a2a = torch.empty_like(x); dist.all_to_all_single(want_a2a, x)
        if not torch.equal(grp.all_to_all(x), want_a2a):
            bad.append(("group.all_to_all",))
        y = x.clone(); want_b = x.clone(); dist.broadcast(want_b, 0)
        if not torch.equal(grp.broadcast(y, 0), want_b):
            bad.append(("group.broadcast",))
        if grp.native_calls != 5 or grp.library_calls != 0:
            bad.append(("group routing", grp.native_calls, grp.library_calls))
        odd = torch.randn(7, device=dev)                     # 28 bytes: not whole 16-byte vectors
        want_odd = odd.clone(); dist.all_reduce(want_odd)
        if not torch.allclose(grp.allreduce(odd), want_odd) or grp.library_calls != 1:
            bad.append(("group fallback", grp.library_calls))
        # point-to-point over the heap: a ring of messages, three rounds (slots and counters recycle)
        grp.enable_native_p2p(1 << 16)
        nxt, prv = (rank + 1) % world, (rank - 1) % world
        before = grp.native_calls
        for rnd in range(3):
            msg = torch.full((1000,), float(100 * rnd + rank), device=dev)
            got = grp.sendrecv(msg, torch.empty_like(msg), nxt) if world == 2 else None
            if world == 2:
                if not torch.all(got == float(100 * rnd + prv)):
                    bad.append(("group.sendrecv", rnd))
            else:
                grp.send(msg, nxt)
                got = grp.recv(torch.empty_like(msg), prv)
                if not torch.all(got == float(100 * rnd + prv)):
                    bad.append(("group.send/recv", rnd))
        if grp.native_calls == before:
            bad.append(("p2p went to the library",))
        ch = grp._chan
        ch.put(nxt, torch.full((64,), float(rank + 7), device=dev), slot=rank)   # one-sided
        torch.cuda.synchronize()
        dist.barrier()
        peek = ch.get(rank, torch.empty(64, device=dev), slot=prv)
        if not torch.all(peek == float(prv + 7)):
            bad.append(("put/get",))
        if ch.status():
            bad.append(("p2p status", ch.status()))
        grp.close()
        torch.cuda.synchronize()
        status = pc.status()
        dist.barrier()
        pc.close()
        ret.put((rank, bad, status))
    except Exception as e:      # report instead of leaving the parent to time out
        import traceback
        ret.put((rank, f"{e!r}\n{traceback.format_exc()}", -1))
        raise
    finally:
        dist.destroy_process_group()


def test_peer_collectives_match_nccl():
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
    for rank, bad, status in results:
        assert not isinstance(bad, str), bad
        assert status == 0, (rank, status)
        assert bad == [], (rank, bad)
