"""The symmetric heap on 2+ GPUs: identical offsets on every rank, peers see each other's blocks,
freed ranges come back zeroed, the heap grows by whole segments behind the existing ones, and (where
the box supports NVLink multicast) the in-switch all-reduce matches NCCL. The offset arena itself is
tested on the CPU (tests/test_parallel_cpu.py)."""
import datetime
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


def _view(ptr, nbytes, dev, dtype=torch.int32):
    from rmlx_b200.parallel.tp_gemm import _RawCuda
    return torch.as_tensor(_RawCuda(ptr, nbytes), device=dev).view(dtype)


def _worker(rank, world, port, multicast, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    os.environ["RMLX_SYMM_SEGMENT_MB"] = "64"
    os.environ["RMLX_SYMM_VA_GB"] = "2"
    os.environ["RMLX_SYMM_MULTICAST"] = "1" if multicast else "0"
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev,
                            timeout=datetime.timedelta(seconds=90))
    from rmlx_b200.parallel import symm_heap
    try:
        support = symm_heap.vmm_support()
        if not support & 1 or (multicast and not support & 2):
            ret.put((rank, "unsupported", support))
            return
        heap = symm_heap.default_heap()
        assert heap is not None and heap.multicast == multicast
        a = heap.alloc(1 << 20)
        b = heap.alloc(3 << 20)
        offs = [None] * world
        dist.all_gather_object(offs, (a.offset, b.offset))
        assert all(o == offs[0] for o in offs) and a.offset == 0 and b.offset == 1 << 20
        # fresh blocks are zero; every rank writes its own copy, peers read it through their mapping
        mine = _view(b.local, b.nbytes, dev)
        assert int(mine.abs().sum()) == 0
        mine.fill_(rank + 1)
        torch.cuda.synchronize()
        dist.barrier()
        for r in range(world):
            peer = _view(b.ptrs[r], b.nbytes, dev)
            assert int(peer[0]) == r + 1 and int(peer[-1]) == r + 1, (rank, r)
        dist.barrier()
        # a freed range is handed out again, zeroed
        _view(a.local, a.nbytes, dev).fill_(7)
        a.close()
        c = heap.alloc(1 << 19)
        assert c.offset == 0 and int(_view(c.local, c.nbytes, dev).abs().sum()) == 0
        # growth: a request larger than what is left adds a segment right behind the first
        d = heap.alloc(80 << 20)
        assert heap.stats["segments"] == 2 and d.offset + d.nbytes <= heap.capacity
        dv = _view(d.local, d.nbytes, dev)
        dv.fill_(100 + rank)
        torch.cuda.synchronize()
        dist.barrier()
        nxt = (rank + 1) % world
        pv = _view(d.ptrs[nxt], d.nbytes, dev)
        assert int(pv[0]) == 100 + nxt and int(pv[-1]) == 100 + nxt
        dist.barrier()
        bad = []
        if multicast:
            from rmlx_b200.parallel.collectives import PeerCollectives
            pc = PeerCollectives(1 << 20, device=dev)
            assert pc.nvls_available
            g = torch.Generator(device=dev).manual_seed(11 + rank)
            for rnd in range(3):
                for dtype in (torch.float32, torch.bfloat16):
                    x = torch.randn(4096 * (rnd + 1), 8, device=dev, generator=g).to(dtype)
                    want = x.clone()
                    dist.all_reduce(want)
                    got = pc.all_reduce_nvls(x)
                    tol = 3e-2 if dtype == torch.bfloat16 else 1e-5
                    if not torch.allclose(got.float(), want.float(), rtol=tol, atol=tol):
                        bad.append((rnd, str(dtype), float((got.float() - want.float()).abs().max())))
            # in place: the producer writes straight into the heap buffer
            buf = pc.nvls_buffer(torch.float32, 8192)
            buf.fill_(float(rank + 1))
            res = pc.all_reduce_nvls(numel=8192, dtype=torch.float32)
            torch.cuda.synchronize()
            if not torch.all(res == float(world * (world + 1) // 2)):
                bad.append(("in place", float(res[0])))
            st = pc.status()
            if st:
                bad.append(("status", st))
            pc.close()
        for blk in (b, c, d):
            blk.close()
        assert heap.bytes_in_use() == 0
        ret.put((rank, bad, heap.stats["segments"]))
    except Exception as e:      # report instead of leaving the parent to time out
        import traceback
        ret.put((rank, f"{e!r}\n{traceback.format_exc()}", -1))
    finally:
        try:
            symm_heap.close_heaps()      # unbinds the multicast objects before the process leaves
        finally:
            dist.destroy_process_group()


@pytest.mark.parametrize("multicast", [False, True])
def test_symmetric_heap(multicast):
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs two GPUs")
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, multicast, q)) for r in range(world)]
    for p in procs:
        p.start()
    try:
        results = [q.get(timeout=150) for _ in range(world)]
    finally:
        for p in procs:
            p.join(timeout=60)
            if p.is_alive():
                p.kill()
    if all(r[1] == "unsupported" for r in results):
        pytest.skip(f"the box does not support what the test needs (support bits {results[0][2]})")
    for rank, bad, segs in results:
        assert not isinstance(bad, str), bad
        assert bad == [], (rank, bad)
        assert segs == 2
