"""Distributed plumbing without GPUs: rank/world resolution, Group collectives and split on gloo
ranks (one OS process per rank, like the mock-transport tests of
crates/rmlx-distributed/tests/tree_allreduce_tests.rs:10-121), health monitor with a host-side
failure, MoE policy hysteresis/cool-down, sparse guard, wire formats, slab ring, EP exchange
against the single-process oracle (crates/rmlx-distributed/tests/moe_tests.rs)."""
import os
import socket
import time

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from rmlx_b200.config import InitConfig, MoeConfig
from rmlx_b200.nn.moe import ExpertGroup, MoeLayer, MoeStrategy
from rmlx_b200.parallel import ep, wire
from rmlx_b200.parallel.group import DistributedError, Group, ReduceOp
from rmlx_b200.parallel.health import DictStore, HealthMonitor, HeartbeatConfig, HeartbeatSender, Watchdog
from rmlx_b200.parallel.init import init, resolve_backend, resolve_rank_world
from rmlx_b200.parallel.moe_policy import GuardAction, MoeBackend, MoePolicy, SparseGuard
from rmlx_b200.parallel.slab_ring import SlabRing, SlabRingConfig
from rmlx_b200.parallel.topology import parse_topo_matrix
from rmlx_b200.runtime.streams import WaitTimeout


def test_rank_resolution_order():
    assert resolve_rank_world(InitConfig(), {}) == (0, 1, 0)
    assert resolve_rank_world(InitConfig(), {"RANK": "3", "WORLD_SIZE": "8", "LOCAL_RANK": "3"}) == (3, 8, 3)
    assert resolve_rank_world(InitConfig(), {"RMLX_RANK": "1", "RMLX_WORLD_SIZE": "2", "RANK": "5",
                                             "WORLD_SIZE": "9"})[:2] == (1, 2)
    assert resolve_rank_world(InitConfig(rank=0, world_size=4), {"RANK": "2"})[:2] == (0, 4)
    assert resolve_rank_world(InitConfig(), {"SLURM_PROCID": "2", "SLURM_NTASKS": "4"})[:2] == (2, 4)
    with pytest.raises(DistributedError):
        resolve_rank_world(InitConfig(rank=4, world_size=2), {})
    assert resolve_backend(InitConfig(backend="gloo"), {}) == "gloo"
    assert resolve_backend(InitConfig(), {"RMLX_BACKEND": "loopback"}) == "loopback"
    ctx = init(InitConfig())
    assert ctx.is_loopback and ctx.world_size == 1
    g = ctx.group
    x = torch.arange(4.0)
    assert torch.equal(g.allreduce(x), x) and torch.equal(g.allgather(x), x)
    with pytest.raises(DistributedError):
        g.send(x, 1)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _group_worker(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"; os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = Group()
        x = torch.full((4,), float(rank + 1))
        ok = torch.equal(g.allreduce(x), torch.full((4,), 10.0))
        ok &= torch.equal(g.allreduce(x, ReduceOp.MAX), torch.full((4,), 4.0))
        hb = g.allreduce(torch.full((3,), 0.1 * (rank + 1), dtype=torch.bfloat16))
        ok &= hb.dtype == torch.bfloat16 and abs(float(hb[0]) - 1.0) < 0.02
        ok &= g.allgather(torch.tensor([rank])).tolist() == [0, 1, 2, 3]
        ok &= torch.equal(g.reduce_scatter(torch.arange(8.0)), torch.arange(8.0)[2 * rank:2 * rank + 2] * 4)
        b = torch.tensor([7.0]) if rank == 2 else torch.zeros(1)
        ok &= float(g.broadcast(b, root=2)) == 7.0
        a2a = g.all_to_all(torch.arange(4.0) + 10 * rank)
        ok &= a2a.tolist() == [rank + 10 * r for r in range(4)]
        var = g.all_to_all(torch.full((rank + 1, 2), float(rank)), [1 if p == 0 else (rank if p == 1 else 0) for p in range(4)][:4]
                           if False else [rank + 1, 0, 0, 0])
        ok &= (var.shape[0] == 10) if rank == 0 else (var.shape[0] == 0)
        peer = rank ^ 1
        got = g.sendrecv(torch.tensor([float(rank)]), torch.zeros(1), peer)
        ok &= float(got) == float(peer)
        sub = g.split(color=rank % 2, key=-rank)          # evens / odds, reversed order
        ok &= sub.world_size == 2 and sub.ranks == ([2, 0] if rank % 2 == 0 else [3, 1])
        ok &= float(sub.allreduce(torch.tensor([float(rank)]))) == (2.0 if rank % 2 == 0 else 4.0)
        g.barrier()
        # expert-parallel exchange against the single-process oracle
        torch.manual_seed(0)
        E, D_, I, T, K = 8, 16, 8, 6, 2
        gate = [torch.randn(I, D_) * 0.1 for _ in range(E)]
        up = [torch.randn(I, D_) * 0.1 for _ in range(E)]
        down = [torch.randn(D_, I) * 0.1 for _ in range(E)]
        router = torch.randn(E, D_)
        cfg = MoeConfig(E, K, D_, I)
        full = MoeLayer(cfg, router, ExpertGroup.from_experts(list(zip(gate, up, down)), dtype=torch.float32),
                        MoeStrategy.PER_EXPERT)
        torch.manual_seed(100 + rank)
        x = torch.randn(T, D_)
        want = full.forward(x)
        el = E // world
        mine = list(zip(gate, up, down))[rank * el:(rank + 1) * el]
        layer = MoeLayer(cfg, router, ExpertGroup.from_experts(mine, dtype=torch.float32)
                         ).with_exchange(ep.EpExchange(g, E))
        got = layer.forward(x)
        ok &= torch.allclose(got, want, atol=1e-5)
        grouped = full.with_strategy(MoeStrategy.GROUPED).forward(x)
        ok &= torch.allclose(grouped, want, atol=1e-5)
        # the same exchange with FP8 rows on the wire: E4M3 codes + one scale per row, both ways
        ex8 = ep.EpExchange(g, E, payload="fp8")
        got8 = MoeLayer(cfg, router, ExpertGroup.from_experts(mine, dtype=torch.float32)).with_exchange(ex8).forward(x)
        rel = float((got8 - want).norm() / want.norm())
        ok &= 1e-4 < rel < 6e-2                           # E4M3: 3 mantissa bits, twice
        # every pair crosses once out and once back: summed over the ranks, 2 x world x T x K rows
        total = float(g.allreduce(torch.tensor([float(ex8.wire_bytes)])))
        ok &= total == 2 * world * (T * K) * (D_ + 4)
        rows = torch.randn(5, D_) * 3
        qr, sr = ep.fp8_quant_rows(rows)
        back = ep.fp8_dequant_rows(qr, sr, torch.float32)
        ok &= qr.dtype == torch.uint8 and float((back - rows).abs().max() / rows.abs().max()) < 0.07
        ok &= torch.allclose(back.abs().amax(-1), rows.abs().amax(-1), rtol=1e-6)   # the row maximum is exact
        q.put((rank, bool(ok)))
    finally:
        dist.destroy_process_group()


def _algo_worker(rank, world, port, q):
    import torch.distributed as dist
    from rmlx_b200.parallel import algorithms as A
    from rmlx_b200.parallel.group import Group
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    try:
        g = Group()
        ok = True
        for n, dtype in ((1, torch.float32), (7, torch.float32), (1000, torch.float32), (2, torch.bfloat16),
                         (513, torch.bfloat16)):
            gen = torch.Generator().manual_seed(100 * n + rank)
            x = torch.randint(-8, 9, (n,), generator=gen).to(dtype)           # small integers: sums are exact
            want = sum(torch.randint(-8, 9, (n,), generator=torch.Generator().manual_seed(100 * n + r)).float()
                       for r in range(world)).to(dtype)
            for fn in (A.tree_allreduce, A.ring_allreduce, A.mesh_allreduce):
                got = fn(g, x)
                ok &= got.dtype == dtype and got.shape == x.shape and torch.equal(got, want)
        y = torch.randn(3, 5, generator=torch.Generator().manual_seed(rank))
        ref = g.allreduce(y)
        for fn in (A.tree_allreduce, A.ring_allreduce, A.mesh_allreduce):
            ok &= torch.allclose(fn(g, y), ref, atol=1e-5)
        out, algo = A.allreduce_auto(g, y)
        ok &= algo is A.AllreduceAlgorithm.TREE and torch.allclose(out, ref, atol=1e-5)
        # the halves of the ring on their own, and the tree broadcast from a root that is not rank 0
        z = torch.arange(11.0) * (rank + 1)
        lo, hi = A.chunk_bounds(11, world)[rank]
        ok &= torch.equal(A.ring_reduce_scatter(g, z), (torch.arange(11.0) * sum(range(1, world + 1)))[lo:hi])
        gathered = A.ring_allgather(g, torch.full((2, 3), float(rank)))
        ok &= gathered.shape == (world, 2, 3) and all(float(gathered[i].mean()) == i for i in range(world))
        root = world - 1
        b = A.tree_broadcast(g, torch.arange(5.0) + 10 * rank, root=root)
        ok &= torch.equal(b, torch.arange(5.0) + 10 * root)
        q.put((rank, bool(ok)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [3, 4])
def test_tree_ring_and_mesh_allreduce_over_point_to_point(world):
    """The three algorithms on gloo ranks (an odd and an even group): exact sums on integer data of
    sizes that do not divide by the group, fp32 and bf16, and agreement with the library."""
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    ps = [ctx.Process(target=_algo_worker, args=(r, world, port, q)) for r in range(world)]
    [p.start() for p in ps]
    res = dict(q.get(timeout=120) for _ in range(world))
    for p in ps:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert res == {r: True for r in range(world)}


def test_allreduce_algorithm_choice_and_chunks():
    from rmlx_b200.parallel import algorithms as A
    assert A.chunk_bounds(10, 4) == [(0, 3), (3, 6), (6, 8), (8, 10)]
    assert A.chunk_bounds(2, 4) == [(0, 1), (1, 2), (2, 2), (2, 2)] and A.chunk_bounds(0, 3) == [(0, 0)] * 3
    T, R, M = A.AllreduceAlgorithm.TREE, A.AllreduceAlgorithm.RING, A.AllreduceAlgorithm.MESH
    assert A.choose_algorithm(4096, 8) is T and A.choose_algorithm(2 << 20, 8) is M
    assert A.choose_algorithm(16 << 20, 8) is R and A.choose_algorithm(16 << 20, 2) is M    # two ranks never ring
    assert A.choose_algorithm(256 << 10, 4, half=True) is R and A.choose_algorithm(256 << 10, 4) is T
    assert A.choose_algorithm(4096, 8, tree_threshold=1024) is M


def test_group_collectives_split_and_ep_exchange_on_gloo():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    ps = [ctx.Process(target=_group_worker, args=(r, 4, port, q)) for r in range(4)]
    [p.start() for p in ps]
    res = dict(q.get(timeout=120) for _ in range(4))
    for p in ps:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert res == {0: True, 1: True, 2: True, 3: True}


def test_health_monitor_detects_a_silent_peer_on_the_host():
    store = DictStore()
    now = [0.0]
    mon = HealthMonitor(store, 0, 3, HeartbeatConfig(1.0, 5.0, 3), clock=lambda: now[0])
    s1, s2 = HeartbeatSender(store, 1), HeartbeatSender(store, 2)
    for step in range(5):
        now[0] += 1.0
        s1.beat()
        if step < 1:
            s2.beat()                       # rank 2 stops after its first beat
        mon.poll()
    assert mon.failed_peers() == [2] and not mon.healthy()
    # the wired form: a watchdog thread flips ok() and calls back; peer 1 never joins
    failures = []
    wd = Watchdog(DictStore(), 0, 2, HeartbeatConfig(0.01, 0.2, 3), on_failure=failures.append)
    wd.start()
    t0 = time.monotonic()
    while wd.ok() and time.monotonic() - t0 < 5:
        time.sleep(0.01)
    wd.stop()
    assert not wd.ok() and failures == [[1]]


def test_moe_policy_and_sparse_guard():
    now = [0.0]
    p = MoePolicy(hysteresis=16, cooldown_s=5.0, cooldown_calls=1000, env={}, clock=lambda: now[0])
    assert p.select(8) == MoeBackend.LOCAL
    now[0] += 10
    assert p.select(70) == MoeBackend.LOCAL           # inside the hysteresis band: no switch
    assert p.select(400) == MoeBackend.FUSED and p.zone_switches == 1
    assert p.select(4) == MoeBackend.FUSED            # cool-down holds the choice
    now[0] += 10
    assert p.select(4) == MoeBackend.LOCAL and p.zone_switches == 2
    assert MoePolicy(env={"RMLX_MOE_BACKEND": "nccl"}).select(1) == MoeBackend.NCCL
    mid = MoePolicy(env={})
    assert mid.select(200, nbytes=4 << 20) == MoeBackend.FUSED
    g = SparseGuard(window=10)
    acts = [g.record_step(1, 10) for _ in range(10)]
    assert acts[-1] == GuardAction.INCREASE_CAPACITY
    acts = [g.record_step(9, 10) for _ in range(30)]
    assert GuardAction.DENSE_FALLBACK in acts
    acts = [g.record_step(0, 10) for _ in range(400)]
    assert GuardAction.RESET in acts and g.state == GuardAction.NONE


def test_wire_formats():
    rows = np.arange(24, dtype=np.uint8).reshape(3, 8)
    buf = wire.pack_v3([0, 2, 1], [5, 0, 65535], rows)
    assert len(buf) == wire.v3_payload_bytes(3, 8)
    e, p, r = wire.unpack_v3(buf, 8)
    assert e == [0, 2, 1] and p == [5, 0, 65535] and np.array_equal(r, rows)
    assert wire.unpack_v3(wire.pack_v3([], [], np.zeros((0, 8), np.uint8)), 8)[0] == []
    with pytest.raises(wire.ProtocolError):
        wire.unpack_v3(buf[:-1], 8)
    x = torch.randn(5, 64)
    y = wire.fp8_unpack_tokens(wire.fp8_pack_tokens(x), 5, 64)
    assert (y - x).abs().max() <= x.abs().max() * 0.07
    f = wire.crc_frame(b"payload")
    assert wire.crc_verify(f) == b"payload"
    with pytest.raises(wire.ProtocolError):
        wire.crc_verify(b"x" + f[1:])


def test_slab_ring_backpressure_and_bounded_waits():
    ring = SlabRing(SlabRingConfig(depth=2, slab_bytes=64))
    a = ring.acquire_for_write(); ring.slab(a)[:4] = torch.tensor([1, 2, 3, 4], dtype=torch.uint8)
    ring.produce(a)
    b = ring.acquire_for_write(); ring.produce(b)
    with pytest.raises(WaitTimeout):
        ring.acquire_for_write(timeout_s=0.01)        # full: consumer has released nothing
    i = ring.consume(0.1)
    assert i == a and ring.slab(i)[:4].tolist() == [1, 2, 3, 4]
    ring.release(i)
    assert ring.acquire_for_write(0.1) == a
    ring.release(ring.consume(0.1))
    with pytest.raises(WaitTimeout):
        ring.consume(0.01)                            # slot a is being written, nothing ready
    assert ring.backpressure_events > 0 and ring.produced == 2 and ring.consumed == 2


def test_capacity_limited_dispatch_matches_reference_semantics():
    torch.manual_seed(0)
    T, K, E, W, D_ = 8, 2, 4, 2, 4
    x = torch.randn(T, D_)
    idx = torch.zeros(T, K, dtype=torch.int64); idx[:, 1] = 1      # everyone wants experts 0 and 1
    wts = torch.full((T, K), 0.5)
    cap = ep.expert_capacity(T, K, E, 1.0)
    assert cap == 4
    bufs, route, overflow = ep.dispatch_with_capacity(x, idx, E, W, src_rank=1, capacity_factor=1.0)
    assert overflow == 8 and (route[:4] >= 0).all() and (route[4:] == -1).all()
    assert int(route[0, 0]) == 0 * W * cap + 1 * cap + 0
    assert torch.equal(bufs[0][0, :4], x[:4]) and bufs[1].abs().sum() == 0
    outs = [torch.zeros(E // W, W * cap, D_) for _ in range(W)]
    outs[0][:, cap:2 * cap] = bufs[0] * 2.0                         # identity-ish experts: y = 2x
    y = ep.combine_with_layout(outs, idx, wts, route, E, W, 1, cap)
    assert torch.allclose(y[:4], 2.0 * x[:4]) and y[4:].abs().sum() == 0


def test_capacity_router_reacts_to_overflow():
    """The overflow guard in the loop: a skewed routing raises the capacity factor, a heavily
    skewed one stops the dropping (every pair fits), balanced steps put the configured factor back;
    the result with room for every pair equals the unrestricted combination."""
    torch.manual_seed(0)
    T, K, E, W, D_ = 16, 2, 8, 2, 4
    x = torch.randn(T, D_)
    wts = torch.full((T, K), 0.5)
    skew = torch.zeros(T, K, dtype=torch.int64); skew[:, 1] = 1          # every token to experts 0 and 1
    even = torch.stack([torch.arange(T) % E, (torch.arange(T) + 4) % E], 1)
    r = ep.GuardedCapacityRouter(E, W, src_rank=0, capacity_factor=1.0, guard=SparseGuard(window=4))
    assert r.capacity(T, K) == 4
    drops = []
    for _ in range(4):                                                  # window 1: ratio 0.75 > 0.20
        _, route, overflow, cap = r.dispatch(x, skew)
        drops.append(overflow)
    assert drops == [24] * 4 and cap == 4 and r.dense and r.dense_fallbacks == 1
    bufs, route, overflow, cap = r.dispatch(x, skew)                    # now nothing is dropped
    assert overflow == 0 and cap == T * K and (route >= 0).all()
    outs = [torch.zeros(E // W, W * cap, D_) for _ in range(W)]
    outs[0][:, :cap] = bufs[0] * 3.0                                    # "experts": y = 3 x (src rank 0's stripe)
    y = r.combine(outs, skew, wts, route, cap)
    assert torch.allclose(y, 3.0 * x, atol=1e-6)
    for _ in range(140):                                                # balanced traffic: the averaged ratio decays
        r.dispatch(x, even)
    assert not r.dense and r.factor == 1.0 and r.resets >= 1
    # a mild skew (a few drops per step) only grows the factor
    mild = even.clone(); mild[:6, 0] = 0
    r2 = ep.GuardedCapacityRouter(E, W, src_rank=0, capacity_factor=1.0, guard=SparseGuard(window=4))
    for _ in range(4):
        _, _, overflow, _ = r2.dispatch(x, mild)
    assert 0 < overflow < 0.2 * T * K and r2.factor == 1.5 and not r2.dense and r2.increases == 1
    assert r2.capacity(T, K) == 6


def test_topology_matrix_parser():
    txt = """\tGPU0\tGPU1\tGPU2\tCPU Affinity
GPU0\t X \tNV18\tNV18\t0-55
GPU1\tNV18\t X \tNV18\t0-55
GPU2\tNV18\tNV18\t X \t56-111
"""
    m = parse_topo_matrix(txt)
    assert m == [["X", "NV18", "NV18"], ["NV18", "X", "NV18"], ["NV18", "NV18", "X"]]


def test_warmup_is_idempotent_and_calibrates():
    """run_warmup semantics (crates/rmlx-distributed/src/warmup.rs tests): both callables run once,
    a second call does nothing, the crossover of the two timed paths becomes the thresholds."""
    from rmlx_b200.parallel.warmup import Warmup, WarmupConfig
    calls = {"comm": 0, "kern": 0}
    w = Warmup(WarmupConfig(calibration_sizes=(4, 32, 128, 512), repeats=1))
    small = lambda n: 10e-6 + n * 1e-6        # latency-optimised path: cheap start, steep slope
    large = lambda n: 60e-6 + n * 0.1e-6      # bandwidth-optimised path
    r = w.run(lambda: calls.__setitem__("comm", calls["comm"] + 1),
              lambda: calls.__setitem__("kern", calls["kern"] + 1), small, large)
    assert r.ran and calls == {"comm": 1, "kern": 1}
    assert r.calibration.large_n_min == 128 and r.calibration.small_n_max == 32
    assert "small_4" in r.timings_us and "large_512" in r.timings_us
    r2 = w.run(lambda: calls.__setitem__("comm", 99))
    assert not r2.ran and calls["comm"] == 1 and r2.calibration == r.calibration
    from rmlx_b200.parallel.moe_policy import MoePolicy
    p = MoePolicy(env={})
    p.apply_calibration(r.calibration)
    assert p.large_n_min == 128


def test_nvtx_ranges_are_noops_without_cuda():
    from rmlx_b200.utils import nvtx
    with nvtx.range("layer0"):
        nvtx.mark("x")
    assert nvtx.enabled() in (False, True)


def _leaver_worker(rank, world, port, q):
    """Three gloo ranks run all-reduce 'steps'; rank 2 leaves between steps (announced on the
    store, nothing in flight); the others learn of it on the host before their next launch, tear the
    group down, re-form a two-rank group and carry on."""
    import datetime
    from rmlx_b200.parallel.init import rejoin
    store = dist.TCPStore("127.0.0.1", port, world, rank == 0, timeout=datetime.timedelta(seconds=60),
                          wait_for_workers=False)
    dist.init_process_group("gloo", store=dist.PrefixStore("gen0", store), rank=rank, world_size=world,
                            timeout=datetime.timedelta(seconds=60))
    try:
        sums = []
        for step in range(3):
            t = torch.tensor([float(rank + 1)])
            dist.all_reduce(t)
            sums.append(t.item())
        if rank == 2:
            store.set("left/2", b"1")        # between steps, no collective in flight
            dist.destroy_process_group()
            q.put((rank, sums, None))
            return
        store.wait(["left/2"], datetime.timedelta(seconds=30))   # host-side notice before the next launch
        ctx = rejoin(store, rank, [0, 1], backend="gloo", generation=1)
        after = []
        for step in range(3):
            t = torch.tensor([float(rank + 1)])
            dist.all_reduce(t)
            after.append(t.item())
        q.put((rank, sums, (ctx.rank, ctx.world_size, after)))
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


def test_rank_leaves_between_steps_and_the_rest_re_rendezvous():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    ps = [ctx.Process(target=_leaver_worker, args=(r, 3, port, q)) for r in range(3)]
    [p.start() for p in ps]
    res = {}
    for _ in range(3):
        r, sums, after = q.get(timeout=120)
        res[r] = (sums, after)
    for p in ps:
        p.join(timeout=60)
        assert p.exitcode == 0
    for r in range(3):
        assert res[r][0] == [6.0, 6.0, 6.0]
    assert res[2][1] is None
    assert res[0][1] == (0, 2, [3.0, 3.0, 3.0]) and res[1][1] == (1, 2, [3.0, 3.0, 3.0])


def test_symmetric_heap_offset_arena_is_deterministic_and_coalesces():
    from rmlx_b200.parallel.symm_heap import OffsetArena
    a, b = OffsetArena(), OffsetArena()
    for ar in (a, b):
        assert ar.take(16) is None
        ar.grow(1000)
    seq = [256, 256, 256]
    offs_a = [a.take(n) for n in seq]
    offs_b = [b.take(n) for n in seq]
    assert offs_a == offs_b == [0, 256, 512]
    a.give(256, 256)
    assert a.take(300) is None              # 256 in the middle, 232 at the end: neither fits
    a.grow(1000)                            # the new segment merges with the free tail
    assert a.take(300) == 768
    a.give(0, 256)
    assert a.free[0] == (0, 512)            # coalesced with its free neighbour
    with pytest.raises(ValueError):
        a.give(100, 50)                     # a range that is already free
    assert a.free_bytes() + 256 + 300 == a.capacity


def test_device_matrix_file_round_trip(tmp_path):
    from rmlx_b200.parallel.topology import GpuInfo, Topology
    t = Topology([GpuInfo(0, "B200", 1 << 30, 18), GpuInfo(1, "B200", 1 << 30, 18)],
                 [[True, True], [True, True]], [["X", "NV18"], ["NV18", "X"]])
    path = str(tmp_path / "devices.json")
    t.save(path)
    back = Topology.load(path)
    assert back.num_gpus == 2 and back.fully_connected() and back.all_nvlink() and back.reachable(0, 1)
    assert back.gpus[1].nvlink_links == 18 and back.link == t.link
    import json
    doc = json.loads(t.to_json())
    doc["peer"] = [[True, True]]
    with open(path, "w") as f:
        json.dump(doc, f)
    with pytest.raises(ValueError):
        Topology.load(path)
