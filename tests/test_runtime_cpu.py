"""Runtime pieces that need no GPU: tuning table, bounded event waits, graph cache bookkeeping,
hazard tracking, logging, metrics, precision guard, shutdown flag (the pure-logic unit tests of
crates/rmlx-metal/src/device.rs:147-209, command.rs, event.rs and crates/rmlx-core/tests/phase7a_tests.rs)."""
import threading
import time

import pytest
import torch

from rmlx_b200.runtime import device, graph, streams
from rmlx_b200.utils import logging as rlog
from rmlx_b200.utils import metrics
from rmlx_b200.utils.precision_guard import GuardAction, PrecisionGuard
from rmlx_b200.utils.shutdown import ShutdownSignal


def test_tuning_from_name():
    t = device.tuning_from_name("NVIDIA B200")
    assert t.supports_tcgen05 and t.sm_count == 148 and t.tmem_columns == 512
    assert device.tuning_from_name("NVIDIA H100 80GB HBM3").supports_tcgen05 is False
    assert device.tuning_from_name("Mystery", (10, 0)).supports_tcgen05
    assert t.gemm_tile_n(8192, 4096) == 256 and t.gemm_tile_n(128, 4096) == 32
    assert t.kv_splits(1, 4, 4096) == 16 and t.kv_splits(64, 4, 4096) == 1


def test_event_wait_is_bounded_and_cancellable():
    ev = streams.GpuEvent()
    ev.record()
    ev.cpu_wait(1.0)                       # host emulation / idle stream: completes at once
    ev._host_done = False                  # a wait that nothing will ever satisfy
    ev._cuda = False
    t0 = time.monotonic()
    with pytest.raises(streams.WaitTimeout):
        ev.cpu_wait(0.05)
    assert time.monotonic() - t0 < 1.0
    threading.Timer(0.02, ev.cancel).start()
    with pytest.raises(streams.WaitCancelled):
        ev.cpu_wait(5.0)
    sm = streams.StreamManager()
    assert set(sm.streams) == {"default", "compute", "copy"}
    sm.compute_to_copy(); sm.synchronize(1.0)


def test_graph_cache_and_buckets():
    calls = []
    gc = graph.GraphCache(max_entries=2)
    if not torch.cuda.is_available():
        g = gc.get_or_capture(("decode", 1), lambda: calls.append(1))
        g.replay(); g.replay()
        assert calls == [1, 1]
        gc.get_or_capture(("decode", 1), lambda: None)
        gc.get_or_capture(("decode", 2), lambda: None)
        gc.get_or_capture(("decode", 4), lambda: None)      # evicts the oldest
        assert gc.hits == 1 and gc.misses == 3 and len(gc) == 2
    assert graph.bucket_for(3) == 4 and graph.bucket_for(64) == 64
    with pytest.raises(ValueError):
        graph.bucket_for(65)


def test_hazard_tracker():
    h = graph.HazardTracker()
    a = h.submit("compute", writes=[(0, 100)])
    assert a == []
    assert h.submit("copy", reads=[(50, 60)]) == [(0, "RAW")]
    assert h.submit("copy", writes=[(90, 120)]) == [(0, "WAW")]
    h.retire(0)
    assert h.submit("compute", writes=[(55, 58)]) == [(1, "WAR")]
    assert h.submit("compute", reads=[(0, 10)], temporaries=[(0, 10)]) == []
    s = graph.HazardTracker(serialize=True)
    s.submit("a", writes=[(0, 1)])
    assert s.submit("b", reads=[(1000, 1001)]) == [(0, "SERIAL")]


def test_logging_metrics_guard_shutdown():
    got = []
    rlog.capture(got)
    rlog.set_level(rlog.LogLevel.WARN)
    rlog.info("t", "dropped")
    rlog.warn("rmlx.alloc", "pool low", free=3)
    rlog.capture(None); rlog.set_level(rlog.LogLevel.INFO)
    assert len(got) == 1 and got[0].fields == {"free": 3}
    assert '"level": "WARN"' in got[0].to_json() and "pool low [free=3]" in got[0].to_text()
    m = metrics.RuntimeMetrics()
    m.record_kernel(12.5, 3); m.add("cache_hits")
    snap = m.snapshot()
    assert snap["kernel_dispatches"] == 3 and snap["kernel_time_us"] == 12.5
    assert "rmlx_kernel_dispatches 3" in metrics.to_prometheus("rmlx", snap)
    mm = metrics.MoeMetrics(4); mm.record_counts([1, 0, 2, 5])
    assert mm.per_expert == [1, 0, 2, 5] and mm.get("tokens_routed") == 8
    g = PrecisionGuard()
    assert g.check(torch.randn(4, 100)) == GuardAction.OK
    assert g.check(torch.randn(4, 100)) == GuardAction.OK
    assert g.check(torch.tensor([[float("nan"), 1.0]])) == GuardAction.FALLBACK
    peaked = torch.zeros(4, 100); peaked[:, 0] = 100
    assert g.check(peaked) in (GuardAction.WARN, GuardAction.FALLBACK)
    s = ShutdownSignal(); h = s.handle()
    assert not h.is_shutdown(); s.trigger(); assert h.is_shutdown() and h.wait(0.01)


def test_stream_manager_submit_tracks_hazards_on_the_host():
    graph.HAZARDS.retire_all()
    sm = streams.StreamManager()
    a = torch.zeros(8)
    op0, _ = sm.submit("compute", lambda: a.add_(1), writes=[a])
    op1, r = sm.submit("copy", lambda: a * 2, reads=[a])
    assert op1 == op0 + 1 and float(r[0]) == 2.0
    # host execution is synchronous: nothing stays in flight, no event wait was needed
    assert graph.HAZARDS.in_flight() == 0 and sm.reap() == 0


def test_hazard_tracker_learns_the_results_of_an_operation():
    h = graph.HazardTracker()
    h.submit("copy", reads=[(0, 10)])
    h.add_writes(h.last_id(), [(100, 140)])
    assert h.submit("compute", reads=[(120, 130)]) == [(0, "RAW")]
    h.retire_all()
    assert h.in_flight() == 0


def test_native_graph_store_bookkeeping_without_a_gpu():
    """The keyed store's host side: misses are counted, an unknown key cannot be launched, nothing
    to drop. (Recording and replaying need a GPU.)"""
    from rmlx_b200 import _lib
    try:
        _lib.cuda()
    except Exception as e:                          # noqa: BLE001
        pytest.skip(f"CUDA library not available: {e}")
    from rmlx_b200.runtime.native_graph import NativeGraphStore
    store = NativeGraphStore(max_entries=3)
    assert not store.has(("decode", 4)) and not store.has("x")
    with pytest.raises(KeyError):
        store.launch(("decode", 4))
    assert store.invalidate(("decode", 4)) == 0 and store.invalidate() == 0
    st = store.stats()
    assert st["entries"] == 0 and st["misses"] == 2 and st["hits"] == 0 and st["captures"] == 0
    store.close()
    store.close()                                   # idempotent


def test_recordings_run_without_cyclic_gc_and_fall_back_when_invalidated(monkeypatch):
    """The graph cache's handling of a recording that gets invalidated, against a stand-in for
    torch.cuda: garbage collection is off inside the recording, a failed recording is tried once
    more, a second failure turns the key into launch-by-launch replay, other errors pass through."""
    import contextlib
    import gc
    import types

    with graph._no_cyclic_gc():
        assert not gc.isenabled()
    assert gc.isenabled()
    gc.disable()
    try:
        with graph._no_cyclic_gc():
            pass
        assert not gc.isenabled()                      # a caller's own setting is kept
    finally:
        gc.enable()

    class _S:
        def wait_stream(self, other):
            pass

    fail = {"left": 0, "msg": "CUDA error: operation failed due to a previous error during capture", "gc": []}

    @contextlib.contextmanager
    def fake_graph(g, stream=None):
        fail["gc"].append(gc.isenabled())
        yield
        if fail["left"] > 0:
            fail["left"] -= 1
            raise RuntimeError(fail["msg"])

    cuda = types.SimpleNamespace(
        is_available=lambda: True, Stream=lambda device=None: _S(), current_stream=lambda device=None: _S(),
        memory_stats=lambda device=None: {"allocation.all.allocated": 0},
        stream=lambda s: contextlib.nullcontext(), synchronize=lambda device=None: None,
        CUDAGraph=lambda: types.SimpleNamespace(replay=lambda: calls.append("replay")), graph=fake_graph)
    monkeypatch.setattr(graph, "torch", types.SimpleNamespace(cuda=cuda))
    calls, restored = [], []
    fn, restore = (lambda: calls.append("fn")), (lambda: restored.append(1))

    cache = graph.GraphCache()
    fail["left"] = 1
    g = cache.get_or_capture("a", fn, warmup=1, restore=restore)
    assert cache.capture_failures == 1 and cache.eager_fallbacks == 0 and calls == ["fn"] * 3
    assert fail["gc"] == [False, False] and gc.isenabled()       # no collection inside either attempt
    g.replay()
    assert calls[-1] == "replay" and len(restored) == 3          # after warm-up, after the failure, after the capture

    fail["left"] = 2
    g2 = cache.get_or_capture("b", fn, warmup=1, restore=restore)
    assert cache.capture_failures == 3 and cache.eager_fallbacks == 1
    n = len(calls)
    g2.replay()
    assert calls[n:] == ["fn"]                                   # launch by launch
    assert cache.get_or_capture("b", fn) is g2 and len(cache) == 2

    fail["left"], fail["msg"] = 1, "invalid argument"
    with pytest.raises(RuntimeError):
        cache.get_or_capture("c", fn, warmup=0)
