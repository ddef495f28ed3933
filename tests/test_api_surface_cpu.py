"""Small API-surface checks for methods that mirror the reference's public interface but are not on
any hot path: each is exercised once so that a rename or a broken delegate shows up here."""
import torch

from rmlx_b200.config import MoeConfig, RotaryConfig, tiny_dense_config
from rmlx_b200.nn.layers import QuantizedLinear, awq_dequantize, gptq_dequantize
from rmlx_b200.nn.moe import ExpertGroup, MoeLayer
from rmlx_b200.parallel.group import Group
from rmlx_b200.parallel.moe_policy import MoeBackend, MoePolicy
from rmlx_b200.parallel.topology import GpuInfo, Topology
from rmlx_b200.parallel.wire import v2_payload_bytes, v3_payload_bytes
from rmlx_b200.runtime.graph import GraphCache, HazardTracker
from rmlx_b200.serve.sampler import Sampler
from rmlx_b200.utils import logging as rlog
from rmlx_b200.utils import nvtx
from rmlx_b200.utils.metrics import Counters, TransportMetrics, to_prometheus
from rmlx_b200.utils.shutdown import ShutdownSignal


def test_config_helpers():
    cfg = tiny_dense_config()
    assert cfg.q_dim == cfg.num_heads * cfg.head_dim and cfg.kv_dim == cfg.num_kv_heads * cfg.head_dim
    r = RotaryConfig(head_dim=64, max_seq_len=128)
    assert (r.base_freq, r.scale, r.traditional) == (10000.0, 1.0, False)


def _pack_nibbles(q: torch.Tensor, order) -> torch.Tensor:
    """[..., 8k] values 0..15 -> int32 [..., k], value order[i] of each group of 8 at bits 4i."""
    g = q.reshape(*q.shape[:-1], -1, 8).long()
    word = torch.zeros(g.shape[:-1], dtype=torch.int64)
    for i, src in enumerate(order):
        word |= g[..., src] << (4 * i)
    word = torch.where(word >= 2**31, word - 2**32, word)
    return word.to(torch.int32)


def test_awq_and_gptq_imports_round_trip():
    g = torch.Generator().manual_seed(0)
    n_in, n_out, gs = 128, 64, 64
    q = torch.randint(0, 16, (n_in, n_out), generator=g)
    z = torch.randint(0, 16, (n_in // gs, n_out), generator=g)
    s = torch.rand(n_in // gs, n_out, generator=g) * 0.1 + 0.01
    grp = torch.arange(n_in) // gs
    want = ((q - z[grp]).float() * s[grp]).t()                       # [out, in]
    # AutoAWQ: value j of a group of eight sits at nibble position order^-1(j); order 0,2,4,6,1,3,5,7
    awq_pos = [0, 2, 4, 6, 1, 3, 5, 7]
    got = awq_dequantize(_pack_nibbles(q, awq_pos), _pack_nibbles(z, awq_pos), s, gs)
    assert torch.allclose(got, want)
    lin = QuantizedLinear.from_awq(_pack_nibbles(q, awq_pos), _pack_nibbles(z, awq_pos), s, gs)
    assert lin.in_features == n_in
    x = torch.randn(3, n_in, generator=g)
    assert torch.allclose(lin(x).float(), x @ want.t(), atol=0.35, rtol=0.1)     # re-quantised to Q4
    # GPTQ: qweight packs eight inputs per word along the input dimension; zeros stored minus one
    qw = _pack_nibbles(q.t().contiguous(), range(8)).t().contiguous()            # [in/8, out]
    qz = _pack_nibbles((z - 1) % 16, range(8))                                   # [groups, out/8]
    got = gptq_dequantize(qw, qz, s)
    want_g = ((q - (((z - 1) % 16) + 1)[grp]).float() * s[grp]).t()
    assert torch.allclose(got, want_g)
    perm = torch.randperm(n_in, generator=g) // gs                               # act-order groups
    got = gptq_dequantize(qw, qz, s, perm)
    assert torch.allclose(got, ((q - (((z - 1) % 16) + 1)[perm]).float() * s[perm]).t())
    assert QuantizedLinear.from_gptq(qw, qz, s).weight.n == n_out
    # the layer classes that keep the checkpoint layout: exact product with the expanded weight
    from rmlx_b200.nn.layers import AwqLinear, GptqLinear, RmsNorm, RMSNorm
    import pytest
    bias = torch.randn(n_out, generator=g)
    awq = AwqLinear(_pack_nibbles(q, awq_pos), _pack_nibbles(z, awq_pos), s, gs, bias=bias)
    assert (awq.in_features, awq.out_features) == (n_in, n_out)
    assert torch.allclose(awq(x), x @ want.t() + bias, atol=1e-4)
    assert awq.to_quantized().weight.n == n_out
    gptq = GptqLinear(qw, qz, s, perm)
    assert gptq.group_size == gs and torch.allclose(gptq(x), x @ gptq.dense_weight().t(), atol=1e-4)
    with pytest.raises(ValueError):
        AwqLinear(_pack_nibbles(q, awq_pos), _pack_nibbles(z, awq_pos), s, gs * 2)      # wrong group size
    with pytest.raises(ValueError):
        GptqLinear(qw, qz, s, perm[:-1])
    assert RmsNorm is RMSNorm


def test_moe_expert_bias_builders_and_update():
    cfg = MoeConfig(num_experts=4, num_experts_per_token=2, hidden_dim=16, intermediate_dim=8)
    g = torch.Generator().manual_seed(1)
    experts = [(torch.randn(8, 16, generator=g), torch.randn(8, 16, generator=g), torch.randn(16, 8, generator=g))
               for _ in range(4)]
    layer = MoeLayer(cfg, torch.randn(4, 16, generator=g), ExpertGroup.from_experts(experts, dtype=torch.float32))
    x = torch.randn(12, 16, generator=g)
    layer.forward(x)
    before = layer.last_counts.clone()
    bias = layer.update_expert_bias(lr=0.5)                 # aux-loss-free balancing: starved experts gain
    assert bias.shape == (4,) and torch.equal(bias.argmax(), before.argmin())
    same = layer.with_expert_bias(torch.tensor([0.0, 0.0, 0.0, 50.0]))
    assert same is layer
    idx, _, counts, _ = layer.route(x)
    assert (idx == 3).any(dim=1).all() and int(counts[3]) == 12


def test_sampler_batch_and_policy_force_and_wire_sizes():
    s = Sampler()
    logits = torch.tensor([[0.0, 3.0, 1.0], [5.0, 0.0, 1.0]])
    assert s.sample_batch(logits) == [1, 0]
    assert s.sample_batch(logits, [[1], []]) == [1, 0]
    p = MoePolicy(env={})
    p.force_backend(MoeBackend.NCCL)
    assert p.select(1, 16) == MoeBackend.NCCL and p.select(10_000, 1 << 30) == MoeBackend.NCCL
    p.force_backend(None)
    assert p.select(1, 16) == MoeBackend.LOCAL
    assert v2_payload_bytes(8, 64) == 8 * 68 and v3_payload_bytes(3, 64) == 4 + 3 * 68


def test_topology_group_metrics_logging_shutdown_nvtx():
    gpus = [GpuInfo(i, "B200", 180 << 30, 18) for i in range(2)]
    t = Topology(gpus, [[True, True], [True, True]], [["X", "NV18"], ["NV18", "X"]])
    assert t.fully_connected() and t.all_nvlink()
    t.link[0][1] = "SYS"
    assert not t.all_nvlink()
    grp = Group.loopback() if hasattr(Group, "loopback") else None
    if grp is not None:
        x = torch.arange(4.0)
        assert grp.allreduce_in_place(x) is x and x.tolist() == [0.0, 1.0, 2.0, 3.0]
    c = Counters(["peak"])
    c.set_max("peak", 3); c.set_max("peak", 2)
    assert c.get("peak") == 3
    tm = TransportMetrics()
    name = next(iter(tm.snapshot()))
    tm.add(name, 5)
    assert f"rmlx_{name} 5" in to_prometheus("rmlx", tm.snapshot()).replace(".0", "")
    lines = []
    old = rlog.get_level()
    rlog.set_sink(lines.append)
    rlog.set_level(rlog.LogLevel.DEBUG)
    rlog.debug("test", "hello", k=1)
    rlog.set_level(old)
    rlog.set_sink(print)
    assert len(lines) == 1 and "hello" in lines[0]
    sig = ShutdownSignal()
    assert not sig.is_triggered() and not sig.handle().is_shutdown()
    sig.trigger()
    assert sig.is_triggered() and sig.handle().is_shutdown()
    nvtx.enable(False)
    assert not nvtx.enabled()
    with nvtx.range("noop"):
        nvtx.mark("m")
    nvtx.enable(True)


def test_graph_cache_invalidate_and_hazard_tracker_streams():
    calls = []
    cache = GraphCache(max_entries=4)
    g1 = cache.get_or_capture(("step", 1), lambda: calls.append(1), warmup=0)
    g1.replay()
    assert len(cache) == 1 and calls
    cache.invalidate(("step", 1))
    assert len(cache) == 0
    cache.get_or_capture("a", lambda: None, warmup=0); cache.get_or_capture("b", lambda: None, warmup=0)
    cache.invalidate()
    assert len(cache) == 0
    h = HazardTracker()
    h.submit("compute", writes=[(0, 100)])
    deps = h.submit("copy", reads=[(50, 60)])
    assert deps == [(0, "RAW")] and h.in_flight() == 2
    h.retire_stream("compute")
    assert h.in_flight() == 1
    assert h.submit("copy2", reads=[(50, 60)]) == []


def test_progress_tracker_error_budget_and_bulk_wait():
    from rmlx_b200.parallel.health import ProgressTracker
    pt = ProgressTracker(max_consecutive_errors=4)
    state = {"a": 2, "b": 0}

    def poll_a():
        state["a"] -= 1
        return state["a"] <= 0

    ia, ib = pt.track(poll_a, "a"), pt.track(lambda: True, "b")
    assert pt.num_pending() == 2
    assert pt.poll() == [ib] and pt.num_pending() == 1
    assert pt.wait_all(timeout_s=1.0) and pt.completed == 2 and not pt.health_warning

    def broken():
        raise OSError("link down")

    pt.track(broken, "c")
    pt.poll(); pt.poll()
    assert pt.consecutive_errors == 2 and not pt.health_warning
    pt.track(lambda: True, "d")
    pt.poll()                                         # one error, then a success: the run is broken
    assert pt.consecutive_errors == 0 and not pt.health_warning
    assert not pt.wait_all(timeout_s=1.0)             # only the broken one is left: four in a row
    assert pt.health_warning and "link down" in pt.last_error and pt.total_errors >= 5
    pt.reset_health()
    assert not pt.health_warning and pt.num_pending() == 1


def test_gpu_error_store_collects_and_clears_status_words():
    from rmlx_b200.runtime.streams import GpuErrorStore
    store = GpuErrorStore()
    gemm, peer = torch.zeros(1, dtype=torch.int32), torch.zeros(1, dtype=torch.int32)
    calls = {"n": 0}

    def tp_status():
        calls["n"] += 1
        return 2 if calls["n"] == 2 else 0

    store.register("gemm", gemm); store.register("ep", peer); store.register("tp", tp_status)
    assert store.collect() == [] and not store.has_errors()
    gemm[0] = 1
    got = store.collect()
    assert ("gemm", 1, "pipeline wait timed out") in got and ("tp", 2, "peer wait timed out") in got
    assert int(gemm) == 0 and store.has_errors() and len(store.records()) == 2
    assert store.collect() == []
    peer[0] = 7
    try:
        store.raise_if_any()
        assert False
    except RuntimeError as e:
        assert "ep" in str(e) and "status 7" in str(e)
    store.clear(); store.unregister("ep")
    assert not store.has_errors()


def test_perf_counters():
    from rmlx_b200.utils.metrics import PERF, PerfCounters
    c = PerfCounters()
    c.record_d2h(torch.zeros(4, 8)); c.record_h2d(torch.zeros(3, dtype=torch.int32)); c.add("graph_replays", 2)
    snap = c.snapshot()
    assert snap["d2h_bytes"] == 128 and snap["host_syncs"] == 1 and snap["h2d_bytes"] == 12 and snap["graph_replays"] == 2
    assert isinstance(PERF, PerfCounters)


def test_ssh_helpers_quote_validate_and_plan():
    import subprocess
    import pytest
    from rmlx_b200.cli import ssh
    assert ssh.shell_quote("abc-1.2/x") == "abc-1.2/x"
    assert ssh.shell_quote("it's; rm -rf /") == "'it'\\''s; rm -rf /'"
    assert ssh.shell_quote("") == "''"
    for bad in ("-oProxyCommand=evil", "host name", "user@-host", "a;b", "$(x)", ""):
        with pytest.raises(ValueError):
            ssh.validate_target(bad)
    assert ssh.validate_target("user@node-1.cluster") == "user@node-1.cluster"
    argv = ssh.ssh_argv("node1", ["python", "-c", "print('hi')"], {"RMLX_RANK": "3", "X": "a b"}, cwd="/opt/my app")
    assert argv[0] == "ssh" and argv[-2] == "node1" and argv[-3] == "--"
    assert argv[-1] == "cd '/opt/my app' && RMLX_RANK=3 X='a b' python -c 'print('\\''hi'\\'')'"
    with pytest.raises(ValueError):
        ssh.remote_command(["x"], {"BAD NAME": "1"})

    def slow(*a, **k):
        raise subprocess.TimeoutExpired(cmd="ssh", timeout=k.get("timeout"))

    assert ssh.run_remote("node1", ["true"], timeout_s=0.1, runner=slow)[0] == 124

    class R:
        returncode, stdout, stderr = 0, "ok\n", ""

    assert ssh.run_remote("node1", ["true"], runner=lambda *a, **k: R()) == (0, "ok\n", "")
    assert ssh.plan_ranks(["a", "b"], 2) == [("a", 0, 0), ("a", 1, 1), ("b", 2, 0), ("b", 3, 1)]


def test_exchange_tags_and_credits():
    import pytest
    from rmlx_b200.parallel.slab_ring import CreditManager
    from rmlx_b200.parallel.wire import TAG_COMBINE, pack_exchange_tag, unpack_exchange_tag
    from rmlx_b200.runtime.streams import WaitTimeout
    w = pack_exchange_tag((1 << 40) - 1, TAG_COMBINE, 7, 255)
    assert w < 1 << 64 and unpack_exchange_tag(w) == ((1 << 40) - 1, TAG_COMBINE, 7, 255)
    with pytest.raises(ValueError):
        pack_exchange_tag(1 << 40, 0, 0, 0)
    cm = CreditManager(window=2)
    assert cm.try_acquire(1, 5) and cm.try_acquire(1, 5) and not cm.try_acquire(1, 5)
    assert cm.available(1, 5) == 0 and cm.available(2, 5) == 2 and cm.stalls == 1
    returned = []

    def progress():
        if not returned:
            cm.release(1, 5); returned.append(1)

    cm.acquire(1, 5, timeout_s=1.0, poll=progress)          # a credit comes back while waiting
    with pytest.raises(WaitTimeout):
        cm.acquire(1, 5, timeout_s=0.02)
    cm.release(1, 5); cm.release(1, 5)
    with pytest.raises(ValueError):
        cm.release(1, 5)


def test_cli_multi_host_dry_run_prints_one_ssh_command_per_rank():
    import io
    from rmlx_b200.cli.main import launch_hosts
    out = io.StringIO()
    rc = launch_hosts(["python", "serve.py"], ["u@n1", "n2"], per_host=2, extra_env={"K": "v w"},
                      cwd="/srv/app", sink=out, dry_run=True)
    lines = out.getvalue().strip().splitlines()
    assert rc == 0 and len(lines) == 4
    assert lines[0].startswith("ssh ") and " -- u@n1 " in lines[0] and " -- n2 " in lines[3]
    assert "RMLX_RANK=3" in lines[3] and "RMLX_LOCAL_SLOT=1" in lines[3] and "RMLX_WORLD_SIZE=4" in lines[3]
    assert "MASTER_ADDR=n1" in lines[2] and "cd /srv/app" in lines[0]


def test_ep_runtime_context_stages_and_delivers_with_credits():
    import pytest
    from rmlx_b200.parallel.ep_runtime import EpRuntimeContext
    from rmlx_b200.parallel.slab_ring import CreditManager
    from rmlx_b200.runtime.streams import WaitTimeout
    ctx = EpRuntimeContext(rank=0, world=2, credits=CreditManager(window=2))
    for k in range(2):
        with ctx.staged(peer=1, tag=1) as buf:
            buf.tensor[:4] = torch.tensor([k, 1, 2, 3], dtype=torch.uint8)
    with pytest.raises(WaitTimeout):                      # window of two: the third has to wait
        with ctx.staged(peer=1, tag=1, timeout_s=0.02):
            pass
    assert ctx.delivered(1, 1)[:4].tolist() == [0, 1, 2, 3]
    ctx.done()
    with ctx.staged(peer=1, tag=1) as buf:                # the returned credit and slab are reusable
        buf.tensor[0] = 9
    assert ctx.delivered(1, 1)[0].item() == 1
    ctx.done()
    # a failing producer publishes nothing and leaks neither the slab nor the credit
    before = (ctx.credits.available(1, 1), ctx.ring.produced)
    with pytest.raises(RuntimeError):
        with ctx.staged(peer=1, tag=1):
            raise RuntimeError("boom")
    assert (ctx.credits.available(1, 1), ctx.ring.produced) == before and ctx.healthy()


def test_logical_topology_striping_and_failover():
    import pytest
    from rmlx_b200.parallel.topology import LinkFailover, LogicalTopology, stripe_plan
    assert LogicalTopology.parse(None).peers(2, 4) == [3, 0, 1]
    assert LogicalTopology.parse("ring").peers(0, 4) == [1, 3] and LogicalTopology.parse("ring").peers(0, 2) == [1]
    hy = LogicalTopology.parse("hybrid:4")
    assert hy.peers(5, 8) == [6, 7, 4, 1] and hy.peers(0, 1) == []
    mat = LogicalTopology.from_env({"RMLX_TOPOLOGY": "[[0,2,1],[2,0,null],[1,1,0]]"})
    assert mat.peers(0, 3) == [2, 1] and mat.peers(1, 3) == [0]
    with pytest.raises(ValueError):
        LogicalTopology.parse("star")
    assert stripe_plan(1000, 4) == [(0, 0, 1000)]
    plan = stripe_plan((256 << 10) + 100, 2)
    assert [p[0] for p in plan] == [0, 1, 0, 1, 0] and plan[-1] == (0, 256 << 10, 100)
    assert sum(p[2] for p in plan) == (256 << 10) + 100 and stripe_plan(0, 2) == []
    fo = LinkFailover(lanes=2, fail_after=2, recover_after=2)
    assert fo.report(1, False) == "active" and fo.report(1, False) == "failed" and fo.usable() == [0]
    assert fo.report(1, True) == "recovering" and fo.report(1, False) == "failed"
    assert fo.report(1, True) == "recovering" and fo.report(1, True) == "active" and fo.usable() == [0, 1]


def test_every_activation_of_the_reference_has_a_closed_form_here():
    """SiLU, GELU (exact / tanh / fast), sigmoid, tanh, ReLU, leaky ReLU, ELU, SELU, Mish, QuickGELU,
    hard swish, hard sigmoid, softplus, softsign, GLU (crates/rmlx-nn/src/activations.rs:1188-1205)."""
    from rmlx_b200.nn.layers import ACTIVATIONS, activation
    x = torch.linspace(-4, 4, 33)
    sig = torch.sigmoid
    forms = {
        "silu": x * sig(x), "sigmoid": sig(x), "tanh": torch.tanh(x), "relu": x.clamp_min(0),
        "leaky_relu": torch.where(x > 0, x, 0.01 * x), "elu": torch.where(x > 0, x, torch.expm1(x)),
        "selu": 1.0507009873554805 * torch.where(x > 0, x, 1.6732632423543772 * torch.expm1(x)),
        "mish": x * torch.tanh(torch.log1p(torch.exp(x))), "quick_gelu": x * sig(1.702 * x),
        "hardswish": x * (x + 3).clamp(0, 6) / 6, "hardsigmoid": (x + 3).clamp(0, 6) / 6,
        "softplus": torch.log1p(torch.exp(x)), "softsign": x / (1 + x.abs()),
        "gelu": 0.5 * x * (1 + torch.erf(x / 2 ** 0.5)),
        "gelu_approx": 0.5 * x * (1 + torch.tanh(0.7978845608 * (x + 0.044715 * x ** 3))),
    }
    for name, want in forms.items():
        assert torch.allclose(activation(name)(x), want, atol=1e-5), name
    assert torch.allclose(activation("gelu_fast")(x), forms["gelu"], atol=3e-2)
    pair = torch.randn(3, 8)
    assert torch.allclose(activation("glu")(pair), pair[:, :4] * sig(pair[:, 4:]))
    assert len(ACTIVATIONS) >= 17


def test_top_level_exports_resolve_lazily():
    """``import rmlx_b200`` is cheap (no model code, no CUDA library) and every exported name
    resolves to the object of its home module."""
    import importlib
    import subprocess
    import sys
    import rmlx_b200
    for name in rmlx_b200.__all__:
        if name == "__version__":
            continue
        obj = getattr(rmlx_b200, name)
        home = importlib.import_module("rmlx_b200." + rmlx_b200._EXPORTS[name])
        assert obj is getattr(home, name), name
    assert "TransformerModel" in dir(rmlx_b200)
    try:
        rmlx_b200.no_such_name
        raise AssertionError("expected AttributeError")
    except AttributeError:
        pass
    code = ("import sys, rmlx_b200; "
            "assert not [m for m in sys.modules if m.startswith('rmlx_b200.')], 'submodules loaded at import'")
    assert subprocess.run([sys.executable, "-c", code], capture_output=True).returncode == 0
