"""Smaller components of the inventory: MoE overlap schedules, the layer pipeline, prefill plans and
scratch pool, convolution wrappers, the dtype table, managed buffers / residency / arena."""
import pytest
import torch

from rmlx_b200 import dtypes
from rmlx_b200.config import FeedForwardType, MoeConfig, TransformerConfig
from rmlx_b200.models.prefill_plan import PrefillPlan, PrefillPool
from rmlx_b200.nn.conv import Conv1d, Conv2d
from rmlx_b200.nn.moe import ExpertGroup, MoeLayer
from rmlx_b200.nn.moe_pipeline import MoePipeline
from rmlx_b200.ops.weights import LinearWeight
from rmlx_b200.parallel.pipeline import LayerPipeline, PipelineConfig, Stage
from rmlx_b200.runtime.alloc import AllocError, ForwardArena, ResidencyManager


def _moe_layer():
    torch.manual_seed(0)
    cfg = MoeConfig(num_experts=4, num_experts_per_token=2, hidden_dim=32, intermediate_dim=64)
    gu = LinearWeight.from_dense(torch.randn(4, 128, 32) * 0.1, None, dtype=torch.float32)
    dn = LinearWeight.from_dense(torch.randn(4, 32, 64) * 0.1, None, dtype=torch.float32)
    layer = MoeLayer(cfg, torch.randn(4, 32) * 0.3, ExpertGroup(gu, dn))
    layer.with_shared_expert(LinearWeight.from_dense(torch.randn(128, 32) * 0.1, None, dtype=torch.float32),
                             LinearWeight.from_dense(torch.randn(32, 64) * 0.1, None, dtype=torch.float32))
    return layer


def test_moe_overlap_schedules_equal_plain_forward():
    layer = _moe_layer()
    x = torch.randn(10, 32)
    want = layer.forward(x)
    pipe = MoePipeline(layer)
    assert torch.allclose(pipe.forward_sbo(x), want, atol=1e-5)
    assert pipe.stats.shared_tokens == 10 and not pipe.stats.used_side_stream
    got = pipe.forward_tbo(x, micro_batches=3)
    assert torch.allclose(got, want, atol=1e-5) and pipe.stats.micro_batches == 3
    assert layer.shared is not None            # restored after the routed-only pass


def test_layer_pipeline_stages_and_stats():
    p = LayerPipeline(PipelineConfig(num_layers=3), device="cpu")
    seen = []
    outs = p.run(lambda l: torch.full((4,), float(l)), lambda l, y: (seen.append(l), y * 2)[1])
    assert seen == [0, 1, 2] and [float(o[0]) for o in outs] == [0.0, 2.0, 4.0]
    assert p.stats.layers_run == 3 and all(s == Stage.COMPLETE for s in p.stats.stages)
    assert 0.0 <= p.stats.overlap_ratio <= 1.0
    ratio = p.measure_overlap(lambda l: torch.ones(8), lambda l, y: y + 1)
    assert ratio > 0
    with pytest.raises(ValueError):
        PipelineConfig(num_layers=0).validate()


def test_prefill_plan_and_pool():
    moe = MoeConfig(num_experts=8, num_experts_per_token=2, hidden_dim=64, intermediate_dim=128)
    cfg = TransformerConfig(hidden_size=64, num_heads=4, num_kv_heads=2, head_dim=16, num_layers=2,
                            vocab_size=100, max_seq_len=128, ff_type=FeedForwardType.moe_(moe)).validate()
    plan = PrefillPlan(cfg, 32)
    names = [s.name for s in plan.steps]
    assert names[:5] == ["attn_norm", "qkv", "rope_kv", "attention", "o_proj"] and "combine" in names
    qkv = plan.steps[1]
    assert (qkv.m, qkv.n, qkv.k) == (32, (4 + 4) * 16, 64) and qkv.flops == 2.0 * 32 * 128 * 64
    assert plan.scratch_bytes >= max(s.out_bytes for s in plan.steps) and plan.flops > 0
    pool = PrefillPool.for_config(cfg, 64, slots=2)
    assert pool.plan(32) is pool.plan(32)
    with pytest.raises(ValueError):
        pool.plan(256)
    a, b = pool.acquire(), pool.acquire()
    assert pool.acquire() is None and a[1].numel() == pool.bytes_per_slot
    pool.release(a[0])
    assert pool.available == 1
    with pytest.raises(ValueError):
        pool.release(a[0])
    dense = cfg.replace(ff_type=FeedForwardType.gated(256))
    assert [s.name for s in PrefillPlan(dense, 8).steps][-2:] == ["gate_up", "down"]


def test_conv_layers_against_the_tap_by_tap_definition():
    """Channels-first layers (the reference's layout) and the channels-last option against the
    explicit definition; weight validation; a layer that waits for its weights."""
    from rmlx_b200.nn.conv import (Conv1dConfig, Conv2dConfig, conv1d_direct, conv2d_direct, conv_out_len)
    torch.manual_seed(1)
    x = torch.randn(2, 6, 19)
    w = torch.randn(8, 3, 4)                                    # groups = 2: 6 / 2 input channels per group
    b = torch.randn(8)
    layer = Conv1d(w, b, stride=2, padding=3, dilation=2, groups=2)
    y = layer(x)
    assert y.shape == (2, 8, layer.out_len(19)) and layer.out_len(19) == conv_out_len(19, 4, 2, 3, 2) == 10
    assert torch.allclose(y, conv1d_direct(x, w, b, 2, 3, 2, 2), atol=1e-4)
    cl = Conv1d(w.permute(0, 2, 1).contiguous(), b, stride=2, padding=3, dilation=2, groups=2, channels_last=True)
    assert torch.allclose(cl(x.transpose(1, 2)), y.transpose(1, 2), atol=1e-5)

    lazy = Conv1d(Conv1dConfig(6, 8, 4, groups=2, has_bias=True))
    assert not lazy.has_weights() and lazy.weight() is None
    with pytest.raises(ValueError):
        lazy(x)                                                 # weights not loaded
    with pytest.raises(ValueError):
        lazy.load_weights(torch.randn(8, 6, 4), b)              # wrong C_in / groups
    with pytest.raises(ValueError):
        lazy.load_weights(w)                                    # the config asks for a bias
    lazy.load_weights(w, b)
    assert lazy.has_weights() and lazy.config().groups == 2 and lazy.bias() is b
    with pytest.raises(ValueError):
        lazy(torch.randn(2, 5, 19))                             # wrong channel count
    with pytest.raises(ValueError):
        Conv1dConfig(6, 8, 3, groups=4).validate()

    x2 = torch.randn(1, 4, 9, 7)
    w2 = torch.randn(6, 2, 3, 2)
    conv = Conv2d(w2, None, stride=(2, 1), padding=(1, 0), dilation=(1, 2), groups=2)
    y2 = conv(x2)
    assert y2.shape == (1, 6, *conv.out_size(9, 7)) and conv.out_size(9, 7) == (5, 5)
    assert torch.allclose(y2, conv2d_direct(x2, w2, None, (2, 1), (1, 0), (1, 2), 2), atol=1e-4)
    nhwc = Conv2d(w2.permute(0, 2, 3, 1).contiguous(), stride=(2, 1), padding=(1, 0), dilation=(1, 2), groups=2,
                  channels_last=True)
    assert torch.allclose(nhwc(x2.permute(0, 2, 3, 1)), y2.permute(0, 2, 3, 1), atol=1e-5)
    lazy2 = Conv2d(Conv2dConfig(4, 6, (3, 2), groups=2))
    with pytest.raises(ValueError):
        lazy2.load_weights(torch.randn(6, 2, 2, 3))
    lazy2.load_weights(w2)
    assert lazy2.has_weights()


def test_dtype_table():
    assert dtypes.Q4_0.nbytes(64) == 36 and dtypes.Q8_0.nbytes(32) == 34 and dtypes.Q4_1.nbytes(32) == 20
    assert dtypes.BF16.nbytes(10) == 20 and not dtypes.BF16.is_quantized and dtypes.Q4_0.is_quantized
    assert dtypes.from_name("BF16") is dtypes.BF16
    assert dtypes.Q4_AFFINE_G64.nbytes(4096) == 4096 // 64 * 36          # 4.5 bits per weight
    with pytest.raises(ValueError):
        dtypes.Q4_0.nbytes(33)
    with pytest.raises(ValueError):
        dtypes.from_name("iq2_xxs")


def test_residency_and_arena():
    r = ResidencyManager(budget_bytes=100)
    r.add("a", 60)
    r.add("a", 60)
    assert len(r) == 1 and r.resident_bytes == 60 and "a" in r
    with pytest.raises(AllocError):
        r.add("b", 50)
    r.remove("a")
    r.add("b", 50)
    arena = ForwardArena(4096)
    t1 = arena.take((4, 8), torch.float32)
    t2 = arena.take((3,), torch.bfloat16)
    assert t1.shape == (4, 8) and t2.dtype == torch.bfloat16 and arena.used >= 128 + 6
    t1.fill_(1.0)
    assert float(t1.sum()) == 32.0
    with pytest.raises(AllocError):
        arena.take((4096,), torch.float32)
    arena.reset()
    assert arena.used == 0 and arena.peak > 0


def test_managed_buffer_returns_memory():
    from rmlx_b200.runtime.alloc import CachingAllocator, ManagedBuffer
    a = CachingAllocator()
    with ManagedBuffer(a, 4096) as b:
        assert b.ptr and b.nbytes >= 4096 and a.stats().bytes_in_use >= 4096
    assert a.stats().bytes_in_use == 0


def test_ncu_summary_parses_raw_csv():
    import importlib.util
    import os
    spec = importlib.util.spec_from_file_location(
        "ncu_summary", os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "benchmarks", "ncu_summary.py"))
    mod = importlib.util.module_from_spec(spec)
    import sys
    sys.modules["ncu_summary"] = mod        # dataclasses look their module up by name
    spec.loader.exec_module(mod)
    parse_raw_csv = mod.parse_raw_csv
    text = "\n".join([
        "==PROF== banner line that is not CSV",
        '"ID","Kernel Name","gpu__time_duration.sum","dram__bytes_read.sum",'
        '"sm__pipe_tensor_cycles_active.avg.pct_of_peak_sustained_active","launch__registers_per_thread",'
        '"smsp__average_warps_issue_stalled_long_scoreboard_per_issue_active.ratio",'
        '"smsp__average_warps_issue_stalled_wait_per_issue_active.ratio"',
        '"","","us","Mbyte","%","register/thread","",""',
        '"0","void my_kernel<128>(int)","57.95","25.2","36.3","131","2.04","1.65"',
        '"1","void my_kernel<128>(int)","1,058.40","25.2","n/a","131","0.5","3.25"',
    ])
    launches = parse_raw_csv(text)
    assert len(launches) == 2
    a, b = launches
    assert a.kernel.startswith("void my_kernel") and a.number("time") == 57.95
    assert a.values["tensor pipe active %"] == ("36.3", "%") and a.stalls[0] == (2.04, "long_scoreboard")
    assert "tensor pipe active %" not in b.values and b.number("time") == 1058.40
    assert b.stalls[0] == (3.25, "wait")
    assert "top stalls" in a.render() and "regs/thread: 131" in a.render()
    assert parse_raw_csv("") == []


def test_moe_layer_picks_its_exchange_through_the_policy_and_overlap_mode():
    from rmlx_b200.parallel.moe_policy import MoeBackend, MoePolicy, ThresholdCalibration

    class Loopback:
        """Single-rank exchange: sorts the (token, slot) pairs by expert, as the real ones do."""
        def __init__(self, n_experts):
            self.e, self.calls = n_experts, 0

        def dispatch(self, x, idx):
            self.calls += 1
            k = idx.shape[1]
            flat = idx.reshape(-1).long()
            order = torch.argsort(flat, stable=True)
            offsets = torch.zeros(self.e + 1, dtype=torch.int64)
            offsets[1:] = torch.cumsum(torch.bincount(flat, minlength=self.e), 0)
            lay = type("L", (), {})()
            lay.offsets, lay.order, lay.k, lay.t = offsets, order, k, x.shape[0]
            return x[order // k], lay

        def combine(self, y, wts, lay):
            out = torch.zeros(lay.t, y.shape[-1])
            out.index_add_(0, lay.order // lay.k, y.float() * wts.reshape(-1)[lay.order].float()[:, None])
            return out

    layer = _moe_layer()
    x_small, x_large = torch.randn(4, 32), torch.randn(40, 32)
    want_small, want_large = layer.forward(x_small), layer.forward(x_large)
    fused, lib = Loopback(4), Loopback(4)
    pol = MoePolicy(ThresholdCalibration(small_n_max=8, large_n_min=32), hysteresis=0, cooldown_s=0.0,
                    cooldown_calls=0, env={})
    layer.with_policy(pol, {MoeBackend.FUSED: fused, MoeBackend.LOCAL: None})
    assert torch.allclose(layer.forward(x_small), want_small, atol=1e-5) and fused.calls == 0
    assert torch.allclose(layer.forward(x_large), want_large, atol=1e-5) and fused.calls == 1
    pol.force_backend(MoeBackend.NCCL)
    layer.exchanges[MoeBackend.NCCL] = lib
    assert torch.allclose(layer.forward(x_small), want_small, atol=1e-5) and lib.calls == 1
    layer.with_policy(None, {})
    for mode in ("sbo", "tbo", None):
        assert torch.allclose(layer.with_overlap(mode).forward_overlapped(x_large), want_large, atol=1e-5)
    with pytest.raises(ValueError):
        layer.with_overlap("both")


def test_prefill_chunk_comes_from_the_static_plan():
    """The prompt chunk of the native forward is the longest one whose per-layer intermediates fit a
    scratch limit according to the layer's static plan."""
    from rmlx_b200.config import moe_a22b_config
    from rmlx_b200.models.prefill import plan_chunk
    from rmlx_b200.models.prefill_plan import PrefillPlan
    from rmlx_b200.models.weights import ParallelLayout

    class _M:
        cfg, layout = moe_a22b_config(2), ParallelLayout()

    assert plan_chunk(_M) == 8192
    small = plan_chunk(_M, 512 << 20)
    assert small % 128 == 0 and 128 <= small < 8192
    assert PrefillPlan(_M.cfg, small, _M.layout).scratch_bytes <= 512 << 20
    assert PrefillPlan(_M.cfg, small + 128, _M.layout).scratch_bytes > 512 << 20
