"""The native execution runtime on a GPU: the keyed graph store (record, replay, eviction), events
with bounded / cancellable host waits, and the decode engine replaying its steps through it; the
grouped narrow-M expert kernels. Collected late: these tests record graphs by hand."""
import pytest
import torch

pytestmark = pytest.mark.gpu

from rmlx_b200.models.decode_engine import CachedDecode          # noqa: E402
from rmlx_b200.models.transformer import TransformerModel        # noqa: E402
from rmlx_b200.models.weights import from_state_dict, random_state_dict   # noqa: E402
from rmlx_b200.ops import decode as D                             # noqa: E402
from rmlx_b200.ops.weights import LinearWeight                    # noqa: E402
from rmlx_b200.runtime.graph import GraphCache                    # noqa: E402
from rmlx_b200.runtime.native_graph import CancelFlag, NativeEvent, NativeGraphStore   # noqa: E402
from test_decode_engine_gpu import tiny_moe_config                # noqa: E402
from test_decode_kernels_gpu import _close, _w                    # noqa: E402


@pytest.fixture(scope="module")
def dev():
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    return torch.device("cuda:0")


def test_store_records_replays_and_evicts(dev):
    torch.manual_seed(0)
    w1 = LinearWeight.random(512, 1024, None, dev)
    w2 = LinearWeight.random(256, 512, None, dev)
    x = torch.randn(2, 1024, device=dev).to(torch.bfloat16)
    mid = torch.empty(2, 512, dtype=torch.bfloat16, device=dev)
    out = torch.empty(2, 256, dtype=torch.bfloat16, device=dev)

    def chain():
        D.rms_gemv(x, w1, out=mid)
        D.rms_gemv(mid, w2, out=out)

    chain()
    torch.cuda.synchronize()
    want = out.clone()
    store = NativeGraphStore(max_entries=2)
    assert not store.has("a")
    nodes = store.capture("a", chain)          # on the store's own stream
    assert nodes >= 2 and store.has("a")
    x.mul_(2)                                  # the graph reads the buffers, not values seen at capture
    out.zero_()
    store.launch("a")
    torch.cuda.synchronize()
    assert torch.allclose(out.float(), 2 * want.float(), rtol=2e-2, atol=2e-2 * float(want.abs().max()))
    store.capture("b", chain)
    store.launch("a")                          # "a" is now the most recently used
    store.capture("c", chain)                  # evicts "b"
    st = store.stats()
    assert st["entries"] == 2 and st["captures"] == 3 and st["evictions"] == 1 and st["launches"] == 2
    assert store.has("a") and store.has("c") and not store.has("b")
    with pytest.raises(KeyError):
        store.launch("b")
    assert store.invalidate("a") == 1 and store.invalidate() == 1
    torch.cuda.synchronize()
    store.close()


def test_event_wait_has_a_deadline_and_a_cancel_flag(dev):
    a = torch.randn(8192, 8192, device=dev, dtype=torch.bfloat16)
    torch.cuda.synchronize()
    first = NativeEvent(timing=True).record()
    for _ in range(60):                        # tens of milliseconds of queued work
        a @ a
    ev = NativeEvent(timing=True).record()
    assert ev.wait(timeout_s=0.0005) == NativeEvent.TIMEOUT
    flag = CancelFlag()
    flag.set()
    assert ev.wait(timeout_s=5.0, cancel=flag) == NativeEvent.CANCELLED
    assert ev.wait(timeout_s=30.0) == NativeEvent.DONE
    assert first.elapsed_ms(ev) > 1.0
    ev.stream_wait()                           # a completed event: the current stream goes straight on
    torch.cuda.synchronize()


def test_decode_engine_replays_through_the_native_store(dev, monkeypatch):
    """On one GPU the engine's step is recorded by the native store (its warm-up run allocates
    nothing: every buffer is the engine's); RMLX_NATIVE_GRAPHS=0 keeps torch's graphs, and the
    tokens are the same either way."""
    cfg = tiny_moe_config()
    model = TransformerModel(from_state_dict(cfg, random_state_dict(cfg, 0), device=dev, quant="q4"))
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g) for n in (9, 14)]

    def run():
        cache = model.new_cache(16, max_seqs=4)
        last = []
        for s in range(2):
            cache.add_sequence(s)
            last.append(int(model.forward(prompts[s].to(dev), cache, [s], last_only=True)[0].argmax()))
        eng = CachedDecode(model, cache, max_batch=2)
        eng.bind([0, 1], last)
        return eng, eng.generate(5)

    monkeypatch.setenv("RMLX_NATIVE_GRAPHS", "0")
    ref, want = run()
    assert not ref.graphs.native and ref.graphs.native_captures == 0
    monkeypatch.delenv("RMLX_NATIVE_GRAPHS")
    eng, got = run()
    assert eng.graphs.native and torch.equal(got, want)
    assert eng.graphs.captures == 1 and eng.graphs.native_captures == 1 and eng.graphs.native_refused == 0


@pytest.mark.parametrize("variant", [0, 1])
def test_narrow_grouped_expert_ffn(dev, variant):
    """The narrow-M grouped expert kernels (a few sorted rows per expert, 4-bit weights) against
    fp32: experts without rows, one row, and more rows than one pass holds; a rank holding a slice
    of the experts leaves the other experts' rows zero."""
    from rmlx_b200.ops.grouped import narrow_expert_ffn, narrow_supported
    e, d, i = 6, 1024, 512
    wgu = _w(2 * i, d, "q4", dev, experts=e, seed=18)
    wdn = _w(d, i, "q4", dev, experts=e, seed=19)
    counts = [3, 0, 1, 11, 0, 8]
    off = torch.tensor([0] + list(torch.tensor(counts).cumsum(0)), dtype=torch.int32, device=dev)
    r = sum(counts)
    assert narrow_supported(wgu, wdn, variant)
    torch.manual_seed(20)
    xs = torch.randn(r, d, device=dev).to(torch.bfloat16)
    gu_d, dn_d = wgu.dequantized(), wdn.dequantized()
    want = torch.zeros(r, d, device=dev)
    want_act = torch.zeros(r, i, device=dev)
    for ex in range(e):
        lo, hi = int(off[ex]), int(off[ex + 1])
        h = xs[lo:hi].float() @ gu_d[ex].t()
        a = (torch.nn.functional.silu(h[:, :i]) * h[:, i:]).to(torch.bfloat16).float()
        want_act[lo:hi] = a
        want[lo:hi] = a @ dn_d[ex].t()
    got = narrow_expert_ffn(xs, off, wgu, wdn, variant=variant)
    _close(got, want)
    # experts 2..4 only (a rank's slice): rows of the other experts stay zero
    sl_gu, sl_dn = wgu.experts_slice(2, 5), wdn.experts_slice(2, 5)
    part = narrow_expert_ffn(xs, off[2:6], sl_gu, sl_dn, zero_rest=True, variant=variant)
    lo, hi = int(off[2]), int(off[5])
    _close(part[lo:hi], want[lo:hi])
    assert float(part[:lo].abs().sum()) == 0.0 and float(part[hi:].abs().sum()) == 0.0
    torch.cuda.synchronize()
    from rmlx_b200 import _lib
    assert _lib.cuda().rmlx_qmv_status() == 0
