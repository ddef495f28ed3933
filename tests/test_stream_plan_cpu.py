"""The streaming mat-vec planner as pure logic (the library loads without a GPU): for every
supported shape the task geometry is consistent, every quad is covered exactly once, the ring and
the block fit shared memory; the model's own projections are supported at every tensor-parallel
degree. The counterpart of the reference's tile-selection tests (crates/rmlx-core/src/ops/matmul.rs:9152-9556)."""
import ctypes
import itertools

import pytest

from rmlx_b200 import _lib

NAMES = "LW qpt TR SQ QS units spl KP nseg seg_rows stage_bytes ns qpc grid smem ok".split()
DENSE, GATE_UP, MOE_DOWN = 0, 1, 2


@pytest.fixture(scope="module")
def query():
    try:
        lib = _lib.cuda()
    except Exception as e:                          # noqa: BLE001
        pytest.skip(f"CUDA library not available: {e}")
    lib.rmlx_sg_plan_query.argtypes = [ctypes.c_int] * 7 + [ctypes.POINTER(ctypes.c_int)]
    lib.rmlx_sg_plan_query.restype = ctypes.c_int

    def q(kind, op, b, n, k, top_k=1, ctas=148):
        out = (ctypes.c_int * 16)()
        rc = lib.rmlx_sg_plan_query(kind, op, b, n, k, top_k, ctas, out)
        return rc, dict(zip(NAMES, out))
    return q


def _quads(op, n):
    return n // 2 if op == GATE_UP else (n + 3) // 4


def _check(p, op, n, ctas_per_problem):
    assert p["LW"] in (8, 16, 32) and p["qpt"] == 32 // p["LW"]
    assert p["TR"] * p["SQ"] == 16 and p["QS"] == p["TR"] * p["qpt"]
    assert p["spl"] * p["LW"] >= p["units"] > (p["spl"] - 1) * p["LW"]          # slices cover a row, no empty slice
    assert 2 <= p["ns"] <= 4 and p["KP"] >= 1
    assert p["qpc"] % p["QS"] == 0                                              # whole stages per block
    quads = _quads(op, n)
    assert p["grid"] * p["qpc"] >= quads > (p["grid"] - 1) * p["qpc"]           # every quad once, no idle block
    assert p["grid"] <= ctas_per_problem
    assert p["seg_rows"] == (2 if op == GATE_UP else 4) * p["QS"]
    assert p["stage_bytes"] % 128 == 0 and p["ns"] * p["stage_bytes"] < p["smem"] <= 200 * 1024


def test_model_projections_are_supported_at_every_tp_degree(query):
    """QKV, O, LM head, dense gate/up, expert down of the 60-layer model, whole and sharded 2/4/8
    ways, 4-bit and 8-bit weights: all supported at batch 1. At batch 4 the staged activations of
    the widest input (K = 8192, unsharded) no longer fit beside the ring; that call is refused and
    the caller uses the tensor-core mat-vec."""
    d, hq, hkv, hd, inter, vocab, top_k = 4096, 64, 4, 128, 1536, 151936, 8
    for kind, tp, b in itertools.product((1, 2), (1, 2, 4, 8), (1, 4)):
        shapes = [(DENSE, (hq // tp + 2 * max(1, hkv // tp)) * hd, d, 1),          # QKV (column parallel)
                  (DENSE, d, hq * hd // tp, 1),                                     # O (row parallel)
                  (DENSE, vocab // tp, d, 1),                                       # LM head
                  (GATE_UP, 12288 // tp, d, 1),                                     # a dense layer's gate/up
                  (MOE_DOWN, d, inter // tp if inter // tp >= 512 else inter, top_k)]
        for op, n, k, tk in shapes:
            bb = 1 if op == MOE_DOWN else b
            rc, p = query(kind, op, bb, n, k, tk)
            assert rc == 0
            if bb == 1 or k < 8192:
                assert p["ok"] == 1, (kind, tp, b, op, n, k, p)
            if p["ok"]:
                _check(p, op, n, 148 // bb if op == MOE_DOWN else 148)


def test_plan_geometry_over_a_sweep_of_shapes(query):
    seen = 0
    for kind, op, b in itertools.product((0, 1, 2), (DENSE, GATE_UP), (1, 2, 4)):
        for n, k, ctas in itertools.product((64, 130, 1024, 9216, 20000), (256, 1024, 4096, 8192), (148, 74, 18)):
            if op == GATE_UP and n % 2:
                continue
            rc, p = query(kind, op, b, n, k, 1, ctas)
            assert rc == 0
            if p["ok"]:
                _check(p, op, n, ctas)
                seen += 1
    assert seen > 300
    for kind, top_k, inter in itertools.product((0, 1, 2), (2, 4, 8), (256, 768, 1536)):
        rc, p = query(kind, MOE_DOWN, 1, 4096, inter, top_k)
        assert rc == 0
        if p["ok"]:
            _check(p, MOE_DOWN, 4096, 148)
            assert p["nseg"] == top_k                                           # one segment per routed slot


def test_planner_refuses_what_it_cannot_run(query):
    assert query(3, DENSE, 1, 64, 256)[0] == -2 and query(1, 5, 1, 64, 256)[0] == -2
    assert query(1, MOE_DOWN, 1, 4096, 1536, 9)[0] == -2                        # more slots than a stage has segments
    rc, p = query(0, MOE_DOWN, 1, 4096, 1536, 8)                                # bf16 experts this wide: two stages do not fit
    assert rc == 0 and p["ok"] == 0                                             # the caller falls back to the per-row kernel


def test_flash_decode_split_heuristic():
    """About one block per SM, never more than 16 splits, never fewer than 8 pages per split."""
    from rmlx_b200.ops.decode import default_splits
    assert default_splits(1, 4, 1, 4096) == 16                   # 4 tiles: as many splits as allowed
    assert default_splits(1, 4, 1, 1024) == 8                    # 64 pages: 8 pages per split
    assert default_splits(1, 4, 1, 100) == 1 and default_splits(64, 4, 1, 8192) == 1
    assert default_splits(8, 4, 1, 8192) == 5                    # 32 tiles -> ceil(148 / 32)
    for b, hkv, ctx in itertools.product((1, 2, 8, 32), (1, 4, 8), (128, 2048, 32768)):
        s = default_splits(b, hkv, 1, ctx)
        assert 1 <= s <= 16 and (s == 1 or ctx // s >= 128)
        assert s == 1 or (s - 1) * b * hkv < 148                 # one split fewer would leave SMs idle
