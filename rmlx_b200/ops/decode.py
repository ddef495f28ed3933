"""Python entry points for the decode-path kernels (csrc/kernels/decode_gemv.cu, decode_moe.cu,
flash_decode.cu, rope_kv.cu, misc.cu). Each function validates shapes, allocates the output when
none is passed, and launches on the current stream; with ``pdl=True`` the launch carries the
programmatic-dependent-launch attribute so its prologue overlaps the previous kernel's tail.

Batches larger than the kernels' activation-tile limit are processed in chunks.
"""
from __future__ import annotations

import math
import os
from typing import Optional, Tuple

import torch

from .. import _lib
from .weights import LinearWeight, W_Q4

_MAXB = 4
_Q4_PATH = os.environ.get("RMLX_Q4_PATH", "auto")
_STREAM = os.environ.get("RMLX_DECODE_STREAM", "1") != "0"
# Which operations take the streaming kernels when streaming is on: any of qkv, gemv (O projection,
# dense down projection, LM head), gate_up, moe_gate_up, moe_down. Measured inside the captured
# step of the 60-layer model (4-bit weights, one GPU, us per layer; per-row kernels everywhere:
# 82.6): streaming the expert down projection saves 3.2, the expert gate/up 3.2, while streaming
# the merged QKV costs 1.3 and the O projection / LM head 2.7 (their per-row kernels request the
# first rows before the dependency wait and have less to set up). Hence the default below; 8-bit
# weights and fp16 scales exist only in the streaming kernels and always take them.
_STREAM_OPS = set(os.environ.get("RMLX_DECODE_STREAM_OPS", "gate_up,moe_gate_up,moe_down").split(","))


def _stream(op: str, w: Optional[LinearWeight] = None) -> bool:
    if not _STREAM:
        return False
    return op in _STREAM_OPS or (w is not None and (w.kind == 2 or w.scales_f16))

_lib.register_cuda_sigs({
    "rmlx_sg_status": ("", "i"),
    "rmlx_sg_debug_drop_stage": ("i", "i"),
    "rmlx_sg_rms_gemv": ("ippppipfpipiiiiiip", "i"),
    "rmlx_sg_rms_qkv_rope": ("ippppipfppppppppiiiiiiiiip", "i"),
    "rmlx_sg_gate_up": ("ippppipfpiiiiip", "i"),
    "rmlx_sg_moe_gate_up": ("ippppipfppiiiiiiiip", "i"),
    "rmlx_sg_moe_down": ("ippppipppipiiiiiiiiip", "i"),
})


def stream_enabled() -> bool:
    """Whether the decode projections run on the persistent weight-streaming kernels
    (csrc/kernels/stream_gemv.cuh: bulk-copy ring, one block per SM). Shapes those kernels do not
    take, and ``RMLX_DECODE_STREAM=0``, use the one-warp-per-row kernels."""
    return _STREAM


ALL_STREAM_OPS = ("qkv", "gemv", "gate_up", "moe_gate_up", "moe_down")
_DEFAULT_STREAM_OPS = set(_STREAM_OPS)


def set_stream(on: bool, ops=None) -> None:
    """Switch the streaming kernels on or off; ``ops``: which operations take them ("all", an
    iterable of names from ``ALL_STREAM_OPS``, or None for the default selection)."""
    global _STREAM, _STREAM_OPS
    _STREAM = bool(on)
    if ops == "all":
        _STREAM_OPS = set(ALL_STREAM_OPS)
    elif ops is None:
        _STREAM_OPS = set(_DEFAULT_STREAM_OPS)
    else:
        _STREAM_OPS = set(ops)


def stream_plan(w_kind: int, op: int, batch: int, n: int, k: int, top_k: int = 1, ctas: int = 0) -> dict:
    """The plan the streaming kernels would use for a projection (host arithmetic only, no device
    needed): ``op`` 0 dense mat-vec of ``n`` rows, 1 gate/up with SwiGLU (``n`` = intermediate
    size), 2 expert down projection over ``top_k`` routed slots of ``k`` weights. ``ok`` is False
    when the launch would be refused (the caller then runs another kernel family)."""
    import ctypes
    lib = _lib.cuda()
    lib.rmlx_sg_plan_query.argtypes = [ctypes.c_int] * 7 + [ctypes.POINTER(ctypes.c_int)]
    lib.rmlx_sg_plan_query.restype = ctypes.c_int
    out = (ctypes.c_int * 16)()
    if lib.rmlx_sg_plan_query(w_kind, op, batch, n, k, top_k, ctas, out) != 0:
        raise ValueError("bad planner query")
    names = "LW qpt TR SQ QS units spl KP nseg seg_rows stage_bytes ns qpc grid smem ok".split()
    plan = dict(zip(names, out))
    plan["ok"] = bool(plan["ok"])
    return plan


def stream_status() -> int:
    """0, or the code of a bounded wait that expired inside a streaming kernel since the last call."""
    return int(_lib.cuda().rmlx_sg_status())



def q4_path() -> str:
    """Which Q4 mat-vec implementation runs: 'mma' (bulk-copy-fed tensor-core path), 'scalar'
    (fp16 FMA path on subnormal-encoded nibbles) or 'auto' (per kernel, whichever measured faster on
    B200: since the scalar inner loop lost its magic-constant subtraction it wins everywhere, so
    'auto' is the scalar path; the tensor-core path stays selectable)."""
    return _Q4_PATH


def set_q4_path(path: str) -> None:
    global _Q4_PATH
    assert path in ("auto", "mma", "scalar")
    _Q4_PATH = path


def _wargs(w: LinearWeight):
    return (w.kernel_kind, w.w.data_ptr(), _lib.ptr(w.scales), _lib.ptr(w.biases))


def rms_gemv(x: torch.Tensor, w: LinearWeight, norm_w: Optional[torch.Tensor] = None,
             eps: float = 1e-6, residual: Optional[torch.Tensor] = None,
             out: Optional[torch.Tensor] = None, out_dtype=torch.bfloat16, pdl: bool = False
             ) -> torch.Tensor:
    """out[b] = residual[b] + W @ rmsnorm(x[b]; norm_w). norm_w None = no norm; x: [B, K] bf16."""
    _lib.require_cuda_tensor(x, w.w)
    assert x.dtype == torch.bfloat16 and x.dim() == 2 and x.stride(1) == 1
    b, k = x.shape
    n = w.n
    assert k == w.k, f"K mismatch {k} vs {w.k}"
    if out is None:
        out = torch.empty(b, n, dtype=out_dtype, device=x.device)
    lib, st = _lib.cuda(), _lib.stream_ptr()
    # Several rows against 4-bit weights: the tensor-core mat-vec carries up to eight rows in the
    # MMA's columns for the price of one, while the CUDA-core kernels pay their unpacking FMAs per
    # row (measured on B200, 9216x4096: four rows 29.5 us streaming; the weights are read once
    # either way).
    mma_rows = (w.kind == W_Q4 and not w.scales_f16 and b >= 2 and q4_path() != "scalar" and
                bool(lib.rmlx_qmv_mma_supported(k, min(8, b), 16)))
    if _stream("gemv", w) and not mma_rows:
        done = True
        for b0 in range(0, b, _MAXB):
            bb = min(_MAXB, b - b0)
            xs, os_ = x[b0:b0 + bb], out[b0:b0 + bb]
            rs = None if residual is None else residual[b0:b0 + bb]
            rc = lib.rmlx_sg_rms_gemv(*_wargs(w), xs.data_ptr(), xs.stride(0), _lib.ptr(norm_w), eps,
                                      _lib.ptr(rs), 0 if rs is None else rs.stride(0), os_.data_ptr(),
                                      os_.stride(0), int(out.dtype == torch.float32), bb, n, k,
                                      int(pdl), st)
            if rc == -2 and b0 == 0:
                done = False
                break
            _lib.check(rc, "sg_rms_gemv")
        if done:
            return out
    if mma_rows or (w.kind == W_Q4 and not w.scales_f16 and q4_path() == "mma" and
                    lib.rmlx_qmv_mma_supported(k, min(8, b), 16)):
        for b0 in range(0, b, 8):
            bb = min(8, b - b0)
            xs, os_ = x[b0:b0 + bb], out[b0:b0 + bb]
            rs = None if residual is None else residual[b0:b0 + bb]
            rc = lib.rmlx_rms_qmv_mma(w.w.data_ptr(), w.scales.data_ptr(), w.biases.data_ptr(),
                                      xs.data_ptr(), xs.stride(0), _lib.ptr(norm_w), eps,
                                      _lib.ptr(rs), 0 if rs is None else rs.stride(0),
                                      os_.data_ptr(), os_.stride(0),
                                      int(out.dtype == torch.float32), bb, n, k, int(pdl), st)
            _lib.check(rc, "rms_qmv_mma")
        return out
    for b0 in range(0, b, _MAXB):
        bb = min(_MAXB, b - b0)
        xs, os_ = x[b0:b0 + bb], out[b0:b0 + bb]
        rs = None if residual is None else residual[b0:b0 + bb]
        rc = lib.rmlx_rms_gemv(*_wargs(w), xs.data_ptr(), xs.stride(0), _lib.ptr(norm_w), eps,
                               _lib.ptr(rs), 0 if rs is None else rs.stride(0), os_.data_ptr(),
                               os_.stride(0), int(out.dtype == torch.float32), bb, n, k, int(pdl), st)
        _lib.check(rc, "rms_gemv")
    return out


def rms_gate_up_swiglu(x: torch.Tensor, w: LinearWeight, norm_w: Optional[torch.Tensor], eps: float,
                       out: Optional[torch.Tensor] = None, pdl: bool = False) -> torch.Tensor:
    """Dense SwiGLU first half: act = silu(Wg xn) * (Wu xn); w holds gate rows then up rows."""
    _lib.require_cuda_tensor(x, w.w)
    b, k = x.shape
    i = w.n // 2
    if out is None:
        out = torch.empty(b, i, dtype=torch.bfloat16, device=x.device)
    lib, st = _lib.cuda(), _lib.stream_ptr()
    if _stream("gate_up", w):
        done = True
        for b0 in range(0, b, _MAXB):
            bb = min(_MAXB, b - b0)
            xs, os_ = x[b0:b0 + bb], out[b0:b0 + bb]
            rc = lib.rmlx_sg_gate_up(*_wargs(w), xs.data_ptr(), xs.stride(0), _lib.ptr(norm_w), eps,
                                     os_.data_ptr(), os_.stride(0), bb, i, k, int(pdl), st)
            if rc == -2 and b0 == 0:
                done = False
                break
            _lib.check(rc, "sg_gate_up")
        if done:
            return out
    for b0 in range(0, b, _MAXB):
        bb = min(_MAXB, b - b0)
        xs, os_ = x[b0:b0 + bb], out[b0:b0 + bb]
        rc = lib.rmlx_rms_gate_up_swiglu(*_wargs(w), xs.data_ptr(), xs.stride(0), _lib.ptr(norm_w),
                                         eps, os_.data_ptr(), os_.stride(0), bb, i, k, int(pdl), st)
        _lib.check(rc, "rms_gate_up_swiglu")
    return out


def swiglu_down(gate_up: torch.Tensor, w: LinearWeight, residual: Optional[torch.Tensor] = None,
                out: Optional[torch.Tensor] = None, pdl: bool = False) -> torch.Tensor:
    """out = residual + W_down @ (silu(gate) * up) with gate_up = [gate | up] per row."""
    _lib.require_cuda_tensor(gate_up, w.w)
    b = gate_up.shape[0]
    i = gate_up.shape[1] // 2
    assert i == w.k
    n = w.n
    if out is None:
        out = torch.empty(b, n, dtype=torch.bfloat16, device=gate_up.device)
    lib, st = _lib.cuda(), _lib.stream_ptr()
    for b0 in range(0, b, _MAXB):
        bb = min(_MAXB, b - b0)
        g, os_ = gate_up[b0:b0 + bb], out[b0:b0 + bb]
        rs = None if residual is None else residual[b0:b0 + bb]
        rc = lib.rmlx_swiglu_down(*_wargs(w), g.data_ptr(), g.stride(0), _lib.ptr(rs),
                                  0 if rs is None else rs.stride(0), os_.data_ptr(), os_.stride(0),
                                  bb, n, i, int(pdl), st)
        _lib.check(rc, "swiglu_down")
    return out


class RouterScratch:
    """Device scratch for the fused router: fp32 logits [B, E] and a zeroed ticket word."""

    def __init__(self, max_batch: int, num_experts: int, device):
        self.logits = torch.empty(max_batch, num_experts, dtype=torch.float32, device=device)
        self.ticket = torch.zeros(1, dtype=torch.int32, device=device)


def moe_router(x: torch.Tensor, gate_w: torch.Tensor, norm_w: Optional[torch.Tensor], eps: float,
               top_k: int, expert_bias: Optional[torch.Tensor] = None,
               scratch: Optional[RouterScratch] = None, idx: Optional[torch.Tensor] = None,
               wts: Optional[torch.Tensor] = None, counts: Optional[torch.Tensor] = None,
               pdl: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    """RMSNorm + gate projection + softmax + top-k + renormalise. x [B, K] bf16, gate_w [E, K] bf16.
    Returns (indices int32 [B, k], weights fp32 [B, k])."""
    _lib.require_cuda_tensor(x, gate_w)
    b, k = x.shape
    e = gate_w.shape[0]
    scratch = scratch or RouterScratch(b, e, x.device)
    if idx is None:
        idx = torch.empty(b, top_k, dtype=torch.int32, device=x.device)
    if wts is None:
        wts = torch.empty(b, top_k, dtype=torch.float32, device=x.device)
    lib, st = _lib.cuda(), _lib.stream_ptr()
    for b0 in range(0, b, _MAXB):
        bb = min(_MAXB, b - b0)
        xs = x[b0:b0 + bb]
        rc = lib.rmlx_moe_router(gate_w.data_ptr(), xs.data_ptr(), xs.stride(0), _lib.ptr(norm_w),
                                 eps, _lib.ptr(expert_bias), scratch.logits[b0:].data_ptr(),
                                 idx[b0:].data_ptr(), wts[b0:].data_ptr(), _lib.ptr(counts),
                                 scratch.ticket.data_ptr(), bb, e, k, top_k, int(pdl), st)
        _lib.check(rc, "moe_router")
    return idx, wts


def topk_route(logits: torch.Tensor, top_k: int, expert_bias: Optional[torch.Tensor] = None,
               want_counts: bool = True):
    """Selection over precomputed fp32 logits [T, E]. Returns (idx, weights, counts, offsets)."""
    _lib.require_cuda_tensor(logits)
    assert logits.dtype == torch.float32 and logits.is_contiguous()
    t, e = logits.shape
    idx = torch.empty(t, top_k, dtype=torch.int32, device=logits.device)
    wts = torch.empty(t, top_k, dtype=torch.float32, device=logits.device)
    counts = torch.empty(e, dtype=torch.int32, device=logits.device) if want_counts else None
    offsets = torch.empty(e + 1, dtype=torch.int32, device=logits.device) if want_counts else None
    rc = _lib.cuda().rmlx_topk_route(logits.data_ptr(), _lib.ptr(expert_bias), idx.data_ptr(),
                                     wts.data_ptr(), _lib.ptr(counts), _lib.ptr(offsets), t, e, top_k,
                                     _lib.stream_ptr())
    _lib.check(rc, "topk_route")
    return idx, wts, counts, offsets


def moe_gate_up(x: torch.Tensor, w: LinearWeight, norm_w: Optional[torch.Tensor], eps: float,
                idx: torch.Tensor, out: Optional[torch.Tensor] = None, expert_base: int = 0,
                pdl: bool = False) -> torch.Tensor:
    """Per (token, slot): act = silu(Wg[e] xn) * (Wu[e] xn). w: stacked [E_local, 2I, K].
    Slots whose expert is outside [expert_base, expert_base + E_local) are left untouched."""
    _lib.require_cuda_tensor(x, w.w, idx)
    b, k = x.shape
    top_k = idx.shape[1]
    i = w.n // 2
    if out is None:
        out = torch.zeros(b * top_k, i, dtype=torch.bfloat16, device=x.device)
    if _stream("moe_gate_up", w):
        rc = _lib.cuda().rmlx_sg_moe_gate_up(*_wargs(w), x.data_ptr(), x.stride(0), _lib.ptr(norm_w),
                                             eps, idx.data_ptr(), out.data_ptr(), out.stride(0), b,
                                             top_k, i, k, expert_base, w.experts, int(pdl),
                                             _lib.stream_ptr())
        if rc != -2:
            _lib.check(rc, "sg_moe_gate_up")
            return out
    if w.kind == W_Q4 and q4_path() == "mma" and _lib.cuda().rmlx_qmv_mma_supported(k, 1, 32):
        rc = _lib.cuda().rmlx_moe_gate_up_q4_mma(
            w.w.data_ptr(), w.scales.data_ptr(), w.biases.data_ptr(), x.data_ptr(), x.stride(0),
            _lib.ptr(norm_w), eps, idx.data_ptr(), out.data_ptr(), out.stride(0), b, top_k, i, k,
            expert_base, w.experts, int(pdl), _lib.stream_ptr())
        _lib.check(rc, "moe_gate_up_q4_mma")
        return out
    rc = _lib.cuda().rmlx_moe_gate_up(*_wargs(w), x.data_ptr(), x.stride(0), _lib.ptr(norm_w), eps,
                                      idx.data_ptr(), out.data_ptr(), out.stride(0), b, top_k, i, k,
                                      expert_base, w.experts, int(pdl), _lib.stream_ptr())
    _lib.check(rc, "moe_gate_up")
    return out


def moe_down(act: torch.Tensor, w: LinearWeight, idx: torch.Tensor, wts: torch.Tensor,
             residual: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
             out_dtype=torch.bfloat16, expert_base: int = 0, pdl: bool = False) -> torch.Tensor:
    """out[b] = residual[b] + sum_slot wts[b,slot] * Wd[e] @ act[b*k+slot]. w: [E_local, N, I]."""
    _lib.require_cuda_tensor(act, w.w, idx, wts)
    b, top_k = idx.shape
    n, i = w.n, w.k
    if out is None:
        out = torch.empty(b, n, dtype=out_dtype, device=act.device)
    if _stream("moe_down", w):
        rc = _lib.cuda().rmlx_sg_moe_down(*_wargs(w), act.data_ptr(), act.stride(0), idx.data_ptr(),
                                          wts.data_ptr(), _lib.ptr(residual),
                                          0 if residual is None else residual.stride(0),
                                          out.data_ptr(), out.stride(0),
                                          int(out.dtype == torch.float32), b, top_k, n, i,
                                          expert_base, w.experts, int(pdl), _lib.stream_ptr())
        if rc != -2:
            _lib.check(rc, "sg_moe_down")
            return out
    if w.kind == W_Q4 and q4_path() == "mma" and _lib.cuda().rmlx_moe_down_q4_mma_supported(i, top_k):
        rc = _lib.cuda().rmlx_moe_down_q4_mma(
            w.w.data_ptr(), w.scales.data_ptr(), w.biases.data_ptr(), act.data_ptr(), act.stride(0),
            idx.data_ptr(), wts.data_ptr(), _lib.ptr(residual),
            0 if residual is None else residual.stride(0), out.data_ptr(), out.stride(0),
            int(out.dtype == torch.float32), b, top_k, n, i, expert_base, w.experts, int(pdl),
            _lib.stream_ptr())
        _lib.check(rc, "moe_down_q4_mma")
        return out
    rc = _lib.cuda().rmlx_moe_down(*_wargs(w), act.data_ptr(), act.stride(0), idx.data_ptr(),
                                   wts.data_ptr(), _lib.ptr(residual),
                                   0 if residual is None else residual.stride(0), out.data_ptr(),
                                   out.stride(0), int(out.dtype == torch.float32), b, top_k, n, i,
                                   expert_base, w.experts, int(pdl), _lib.stream_ptr())
    _lib.check(rc, "moe_down")
    return out


_lib.register_cuda_sigs({
    "rmlx_flash_decode_cluster_plan": ("iii", "i"),
    "rmlx_flash_decode_cluster_part_o_elems": ("iii", "q"),
    "rmlx_flash_decode_cluster_part_ml_elems": ("ii", "q"),
    "rmlx_flash_decode_cluster": ("pppppppppiiiiiiifip", "i"),
})
_FD_CLUSTER = os.environ.get("RMLX_FLASH_DECODE_CLUSTER", "1") != "0"


class FlashDecodeScratch:
    """Split-KV scratch: partial outputs, (max, sum) pairs and the per-tile ticket counters.

    With ``max_len`` given, the scratch also plans the cluster kernel (flash_decode_cluster.cu:
    thread-block clusters merging through distributed shared memory), which takes over when a
    few sequences have to fill the machine; ``clusters`` is then its plan
    ((cluster size << 8) | clusters per tile)."""

    def __init__(self, batch: int, hq: int, hkv: int, head_dim: int, splits: int, device,
                 max_len: Optional[int] = None):
        lib = _lib.cuda()
        self.splits = splits
        self.part_o = torch.empty(lib.rmlx_flash_decode_part_o_elems(batch, hq, hkv, splits, head_dim),
                                  dtype=torch.float32, device=device)
        self.part_ml = torch.empty(lib.rmlx_flash_decode_part_ml_elems(batch, hq, hkv, splits),
                                   dtype=torch.float32, device=device)
        self.tickets = torch.zeros(lib.rmlx_flash_decode_ticket_elems(batch, hq, hkv),
                                   dtype=torch.int32, device=device)
        self.clusters = 0
        if max_len is not None and _FD_CLUSTER:
            tiles = batch * hkv * lib.rmlx_flash_decode_gtiles(hq, hkv)
            with torch.cuda.device(device):
                self.clusters = int(lib.rmlx_flash_decode_cluster_plan(tiles, int(max_len), head_dim))
            if (self.clusters & 0xff) > 1:
                self.c_part_o = torch.empty(
                    lib.rmlx_flash_decode_cluster_part_o_elems(tiles, self.clusters & 0xff, head_dim),
                    dtype=torch.float32, device=device)
                self.c_part_ml = torch.empty(
                    lib.rmlx_flash_decode_cluster_part_ml_elems(tiles, self.clusters & 0xff),
                    dtype=torch.float32, device=device)
                self.c_tickets = torch.zeros(tiles, dtype=torch.int32, device=device)


def default_splits(batch: int, hkv: int, gtiles: int, max_len: int, sm_count: int = 148) -> int:
    """About one block per SM, capped so a split keeps at least 8 pages (two per warp)."""
    tiles = max(1, batch * hkv * gtiles)
    want = max(1, (sm_count + tiles - 1) // tiles)
    cap = max(1, max_len // 128)
    return int(min(16, want, cap))


def flash_decode_paged(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                       block_table: torch.Tensor, seq_lens: torch.Tensor,
                       scale: Optional[float] = None, splits: Optional[int] = None,
                       scratch: Optional[FlashDecodeScratch] = None, window: int = 0,
                       out: Optional[torch.Tensor] = None, pdl: bool = False,
                       k_sb: Optional[torch.Tensor] = None,
                       v_sb: Optional[torch.Tensor] = None) -> torch.Tensor:
    """q [B, Hq, D] bf16; caches [blocks, Hkv, 16, D] bf16; block_table int32 [B, max_blocks];
    seq_lens int32 [B] (context length including the current token). With ``k_sb`` / ``v_sb``
    (bf16 [blocks, Hkv, 16, D/64, 2]) the caches are the uint8 codes of the 8-bit format and the
    kernel expands pages in shared memory."""
    _lib.require_cuda_tensor(q, k_cache, v_cache, block_table, seq_lens)
    b, hq, d = q.shape
    hkv, page = k_cache.shape[1], k_cache.shape[2]
    assert page == 16 and k_cache.shape[3] == d and q.is_contiguous()
    assert block_table.dtype == torch.int32 and seq_lens.dtype == torch.int32
    if scale is None:
        scale = 1.0 / math.sqrt(d)
    lib = _lib.cuda()
    if splits is None:
        splits = scratch.splits if scratch is not None else default_splits(
            b, hkv, lib.rmlx_flash_decode_gtiles(hq, hkv), block_table.shape[1] * page)
    if splits > 1 and scratch is None:
        scratch = FlashDecodeScratch(b, hq, hkv, d, splits, q.device)
    if out is None:
        out = torch.empty_like(q)
    if k_sb is not None:
        assert k_cache.dtype == torch.uint8 and v_sb is not None and k_sb.dtype == torch.bfloat16
        rc = lib.rmlx_flash_decode_paged_q8(
            q.data_ptr(), k_cache.data_ptr(), k_sb.data_ptr(), v_cache.data_ptr(), v_sb.data_ptr(),
            block_table.data_ptr(), seq_lens.data_ptr(), out.data_ptr(),
            None if scratch is None else scratch.part_o.data_ptr(),
            None if scratch is None else scratch.part_ml.data_ptr(),
            None if scratch is None else scratch.tickets.data_ptr(),
            b, hq, hkv, d, block_table.stride(0), splits, window, scale, int(pdl), _lib.stream_ptr())
        _lib.check(rc, "flash_decode_paged_q8")
        return out
    if scratch is not None and scratch.clusters > 0 and (splits is None or splits == scratch.splits):
        nc = scratch.clusters & 0xff
        rc = lib.rmlx_flash_decode_cluster(
            q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), block_table.data_ptr(),
            seq_lens.data_ptr(), out.data_ptr(),
            scratch.c_part_o.data_ptr() if nc > 1 else None,
            scratch.c_part_ml.data_ptr() if nc > 1 else None,
            scratch.c_tickets.data_ptr() if nc > 1 else None,
            b, hq, hkv, d, block_table.stride(0), scratch.clusters, window, scale, int(pdl),
            _lib.stream_ptr())
        _lib.check(rc, "flash_decode_cluster")
        return out
    rc = lib.rmlx_flash_decode_paged(
        q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), block_table.data_ptr(),
        seq_lens.data_ptr(), out.data_ptr(),
        None if scratch is None else scratch.part_o.data_ptr(),
        None if scratch is None else scratch.part_ml.data_ptr(),
        None if scratch is None else scratch.tickets.data_ptr(),
        b, hq, hkv, d, block_table.stride(0), splits, window, scale, int(pdl), _lib.stream_ptr())
    _lib.check(rc, "flash_decode_paged")
    return out


def rope_kv_write(qkv: torch.Tensor, q_out: torch.Tensor, k_cache: torch.Tensor,
                  v_cache: torch.Tensor, block_table: torch.Tensor, positions: torch.Tensor,
                  cos: torch.Tensor, sin: torch.Tensor, hq: int, hkv: int,
                  token_seq: Optional[torch.Tensor] = None, traditional: bool = False,
                  pdl: bool = False, k_sb: Optional[torch.Tensor] = None,
                  v_sb: Optional[torch.Tensor] = None) -> torch.Tensor:
    """RoPE(Q) -> q_out, RoPE(K) and V -> their page slots. qkv [T, (Hq+2Hkv)*D] bf16. With
    ``k_sb`` / ``v_sb`` the caches are in the 8-bit format: K and V are quantised as they are
    written."""
    _lib.require_cuda_tensor(qkv, q_out, k_cache, v_cache, block_table, positions, cos, sin)
    t = qkv.shape[0]
    d = k_cache.shape[3]
    assert qkv.is_contiguous() and qkv.shape[1] == (hq + 2 * hkv) * d
    assert positions.dtype == torch.int32 and cos.dtype == torch.float32
    if k_sb is not None:
        assert k_cache.dtype == torch.uint8 and v_sb is not None
        rc = _lib.cuda().rmlx_rope_kv_write_q8(
            qkv.data_ptr(), q_out.data_ptr(), k_cache.data_ptr(), k_sb.data_ptr(), v_cache.data_ptr(),
            v_sb.data_ptr(), block_table.data_ptr(), positions.data_ptr(), _lib.ptr(token_seq),
            cos.data_ptr(), sin.data_ptr(), t, hq, hkv, d, block_table.stride(0), k_cache.shape[2],
            int(traditional), int(pdl), _lib.stream_ptr())
        _lib.check(rc, "rope_kv_write_q8")
        return q_out
    rc = _lib.cuda().rmlx_rope_kv_write(
        qkv.data_ptr(), q_out.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(),
        block_table.data_ptr(), positions.data_ptr(), _lib.ptr(token_seq), cos.data_ptr(),
        sin.data_ptr(), t, hq, hkv, d, block_table.stride(0), k_cache.shape[2], int(traditional),
        int(pdl), _lib.stream_ptr())
    _lib.check(rc, "rope_kv_write")
    return q_out


_lib.register_cuda_sigs({
    "rmlx_rms_qkv_rope": ("ippppipfppppppppiiiiiiiiip", "i"),
    "rmlx_flash_decode_paged_q8": ("pppppppppppiiiiiiifip", "i"),
    "rmlx_rope_kv_write_q8": ("pppppppppppiiiiiiiip", "i"),
    "rmlx_kv_dequant_pages": ("ppppiiiip", "i"),
})


def kv_dequant_pages(codes: torch.Tensor, sb: torch.Tensor, table_row: torch.Tensor, n_pages: int,
                     out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Expand the first ``n_pages`` pages of one sequence (``table_row`` int32) of an 8-bit cache
    into contiguous bf16 pages [n_pages, Hkv, page, D] (page i of the result is page
    ``table_row[i]`` of the cache)."""
    _lib.require_cuda_tensor(codes, sb, table_row)
    _, hkv, page, d = codes.shape
    if out is None:
        out = torch.empty(n_pages, hkv, page, d, dtype=torch.bfloat16, device=codes.device)
    rc = _lib.cuda().rmlx_kv_dequant_pages(codes.data_ptr(), sb.data_ptr(), table_row.data_ptr(),
                                           out.data_ptr(), n_pages, hkv, page, d, _lib.stream_ptr())
    _lib.check(rc, "kv_dequant_pages")
    return out


def rms_qkv_rope(x: torch.Tensor, w: LinearWeight, norm_w: Optional[torch.Tensor], eps: float,
                 q_out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                 block_table: torch.Tensor, positions: torch.Tensor, cos: torch.Tensor,
                 sin: torch.Tensor, hq: int, hkv: int, row_seq: Optional[torch.Tensor] = None,
                 traditional: bool = False, pdl: bool = False) -> torch.Tensor:
    """RMSNorm + merged QKV projection + RoPE(Q, K) + paged K/V append in one kernel (up to 4 rows).
    x [B, K] bf16; q_out [B, Hq, D]; the new K/V rows go straight to their page slots."""
    _lib.require_cuda_tensor(x, w.w, q_out, k_cache, v_cache, block_table, positions, cos, sin)
    b, k = x.shape
    d = k_cache.shape[3]
    assert w.n == (hq + 2 * hkv) * d and w.k == k and x.stride(1) == 1 and q_out.is_contiguous()
    assert positions.dtype == torch.int32 and block_table.dtype == torch.int32 and cos.dtype == torch.float32
    for b0 in range(0, b, _MAXB):          # the kernel takes up to four rows per launch
        bb = min(_MAXB, b - b0)
        xs, qs = x[b0:b0 + bb], q_out[b0:b0 + bb]
        # without an explicit map, row r of this launch is sequence b0 + r: shift the table instead
        bt = block_table if row_seq is not None else block_table[b0:]
        rs = None if row_seq is None else row_seq[b0:]
        fn = _lib.cuda().rmlx_sg_rms_qkv_rope if _stream("qkv", w) else None
        if fn is not None:
            rc = fn(w.kernel_kind, w.w.data_ptr(), _lib.ptr(w.scales), _lib.ptr(w.biases), xs.data_ptr(),
                    xs.stride(0), _lib.ptr(norm_w), eps, qs.data_ptr(), k_cache.data_ptr(),
                    v_cache.data_ptr(), bt.data_ptr(), positions[b0:].data_ptr(), _lib.ptr(rs),
                    cos.data_ptr(), sin.data_ptr(), bb, k, hq, hkv, d, block_table.stride(0),
                    k_cache.shape[2], int(traditional), int(pdl), _lib.stream_ptr())
            if rc != -2:
                _lib.check(rc, "sg_rms_qkv_rope")
                continue
        rc = _lib.cuda().rmlx_rms_qkv_rope(
            w.kernel_kind, w.w.data_ptr(), _lib.ptr(w.scales), _lib.ptr(w.biases), xs.data_ptr(), xs.stride(0),
            _lib.ptr(norm_w), eps, qs.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(),
            bt.data_ptr(), positions[b0:].data_ptr(), _lib.ptr(rs), cos.data_ptr(), sin.data_ptr(),
            bb, k, hq, hkv, d, block_table.stride(0), k_cache.shape[2], int(traditional), int(pdl),
            _lib.stream_ptr())
        _lib.check(rc, "rms_qkv_rope")
    return q_out


def rope(x: torch.Tensor, positions: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor,
         traditional: bool = False, inverse: bool = False) -> torch.Tensor:
    """x [T, H, D] bf16."""
    _lib.require_cuda_tensor(x, positions, cos, sin)
    t, h, d = x.shape
    out = torch.empty_like(x)
    rc = _lib.cuda().rmlx_rope(x.data_ptr(), out.data_ptr(), positions.data_ptr(), cos.data_ptr(),
                               sin.data_ptr(), t, h, d, int(traditional), int(inverse),
                               _lib.stream_ptr())
    _lib.check(rc, "rope")
    return out


def embedding(table: torch.Tensor, ids: torch.Tensor, out: Optional[torch.Tensor] = None,
              pdl: bool = False) -> torch.Tensor:
    _lib.require_cuda_tensor(table, ids)
    assert ids.dtype == torch.int32 and table.dtype == torch.bfloat16
    t = ids.numel()
    if out is None:
        out = torch.empty(t, table.shape[1], dtype=torch.bfloat16, device=table.device)
    rc = _lib.cuda().rmlx_embedding(table.data_ptr(), ids.data_ptr(), out.data_ptr(), t,
                                    table.shape[1], table.shape[0], int(pdl), _lib.stream_ptr())
    _lib.check(rc, "embedding")
    return out


def rms_norm(x: torch.Tensor, w: Optional[torch.Tensor], eps: float,
             residual: Optional[torch.Tensor] = None, sum_out: Optional[torch.Tensor] = None,
             out: Optional[torch.Tensor] = None, pdl: bool = False) -> torch.Tensor:
    """rmsnorm(x [+ residual]) * w over the last dim; bf16 [T, D]."""
    _lib.require_cuda_tensor(x)
    x2 = x.reshape(-1, x.shape[-1])
    assert x2.is_contiguous() and x2.dtype == torch.bfloat16
    if out is None:
        out = torch.empty_like(x2)
    if residual is not None and sum_out is None:
        sum_out = torch.empty_like(x2)
    rc = _lib.cuda().rmlx_rms_norm(x2.data_ptr(), _lib.ptr(residual), _lib.ptr(w), out.data_ptr(),
                                   _lib.ptr(sum_out), x2.shape[0], x2.shape[1], eps, int(pdl),
                                   _lib.stream_ptr())
    _lib.check(rc, "rms_norm")
    return out.view(x.shape)


class ArgmaxScratch:
    """Zeroed merge keys and tickets for the multi-block arg-max (left zero by every launch)."""

    def __init__(self, rows: int, device):
        self.keys = torch.zeros(rows, dtype=torch.int64, device=device)
        self.tickets = torch.zeros(rows, dtype=torch.int32, device=device)


def argmax(logits: torch.Tensor, out: Optional[torch.Tensor] = None,
           scratch: Optional[ArgmaxScratch] = None, pdl: bool = False) -> torch.Tensor:
    _lib.require_cuda_tensor(logits)
    assert logits.dtype == torch.float32 and logits.dim() == 2
    if out is None:
        out = torch.empty(logits.shape[0], dtype=torch.int32, device=logits.device)
    scratch = scratch or ArgmaxScratch(logits.shape[0], logits.device)
    rc = _lib.cuda().rmlx_argmax(logits.data_ptr(), out.data_ptr(), logits.shape[0], logits.shape[1],
                                 logits.stride(0), scratch.keys.data_ptr(),
                                 scratch.tickets.data_ptr(), int(pdl), _lib.stream_ptr())
    _lib.check(rc, "argmax")
    return out


def silu_mul(gate_up: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    _lib.require_cuda_tensor(gate_up)
    t, two_i = gate_up.shape
    assert gate_up.is_contiguous()
    if out is None:
        out = torch.empty(t, two_i // 2, dtype=torch.bfloat16, device=gate_up.device)
    rc = _lib.cuda().rmlx_silu_mul(gate_up.data_ptr(), out.data_ptr(), t, two_i // 2, _lib.stream_ptr())
    _lib.check(rc, "silu_mul")
    return out
