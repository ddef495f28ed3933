"""Binding of the persistent decode-step kernel (csrc/kernels/decode_step.cu): one cooperative
launch runs every layer of a batch-1 decode step of a mixture-of-experts decoder, with grid-wide
barriers where the separate-kernel engine has kernel boundaries.

``DecodeStepKernel.supported(model, comm)`` says whether a model fits (all layers routed-expert
layers, one sequence, single GPU, head_dim 64 or 128); ``CachedDecode`` falls back to its chain of
kernels otherwise. The reference's counterpart is the 7-dispatch layer replayed from one command
buffer (crates/rmlx-nn/src/transformer.rs:2306-2555).
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_void_p

import torch

from .. import _lib

_lib.register_cuda_sigs({
    "rmlx_decode_step_layer_bytes": ("", "i"),
    "rmlx_decode_step_desc_bytes": ("", "i"),
    "rmlx_decode_step_layer_desc_bytes": ("", "i"),
    "rmlx_decode_step_fd_part_o_elems": ("iiii", "q"),
    "rmlx_decode_step_fd_part_ml_elems": ("iii", "q"),
    "rmlx_decode_step_grid": ("", "i"),
    "rmlx_decode_step_status": ("", "i"),
    "rmlx_decode_step_prepare": ("pp", "i"),
    "rmlx_decode_step_launch": ("ppp", "i"),
})


class _LayerDesc(ctypes.Structure):
    _fields_ = [(n, c_void_p) for n in (
        "wqkv", "wqkv_s", "wqkv_b", "wo", "wo_s", "wo_b", "wgu", "wgu_s", "wgu_b",
        "wdn", "wdn_s", "wdn_b", "norm1", "norm2", "router", "expert_bias", "k_cache", "v_cache")] + [
        ("expert_base", c_int), ("experts_local", c_int)]


class _StepDesc(ctypes.Structure):
    _fields_ = [(n, c_int) for n in ("num_layers", "D", "Hq", "Hkv", "HD", "I", "E", "top_k", "V", "q4")] + [
        ("eps", c_float), ("scale", c_float),
        ("max_blocks", c_int), ("window", c_int), ("traditional", c_int)] + [(n, c_void_p) for n in (
            "tokens", "positions", "seq_lens", "block_table", "cos_t", "sin_t", "embed", "final_norm",
            "lm", "lm_s", "lm_b", "h", "h2", "q", "attn", "act", "router_logits", "topk_idx", "topk_w",
            "fd_part_o", "fd_part_ml", "logits", "grid_bar", "trace", "layers_dev")]


def enabled() -> bool:
    """The persistent step kernel is opt-in (``RMLX_DECODE_STEP_KERNEL=1`` or
    ``CachedDecode(step_kernel=True)``): measured on B200 at the 60-layer model it takes 130 us per
    layer against 81 us for the chain of kernels, because its short phases start cold (see the
    phase trace, ``RMLX_STEP_TRACE=1``)."""
    return os.environ.get("RMLX_DECODE_STEP_KERNEL", "0") == "1"


class DecodeStepKernel:
    """Owns the device-side layer table and the scratch of the persistent step kernel and launches
    it on the current stream. Buffers (h, h2, q, attn, act, logits, tokens ...) are the engine's."""

    @staticmethod
    def supported(model, max_batch: int, comm, force: bool = False) -> bool:
        cfg = model.cfg
        if not (force or enabled()) or max_batch != 1 or comm is not None or model.layout.world != 1:
            return False
        if cfg.ff_type.moe is None or cfg.head_dim not in (64, 128):
            return False
        if cfg.ff_type.moe.num_shared_experts:
            return False
        kinds = set()
        for l in model.w.layers:
            if l.router is None or l.experts_gate_up is None or l.shared_gate_up is not None:
                return False
            kinds.update((l.wqkv.kind, l.wo.kind, l.experts_gate_up.kind, l.experts_down.kind))
        kinds.add(model.w.lm_head.kind)
        return len(kinds) == 1

    def __init__(self, eng):
        lib = _lib.cuda()
        assert lib.rmlx_decode_step_desc_bytes() == ctypes.sizeof(_StepDesc)
        assert lib.rmlx_decode_step_layer_desc_bytes() == ctypes.sizeof(_LayerDesc)
        m, cfg, w = eng.model, eng.cfg, eng.model.w
        dev = m.device
        moe = cfg.ff_type.moe
        self.grid = int(lib.rmlx_decode_step_grid())
        hq, hkv, hd = m.hq, m.hkv, cfg.head_dim
        f32 = dict(dtype=torch.float32, device=dev)
        self.fd_part_o = torch.empty(lib.rmlx_decode_step_fd_part_o_elems(self.grid, hq, hkv, hd), **f32)
        self.fd_part_ml = torch.empty(lib.rmlx_decode_step_fd_part_ml_elems(self.grid, hq, hkv), **f32)
        self.router_logits = torch.zeros(moe.num_experts, **f32)
        self.grid_bar = torch.zeros(1, dtype=torch.int32, device=dev)
        nl = len(w.layers)
        self.layers_dev = torch.zeros(nl * lib.rmlx_decode_step_layer_bytes(), dtype=torch.uint8, device=dev)
        self._layer_descs = (_LayerDesc * nl)()
        p = _lib.ptr
        for i, lw in enumerate(w.layers):
            d = self._layer_descs[i]
            d.wqkv, d.wqkv_s, d.wqkv_b = lw.wqkv.w.data_ptr(), p(lw.wqkv.scales), p(lw.wqkv.biases)
            d.wo, d.wo_s, d.wo_b = lw.wo.w.data_ptr(), p(lw.wo.scales), p(lw.wo.biases)
            gu, dn = lw.experts_gate_up, lw.experts_down
            d.wgu, d.wgu_s, d.wgu_b = gu.w.data_ptr(), p(gu.scales), p(gu.biases)
            d.wdn, d.wdn_s, d.wdn_b = dn.w.data_ptr(), p(dn.scales), p(dn.biases)
            d.norm1, d.norm2, d.router = lw.norm1.data_ptr(), lw.norm2.data_ptr(), lw.router.data_ptr()
            d.expert_bias = p(lw.expert_bias)
            d.k_cache, d.v_cache = eng.cache.k[i].data_ptr(), eng.cache.v[i].data_ptr()
            d.expert_base, d.experts_local = lw.expert_base, gu.experts
        s = self._desc = _StepDesc()
        s.num_layers, s.D, s.Hq, s.Hkv, s.HD = nl, cfg.hidden_size, hq, hkv, hd
        s.I, s.E, s.top_k = w.layers[0].experts_gate_up.n // 2, moe.num_experts, moe.num_experts_per_token
        s.V, s.q4 = w.lm_head.n, int(w.lm_head.kind)      # weight kind: 0 bf16, 1 Q4, 2 Q8
        s.eps, s.scale = cfg.rms_norm_eps, m.scale
        s.max_blocks, s.window = eng.block_table.stride(0), int(cfg.sliding_window or 0)
        s.traditional = int(cfg.rope_traditional)
        s.tokens, s.positions, s.seq_lens = eng.tokens.data_ptr(), eng.positions.data_ptr(), eng.seq_lens.data_ptr()
        s.block_table, s.cos_t, s.sin_t = eng.block_table.data_ptr(), m.cos.data_ptr(), m.sin.data_ptr()
        s.embed, s.final_norm = w.embed.data_ptr(), w.final_norm.data_ptr()
        s.lm, s.lm_s, s.lm_b = w.lm_head.w.data_ptr(), p(w.lm_head.scales), p(w.lm_head.biases)
        s.h, s.h2, s.q, s.attn, s.act = (eng.h.data_ptr(), eng.h2.data_ptr(), eng.q.data_ptr(),
                                          eng.attn.data_ptr(), eng.act.data_ptr())
        s.router_logits, s.topk_idx, s.topk_w = self.router_logits.data_ptr(), eng.idx.data_ptr(), eng.wts.data_ptr()
        s.fd_part_o, s.fd_part_ml, s.logits = self.fd_part_o.data_ptr(), self.fd_part_ml.data_ptr(), eng.logits.data_ptr()
        s.grid_bar, s.layers_dev = self.grid_bar.data_ptr(), self.layers_dev.data_ptr()
        self.trace = None
        if os.environ.get("RMLX_STEP_TRACE"):
            # block 0 stamps the global timer at every phase end: [layers, 32] nanoseconds
            self.trace = torch.zeros(nl, 32, dtype=torch.int64, device=dev)
            s.trace = self.trace.data_ptr()
        with torch.cuda.device(dev):
            rc = lib.rmlx_decode_step_prepare(ctypes.byref(s), self._layer_descs)
        self.ok = rc == 0
        if rc not in (0, -2):
            _lib.check(rc, "decode_step_prepare")

    def launch(self) -> None:
        self.grid_bar.zero_()
        rc = _lib.cuda().rmlx_decode_step_launch(ctypes.byref(self._desc), self._layer_descs,
                                                 _lib.stream_ptr())
        _lib.check(rc, "decode_step_launch")

    @staticmethod
    def status() -> int:
        return int(_lib.cuda().rmlx_decode_step_status())
