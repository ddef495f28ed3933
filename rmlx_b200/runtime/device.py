"""Device probe and tuning table. ``DeviceTuning`` plays the role of the reference's ``ChipTuning``
(crates/rmlx-metal/src/device.rs:44-235: per-chip limits that feed kernel-selection heuristics);
here the chip is recognised from the CUDA device name / compute capability and the numbers are the
B200's: 148 SMs, 227 KB shared memory per block, 256 KB tensor memory per SM, 126 MB L2.
``self_check`` is the start-up diagnostic of crates/rmlx-metal/src/self_check.rs:7-61."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional

import torch


@dataclass(frozen=True)
class DeviceTuning:
    name: str
    sm_count: int
    smem_per_block: int
    tmem_columns: int            # 32-bit tensor-memory columns per SM (x 128 lanes)
    l2_bytes: int
    hbm_bytes: int
    supports_tcgen05: bool
    supports_tma: bool
    max_cluster: int
    gemv_max_batch: int          # activations per GEMV launch before the GEMM path takes over
    decode_graph_batch_buckets: tuple = (1, 2, 4, 8, 16, 32, 64)

    def kv_splits(self, batch: int, kv_heads: int, max_len: int) -> int:
        tiles = max(1, batch * kv_heads)
        return int(min(16, max(1, (self.sm_count + tiles - 1) // tiles), max(1, max_len // 128)))

    def gemm_tile_n(self, m: int, n: int) -> int:
        tm = (m + 127) // 128
        for bn in (256, 128, 64, 32):
            if tm * ((n + bn - 1) // bn) >= self.sm_count or bn == 32:
                return bn
        return 32


_B200 = DeviceTuning("NVIDIA B200", 148, 227 * 1024, 512, 126 << 20, 180 * 10 ** 9, True, True, 8, 8)
_GENERIC = DeviceTuning("generic", 108, 99 * 1024, 0, 40 << 20, 40 * 10 ** 9, False, False, 1, 4)


def tuning_from_name(name: str, capability: Optional[tuple] = None) -> DeviceTuning:
    """Pure function (testable without a GPU)."""
    n = name.upper()
    if "B200" in n or "B100" in n or "GB200" in n or (capability and capability[0] == 10):
        return DeviceTuning(name, _B200.sm_count, _B200.smem_per_block, 512, _B200.l2_bytes,
                            _B200.hbm_bytes, True, True, 8, 8)
    if "H100" in n or "H200" in n or (capability and capability[0] == 9):
        return DeviceTuning(name, 132, 227 * 1024, 0, 50 << 20, 80 * 10 ** 9, False, True, 8, 4)
    return DeviceTuning(name, _GENERIC.sm_count, _GENERIC.smem_per_block, 0, _GENERIC.l2_bytes,
                        _GENERIC.hbm_bytes, False, False, 1, 4)


def probe(device: int = 0) -> DeviceTuning:
    if not torch.cuda.is_available():
        return _GENERIC
    p = torch.cuda.get_device_properties(device)
    t = tuning_from_name(p.name, (p.major, p.minor))
    return DeviceTuning(p.name, p.multi_processor_count, t.smem_per_block, t.tmem_columns,
                        getattr(p, "L2_cache_size", t.l2_bytes), p.total_memory, t.supports_tcgen05,
                        t.supports_tma, t.max_cluster, t.gemv_max_batch)


def self_check(device: int = 0) -> Dict[str, object]:
    """Start-up diagnostics: device present, architecture, native library loadable, memory."""
    out: Dict[str, object] = {"cuda_available": torch.cuda.is_available()}
    if not out["cuda_available"]:
        out["ok"] = False
        out["reason"] = "no CUDA device"
        return out
    p = torch.cuda.get_device_properties(device)
    out.update(name=p.name, capability=f"{p.major}.{p.minor}", sm_count=p.multi_processor_count,
               total_memory=p.total_memory)
    try:
        from .. import _lib
        out["native_library"] = _lib.cuda().rmlx_gemv_max_batch() >= 1
    except Exception as e:  # pragma: no cover
        out["native_library"] = False
        out["reason"] = str(e)
    out["sm100"] = p.major == 10
    out["ok"] = bool(out["native_library"] and out["sm100"])
    return out
