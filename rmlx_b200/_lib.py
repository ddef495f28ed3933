"""ctypes bindings for the two native libraries.

``cuda()`` loads ``lib/librmlx_b200_cuda.so`` (every sm_100a kernel, exported as ``extern "C"``
launchers that take raw device pointers and a stream) and ``host()`` loads
``lib/librmlx_b200_host.so`` (allocator, block manager and other pure C++ runtime pieces). Missing
libraries are built on first use when a compiler is present; on a machine with a GPU a missing
CUDA library is an error, never a silent fallback.

This registry of exported launchers, looked up by name and bound once, is the analogue of the
reference's KernelRegistry (crates/rmlx-core/src/kernels/mod.rs:95-125) for ahead-of-time
compiled kernels.
"""
from __future__ import annotations

import ctypes
import os
import threading
from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import Any, Dict, Optional

import torch

from . import _build

_CODES = {"p": c_void_p, "i": c_int, "f": c_float, "q": c_longlong, "Q": ctypes.c_ulonglong, None: None}

# name -> (argument codes, restype code)
_CUDA_SIGS: Dict[str, tuple] = {
    "rmlx_error_string": ("i", "p"),
    "rmlx_gemv_max_batch": ("", "i"),
    "rmlx_rms_gemv": ("ippppipfpipiiiiiip", "i"),
    "rmlx_rms_gate_up_swiglu": ("ippppipfpiiiiip", "i"),
    "rmlx_swiglu_down": ("ippppipipiiiiip", "i"),
    "rmlx_moe_router": ("ppipfppppppiiiiip", "i"),
    "rmlx_topk_route": ("ppppppiiip", "i"),
    "rmlx_moe_gate_up": ("ippppipfppiiiiiiiip", "i"),
    "rmlx_moe_down": ("ippppipppipiiiiiiiiip", "i"),
    "rmlx_flash_decode_gtiles": ("ii", "i"),
    "rmlx_flash_decode_part_o_elems": ("iiiii", "q"),
    "rmlx_flash_decode_part_ml_elems": ("iiii", "q"),
    "rmlx_flash_decode_ticket_elems": ("iii", "q"),
    "rmlx_flash_decode_paged": ("pppppppppiiiiiiifip", "i"),
    "rmlx_rope_kv_write": ("pppppppppiiiiiiiip", "i"),
    "rmlx_rope": ("pppppiiiiip", "i"),
    "rmlx_embedding": ("pppiiiip", "i"),
    "rmlx_rms_norm": ("pppppiifip", "i"),
    "rmlx_argmax": ("ppiiippip", "i"),
    "rmlx_qmv_mma_max_batch": ("", "i"),
    "rmlx_qmv_status": ("", "i"),
    "rmlx_qmv_mma_supported": ("iii", "i"),
    "rmlx_moe_down_q4_mma_supported": ("ii", "i"),
    "rmlx_rms_qmv_mma": ("ppppipfpipiiiiiip", "i"),
    "rmlx_moe_gate_up_q4_mma": ("ppppipfppiiiiiiiip", "i"),
    "rmlx_moe_down_q4_mma": ("ppppipppipiiiiiiiiip", "i"),
    "rmlx_gemm_pick_bn": ("ii", "i"),
    "rmlx_gemm_bf16": ("ppppiiiiiiipip", "i"),
    "rmlx_silu_mul": ("ppqip", "i"),
    "rmlx_decode_advance": ("pppppiip", "i"),
    "rmlx_fp8_quant_rows": ("pppiip", "i"),
    "rmlx_fp8_dequant_rows": ("pppiip", "i"),
}

_lock = threading.Lock()
_cuda_lib: Optional[ctypes.CDLL] = None
_host_lib: Optional[ctypes.CDLL] = None


class NativeError(RuntimeError):
    pass


def _bind(lib: ctypes.CDLL, sigs: Dict[str, tuple]) -> None:
    for name, (args, ret) in sigs.items():
        try:
            fn = getattr(lib, name)
        except AttributeError:
            continue  # optional symbol (a source file may be excluded from some builds)
        fn.argtypes = [_CODES[c] for c in args]
        fn.restype = _CODES[ret] if ret != "p" else ctypes.c_char_p if name == "rmlx_error_string" else c_void_p


def register_cuda_sigs(sigs: Dict[str, tuple]) -> None:
    """Other modules add their launchers' signatures here before first use."""
    _CUDA_SIGS.update(sigs)
    if _cuda_lib is not None:
        _bind(_cuda_lib, sigs)


def cuda() -> ctypes.CDLL:
    global _cuda_lib
    if _cuda_lib is None:
        with _lock:
            if _cuda_lib is None:
                # RMLX_BOUNDS=1: the bounds-checked build of the same kernels
                bounds = os.environ.get("RMLX_BOUNDS", "0") == "1"
                path = _build.CUDA_BOUNDS_LIB if bounds else _build.CUDA_LIB
                if not path.exists():
                    _build.build(kinds=("cuda_bounds" if bounds else "cuda",))
                lib = ctypes.CDLL(str(path))
                lib.rmlx_bounds_build.restype = c_int
                if bool(lib.rmlx_bounds_build()) != bounds:
                    raise NativeError(f"{path.name} is {'not ' if bounds else ''}a bounds-checked build")
                _bind(lib, _CUDA_SIGS)
                _register_status_words(lib)
                _cuda_lib = lib
    return _cuda_lib


def _register_status_words(lib: ctypes.CDLL) -> None:
    """The kernels' status words (set by a bounded wait that ran out) become sources of the
    process-wide error store; ``ERRORS.collect()`` reads and clears them."""
    from .runtime.streams import ERRORS
    for title, sym in (("weight-streaming mat-vec", "rmlx_sg_status"),
                       ("tensor-core mat-vec", "rmlx_qmv_status"),
                       ("tensor-parallel decode", "rmlx_tp_status"),
                       ("decode step kernel", "rmlx_decode_step_status"),
                       ("latent-attention decode", "rmlx_mla_status")):
        fn = getattr(lib, sym, None)
        if fn is not None:
            fn.restype = c_int
            ERRORS.register(title, lambda fn=fn: int(fn()) & 0xff if torch.cuda.is_available() else 0)


def host() -> ctypes.CDLL:
    global _host_lib
    if _host_lib is None:
        with _lock:
            if _host_lib is None:
                if not _build.HOST_LIB.exists():
                    _build.build(kinds=("host",))
                _host_lib = ctypes.CDLL(str(_build.HOST_LIB))
    return _host_lib


def ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def stream_ptr(stream: Optional[torch.cuda.Stream] = None) -> int:
    return (stream or torch.cuda.current_stream()).cuda_stream


_launch_count = 0
# RMLX_DEBUG_SERIALIZE=1: every launch is followed by a device synchronisation and a read of the
# kernels' status words, so a fault or an expired wait is reported with the name of the launch that
# caused it (the stand-in for a race / memory checker on boxes where none can run). Launches made
# during stream capture are left alone; the engines run un-captured in this mode.
_debug_serialize = os.environ.get("RMLX_DEBUG_SERIALIZE", "0") == "1"
_serial_trace: list = []


def set_debug_serialize(on: bool) -> None:
    global _debug_serialize
    _debug_serialize = bool(on)


def debug_serialize() -> bool:
    return _debug_serialize


def serial_trace() -> list:
    """Names of the launches checked one by one since the last call (debug-serialize mode)."""
    out = list(_serial_trace)
    _serial_trace.clear()
    return out


def launch_count() -> int:
    """Number of kernel launches issued through ``check`` by this process."""
    return _launch_count


def check(rc: int, what: str) -> None:
    global _launch_count
    _launch_count += 1
    if rc == 0:
        if _debug_serialize and torch.cuda.is_available() and not torch.cuda.is_current_stream_capturing():
            _check_serialized(what)
        return
    if rc == -2:
        raise NativeError(f"{what}: invalid argument or unsupported shape")
    msg = cuda().rmlx_error_string(rc)
    raise NativeError(f"{what}: CUDA error {rc}: {msg.decode() if msg else '?'}")


def is_bounds_build() -> bool:
    """Whether the loaded kernels are the bounds-checked build (RMLX_BOUNDS=1)."""
    return bool(cuda().rmlx_bounds_build())


def bounds_status():
    """Bounds-checked build only: the first out-of-range index a kernel recorded since the last
    call, as (source file, source line, index, limit), or None. Raises on a normal build."""
    lib = cuda()
    lib.rmlx_bounds_status.argtypes = [c_void_p, ctypes.c_char_p, c_int]
    lib.rmlx_bounds_status.restype = c_int
    rec = (c_int * 4)()
    name = ctypes.create_string_buffer(64)
    rc = lib.rmlx_bounds_status(ctypes.cast(rec, c_void_p), name, 64)
    if rc == -3:
        raise NativeError("not a bounds-checked build (set RMLX_BOUNDS=1 before the first kernel)")
    if rc < 0:
        raise NativeError("bounds status could not be read")
    return (name.value.decode(), rec[1], rec[2], rec[3]) if rc == 1 else None


def _check_serialized(what: str) -> None:
    try:
        torch.cuda.synchronize()
    except RuntimeError as e:                      # a sticky CUDA error: name the launch
        raise NativeError(f"{what}: {e}") from e
    from .runtime.streams import ERRORS
    from .runtime.graph import HAZARDS
    HAZARDS.retire_all()                           # everything before this point has completed
    _serial_trace.append(what)
    new = ERRORS.collect()
    if new:
        raise NativeError(f"{what}: device status " + ", ".join(f"{n}={c} ({m})" for n, c, m in new))


def require_cuda_tensor(*ts: Any) -> None:
    for t in ts:
        if t is not None and not (isinstance(t, torch.Tensor) and t.is_cuda):
            raise NativeError("native kernels need CUDA tensors; use rmlx_b200.reference on CPU")
