"""Memory-mapped .safetensors access through the native host library
(csrc/host/safetensors_io.cpp).

``SafetensorsFile`` lists a file's tensors without reading them and hands each one out as a tensor
that views the mapping (no copy), so ``.to(device)`` moves bytes from the page cache straight to the
GPU and a rank only ever touches the tensors it asks for; ``read_into`` fills a caller buffer
(typically pinned memory) with a multi-threaded copy. The reference's loader parses the same header
(crates/rmlx-nn/src/safetensors_loader.rs:7-19,122-162).
"""
from __future__ import annotations

import ctypes
from ctypes import POINTER, c_char_p, c_int, c_int64, c_uint64, c_void_p
from typing import Dict, Iterator, List, Tuple

import torch

from .. import _lib

_DTYPES = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8,
    "BOOL": torch.bool, "U16": torch.uint16, "U32": torch.uint32, "U64": torch.uint64,
    "F8_E4M3": torch.float8_e4m3fn, "F8_E5M2": torch.float8_e5m2,
}
_bound = False


def _host():
    global _bound
    lib = _lib.host()
    if not _bound:
        sig = {
            "rmlx_st_open": (c_void_p, [c_char_p, c_char_p, c_int]),
            "rmlx_st_close": (None, [c_void_p]),
            "rmlx_st_count": (c_int, [c_void_p]),
            "rmlx_st_find": (c_int, [c_void_p, c_char_p]),
            "rmlx_st_name": (c_char_p, [c_void_p, c_int]),
            "rmlx_st_dtype": (c_char_p, [c_void_p, c_int]),
            "rmlx_st_ndim": (c_int, [c_void_p, c_int]),
            "rmlx_st_shape": (None, [c_void_p, c_int, POINTER(c_int64)]),
            "rmlx_st_nbytes": (c_uint64, [c_void_p, c_int]),
            "rmlx_st_data": (c_void_p, [c_void_p, c_int]),
            "rmlx_st_read": (c_int, [c_void_p, c_int, c_void_p, c_uint64, c_uint64, c_int]),
        }
        for name, (res, args) in sig.items():
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = res, args
        _bound = True
    return lib


def available() -> bool:
    try:
        _host()
        return True
    except Exception:
        return False


class SafetensorsFile:
    """One mapped checkpoint file. Tensors returned by ``tensor`` view the mapping and keep this
    object alive; they must not be written to."""

    def __init__(self, path: str):
        self._lib = _host()
        err = ctypes.create_string_buffer(256)
        self._h = self._lib.rmlx_st_open(str(path).encode(), err, len(err))
        if not self._h:
            raise ValueError(f"{path}: {err.value.decode(errors='replace')}")
        self.path = str(path)
        self._names: List[str] = [self._lib.rmlx_st_name(self._h, i).decode()
                                  for i in range(self._lib.rmlx_st_count(self._h))]

    def close(self) -> None:
        h, self._h = getattr(self, "_h", None), None
        if h:
            self._lib.rmlx_st_close(h)

    def __del__(self):
        self.close()

    # ------------------------------------------------------------------ directory
    def keys(self) -> List[str]:
        return list(self._names)

    def __contains__(self, name: str) -> bool:
        return self._lib.rmlx_st_find(self._h, name.encode()) >= 0

    def _index(self, name: str) -> int:
        i = self._lib.rmlx_st_find(self._h, name.encode())
        if i < 0:
            raise KeyError(name)
        return i

    def info(self, name: str) -> Tuple[torch.dtype, Tuple[int, ...], int]:
        """(dtype, shape, size in bytes) without touching the data."""
        i = self._index(name)
        code = self._lib.rmlx_st_dtype(self._h, i).decode()
        if code not in _DTYPES:
            raise ValueError(f"{name}: unsupported safetensors dtype {code}")
        nd = self._lib.rmlx_st_ndim(self._h, i)
        shape = (c_int64 * max(1, nd))()
        self._lib.rmlx_st_shape(self._h, i, shape)
        return _DTYPES[code], tuple(int(s) for s in shape[:nd]), int(self._lib.rmlx_st_nbytes(self._h, i))

    # ------------------------------------------------------------------ data
    def tensor(self, name: str) -> torch.Tensor:
        """The tensor as a zero-copy view of the mapping (CPU)."""
        i = self._index(name)
        dtype, shape, nbytes = self.info(name)
        if nbytes == 0:
            return torch.empty(shape, dtype=dtype)
        buf = (ctypes.c_char * nbytes).from_address(self._lib.rmlx_st_data(self._h, i))
        # the tensor's storage keeps ``buf`` alive and ``buf`` keeps the mapping alive, so views
        # derived from the tensor are safe after the caller drops this object
        buf._rmlx_owner = self
        return torch.frombuffer(buf, dtype=dtype).view(shape)

    def read_into(self, name: str, dst: torch.Tensor, threads: int = 0) -> torch.Tensor:
        """Copy the tensor's bytes into ``dst`` (CPU, contiguous, same size in bytes; pinned memory
        makes the following host-to-device copy asynchronous)."""
        i = self._index(name)
        _, _, nbytes = self.info(name)
        if dst.device.type != "cpu" or not dst.is_contiguous() or dst.numel() * dst.element_size() != nbytes:
            raise ValueError("destination must be a contiguous CPU tensor of the same byte size")
        rc = self._lib.rmlx_st_read(self._h, i, dst.data_ptr(), 0, nbytes, threads)
        if rc != 0:
            raise ValueError(f"read of {name} failed ({rc})")
        return dst

    def items(self) -> Iterator[Tuple[str, torch.Tensor]]:
        for n in self._names:
            yield n, self.tensor(n)


def load_file(path: str) -> Dict[str, torch.Tensor]:
    """Every tensor of one file as views of its mapping (the shape of ``safetensors.torch.load_file``,
    without reading the file into memory)."""
    return dict(SafetensorsFile(path).items())
