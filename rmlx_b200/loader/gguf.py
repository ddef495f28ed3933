"""GGUF v2/v3 reader (and a minimal writer for tests): header, typed metadata, tensor directory,
and dequantisation of the GGML block formats F32, F16, BF16, Q4_0, Q4_1, Q8_0, Q4_K and Q6_K to
fp32.

Covers the reference's ``formats::gguf`` parser and loader (crates/rmlx-core/src/formats/gguf.rs:23-819,
crates/rmlx-nn/src/gguf_loader.rs:112-450) and its K-quant dequantisers
(crates/rmlx-nn/src/quantized_linear.rs:738-1149). ``gguf_name_to_hf`` maps llama.cpp tensor names to
the HF names the weight builder consumes.
"""
from __future__ import annotations

import struct
from dataclasses import dataclass
from typing import Any, BinaryIO, Dict, Tuple

import numpy as np

MAGIC = 0x46554747  # "GGUF"

# ggml type id -> (name, block elements, block bytes)
GGML_TYPES = {
    0: ("F32", 1, 4), 1: ("F16", 1, 2), 2: ("Q4_0", 32, 18), 3: ("Q4_1", 32, 20), 6: ("Q5_0", 32, 22),
    7: ("Q5_1", 32, 24), 8: ("Q8_0", 32, 34), 10: ("Q2_K", 256, 84), 11: ("Q3_K", 256, 110),
    12: ("Q4_K", 256, 144), 13: ("Q5_K", 256, 176), 14: ("Q6_K", 256, 210), 30: ("BF16", 1, 2),
}
_T = {v[0]: k for k, v in GGML_TYPES.items()}

_SCALARS = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 7: "<?", 10: "<Q",
            11: "<q", 12: "<d"}


@dataclass
class GgufTensorInfo:
    name: str
    shape: Tuple[int, ...]      # outermost first (GGUF stores innermost first; reversed here)
    ggml_type: int
    offset: int                 # from the start of the data section

    @property
    def type_name(self) -> str:
        return GGML_TYPES[self.ggml_type][0]

    def nbytes(self) -> int:
        _, be, bb = GGML_TYPES[self.ggml_type]
        n = int(np.prod(self.shape)) if self.shape else 1
        return n // be * bb


@dataclass
class GgufFile:
    version: int
    metadata: Dict[str, Any]
    tensors: Dict[str, GgufTensorInfo]
    data_offset: int
    path: str

    def raw(self, name: str) -> np.ndarray:
        t = self.tensors[name]
        return np.fromfile(self.path, dtype=np.uint8, count=t.nbytes(), offset=self.data_offset + t.offset)

    def tensor_f32(self, name: str) -> np.ndarray:
        t = self.tensors[name]
        return dequantize(self.raw(name), t.ggml_type).reshape(t.shape)


def _read_str(f: BinaryIO) -> str:
    (n,) = struct.unpack("<Q", f.read(8))
    return f.read(n).decode("utf-8")


def _read_value(f: BinaryIO, vt: int):
    if vt in _SCALARS:
        fmt = _SCALARS[vt]
        return struct.unpack(fmt, f.read(struct.calcsize(fmt)))[0]
    if vt == 8:
        return _read_str(f)
    if vt == 9:
        (et,) = struct.unpack("<I", f.read(4))
        (n,) = struct.unpack("<Q", f.read(8))
        return [_read_value(f, et) for _ in range(n)]
    raise ValueError(f"unknown GGUF metadata type {vt}")


def read_gguf(path: str) -> GgufFile:
    with open(path, "rb") as f:
        magic, version = struct.unpack("<II", f.read(8))
        if magic != MAGIC:
            raise ValueError("not a GGUF file")
        if version not in (2, 3):
            raise ValueError(f"unsupported GGUF version {version}")
        n_tensors, n_kv = struct.unpack("<QQ", f.read(16))
        meta: Dict[str, Any] = {}
        for _ in range(n_kv):
            k = _read_str(f)
            (vt,) = struct.unpack("<I", f.read(4))
            meta[k] = _read_value(f, vt)
        infos: Dict[str, GgufTensorInfo] = {}
        for _ in range(n_tensors):
            name = _read_str(f)
            (nd,) = struct.unpack("<I", f.read(4))
            dims = struct.unpack(f"<{nd}Q", f.read(8 * nd))
            gt, off = struct.unpack("<IQ", f.read(12))
            if gt not in GGML_TYPES:
                raise ValueError(f"tensor {name}: unsupported ggml type {gt}")
            infos[name] = GgufTensorInfo(name, tuple(reversed(dims)), gt, off)
        align = int(meta.get("general.alignment", 32))
        pos = f.tell()
        data_offset = (pos + align - 1) // align * align
    return GgufFile(version, meta, infos, data_offset, path)


# ------------------------------------------------------------------------------------------------
# Dequantisation (vectorised numpy)
# ------------------------------------------------------------------------------------------------
def _f16(b: np.ndarray) -> np.ndarray:
    return b.copy().view(np.float16).astype(np.float32)


def _native_lib():
    """The host library with the block dequantisers bound, or None (``RMLX_NATIVE_LOADER=0``, or the
    library cannot be built or loaded)."""
    import ctypes
    import os
    if os.environ.get("RMLX_NATIVE_LOADER", "1") == "0":
        return None
    try:
        from .. import _lib
        lib = _lib.host()
        fn = lib.rmlx_ggml_dequant
        fn.restype = ctypes.c_int
        fn.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_uint64, ctypes.c_void_p, ctypes.c_int]
        return lib
    except Exception:
        return None


def dequantize(raw: np.ndarray, ggml_type: int) -> np.ndarray:
    """Blocks of a GGML type to fp32: through the native multi-threaded dequantisers
    (csrc/host/ggml_dequant.cpp) when available, else ``dequantize_numpy`` (same results)."""
    lib = _native_lib()
    if lib is None:
        return dequantize_numpy(raw, ggml_type)
    _, be, bb = GGML_TYPES[ggml_type]
    raw = np.ascontiguousarray(raw, dtype=np.uint8)
    if raw.size % bb:
        raise ValueError(f"{raw.size} bytes is not a whole number of {bb}-byte blocks")
    nblocks = raw.size // bb
    out = np.empty(nblocks * be, np.float32)
    if lib.rmlx_ggml_dequant(ggml_type, raw.ctypes.data, nblocks, out.ctypes.data, 0) != 0:
        raise ValueError(f"no dequantiser for {GGML_TYPES[ggml_type][0]}")
    return out


def dequantize_numpy(raw: np.ndarray, ggml_type: int) -> np.ndarray:
    name, be, bb = GGML_TYPES[ggml_type]
    if name == "F32":
        return raw.view(np.float32).copy()
    if name == "F16":
        return raw.view(np.float16).astype(np.float32)
    if name == "BF16":
        return (raw.view(np.uint16).astype(np.uint32) << 16).view(np.float32)
    blk = raw.reshape(-1, bb)
    if name == "Q4_0":
        d = _f16(blk[:, :2])
        qs = blk[:, 2:]
        lo, hi = (qs & 0xF).astype(np.int8) - 8, (qs >> 4).astype(np.int8) - 8
        return (np.concatenate([lo, hi], 1).astype(np.float32) * d).reshape(-1)
    if name == "Q4_1":
        d, m = _f16(blk[:, :2]), _f16(blk[:, 2:4])
        qs = blk[:, 4:]
        q = np.concatenate([qs & 0xF, qs >> 4], 1).astype(np.float32)
        return (q * d + m).reshape(-1)
    if name == "Q8_0":
        d = _f16(blk[:, :2])
        return (blk[:, 2:].view(np.int8).astype(np.float32) * d).reshape(-1)
    if name in ("Q5_0", "Q5_1"):
        off = 2 if name == "Q5_0" else 4
        d = _f16(blk[:, :2])
        qh = blk[:, off:off + 4].copy().view(np.uint32)                     # [n, 1]: bit j = 5th bit of value j
        qs = blk[:, off + 4:]
        bits = ((qh >> np.arange(32, dtype=np.uint32)) & 1).astype(np.uint8)  # [n, 32]
        q = np.concatenate([qs & 0xF, qs >> 4], 1) | (bits << 4)
        if name == "Q5_0":
            return ((q.astype(np.int8) - 16).astype(np.float32) * d).reshape(-1)
        return (q.astype(np.float32) * d + _f16(blk[:, 2:4])).reshape(-1)
    if name == "Q2_K":
        sc, qs = blk[:, :16], blk[:, 16:80]
        d, dmin = _f16(blk[:, 80:82]), _f16(blk[:, 82:84])
        out = np.zeros((blk.shape[0], 256), np.float32)
        for n in range(2):                       # 128 values per half, 32 bytes of quants each
            q = qs[:, 32 * n:32 * n + 32]
            for j in range(4):                   # bit pair j of every byte
                v = (q >> (2 * j)) & 3
                for h in range(2):               # 16 values per 4-bit scale / 4-bit minimum
                    s_ = sc[:, 8 * n + 2 * j + h]
                    dl, ml = d[:, 0] * (s_ & 0xF), dmin[:, 0] * (s_ >> 4)
                    base = 128 * n + 32 * j + 16 * h
                    out[:, base:base + 16] = dl[:, None] * v[:, 16 * h:16 * h + 16] - ml[:, None]
        return out.reshape(-1)
    if name == "Q3_K":
        hm, qs, sraw = blk[:, :32], blk[:, 32:96], blk[:, 96:108]
        d = _f16(blk[:, 108:110])
        # sixteen 6-bit scales: low 4 bits in bytes 0..7 (two per byte), high 2 bits in bytes 8..11
        lo = np.concatenate([sraw[:, :8] & 0xF, sraw[:, :8] >> 4], 1)                     # [n, 16]
        hi = np.concatenate([(sraw[:, 8:12] >> (2 * k)) & 3 for k in range(4)], 1)        # [n, 16]
        scales = (lo | (hi << 4)).astype(np.int8).astype(np.float32) - 32
        out = np.zeros((blk.shape[0], 256), np.float32)
        for n in range(2):
            q = qs[:, 32 * n:32 * n + 32]
            for j in range(4):
                v = ((q >> (2 * j)) & 3).astype(np.int8)
                m = ((hm >> (4 * n + j)) & 1).astype(np.int8)                              # high bit set: no -4
                v = v - 4 * (1 - m)
                for h in range(2):
                    dl = d[:, 0] * scales[:, 8 * n + 2 * j + h]
                    base = 128 * n + 32 * j + 16 * h
                    out[:, base:base + 16] = dl[:, None] * v[:, 16 * h:16 * h + 16]
        return out.reshape(-1)
    if name == "Q5_K":
        d, dmin = _f16(blk[:, 0:2]), _f16(blk[:, 2:4])
        sc_raw, qh, qs = blk[:, 4:16], blk[:, 16:48], blk[:, 48:176]
        sc = np.zeros((blk.shape[0], 8), np.float32)
        mn = np.zeros((blk.shape[0], 8), np.float32)
        for j in range(8):
            if j < 4:
                sc[:, j] = sc_raw[:, j] & 63
                mn[:, j] = sc_raw[:, j + 4] & 63
            else:
                sc[:, j] = (sc_raw[:, j + 4] & 0xF) | ((sc_raw[:, j - 4] >> 6) << 4)
                mn[:, j] = (sc_raw[:, j + 4] >> 4) | ((sc_raw[:, j] >> 6) << 4)
        out = np.zeros((blk.shape[0], 256), np.float32)
        for j in range(4):
            q = qs[:, 32 * j:32 * j + 32]
            lo = (q & 0xF) + (((qh >> (2 * j)) & 1) << 4)
            hi = (q >> 4) + (((qh >> (2 * j + 1)) & 1) << 4)
            out[:, 64 * j:64 * j + 32] = d * sc[:, [2 * j]] * lo - dmin * mn[:, [2 * j]]
            out[:, 64 * j + 32:64 * j + 64] = d * sc[:, [2 * j + 1]] * hi - dmin * mn[:, [2 * j + 1]]
        return out.reshape(-1)
    if name == "Q4_K":
        d, dmin = _f16(blk[:, 0:2]), _f16(blk[:, 2:4])
        sc_raw = blk[:, 4:16].astype(np.uint8)
        qs = blk[:, 16:144]
        sc = np.zeros((blk.shape[0], 8), np.float32)
        mn = np.zeros((blk.shape[0], 8), np.float32)
        for j in range(8):
            if j < 4:
                sc[:, j] = sc_raw[:, j] & 63
                mn[:, j] = sc_raw[:, j + 4] & 63
            else:
                sc[:, j] = (sc_raw[:, j + 4] & 0xF) | ((sc_raw[:, j - 4] >> 6) << 4)
                mn[:, j] = (sc_raw[:, j + 4] >> 4) | ((sc_raw[:, j] >> 6) << 4)
        out = np.zeros((blk.shape[0], 256), np.float32)
        for j in range(4):
            q = qs[:, 32 * j:32 * j + 32]
            out[:, 64 * j:64 * j + 32] = d * sc[:, [2 * j]] * (q & 0xF) - dmin * mn[:, [2 * j]]
            out[:, 64 * j + 32:64 * j + 64] = d * sc[:, [2 * j + 1]] * (q >> 4) - dmin * mn[:, [2 * j + 1]]
        return out.reshape(-1)
    if name == "Q6_K":
        ql, qh = blk[:, :128], blk[:, 128:192]
        sc = blk[:, 192:208].view(np.int8).astype(np.float32)
        d = _f16(blk[:, 208:210])
        out = np.zeros((blk.shape[0], 256), np.float32)
        for half in range(2):
            l_ = ql[:, 64 * half:64 * half + 64]
            h_ = qh[:, 32 * half:32 * half + 32]
            s_ = sc[:, 8 * half:8 * half + 8]
            a, b = l_[:, :32], l_[:, 32:]
            q1 = ((a & 0xF) | (((h_ >> 0) & 3) << 4)).astype(np.int16) - 32
            q2 = ((b & 0xF) | (((h_ >> 2) & 3) << 4)).astype(np.int16) - 32
            q3 = ((a >> 4) | (((h_ >> 4) & 3) << 4)).astype(np.int16) - 32
            q4 = ((b >> 4) | (((h_ >> 6) & 3) << 4)).astype(np.int16) - 32
            idx = np.arange(32) // 16
            base = 128 * half
            out[:, base:base + 32] = d * s_[:, idx] * q1
            out[:, base + 32:base + 64] = d * s_[:, idx + 2] * q2
            out[:, base + 64:base + 96] = d * s_[:, idx + 4] * q3
            out[:, base + 96:base + 128] = d * s_[:, idx + 6] * q4
        return out.reshape(-1)
    raise ValueError(f"no dequantiser for {name}")


def quantize_q8_0(x: np.ndarray) -> np.ndarray:
    """fp32 -> Q8_0 blocks (for tests and for writing small files)."""
    b = x.reshape(-1, 32).astype(np.float32)
    d = np.abs(b).max(1, keepdims=True) / 127.0
    q = np.where(d > 0, np.round(b / np.where(d > 0, d, 1)), 0).astype(np.int8)
    out = np.zeros((b.shape[0], 34), np.uint8)
    out[:, :2] = d.astype(np.float16).view(np.uint8).reshape(-1, 2)
    out[:, 2:] = q.view(np.uint8)
    return out.reshape(-1)


def quantize_q4_0(x: np.ndarray) -> np.ndarray:
    b = x.reshape(-1, 32).astype(np.float32)
    amax_idx = np.abs(b).argmax(1)
    mx = b[np.arange(b.shape[0]), amax_idx]
    d = mx / -8.0
    inv = np.where(d != 0, 1.0 / np.where(d != 0, d, 1), 0)
    q = np.clip(np.round(b * inv[:, None]) + 8, 0, 15).astype(np.uint8)
    out = np.zeros((b.shape[0], 18), np.uint8)
    out[:, :2] = d.astype(np.float16).view(np.uint8).reshape(-1, 2)
    out[:, 2:] = q[:, :16] | (q[:, 16:] << 4)
    return out.reshape(-1)


# ------------------------------------------------------------------------------------------------
# Writer (enough for round-trip tests and tiny random-init files)
# ------------------------------------------------------------------------------------------------
def _w_str(f, s: str):
    b = s.encode("utf-8")
    f.write(struct.pack("<Q", len(b)))
    f.write(b)


def write_gguf(path: str, metadata: Dict[str, Any], tensors: Dict[str, Tuple[np.ndarray, str]],
               version: int = 3, alignment: int = 32) -> None:
    """tensors: name -> (fp32 array, ggml type name in {F32, F16, Q8_0, Q4_0})."""
    blobs, infos, off = [], [], 0
    for name, (arr, tname) in tensors.items():
        if tname == "F32":
            raw = arr.astype(np.float32).tobytes()
        elif tname == "F16":
            raw = arr.astype(np.float16).tobytes()
        elif tname == "Q8_0":
            raw = quantize_q8_0(arr).tobytes()
        elif tname == "Q4_0":
            raw = quantize_q4_0(arr).tobytes()
        else:
            raise ValueError(tname)
        infos.append((name, arr.shape, _T[tname], off))
        pad = (-len(raw)) % alignment
        blobs.append(raw + b"\0" * pad)
        off += len(raw) + pad
    with open(path, "wb") as f:
        f.write(struct.pack("<IIQQ", MAGIC, version, len(infos), len(metadata) + 1))
        _w_str(f, "general.alignment"); f.write(struct.pack("<II", 4, alignment))
        for k, v in metadata.items():
            _w_str(f, k)
            if isinstance(v, str):
                f.write(struct.pack("<I", 8)); _w_str(f, v)
            elif isinstance(v, bool):
                f.write(struct.pack("<I?", 7, v))
            elif isinstance(v, int):
                f.write(struct.pack("<Iq", 11, v))
            elif isinstance(v, float):
                f.write(struct.pack("<If", 6, v))
            else:
                raise ValueError(f"metadata {k}: unsupported value")
        for name, shape, gt, o in infos:
            _w_str(f, name)
            f.write(struct.pack("<I", len(shape)))
            f.write(struct.pack(f"<{len(shape)}Q", *reversed(shape)))
            f.write(struct.pack("<IQ", gt, o))
        pos = f.tell()
        f.write(b"\0" * ((-pos) % alignment))
        for b in blobs:
            f.write(b)


_GGUF_MAP = (("token_embd.", "model.embed_tokens."), ("output_norm.", "model.norm."),
             ("output.", "lm_head."), ("blk.", "model.layers."), (".attn_norm.", ".input_layernorm."),
             (".ffn_norm.", ".post_attention_layernorm."), (".attn_q.", ".self_attn.q_proj."),
             (".attn_k.", ".self_attn.k_proj."), (".attn_v.", ".self_attn.v_proj."),
             (".attn_output.", ".self_attn.o_proj."), (".ffn_gate_inp.", ".mlp.gate."),
             (".ffn_gate.", ".mlp.gate_proj."), (".ffn_up.", ".mlp.up_proj."),
             (".ffn_down.", ".mlp.down_proj."))


def gguf_name_to_hf(name: str) -> str:
    for a, b in _GGUF_MAP:
        name = name.replace(a, b)
    return name


def load_state_dict(path: str, name_filter=None):
    """fp32 torch state dict with HF names from a GGUF file (dequantised on the host)."""
    import torch
    g = read_gguf(path)
    out = {}
    for name in g.tensors:
        hf = gguf_name_to_hf(name)
        if name_filter is not None and not name_filter(hf):
            continue
        out[hf] = torch.from_numpy(g.tensor_f32(name).copy())
    return out, g.metadata
