"""Host-side wire formats for MoE token exchange over byte transports.

v3 (variable length), crates/rmlx-distributed/src/v3_protocol.rs:1-125:
    [count: u32] ( [meta: u32 = local_expert << 16 | position] [token bytes] ) * count
v2 (fixed), crates/rmlx-distributed/src/moe_exchange.rs: ``count * (4 + token_stride)`` with an
expert-id prefix per token. FP8 payload, crates/rmlx-distributed/src/fp8_exchange.rs:85-330: per
token ``[E4M3 bytes][fp32 scale]`` with ``scale = max|x| / 448``. CRC32 framing for unreliable
transports: crates/rmlx-rdma/src/crc.rs:21-85.

On NVLink the device-side dispatch writes plain rows into peer slabs and needs none of this; the
formats are kept for the NCCL/gloo byte-transport path and for parity with stored traces.
"""
from __future__ import annotations

import struct
from typing import List, Tuple

import numpy as np
import torch


class ProtocolError(ValueError):
    pass


def pack_v3(local_experts: List[int], positions: List[int], tokens: np.ndarray) -> bytes:
    """tokens: uint8 [count, token_stride]."""
    count = len(local_experts)
    if tokens.shape[0] != count or len(positions) != count:
        raise ProtocolError("length mismatch")
    out = bytearray(struct.pack("<I", count))
    for e, p, row in zip(local_experts, positions, tokens):
        if not (0 <= e < 65536 and 0 <= p < 65536):
            raise ProtocolError("expert or position does not fit 16 bits")
        out += struct.pack("<I", (e << 16) | p)
        out += row.tobytes()
    return bytes(out)


def unpack_v3(buf: bytes, token_stride: int) -> Tuple[List[int], List[int], np.ndarray]:
    if len(buf) < 4:
        raise ProtocolError("truncated: no count header")
    (count,) = struct.unpack_from("<I", buf, 0)
    need = 4 + count * (4 + token_stride)
    if len(buf) < need:
        raise ProtocolError(f"truncated: need {need} bytes, have {len(buf)}")
    experts, positions = [], []
    rows = np.empty((count, token_stride), np.uint8)
    off = 4
    for i in range(count):
        (meta,) = struct.unpack_from("<I", buf, off)
        experts.append(meta >> 16)
        positions.append(meta & 0xFFFF)
        rows[i] = np.frombuffer(buf, np.uint8, token_stride, off + 4)
        off += 4 + token_stride
    return experts, positions, rows


def v3_payload_bytes(count: int, token_stride: int) -> int:
    return 4 + count * (4 + token_stride)


def v2_payload_bytes(capacity: int, token_stride: int) -> int:
    return capacity * (4 + token_stride)


def fp8_pack_tokens(x: torch.Tensor) -> bytes:
    """bf16/fp32 [n, d] -> per token [d E4M3 bytes][fp32 scale]."""
    xf = x.float()
    amax = xf.abs().amax(-1, keepdim=True)
    scale = torch.where(amax > 0, amax / 448.0, torch.ones_like(amax))
    q = (xf / scale).to(torch.float8_e4m3fn).view(torch.uint8).cpu().numpy()
    s = scale.squeeze(-1).cpu().numpy().astype("<f4")
    out = bytearray()
    for i in range(q.shape[0]):
        out += q[i].tobytes() + s[i].tobytes()
    return bytes(out)


def fp8_unpack_tokens(buf: bytes, n: int, d: int) -> torch.Tensor:
    if len(buf) < n * (d + 4):
        raise ProtocolError("truncated FP8 payload")
    raw = np.frombuffer(buf, np.uint8, n * (d + 4)).reshape(n, d + 4)
    q = torch.from_numpy(raw[:, :d].copy()).view(torch.float8_e4m3fn).float()
    s = torch.from_numpy(raw[:, d:].copy().view("<f4").reshape(n, 1).astype(np.float32))
    return q * s


def crc_frame(payload: bytes) -> bytes:
    from ..runtime.alloc import crc32
    return payload + struct.pack("<I", crc32(payload))


def crc_verify(frame: bytes) -> bytes:
    from ..runtime.alloc import crc32
    if len(frame) < 4:
        raise ProtocolError("frame shorter than its checksum")
    payload, (want,) = frame[:-4], struct.unpack("<I", frame[-4:])
    if crc32(payload) != want:
        raise ProtocolError("CRC mismatch")
    return payload


# ------------------------------------------------------------------------------------------------
# Exchange tags: one 64-bit id per in-flight message, so that completions, traces and slot
# bookkeeping can be matched without a side table. Layout as in the reference's work-request ids
# (crates/rmlx-rdma/src/exchange_tag.rs): sequence (40 bits) . tag (8) . buffer slot (8) . peer (8).
# ------------------------------------------------------------------------------------------------
TAG_DISPATCH, TAG_COMBINE, TAG_ALLREDUCE, TAG_BARRIER = 1, 2, 3, 4


def pack_exchange_tag(seq: int, tag: int, slot: int, peer: int) -> int:
    if not (0 <= seq < 1 << 40 and 0 <= tag < 256 and 0 <= slot < 256 and 0 <= peer < 256):
        raise ValueError("exchange tag field out of range")
    return (seq << 24) | (tag << 16) | (slot << 8) | peer


def unpack_exchange_tag(word: int):
    """-> (seq, tag, slot, peer)"""
    return word >> 24, (word >> 16) & 0xFF, (word >> 8) & 0xFF, word & 0xFF
