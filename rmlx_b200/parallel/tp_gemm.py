"""Tensor-parallel GEMMs whose collective runs inside the tensor-core kernel
(csrc/comm/tp_gemm.cu): ``gemm_allreduce`` for row-parallel layers and ``allgather_gemm`` for
column-parallel layers fed by row-sharded activations. ``NcclGemmComm`` is the library baseline with
the same interface (GEMM kernel, then ``torch.distributed`` collective).

The reference's counterpart is ``RowParallelLinear`` / ``ColumnParallelLinear``
(crates/rmlx-nn/src/parallel.rs:52-693), where the sum over ranks is a separate host-driven
all-reduce after the matmul's command buffer has completed.
"""
from __future__ import annotations

import ctypes
from typing import Dict, Optional, Tuple

import torch
import torch.distributed as dist

from .. import _lib
from ..ops.gemm import GemmStatus, gemm_bf16
from ..ops.quantized import qmm
from ..ops.weights import LinearWeight, W_BF16
from .comm import SymmetricRegion

_lib.register_cuda_sigs({
    "rmlx_tp_gemm_stage_bytes": ("iiii", "q"),
    "rmlx_tp_gemm_allreduce": ("ippppppppppiiiiiiiiippp", "i"),
    "rmlx_tp_allgather_gemm": ("ipiippppppppiiiiiippp", "i"),
})


class _RawCuda:
    """Zero-copy view of device memory for ``torch.as_tensor``."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False),
                                         "version": 2}


def _align(n: int, a: int = 256) -> int:
    return (n + a - 1) // a * a


class FusedGemmComm:
    """Owns the peer-mapped buffers (staging slab, two output buffers, gathered-activation buffers,
    counters) for GEMMs of up to ``max_tokens`` rows, ``max_n`` output and ``max_k`` input columns."""

    kind = "fused"
    COUNTER_BYTES = 1 << 20

    def __init__(self, max_tokens: int, max_n: int, max_k: int, group=None, device=None):
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.max_tokens, self.max_n, self.max_k = max_tokens, max_n, max_k
        lib = _lib.cuda()
        mt = _align(max_tokens, 128)
        self.stage_bytes = int(max(lib.rmlx_tp_gemm_stage_bytes(self.world, mt, max_n, bn) for bn in (128, 256)))
        self.out_bytes = _align(mt * max_n * 2)
        self.full_bytes = _align(2 * mt * max_k * 2)
        self.off_stage = 0
        self.off_out = [_align(self.stage_bytes), _align(self.stage_bytes) + self.out_bytes]
        self.off_full = self.off_out[1] + self.out_bytes
        self.off_ctr = self.off_full + self.full_bytes
        self.region = SymmetricRegion(self.off_ctr + self.COUNTER_BYTES, group)
        self._ctr_used = 0
        self._sites: Dict[Tuple, int] = {}
        self._flip = 0
        self._out_views = [torch.as_tensor(_RawCuda(self.region.local + o, self.out_bytes), device=self.device)
                           for o in self.off_out]
        self._stage = self.region.peer_array(self.off_stage)
        self.trace: Optional[torch.Tensor] = None

    # ------------------------------------------------------------------ counters per call shape
    def _site(self, key: Tuple, words: int) -> int:
        """Byte offset (same on every rank) of a zero-initialised counter block for this shape."""
        off = self._sites.get(key)
        if off is None:
            need = _align(words * 4, 64)
            if self._ctr_used + need > self.COUNTER_BYTES:
                raise _lib.NativeError("too many distinct tensor-parallel GEMM shapes for the counter area")
            off = self.off_ctr + self._ctr_used
            self._ctr_used += need
            self._sites[key] = off
        return off

    # ------------------------------------------------------------------ row-parallel: GEMM + all-reduce
    def gemm_reduce_scatter(self, x: torch.Tensor, w: LinearWeight,
                            residual: Optional[torch.Tensor] = None, bn: int = 0) -> torch.Tensor:
        """x [M, K_local] bf16, w [N, K_local] -> this rank's share of sum over ranks (+ residual):
        the 128-row blocks b with b % world == rank, in order, as [M / world, N] (a strided view of a
        peer-mapped buffer, valid until the call after next). Nothing is broadcast: a finished tile
        stays with the rank that reduced it. M must be a whole number of 128-row blocks per rank.
        ``owned_rows(M)`` lists the row indices (crates/rmlx-distributed/src/group.rs:728,
        reduce_scatter)."""
        m = x.shape[0]
        if m % (128 * self.world):
            raise ValueError("reduce-scatter needs M to be a multiple of 128 x world")
        full = self.gemm_allreduce(x, w, residual, bn, _scatter=True)
        return full.view(m // 128, 128, w.n)[self.rank::self.world].reshape(m // self.world, w.n)

    def owned_rows(self, m: int) -> torch.Tensor:
        """Row indices of the [M, N] result that ``gemm_reduce_scatter`` leaves on this rank."""
        blocks = torch.arange(self.rank, m // 128, self.world)
        return (blocks[:, None] * 128 + torch.arange(128)[None, :]).reshape(-1)

    def gemm_allreduce(self, x: torch.Tensor, w: LinearWeight, residual: Optional[torch.Tensor] = None,
                       bn: int = 0, _scatter: bool = False) -> torch.Tensor:
        """x [M, K_local] bf16, w [N, K_local] -> sum over ranks (+ residual) as [M, N], complete on
        every rank. The result is a view of one of two peer-mapped buffers, valid until the call
        after next."""
        m, k = x.shape
        n = w.n
        bn = bn or 128
        assert m <= self.max_tokens and n <= self.max_n and x.stride(1) == 1 and k == w.k
        tiles = ((m + 127) // 128) * ((n + bn - 1) // bn)
        owned = (tiles + self.world - 1) // self.world
        # block: [0] epoch, [1] ticket, [2] done, [4..] per-tile arrival counters
        off = self._site(("rs" if _scatter else "ar", m, n, bn), 4 + owned)
        self._flip ^= 1
        out = self._out_views[self._flip][: m * n * 2].view(torch.bfloat16).view(m, n)
        if residual is not None:
            assert residual.shape == (m, n) and residual.is_contiguous()
        rg = self.region
        rc = _lib.cuda().rmlx_tp_gemm_allreduce(
            w.kind, x.data_ptr(), w.w.data_ptr(), _lib.ptr(w.scales), _lib.ptr(w.biases),
            _lib.ptr(residual), self._stage, rg.peer_array(off + 16), rg.peer_array(self.off_out[self._flip]),
            rg.peer_array(off + 8), ctypes.c_void_p(rg.local + off), self.rank, self.world, m, n, k,
            x.stride(0), n, bn, int(_scatter), GemmStatus.get(self.device).data_ptr(), _lib.ptr(self.trace),
            _lib.stream_ptr())
        _lib.check(rc, "tp_gemm_allreduce")
        return out

    # ------------------------------------------------------------------ column-parallel: all-gather + GEMM
    def allgather_gemm(self, x_shard: torch.Tensor, w: LinearWeight,
                       residual: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
                       bn: int = 0) -> torch.Tensor:
        """x_shard [M/world, K] bf16 (this rank's rows), w [N_local, K] -> [M, N_local] (local)."""
        ms, k = x_shard.shape
        m = ms * self.world
        assert m <= _align(self.max_tokens, 128) and k <= self.max_k and x_shard.stride(1) == 1 and k == w.k
        assert ms % 128 == 0, "row shards are whole 128-row blocks"
        off = self._site(("ag", ms, k), 4 + m // 128)
        if out is None:
            out = torch.empty(m, w.n, dtype=torch.bfloat16, device=self.device)
        rg = self.region
        # the gathered buffer holds two parities of [m, k]; the kernel alternates between them
        rc = _lib.cuda().rmlx_tp_allgather_gemm(
            w.kind, x_shard.data_ptr(), x_shard.stride(0), ms, rg.peer_array(self.off_full),
            rg.peer_array(off + 16), ctypes.c_void_p(rg.local + off), w.w.data_ptr(), _lib.ptr(w.scales),
            _lib.ptr(w.biases), out.data_ptr(), _lib.ptr(residual), self.rank, self.world, w.n, k,
            out.stride(0), bn, GemmStatus.get(self.device).data_ptr(), _lib.ptr(self.trace), _lib.stream_ptr())
        _lib.check(rc, "tp_allgather_gemm")
        return out

    def enable_trace(self, on: bool = True) -> None:
        """Record per-CTA phase timestamps of the next calls (see ``trace_summary``)."""
        self.trace = torch.zeros(256, 8, dtype=torch.int64, device=self.device) if on else None

    def trace_summary(self) -> Dict[str, float]:
        """Microseconds from the first CTA's start to the latest CTA's mark, per phase, for the
        last traced call: last MMA issued, epilogue done, collective warps done, exit."""
        t = self.trace.cpu()
        t = t[t[:, 0] > 0]
        t0 = int(t[:, 0].min())
        names = ("start_spread", "mma_issued", "epilogue_done", "collective_done", "exit")
        return {n: (int(t[:, i].max()) - t0) / 1e3 for i, n in enumerate(names)}

    def status(self) -> int:
        return int(GemmStatus.get(self.device).item())

    def close(self) -> None:
        self._out_views = []
        self.region.close()


class NcclGemmComm:
    """Same interface on library collectives: the baseline the fused kernels are measured against."""

    kind = "nccl"

    def __init__(self, max_tokens: int, max_n: int, max_k: int, group=None, device=None):
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.device = device or torch.device("cuda", torch.cuda.current_device())

    @staticmethod
    def _mm(x, w, residual=None):
        return gemm_bf16(x, w.w, residual=residual) if w.kind == W_BF16 else qmm(x, w, residual=residual)

    def gemm_allreduce(self, x, w, residual=None, bn=0):
        y = self._mm(x, w)
        dist.all_reduce(y, group=self.group)
        return y if residual is None else y + residual

    def gemm_reduce_scatter(self, x, w, residual=None, bn=0):
        m = x.shape[0]
        y = self.gemm_allreduce(x, w, residual, bn)
        return y.view(m // 128, 128, w.n)[self.rank::self.world].reshape(m // self.world, w.n)

    def owned_rows(self, m: int) -> torch.Tensor:
        blocks = torch.arange(self.rank, m // 128, self.world)
        return (blocks[:, None] * 128 + torch.arange(128)[None, :]).reshape(-1)

    def allgather_gemm(self, x_shard, w, residual=None, out=None, bn=0):
        full = torch.empty(x_shard.shape[0] * self.world, x_shard.shape[1], dtype=x_shard.dtype,
                           device=x_shard.device)
        dist.all_gather_into_tensor(full, x_shard.contiguous(), group=self.group)
        y = self._mm(full, w, residual)
        if out is not None:
            out.copy_(y)
            return out
        return y

    def status(self) -> int:
        return 0

    def close(self) -> None:
        pass


def make_gemm_comm(kind: str, max_tokens: int, max_n: int, max_k: int, group=None, device=None):
    cls = {"fused": FusedGemmComm, "nccl": NcclGemmComm}[kind]
    return cls(max_tokens, max_n, max_k, group, device)
