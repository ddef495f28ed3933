"""All-reduce algorithms built on a group's point-to-point calls: tree, ring and mesh, and the
size-based choice among them.

The reference implements the same family over its transport
(crates/rmlx-distributed/src/group.rs:1660-1850: ``tree_allreduce`` for small tensors, O(log N)
steps; ring for large tensors on more than two ranks, bandwidth optimal; mesh otherwise, one round
of pairwise exchanges; ``allreduce_auto`` picks by size). On B200s the product path for CUDA tensors
is the peer-memory kernels behind ``Group.allreduce`` (one-shot / two-shot pushes, in-switch
reduction); these functions are the transport-agnostic forms: they run on any ``Group`` that can
``sendrecv`` / ``shift`` (gloo ranks on CPUs in the tests, the peer mailboxes of
``parallel/p2p.py`` on GPUs) and serve as the oracle for chunk boundaries and reduction order.
Half-precision inputs are accumulated in fp32 and rounded once at the end, in a fixed order, so
every rank returns the same bits.
"""
from __future__ import annotations

from enum import Enum
from typing import List, Tuple

import torch

from .group import Group

TREE_THRESHOLD_BYTES = 1 << 20           # below: tree
RING_THRESHOLD_BYTES = 8 << 20           # at or above, on more than two ranks: ring
RING_THRESHOLD_BYTES_HALF = 128 << 10    # the same for 16-bit element types


class AllreduceAlgorithm(Enum):
    TREE = "tree"
    RING = "ring"
    MESH = "mesh"


def chunk_bounds(n: int, parts: int) -> List[Tuple[int, int]]:
    """``parts`` contiguous [lo, hi) ranges covering n elements; the first n % parts ranges are
    one element longer (empty ranges when n < parts)."""
    base, extra = divmod(n, parts)
    out, lo = [], 0
    for i in range(parts):
        hi = lo + base + (1 if i < extra else 0)
        out.append((lo, hi))
        lo = hi
    return out


def _acc(t: torch.Tensor) -> torch.Tensor:
    flat = t.reshape(-1)
    return flat.float() if t.dtype in (torch.bfloat16, torch.float16) else flat.clone()


def tree_allreduce(group: Group, t: torch.Tensor) -> torch.Tensor:
    """Binary-tree reduction to the group's rank 0, then the mirror-image broadcast:
    2 ceil(log2 N) steps, whole tensor per step."""
    n, r = group.world_size, group.local_rank
    if n == 1:
        return t.clone()
    acc = _acc(t)
    buf = torch.empty_like(acc)
    step = 1
    while step < n:                                   # reduce: r with bit `step` set sends to r - step
        if r % (2 * step) == step:
            group.send(acc, r - step)
        elif r % (2 * step) == 0 and r + step < n:
            group.recv(buf, r + step)
            acc += buf
        step *= 2
    step //= 2
    while step >= 1:                                  # broadcast back down the same tree
        if r % (2 * step) == 0 and r + step < n:
            group.send(acc, r + step)
        elif r % (2 * step) == step:
            group.recv(acc, r - step)
        step //= 2
    return acc.to(t.dtype).reshape(t.shape)


def ring_allreduce(group: Group, t: torch.Tensor) -> torch.Tensor:
    """Reduce-scatter then all-gather around the ring: 2 (N - 1) steps of 1/N of the tensor each."""
    n, r = group.world_size, group.local_rank
    if n == 1:
        return t.clone()
    acc = _acc(t)
    bounds = chunk_bounds(acc.numel(), n)
    right, left = (r + 1) % n, (r - 1) % n
    longest = max(hi - lo for lo, hi in bounds)
    buf = torch.empty(longest, dtype=acc.dtype, device=acc.device)
    for s in range(n - 1):                            # after step s rank r holds the sum of s + 2 ranks of chunk r - s - 1
        lo, hi = bounds[(r - s) % n]
        rlo, rhi = bounds[(r - s - 1) % n]
        got = group.shift(acc[lo:hi].contiguous(), buf[:rhi - rlo], right, left)
        acc[rlo:rhi] += got
    for s in range(n - 1):                            # circulate the finished chunks
        lo, hi = bounds[(r + 1 - s) % n]
        rlo, rhi = bounds[(r - s) % n]
        got = group.shift(acc[lo:hi].contiguous(), buf[:rhi - rlo], right, left)
        acc[rlo:rhi] = got
    return acc.to(t.dtype).reshape(t.shape)


def ring_reduce_scatter(group: Group, t: torch.Tensor) -> torch.Tensor:
    """The first half of the ring: returns this rank's chunk (``chunk_bounds(numel, N)[rank]``)
    of the sum over ranks, flat, in the input's dtype."""
    n, r = group.world_size, group.local_rank
    acc = _acc(t)
    bounds = chunk_bounds(acc.numel(), n)
    if n > 1:
        right, left = (r + 1) % n, (r - 1) % n
        buf = torch.empty(max(hi - lo for lo, hi in bounds), dtype=acc.dtype, device=acc.device)
        for s in range(n - 1):                        # chunks start one place earlier, so r ends with chunk r
            lo, hi = bounds[(r - s - 1) % n]
            rlo, rhi = bounds[(r - s - 2) % n]
            got = group.shift(acc[lo:hi].contiguous(), buf[:rhi - rlo], right, left)
            acc[rlo:rhi] += got
    lo, hi = bounds[r]
    return acc[lo:hi].to(t.dtype)


def ring_allgather(group: Group, shard: torch.Tensor) -> torch.Tensor:
    """Shards of equal shape from every rank, concatenated along a new leading axis in rank
    order: N - 1 steps, each passing on the shard received in the step before."""
    n, r = group.world_size, group.local_rank
    out = torch.empty((n, *shard.shape), dtype=shard.dtype, device=shard.device)
    out[r] = shard
    right, left = (r + 1) % n, (r - 1) % n
    for s in range(n - 1):
        src = (r - s - 1) % n
        group.shift(out[(r - s) % n].contiguous(), out[src], right, left)
    return out


def tree_broadcast(group: Group, t: torch.Tensor, root: int = 0) -> torch.Tensor:
    """``root``'s tensor to every rank in ceil(log2 N) steps (ranks renumbered so that the root is
    0; in step k every rank that already holds the data passes it to the rank 2^k away)."""
    n, r = group.world_size, group.local_rank
    if n == 1:
        return t
    v = (r - root) % n                                # position in the tree rooted at `root`
    buf = t.contiguous() if v == 0 else torch.empty_like(t)
    step = 1
    while step < n:
        if v < step and v + step < n:
            group.send(buf, (v + step + root) % n)
        elif step <= v < 2 * step:
            group.recv(buf, (v - step + root) % n)
        step *= 2
    return buf


def mesh_allreduce(group: Group, t: torch.Tensor) -> torch.Tensor:
    """Every rank exchanges its whole tensor with every other rank (N - 1 pairwise exchanges, a
    round-robin schedule so that each round is a perfect matching) and sums in rank order."""
    n, r = group.world_size, group.local_rank
    if n == 1:
        return t.clone()
    mine = _acc(t)
    parts = {r: mine}
    m = n if n % 2 == 0 else n + 1                    # odd groups: one rank idles per round
    for rnd in range(m - 1):
        if r == m - 1:
            peer = rnd
        elif r == rnd:
            peer = m - 1
        else:
            peer = (2 * rnd - r) % (m - 1)
        if peer >= n or peer == r:
            continue
        parts[peer] = group.sendrecv(mine, torch.empty_like(mine), peer)
    acc = torch.zeros_like(mine)
    for i in range(n):                                # the same order everywhere: identical bits
        acc += parts[i]
    return acc.to(t.dtype).reshape(t.shape)


def choose_algorithm(nbytes: int, world: int, half: bool = False,
                     tree_threshold: int = TREE_THRESHOLD_BYTES) -> AllreduceAlgorithm:
    ring_at = RING_THRESHOLD_BYTES_HALF if half else RING_THRESHOLD_BYTES
    if world > 2 and nbytes >= ring_at:
        return AllreduceAlgorithm.RING
    if nbytes < tree_threshold:
        return AllreduceAlgorithm.TREE
    return AllreduceAlgorithm.MESH


def allreduce_auto(group: Group, t: torch.Tensor, tree_threshold: int = TREE_THRESHOLD_BYTES
                   ) -> Tuple[torch.Tensor, AllreduceAlgorithm]:
    """Large tensors on more than two ranks: ring; small ones: tree; the rest: mesh."""
    half = t.dtype in (torch.bfloat16, torch.float16)
    algo = choose_algorithm(t.numel() * t.element_size(), group.world_size, half, tree_threshold)
    fn = {AllreduceAlgorithm.RING: ring_allreduce, AllreduceAlgorithm.TREE: tree_allreduce,
          AllreduceAlgorithm.MESH: mesh_allreduce}[algo]
    return fn(group, t), algo
