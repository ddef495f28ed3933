"""Single-box GPU topology discovery: which GPUs exist, whether every pair can reach each other
over peer access / NVLink, and the rank -> device map the launcher exports.

Replaces the reference's Thunderbolt discovery and rank x rank RDMA device matrix
(crates/rmlx-cli/src/tb_discovery.rs, crates/rmlx-rdma/src/device_file.rs:1-150). Sources, in order:
NVML through ``pynvml`` (link states, when present), then ``torch.cuda`` peer-access queries.
Everything is read-only: no clocks, power limits or modes are touched. ``parse_topo_matrix``
parses the text of ``nvidia-smi topo -m`` (kept pure so it is testable with canned output)."""
from __future__ import annotations

import json
from dataclasses import dataclass, field
from typing import Dict, List, Optional


@dataclass
class GpuInfo:
    index: int
    name: str
    memory_bytes: int
    nvlink_links: int = 0


@dataclass
class Topology:
    gpus: List[GpuInfo] = field(default_factory=list)
    peer: List[List[bool]] = field(default_factory=list)     # peer[i][j]: i can map j's memory
    link: List[List[str]] = field(default_factory=list)      # "NV18", "PIX", "SYS", "X" ...

    @property
    def num_gpus(self) -> int:
        return len(self.gpus)

    def fully_connected(self) -> bool:
        n = self.num_gpus
        return all(self.peer[i][j] for i in range(n) for j in range(n) if i != j)

    def all_nvlink(self) -> bool:
        n = self.num_gpus
        return bool(self.link) and all(self.link[i][j].startswith("NV")
                                       for i in range(n) for j in range(n) if i != j)

    def device_map(self, world: int) -> List[int]:
        if world > self.num_gpus:
            raise ValueError(f"{world} ranks requested, {self.num_gpus} GPUs present")
        return list(range(world))

    def to_json(self) -> str:
        return json.dumps({"gpus": [g.__dict__ for g in self.gpus], "peer": self.peer,
                           "link": self.link})

    # The device-matrix file: what rank i uses to reach rank j, written once by ``config`` and read
    # by every rank at start-up instead of probing again (the reference keeps a rank x rank table
    # of RDMA device names, crates/rmlx-rdma/src/device_file.rs:1-150; here an entry is the link
    # label between two GPUs and whether peer mapping works).
    def save(self, path: str) -> None:
        with open(path, "w") as f:
            f.write(self.to_json())

    @staticmethod
    def load(path: str) -> "Topology":
        with open(path) as f:
            doc = json.load(f)
        n = len(doc.get("gpus", []))
        peer, link = doc.get("peer", []), doc.get("link", [])
        if len(peer) != n or any(len(r) != n for r in peer) or (link and (len(link) != n or any(len(r) != n for r in link))):
            raise ValueError("device matrix file: peer / link tables must be rank x rank")
        if any(peer[i][i] is not True for i in range(n)):
            raise ValueError("device matrix file: a device must reach itself")
        return Topology([GpuInfo(**g) for g in doc["gpus"]], [[bool(v) for v in r] for r in peer],
                        [[str(v) for v in r] for r in link])

    def reachable(self, i: int, j: int) -> bool:
        return bool(self.peer[i][j])


def parse_topo_matrix(text: str) -> List[List[str]]:
    """Rows ``GPUi  X  NV18 ...`` of ``nvidia-smi topo -m`` -> matrix of link labels."""
    rows = []
    lines = [l for l in text.splitlines() if l.strip()]
    hdr = next((l for l in lines if l.split() and l.split()[0].startswith("GPU0")), None)
    if hdr is None:
        return rows
    ngpu = sum(1 for t in hdr.split() if t.startswith("GPU"))
    for l in lines:
        t = l.split()
        if t and t[0].startswith("GPU") and t[0][3:].isdigit() and len(t) >= 1 + ngpu and l is not hdr:
            rows.append(t[1:1 + ngpu])
    return rows


def discover(max_gpus: Optional[int] = None) -> Topology:
    import torch
    topo = Topology()
    if not torch.cuda.is_available():
        return topo
    n = torch.cuda.device_count()
    if max_gpus:
        n = min(n, max_gpus)
    links: Dict[int, int] = {}
    try:
        import pynvml
        pynvml.nvmlInit()
        for i in range(n):
            h = pynvml.nvmlDeviceGetHandleByIndex(i)
            cnt = 0
            for l in range(18):
                try:
                    if pynvml.nvmlDeviceGetNvLinkState(h, l):
                        cnt += 1
                except Exception:
                    break
            links[i] = cnt
    except Exception:
        pass
    for i in range(n):
        p = torch.cuda.get_device_properties(i)
        topo.gpus.append(GpuInfo(i, p.name, p.total_memory, links.get(i, 0)))
    topo.peer = [[i == j or torch.cuda.can_device_access_peer(i, j) for j in range(n)] for i in range(n)]
    topo.link = [["X" if i == j else ("NV%d" % links[i] if links.get(i) else ("P2P" if topo.peer[i][j] else "SYS"))
                  for j in range(n)] for i in range(n)]
    return topo


# ------------------------------------------------------------------------------------------------
# Logical topologies, striping plans and link fail-over: the host-side logic of the reference's
# multi-port module (crates/rmlx-rdma/src/multi_port.rs:60-300) and its RMLX_TOPOLOGY setting
# (crates/rmlx-distributed/src/init.rs:247-263). On an NVSwitch box every pair of GPUs is one hop
# apart, so "mesh" is the default and the others matter for algorithms that want a neighbour order
# (ring collectives, hierarchical exchanges) or for boxes without a switch.
# ------------------------------------------------------------------------------------------------
class LogicalTopology:
    def __init__(self, kind: str = "mesh", group_size: int = 0, hops: Optional[List[List[int]]] = None):
        if kind not in ("ring", "mesh", "hybrid", "matrix"):
            raise ValueError(f"unknown topology {kind!r}")
        if kind == "hybrid" and group_size < 1:
            raise ValueError("hybrid topology needs a group size")
        self.kind, self.group_size, self.hops = kind, group_size, hops

    @staticmethod
    def parse(text: Optional[str]) -> "LogicalTopology":
        """``ring`` | ``mesh`` | ``hybrid:<group>`` | a JSON rank x rank hop matrix (0 = self,
        1 = direct, larger = more hops, null / negative = unreachable)."""
        text = (text or "mesh").strip()
        if text.startswith("["):
            import json
            m = json.loads(text)
            if not m or any(len(r) != len(m) for r in m):
                raise ValueError("hop matrix must be square")
            return LogicalTopology("matrix", hops=[[(-1 if v is None else int(v)) for v in r] for r in m])
        if text.startswith("hybrid"):
            _, _, g = text.partition(":")
            return LogicalTopology("hybrid", int(g or 2))
        return LogicalTopology(text)

    @staticmethod
    def from_env(env=None) -> "LogicalTopology":
        import os
        return LogicalTopology.parse((os.environ if env is None else env).get("RMLX_TOPOLOGY"))

    def peers(self, rank: int, world: int) -> List[int]:
        """Ranks this rank talks to directly, nearest first."""
        if not 0 <= rank < world:
            raise ValueError("rank out of range")
        if world == 1:
            return []
        if self.kind == "mesh":
            return [(rank + d) % world for d in range(1, world)]
        if self.kind == "ring":
            out = [(rank + 1) % world, (rank - 1) % world]
            return out[:1] if out[0] == out[1] else out
        if self.kind == "hybrid":
            g = self.group_size
            base = rank // g * g
            local = [base + (rank - base + d) % g for d in range(1, g) if base + (rank - base + d) % g < world]
            ngroups = (world + g - 1) // g
            remote = [((rank // g + d) % ngroups) * g + rank % g for d in range(1, ngroups)]
            return local + [r for r in remote if r < world and r != rank]
        row = self.hops[rank]
        if len(row) != world:
            raise ValueError("hop matrix does not match the world size")
        return [r for _, r in sorted((h, r) for r, h in enumerate(row) if r != rank and h > 0)]


def stripe_plan(nbytes: int, lanes: int, chunk: int = 64 << 10, threshold: int = 256 << 10) -> List[tuple]:
    """(lane, offset, length) pieces of one transfer: below ``threshold`` a single piece on lane 0,
    above it chunks of ``chunk`` bytes dealt round-robin over ``lanes`` (the last one may be short).
    Lanes are links in the reference; here they are the blocks of a copy kernel or several streams."""
    if nbytes < 0 or lanes < 1 or chunk < 1:
        raise ValueError("bad striping arguments")
    if nbytes == 0:
        return []
    if lanes == 1 or nbytes < threshold:
        return [(0, 0, nbytes)]
    return [(i % lanes, off, min(chunk, nbytes - off)) for i, off in enumerate(range(0, nbytes, chunk))]


class LinkFailover:
    """Active -> Failed -> Recovering -> Active state per lane, with a count of consecutive errors
    before a lane is taken out and of clean probes before it is trusted again."""
    ACTIVE, FAILED, RECOVERING = "active", "failed", "recovering"

    def __init__(self, lanes: int, fail_after: int = 3, recover_after: int = 2):
        self.state = [self.ACTIVE] * lanes
        self._errors = [0] * lanes
        self._clean = [0] * lanes
        self.fail_after, self.recover_after = fail_after, recover_after

    def report(self, lane: int, ok: bool) -> str:
        if ok:
            self._errors[lane] = 0
            if self.state[lane] == self.FAILED:
                self.state[lane], self._clean[lane] = self.RECOVERING, 1
            elif self.state[lane] == self.RECOVERING:
                self._clean[lane] += 1
            if self.state[lane] == self.RECOVERING and self._clean[lane] >= self.recover_after:
                self.state[lane] = self.ACTIVE
        else:
            self._clean[lane] = 0
            self._errors[lane] += 1
            if self.state[lane] == self.RECOVERING or self._errors[lane] >= self.fail_after:
                self.state[lane] = self.FAILED
        return self.state[lane]

    def usable(self) -> List[int]:
        return [i for i, s in enumerate(self.state) if s == self.ACTIVE]
