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
