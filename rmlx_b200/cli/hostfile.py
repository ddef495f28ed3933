"""Hostfile: the JSON list of machines a multi-host launch spans.

Schema (one object per host, as written by ``rmlx_b200 config --hostfile``):

    [{"ssh": "user@node0", "ips": ["10.0.0.1"], "gpus": 8, "nvlink": true},
     {"ssh": "node1", "ips": [], "gpus": 8}]

``ssh`` is the target handed to ssh (validated against option injection), ``ips`` the addresses the
rendezvous may use (the first host's first address is the coordinator), ``gpus`` the ranks to start
there (defaults to the launcher's ``--nproc``), ``nvlink`` whether the host's GPUs are fully
connected. The reference's hostfile has the same role and the same ``ssh`` / ``ips`` fields plus
an RDMA device matrix that has no meaning on NVLink (crates/rmlx-cli/src/hostfile.rs:4-70,
config.rs:209-335).
"""
from __future__ import annotations

import json
from dataclasses import asdict, dataclass, field
from typing import List, Optional, Sequence

from .ssh import validate_target


@dataclass
class HostEntry:
    ssh: str
    ips: List[str] = field(default_factory=list)
    gpus: Optional[int] = None
    nvlink: Optional[bool] = None

    def address(self) -> str:
        """What other hosts connect to: the first listed address, else the ssh host name."""
        return self.ips[0] if self.ips else self.ssh.split("@")[-1]


def load_host_entries(path: str) -> List[HostEntry]:
    try:
        with open(path) as f:
            raw = json.load(f)
    except OSError as e:
        raise ValueError(f"failed to read hostfile {path}: {e}") from e
    except json.JSONDecodeError as e:
        raise ValueError(f"failed to parse hostfile {path}: {e}") from e
    if not isinstance(raw, list) or not raw:
        raise ValueError("hostfile has no hosts")
    out = []
    for i, item in enumerate(raw):
        if not isinstance(item, dict) or "ssh" not in item:
            raise ValueError(f"hostfile entry {i}: an object with an 'ssh' field is required")
        unknown = set(item) - {"ssh", "ips", "gpus", "nvlink"}
        if unknown:
            raise ValueError(f"hostfile entry {i}: unknown fields {sorted(unknown)}")
        e = HostEntry(validate_target(str(item["ssh"])), [str(a) for a in item.get("ips", [])],
                      item.get("gpus"), item.get("nvlink"))
        if e.gpus is not None and (not isinstance(e.gpus, int) or e.gpus < 1):
            raise ValueError(f"hostfile entry {i}: 'gpus' must be a positive integer")
        out.append(e)
    return out


def save_host_entries(path: str, entries: Sequence[HostEntry]) -> None:
    doc = [{k: v for k, v in asdict(e).items() if v not in (None, [])} | {"ssh": e.ssh} for e in entries]
    with open(path, "w") as f:
        json.dump(doc, f, indent=1)


def resolve_hosts(hosts_csv: Optional[str], hostfile: Optional[str]) -> List[HostEntry]:
    """Exactly one of a comma-separated list and a hostfile path."""
    if hosts_csv and hostfile:
        raise ValueError("provide only one of --hosts or --hostfile")
    if hostfile:
        return load_host_entries(hostfile)
    if hosts_csv:
        return [HostEntry(validate_target(h)) for h in hosts_csv.split(",") if h]
    raise ValueError("provide exactly one of --hosts or --hostfile")
