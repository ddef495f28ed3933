"""Process-group bring-up. Resolution order for rank / world size: explicit config, then
``RMLX_RANK`` / ``RMLX_WORLD_SIZE``, then torchrun's ``RANK`` / ``WORLD_SIZE``, then
OMPI / PMI / SLURM variables, else a single-rank loopback context
(crates/rmlx-distributed/src/init.rs:100-152). The backend is ``RMLX_BACKEND`` or "auto"
(NCCL when CUDA is present, else gloo). Failure to initialise falls back to loopback unless
``strict`` (init.rs:596-608)."""
from __future__ import annotations

import datetime
import os
from dataclasses import dataclass
from typing import Mapping, Optional, Tuple

import torch
import torch.distributed as dist

from ..config import InitConfig
from ..utils import logging as rlog
from .group import DistributedError, Group

_ENV_RANK = ("RMLX_RANK", "RANK", "OMPI_COMM_WORLD_RANK", "PMI_RANK", "SLURM_PROCID")
_ENV_WORLD = ("RMLX_WORLD_SIZE", "WORLD_SIZE", "OMPI_COMM_WORLD_SIZE", "PMI_SIZE", "SLURM_NTASKS")
_ENV_LOCAL = ("RMLX_LOCAL_SLOT", "LOCAL_RANK", "OMPI_COMM_WORLD_LOCAL_RANK", "SLURM_LOCALID")


@dataclass
class DistributedContext:
    group: Group
    rank: int
    world_size: int
    local_rank: int
    backend: str          # nccl | gloo | loopback

    @property
    def is_loopback(self) -> bool:
        return self.backend == "loopback"


def _first(env: Mapping[str, str], names) -> Optional[int]:
    for n in names:
        v = env.get(n)
        if v is not None and v != "":
            return int(v)
    return None


def resolve_rank_world(cfg: InitConfig, env: Optional[Mapping[str, str]] = None) -> Tuple[int, int, int]:
    env = os.environ if env is None else env
    rank = cfg.rank if cfg.rank is not None else _first(env, _ENV_RANK)
    world = cfg.world_size if cfg.world_size is not None else _first(env, _ENV_WORLD)
    local = _first(env, _ENV_LOCAL)
    rank = 0 if rank is None else rank
    world = 1 if world is None else world
    if not 0 <= rank < world:
        raise DistributedError(f"rank {rank} outside world of {world}")
    return rank, world, (rank if local is None else local)


def resolve_backend(cfg: InitConfig, env: Optional[Mapping[str, str]] = None) -> str:
    env = os.environ if env is None else env
    b = (cfg.backend if cfg.backend != "auto" else env.get("RMLX_BACKEND", "auto")).lower()
    if b == "auto":
        return "nccl" if torch.cuda.is_available() else "gloo"
    if b not in ("nccl", "gloo", "loopback"):
        raise DistributedError(f"unknown backend {b!r}")
    return b


def loopback_context() -> DistributedContext:
    return DistributedContext(Group(), 0, 1, 0, "loopback")


def init(cfg: Optional[InitConfig] = None) -> DistributedContext:
    cfg = cfg or InitConfig()
    rank, world, local = resolve_rank_world(cfg)
    backend = resolve_backend(cfg)
    if world <= 1 or backend == "loopback":
        return loopback_context()
    try:
        if not dist.is_initialized():
            addr = os.environ.get("RMLX_COORDINATOR", os.environ.get("MASTER_ADDR", cfg.master_addr))
            port = os.environ.get("RMLX_COORDINATOR_PORT", os.environ.get("MASTER_PORT", cfg.master_port))
            kw = {}
            if backend == "nccl":
                torch.cuda.set_device(local)
                kw["device_id"] = torch.device("cuda", local)
            dist.init_process_group(backend, init_method=f"tcp://{addr}:{port}", rank=rank,
                                    world_size=world,
                                    timeout=datetime.timedelta(seconds=cfg.timeout_s), **kw)
        rlog.info("rmlx.distributed", "process group up", rank=rank, world=world, backend=backend)
        return DistributedContext(Group(), rank, world, local, backend)
    except Exception as e:
        if cfg.strict:
            raise DistributedError(f"distributed init failed: {e}") from e
        rlog.warn("rmlx.distributed", "init failed, falling back to loopback", error=str(e))
        return loopback_context()


def shutdown() -> None:
    if dist.is_available() and dist.is_initialized():
        dist.destroy_process_group()


def rejoin(store, old_rank: int, survivors, backend: str = "gloo", generation: int = 1,
           timeout_s: float = 30.0):
    """Teardown + re-rendezvous after a rank has left between steps: the reference has no elastic
    re-ranking (a dead peer ends the job); recovery here is to destroy the process group and form a
    new, smaller one from the ranks that are still alive.

    ``survivors`` is the sorted list of old ranks that continue (every survivor passes the same
    list, learned on the host from the store or the heartbeat monitor before the next launch).
    The new rank is the position in that list. ``store`` is any ``torch.distributed`` store all
    survivors can reach (the job's TCPStore); keys are prefixed with the generation so several
    recoveries do not collide. Returns the new ``DistributedContext``."""
    survivors = sorted(int(r) for r in survivors)
    if old_rank not in survivors:
        raise DistributedError(f"rank {old_rank} is not among the survivors {survivors}")
    if dist.is_initialized():
        dist.destroy_process_group()
    new_rank, new_world = survivors.index(old_rank), len(survivors)
    if new_world == 1:
        return loopback_context()
    pstore = dist.PrefixStore(f"rmlx_gen{generation}", store)
    dist.init_process_group(backend, store=pstore, rank=new_rank, world_size=new_world,
                            timeout=datetime.timedelta(seconds=timeout_s))
    rlog.info("rmlx.distributed", "process group re-formed", rank=new_rank, world=new_world,
              generation=generation)
    return DistributedContext(Group(), new_rank, new_world, new_rank, backend)
