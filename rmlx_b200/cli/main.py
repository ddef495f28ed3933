"""``python -m rmlx_b200.cli {config,launch}`` — the single-box counterpart of the reference's
``rmlx`` binary (crates/rmlx-cli/src/main.rs:18-32).

``config`` probes the machine (GPUs, peer access, NVLink) and writes a hostfile-like JSON
(crates/rmlx-cli/src/config.rs:115-345 does this over SSH with Thunderbolt discovery).
``launch`` starts one process per GPU with the rank contract exported in the environment
(RMLX_RANK, RMLX_WORLD_SIZE, RMLX_LOCAL_SLOT, RMLX_BACKEND, RMLX_COORDINATOR, RMLX_COORDINATOR_PORT
plus torchrun's RANK / WORLD_SIZE / LOCAL_RANK / MASTER_ADDR / MASTER_PORT), prefixes every output
line with ``[rank=R]``, and kills the whole job as soon as one rank exits non-zero
(crates/rmlx-cli/src/launch.rs:95-120,343-416)."""
from __future__ import annotations

import argparse
import json
import os
import signal
import subprocess
import sys
import threading
import time
from typing import Dict, List, Optional, Sequence

VALID_BACKENDS = ("auto", "nccl", "gloo", "loopback")


def build_env(rank: int, world: int, backend: str, addr: str, port: int,
              extra: Optional[Dict[str, str]] = None, device_map: Optional[Sequence[int]] = None
              ) -> Dict[str, str]:
    local = rank if device_map is None else device_map[rank]
    env = {"RMLX_RANK": str(rank), "RMLX_WORLD_SIZE": str(world), "RMLX_LOCAL_SLOT": str(local),
           "RMLX_BACKEND": backend, "RMLX_COORDINATOR": addr, "RMLX_COORDINATOR_PORT": str(port),
           "RANK": str(rank), "WORLD_SIZE": str(world), "LOCAL_RANK": str(local),
           "MASTER_ADDR": addr, "MASTER_PORT": str(port)}
    env.update(extra or {})
    return env


def parse_env_args(items: Sequence[str]) -> Dict[str, str]:
    out = {}
    for it in items:
        if "=" not in it or it.startswith("="):
            raise ValueError(f"--env expects KEY=VALUE, got {it!r}")
        k, v = it.split("=", 1)
        if not k.replace("_", "").isalnum():
            raise ValueError(f"invalid environment variable name {k!r}")
        out[k] = v
    return out


def resolve_backend(requested: str, have_cuda: bool) -> str:
    if requested not in VALID_BACKENDS:
        raise ValueError(f"unknown backend {requested!r}; choose from {VALID_BACKENDS}")
    if requested == "auto":
        return "nccl" if have_cuda else "gloo"
    return requested


def _pump(rank: int, stream, sink, lock):
    for line in iter(stream.readline, ""):
        with lock:
            sink.write(f"[rank={rank}] {line}")
            sink.flush()
    stream.close()


def launch(cmd: Sequence[str], nproc: int, backend: str = "auto", addr: str = "127.0.0.1",
           port: int = 18520, extra_env: Optional[Dict[str, str]] = None, sink=None,
           poll_s: float = 0.05, device_map: Optional[Sequence[int]] = None) -> int:
    """Run ``cmd`` as ``nproc`` ranks. Returns 0 if all succeeded, else 1 after killing the rest."""
    specs = []
    for r in range(nproc):
        env = dict(os.environ)
        env.update(build_env(r, nproc, backend, addr, port, extra_env, device_map))
        specs.append((list(cmd), env))
    return _run_all(specs, sink or sys.stdout, poll_s)


def launch_hosts(cmd: Sequence[str], hosts: Sequence[str], per_host: int, backend: str = "nccl",
                 port: int = 18520, extra_env: Optional[Dict[str, str]] = None, cwd: Optional[str] = None,
                 sink=None, poll_s: float = 0.05, dry_run: bool = False,
                 coordinator: Optional[str] = None) -> int:
    """One rank per GPU on every host, spawned through ssh; the first host is the coordinator
    (``coordinator``: the address the ranks rendezvous at, default the first host's name).
    ``dry_run`` prints the ssh command lines instead of running them
    (crates/rmlx-cli/src/launch.rs:95-120: hosts list, per-rank environment, fail-fast)."""
    from . import ssh
    sink = sink or sys.stdout
    plan = ssh.plan_ranks(hosts, per_host)
    world = len(plan)
    addr = coordinator or hosts[0].split("@")[-1]
    specs = []
    for host, rank, slot in plan:
        env = build_env(rank, world, backend, addr, port, extra_env, device_map=None)
        env["RMLX_LOCAL_SLOT"] = env["LOCAL_RANK"] = str(slot)
        specs.append((ssh.ssh_argv(host, cmd, env, cwd), dict(os.environ)))
    if dry_run:
        for argv, _ in specs:
            sink.write(" ".join(ssh.shell_quote(a) for a in argv) + "\n")
        return 0
    return _run_all(specs, sink, poll_s)


def _run_all(specs, sink, poll_s: float) -> int:
    """Start every (argv, env), prefix their output with the rank, stop everything at the first
    non-zero exit. Returns 0 if all succeeded, else 1."""
    nproc = len(specs)
    lock = threading.Lock()
    procs: List[subprocess.Popen] = []
    threads = []
    for r, (argv, env) in enumerate(specs):
        p = subprocess.Popen(argv, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT,
                             text=True, bufsize=1, start_new_session=True)
        procs.append(p)
        t = threading.Thread(target=_pump, args=(r, p.stdout, sink, lock), daemon=True)
        t.start()
        threads.append(t)
    rc = 0
    alive = set(range(nproc))
    while alive:
        for r in list(alive):
            code = procs[r].poll()
            if code is None:
                continue
            alive.discard(r)
            if code != 0 and rc == 0:
                rc = 1
                with lock:
                    sink.write(f"[launch] rank {r} exited with {code}; stopping the job\n")
                for o in alive:           # fail fast: exact process groups we started
                    try:
                        os.killpg(procs[o].pid, signal.SIGTERM)
                    except ProcessLookupError:
                        pass
        time.sleep(poll_s)
    for t in threads:
        t.join(timeout=2)
    return rc


def config(path: Optional[str]) -> dict:
    from ..parallel.topology import discover
    from ..runtime.device import self_check
    topo = discover()
    doc = {"host": "localhost", "gpus": [g.__dict__ for g in topo.gpus], "peer_access": topo.peer,
           "links": topo.link, "fully_connected": topo.fully_connected() if topo.num_gpus else False,
           "self_check": self_check() if topo.num_gpus else {"ok": False, "reason": "no CUDA device"}}
    if path:
        with open(path, "w") as f:
            json.dump(doc, f, indent=1)
    return doc


def main(argv: Optional[Sequence[str]] = None) -> int:
    ap = argparse.ArgumentParser(prog="rmlx_b200")
    sub = ap.add_subparsers(dest="cmd", required=True)
    c = sub.add_parser("config", help="probe GPUs and NVLink topology")
    c.add_argument("--output", "-o", default=None)
    c.add_argument("--hostfile", default=None,
                   help="also write a one-entry hostfile for this machine (ssh target = --ssh)")
    c.add_argument("--ssh", default="localhost", help="ssh target recorded in the hostfile")
    sub.add_parser("plan", add_help=False,
                   help="memory and decode plans of a model on B200s (see `rmlx_b200 plan --help`)")
    l = sub.add_parser("launch", help="run a command as one rank per GPU")
    l.add_argument("--nproc", "-n", type=int, default=0, help="ranks (default: all GPUs)")
    l.add_argument("--backend", default="auto")
    l.add_argument("--coordinator", default="127.0.0.1")
    l.add_argument("--port", type=int, default=18520)
    l.add_argument("--env", action="append", default=[])
    l.add_argument("--hosts", default="", help="comma-separated [user@]host list: spawn over ssh, --nproc ranks per host")
    l.add_argument("--hostfile", default=None, help="JSON hostfile (see cli/hostfile.py) instead of --hosts")
    l.add_argument("--cwd", default=None, help="working directory on the remote hosts")
    l.add_argument("--dry-run", action="store_true", help="with --hosts: print the ssh commands only")
    l.add_argument("command", nargs=argparse.REMAINDER)
    args = list(sys.argv[1:] if argv is None else argv)
    if args and args[0] == "plan":                  # the planner owns its own options
        from .plan import main as plan_main
        return plan_main(args[1:])
    a = ap.parse_args(argv)
    if a.cmd == "config":
        doc = config(a.output)
        if a.hostfile:
            from .hostfile import HostEntry, save_host_entries
            save_host_entries(a.hostfile, [HostEntry(a.ssh, [], len(doc["gpus"]) or None,
                                                     bool(doc["fully_connected"]))])
        print(json.dumps(doc, indent=1))
        return 0
    cmd = a.command[1:] if a.command and a.command[0] == "--" else a.command
    if not cmd:
        ap.error("launch needs a command after --")
    if a.hosts or a.hostfile:
        from .hostfile import resolve_hosts
        try:
            entries = resolve_hosts(a.hosts or None, a.hostfile)
        except ValueError as e:
            ap.error(str(e))
        per_host = a.nproc or min((e.gpus for e in entries if e.gpus), default=8)
        backend = "nccl" if a.backend == "auto" else resolve_backend(a.backend, True)
        return launch_hosts(cmd, [e.ssh for e in entries], per_host, backend, a.port,
                            parse_env_args(a.env), a.cwd, dry_run=a.dry_run,
                            coordinator=entries[0].address())
    import torch
    n = a.nproc or max(1, torch.cuda.device_count())
    backend = resolve_backend(a.backend, torch.cuda.is_available())
    return launch(cmd, n, backend, a.coordinator, a.port, parse_env_args(a.env))


if __name__ == "__main__":
    sys.exit(main())
