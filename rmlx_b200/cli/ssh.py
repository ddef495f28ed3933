"""Remote spawning for multi-host launches: quoting, target validation, command construction and a
bounded ``run_remote``. Mirrors crates/rmlx-cli/src/ssh.rs (``shell_quote``, option-injection-safe
target validation, ``run_remote`` with timeout, ``spawn_remote``). The fused kernels need all ranks
on one NVLink domain; a multi-host launch is for the library (NCCL) backend and for bring-up tools.
"""
from __future__ import annotations

import re
import subprocess
from typing import Dict, List, Optional, Sequence

_TARGET = re.compile(r"^(?:[A-Za-z_][A-Za-z0-9_.-]*@)?[A-Za-z0-9][A-Za-z0-9_.:-]*$")
SSH_OPTIONS = ["-o", "BatchMode=yes", "-o", "StrictHostKeyChecking=accept-new", "-o", "ConnectTimeout=5"]


def shell_quote(s: str) -> str:
    """Single-quote ``s`` for a POSIX shell (``'`` becomes ``'\\''``); safe strings pass unchanged."""
    if s and re.fullmatch(r"[A-Za-z0-9_@%+=:,./-]+", s):
        return s
    return "'" + s.replace("'", "'\\''") + "'"


def validate_target(target: str) -> str:
    """``[user@]host`` only: nothing that ssh could read as an option, no whitespace, no shell
    metacharacters."""
    if not _TARGET.match(target) or target.startswith("-") or "@-" in target:
        raise ValueError(f"invalid ssh target {target!r}")
    return target


def remote_command(cmd: Sequence[str], env: Optional[Dict[str, str]] = None,
                   cwd: Optional[str] = None) -> str:
    """The single string handed to the remote shell: ``cd``, exported variables, quoted command."""
    parts: List[str] = []
    if cwd:
        parts.append(f"cd {shell_quote(cwd)} &&")
    for k, v in sorted((env or {}).items()):
        if not re.fullmatch(r"[A-Za-z_][A-Za-z0-9_]*", k):
            raise ValueError(f"invalid environment variable name {k!r}")
        parts.append(f"{k}={shell_quote(v)}")
    parts += [shell_quote(c) for c in cmd]
    return " ".join(parts)


def ssh_argv(target: str, cmd: Sequence[str], env: Optional[Dict[str, str]] = None,
             cwd: Optional[str] = None) -> List[str]:
    return ["ssh", *SSH_OPTIONS, "--", validate_target(target), remote_command(cmd, env, cwd)]


def run_remote(target: str, cmd: Sequence[str], timeout_s: float = 10.0, runner=subprocess.run):
    """Run ``cmd`` on ``target`` and wait at most ``timeout_s``. Returns (exit code, stdout, stderr);
    a timeout is reported as exit code 124."""
    try:
        r = runner(ssh_argv(target, cmd), capture_output=True, text=True, timeout=timeout_s)
        return r.returncode, r.stdout, r.stderr
    except subprocess.TimeoutExpired:
        return 124, "", f"timed out after {timeout_s} s"


def spawn_remote(target: str, cmd: Sequence[str], env: Optional[Dict[str, str]] = None,
                 cwd: Optional[str] = None, popen=subprocess.Popen):
    return popen(ssh_argv(target, cmd, env, cwd), stdout=subprocess.PIPE, stderr=subprocess.STDOUT,
                 text=True, bufsize=1, start_new_session=True)


def plan_ranks(hosts: Sequence[str], per_host: int) -> List[tuple]:
    """(host, global rank, local slot) for ``per_host`` ranks on each host, hosts in the given order."""
    out = []
    for h_i, h in enumerate(hosts):
        validate_target(h)
        for s in range(per_host):
            out.append((h, h_i * per_host + s, s))
    return out
