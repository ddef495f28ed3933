"""Launcher logic (crates/rmlx-cli/src/launch.rs:422-457 style): env contract, argument
validation, output prefixing, fail-fast."""
import io
import sys

import pytest

from rmlx_b200.cli.main import build_env, launch, parse_env_args, resolve_backend


def test_env_contract_and_validation():
    e = build_env(2, 4, "nccl", "127.0.0.1", 18520, {"X": "1"})
    assert e["RMLX_RANK"] == "2" and e["RMLX_WORLD_SIZE"] == "4" and e["LOCAL_RANK"] == "2"
    assert e["MASTER_PORT"] == "18520" and e["RMLX_BACKEND"] == "nccl" and e["X"] == "1"
    assert parse_env_args(["A=1", "B_C=x=y"]) == {"A": "1", "B_C": "x=y"}
    for bad in ("novalue", "=x", "a;b=1"):
        with pytest.raises(ValueError):
            parse_env_args([bad])
    assert resolve_backend("auto", False) == "gloo" and resolve_backend("auto", True) == "nccl"
    with pytest.raises(ValueError):
        resolve_backend("tb5", True)


def test_launch_prefixes_output_and_fails_fast():
    out = io.StringIO()
    rc = launch([sys.executable, "-c", "import os; print('hi', os.environ['RMLX_RANK'])"], 3,
                backend="gloo", port=18999, sink=out)
    assert rc == 0
    lines = sorted(out.getvalue().splitlines())
    assert lines == ["[rank=0] hi 0", "[rank=1] hi 1", "[rank=2] hi 2"]
    out = io.StringIO()
    prog = ("import os,sys,time\n"
            "r=int(os.environ['RMLX_RANK'])\n"
            "sys.exit(3) if r==1 else time.sleep(60)\n")
    import time
    t0 = time.time()
    rc = launch([sys.executable, "-c", prog], 3, backend="gloo", port=18998, sink=out)
    assert rc == 1 and time.time() - t0 < 20
    assert "rank 1 exited with 3" in out.getvalue()


def test_hostfile_schema_round_trip_and_launch_plan(tmp_path):
    import io
    import json
    from rmlx_b200.cli import main as cli
    from rmlx_b200.cli.hostfile import (HostEntry, load_host_entries, resolve_hosts,
                                        save_host_entries)
    path = str(tmp_path / "hosts.json")
    save_host_entries(path, [HostEntry("user@node0", ["10.0.0.1"], 2, True), HostEntry("node1")])
    entries = load_host_entries(path)
    assert [e.ssh for e in entries] == ["user@node0", "node1"]
    assert entries[0].address() == "10.0.0.1" and entries[1].address() == "node1"
    assert entries[0].gpus == 2 and entries[1].gpus is None
    assert [e.ssh for e in resolve_hosts("a,b", None)] == ["a", "b"]
    for bad in ([], [{"ips": []}], [{"ssh": "-oProxyCommand=x"}], [{"ssh": "n", "gpus": 0}],
                [{"ssh": "n", "rdma": []}]):
        with open(path, "w") as f:
            json.dump(bad, f)
        with pytest.raises(ValueError):
            load_host_entries(path)
    with pytest.raises(ValueError):
        resolve_hosts("a", path)
    with pytest.raises(ValueError):
        resolve_hosts(None, None)
    # the launcher takes the ranks per host and the coordinator address from the file
    save_host_entries(path, [HostEntry("user@node0", ["10.0.0.1"], 2), HostEntry("node1", [], 2)])
    buf = io.StringIO()
    entries = load_host_entries(path)
    rc = cli.launch_hosts(["python", "x.py"], [e.ssh for e in entries], 2, sink=buf, dry_run=True,
                          coordinator=entries[0].address())
    lines = buf.getvalue().strip().splitlines()
    assert rc == 0 and len(lines) == 4
    assert all("MASTER_ADDR=10.0.0.1" in ln for ln in lines) and "node1" in lines[2]
