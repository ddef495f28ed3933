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


def test_plan_matches_the_loaders_sharding_and_the_real_weights():
    """``rmlx plan``: the analytic weight bytes equal what the loader builds for a small model at
    TP 1 and 2 (sliced and partitioned experts, 4-bit and bf16); the 60-layer model's headline
    facts (bf16 does not fit one GPU, 4-bit does; KV bytes per token) and the CLI exit codes."""
    import torch
    from rmlx_b200.cli import plan as P
    from rmlx_b200.cli.main import main as cli_main
    from rmlx_b200.config import FeedForwardType, MoeConfig, TransformerConfig
    from rmlx_b200.models.weights import ParallelLayout, from_state_dict, random_state_dict
    moe = MoeConfig(num_experts=4, num_experts_per_token=2, hidden_dim=128, intermediate_dim=128)
    cfg = TransformerConfig(hidden_size=128, num_heads=4, num_kv_heads=2, head_dim=32, num_layers=2,
                            vocab_size=512, max_seq_len=128, ff_type=FeedForwardType.moe_(moe), name="tiny").validate()
    sd = random_state_dict(cfg, 0)
    for quant, fmt in ((None, "bf16"), ("q4", "q4")):
        for tp, ep in ((1, False), (2, False), (2, True)):
            w = from_state_dict(cfg, sd, dtype=torch.bfloat16, quant=quant, layout=ParallelLayout(0, tp, ep))
            parts = P.weight_bytes_per_gpu(cfg, fmt, tp, ep)
            # ModelWeights.nbytes counts the projections, embedding and LM head (not norms / router)
            want = parts["total"] - parts["norms"] - cfg.num_layers * moe.num_experts * cfg.hidden_size * 2
            assert w.nbytes() == want, (fmt, tp, ep, w.nbytes(), want)
    big = P.plan("moe-a22b", "bf16", tp=1)
    assert not big["fits"] and 295e9 < big["weight_bytes_per_gpu"]["total"] < 305e9
    q4 = P.plan("moe-a22b", "q4", tp=1, batch=1, ctx=4096)
    assert q4["fits"] and q4["kv_bytes_per_token_per_gpu"] == 60 * 2 * 4 * 128 * 2
    assert q4["kv_tokens_that_fit"] > 500_000
    assert P.plan("moe-a22b", "q4", tp=8)["kv_bytes_per_token_per_gpu"] == 60 * 2 * 1 * 128 * 2   # kv heads replicated
    assert P.kv_bytes_per_token_per_gpu(P.presets()["moe-a22b"], 1, "q8") == int(60 * 2 * 4 * 128 * (1 + 4 / 64))
    if q4["decode_stream_plans"]:                                    # the library is there: plans are filled in
        assert q4["decode_stream_plans"]["qkv"]["supported"] and q4["decode_stream_plans"]["qkv"]["blocks"] <= 148
    assert P.plan("moe-a22b", "q4", batch=64)["decode_stream_plans"] == {}
    roof = P.decode_roofline(P.presets()["moe-a22b"], "q4", 1, 4096, hbm_gbs=6533.0)
    assert 20.0 < roof["us_per_layer"] < 21.0 and 750 < roof["tokens_per_s"] < 810     # the 20.6 us of bytes per layer
    assert P.decode_roofline(P.presets()["moe-a22b"], "q4", 8, 4096, hbm_gbs=6533.0)["us_per_layer"] < 0.2 * roof["us_per_layer"]
    assert "DOES NOT FIT" in P.render(big) and "fits" in P.render(q4)
    assert cli_main(["plan", "--weights", "q4"]) == 0 and cli_main(["plan", "--weights", "bf16"]) == 1
    ds8, ds2 = P.plan("deepseek-v3", "q4", tp=8, batch=8, ctx=32768), P.plan("deepseek-v3", "q4", tp=2)
    assert ds8["fits"] and not ds2["fits"] and ds8["kv_compression"] > 50
    w8 = ds8["weight_bytes_per_gpu"]
    quantised = 8 * w8["routed_experts"] + w8["attention"] + w8["dense_layers"] + w8["lm_head"] + \
        w8["shared_experts_and_router"] - 60 * 256 * 7168 * 2        # the routers stay bf16
    params = quantised / (4.5 / 8) + (w8["embedding"] + 60 * 256 * 7168 * 2) / 2
    # this preset keeps ONE leading dense layer (the released model has three): 60 x 256 routed experts
    assert 685e9 < params < 700e9
    assert ds8["kv_bytes_per_token_per_gpu"] == 61 * (512 + 64 + 8) * 2 and "latent cache" in P.render(ds8)
