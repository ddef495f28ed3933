#!/usr/bin/env python
"""Short text summaries of Nsight Compute reports: per captured launch the duration, DRAM traffic and
throughput, tensor-pipe and special-function-pipe activity, occupancy, registers, and the warp stall
reasons that dominate. A report condenser for the benchmark scripts beside it, not a capture API.

    ncu --set full --clock-control none -k regex:<kernel> -c 3 -o report <command>
    python benchmarks/ncu_summary.py report.ncu-rep        # needs `ncu` on PATH, no GPU
    ncu -i report.ncu-rep --page raw --csv | python benchmarks/ncu_summary.py -
"""
from __future__ import annotations

import csv
import subprocess
import sys
from dataclasses import dataclass, field
from typing import Dict, List, Tuple

# (metric name in the raw page, label in the summary)
METRICS: List[Tuple[str, str]] = [
    ("gpu__time_duration.sum", "time"),
    ("dram__bytes_read.sum", "dram read"),
    ("dram__bytes_write.sum", "dram write"),
    ("gpu__dram_throughput.avg.pct_of_peak_sustained_elapsed", "dram throughput %"),
    ("sm__pipe_tensor_cycles_active.avg.pct_of_peak_sustained_active", "tensor pipe active %"),
    ("sm__inst_executed_pipe_xu.avg.pct_of_peak_sustained_active", "xu pipe %"),
    ("sm__inst_executed_pipe_alu.avg.pct_of_peak_sustained_active", "alu pipe %"),
    ("sm__inst_executed_pipe_fma.avg.pct_of_peak_sustained_active", "fma pipe %"),
    ("smsp__issue_active.avg.pct_of_peak_sustained_active", "issue active %"),
    ("sm__warps_active.avg.pct_of_peak_sustained_active", "warps active %"),
    ("launch__registers_per_thread", "regs/thread"),
    ("launch__grid_size", "grid"),
    ("launch__block_size", "block"),
    ("launch__shared_mem_per_block_dynamic", "dyn smem"),
    ("lts__t_sector_hit_rate.pct", "L2 hit %"),
]
_STALL_PREFIX = "smsp__average_warps_issue_stalled_"
_STALL_SUFFIX = "_per_issue_active.ratio"


@dataclass
class LaunchSummary:
    kernel: str
    values: Dict[str, Tuple[str, str]] = field(default_factory=dict)     # label -> (value, unit)
    stalls: List[Tuple[float, str]] = field(default_factory=list)        # (warps per issue, reason)

    def number(self, label: str) -> float:
        return float(self.values[label][0].replace(",", ""))

    def render(self, top_stalls: int = 5, name_width: int = 60) -> str:
        parts = [f"kernel: {self.kernel[:name_width]}"]
        parts += [f"{label}: {v} {u}".strip() for label, (v, u) in self.values.items()]
        stalls = ", ".join(f"{n}={v:.2f}" for v, n in self.stalls[:top_stalls])
        return "; ".join(parts) + f"\n   top stalls (warps per issue): {stalls}"


def parse_raw_csv(text: str) -> List[LaunchSummary]:
    """Summaries from the output of ``ncu -i <report> --page raw --csv`` (header row, unit row, then
    one row per captured launch). Lines before the header (profiler banners) are skipped."""
    lines = text.splitlines()
    start = next((i for i, l in enumerate(lines) if l.startswith('"ID"') or l.startswith("ID,")), 0)
    rows = list(csv.reader(lines[start:]))
    if len(rows) < 3:
        return []
    hdr, units = rows[0], rows[1]
    out: List[LaunchSummary] = []
    for vals in rows[2:]:
        if len(vals) != len(hdr):
            continue
        d = {h: (v, u) for h, v, u in zip(hdr, vals, units)}
        s = LaunchSummary(d.get("Kernel Name", ("?", ""))[0])
        for key, label in METRICS:
            if key in d and d[key][0] not in ("", "n/a"):
                s.values[label] = d[key]
        for h, (v, _) in d.items():
            if h.startswith(_STALL_PREFIX) and h.endswith(_STALL_SUFFIX):
                try:
                    s.stalls.append((float(v.replace(",", "")), h[len(_STALL_PREFIX):-len(_STALL_SUFFIX)]))
                except ValueError:
                    pass
        s.stalls.sort(reverse=True)
        out.append(s)
    return out


def summarize_report(path: str) -> List[LaunchSummary]:
    """Run ``ncu -i`` on a ``.ncu-rep`` file (no GPU needed) and parse its raw page."""
    res = subprocess.run(["ncu", "-i", path, "--page", "raw", "--csv"], capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"ncu could not read {path}: {res.stderr.strip()[:200]}")
    return parse_raw_csv(res.stdout)


def main(argv=None) -> int:
    argv = sys.argv[1:] if argv is None else argv
    if len(argv) != 1:
        print(__doc__)
        return 2
    launches = parse_raw_csv(sys.stdin.read()) if argv[0] == "-" else summarize_report(argv[0])
    for s in launches:
        print(s.render())
    return 0 if launches else 1


if __name__ == "__main__":
    sys.exit(main())
