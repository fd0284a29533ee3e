"""Turn an Nsight Compute report into the short text summary kept under ``profiles/``.

  ncu --set full --clock-control none -k regex:fused_gemm_kernel -c 1 -o prof_gemm \\
      python bench/probe_gemm.py --shapes "8192,8192,4096" --once          # on the GPU box, small case
  python bench/ncu_summary.py prof_gemm.ncu-rep --title "fused_gemm_kernel, plain 8192x8192x4096 bf16" \\
      --command 'ncu --set full ... python bench/probe_gemm.py --shapes "8192,8192,4096" --once' \\
      --flops 549755813888 --bytes 268435456 --out profiles/fused_gemm_plain_8192x8192x4096.md

Reads the report with ``ncu -i <report> --page raw --csv`` (works without a GPU), or a CSV exported
that way (``--csv``). Per captured launch it lists the handful of counters that decide where a kernel
stands (duration, tensor-pipe activity, DRAM bytes and throughput, L2 hit rate, occupancy, the
dominant warp stalls) and, when the algorithmic FLOPs / bytes of the launch are given, the achieved
rates against the measured peaks of this machine pool (``MEASURED_PEAKS.json``; a stated fallback
otherwise). Numbers under a profiler are for shares and counters, never benchmark values.
"""
from __future__ import annotations

import argparse
import csv
import io
import os
import subprocess
import sys
from typing import Dict, List, Optional

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

METRICS = [
    "gpu__time_duration.sum",
    "launch__grid_size",
    "launch__cluster_size",
    "launch__block_size",
    "launch__registers_per_thread",
    "sm__pipe_tensor_cycles_active.avg.pct_of_peak_sustained_elapsed",
    "sm__pipe_tensor_cycles_active.avg.pct_of_peak_sustained_active",
    "sm__throughput.avg.pct_of_peak_sustained_elapsed",
    "dram__bytes_read.sum",
    "dram__bytes_write.sum",
    "gpu__dram_throughput.avg.pct_of_peak_sustained_elapsed",
    "lts__t_sector_hit_rate.pct",
    "lts__throughput.avg.pct_of_peak_sustained_elapsed",
    "l1tex__m_xbar2l1tex_read_bytes.sum.per_second",
    "sm__warps_active.avg.per_cycle_active",
    "sm__cycles_elapsed.avg.per_second",
    "smsp__average_warps_issue_stalled_barrier_per_issue_active.ratio",
    "smsp__average_warps_issue_stalled_long_scoreboard_per_issue_active.ratio",
    "smsp__average_warps_issue_stalled_wait_per_issue_active.ratio",
    "smsp__average_warps_issue_stalled_lg_throttle_per_issue_active.ratio",
]

_TO_BYTES = {"byte": 1.0, "Kbyte": 1e3, "Mbyte": 1e6, "Gbyte": 1e9, "Tbyte": 1e12}
_TO_SECONDS = {"ns": 1e-9, "us": 1e-6, "ms": 1e-3, "s": 1.0, "nsecond": 1e-9, "usecond": 1e-6, "msecond": 1e-3,
               "second": 1.0}


def read_raw_csv(text: str) -> List[Dict[str, Dict[str, str]]]:
    """Rows of ``--page raw --csv`` as ``{metric: {"value": .., "unit": ..}}`` per captured launch."""
    rows = [r for r in csv.reader(io.StringIO(text)) if r]
    start = next((i for i, r in enumerate(rows) if "Kernel Name" in r), None)
    if start is None or len(rows) < start + 3:
        return []
    hdr, units = rows[start], rows[start + 1]
    out = []
    for r in rows[start + 2:]:
        if len(r) != len(hdr):
            continue
        out.append({h: {"value": v, "unit": u} for h, v, u in zip(hdr, r, units)})
    return out


def _num(cell: Optional[Dict[str, str]]) -> Optional[float]:
    if not cell or cell["value"] in ("", "n/a"):
        return None
    try:
        return float(cell["value"].replace(",", ""))
    except ValueError:
        return None


def derived(launch: Dict[str, Dict[str, str]], flops: float, nbytes: float, peaks: Dict) -> List[str]:
    """Achieved rates of one launch against the machine's measured peaks."""
    lines = []
    dur = _num(launch.get("gpu__time_duration.sum"))
    if dur is None:
        return lines
    secs = dur * _TO_SECONDS.get(launch["gpu__time_duration.sum"]["unit"], 1e-9)
    tag = "of measured" if peaks.get("source") == "measured" else "of fallback"
    if flops > 0:
        tf = flops / secs / 1e12
        lines.append(f"* {tf:.0f} TFLOP/s under the profiler = {tf / peaks['bf16_tflops']:.2f} {tag} "
                     f"cuBLAS bf16 burst ({peaks['bf16_tflops']:.0f} TFLOP/s)")
    rd, wr = launch.get("dram__bytes_read.sum"), launch.get("dram__bytes_write.sum")
    if _num(rd) is not None and _num(wr) is not None:
        traffic = _num(rd) * _TO_BYTES.get(rd["unit"], 1.0) + _num(wr) * _TO_BYTES.get(wr["unit"], 1.0)
        gbs = traffic / secs / 1e9
        lines.append(f"* DRAM traffic {traffic / 1e6:.0f} MB = {gbs:.0f} GB/s = {gbs / peaks['hbm_gbs']:.2f} {tag} "
                     f"copy bandwidth ({peaks['hbm_gbs']:.0f} GB/s)")
        if nbytes > 0:
            lines.append(f"* {traffic / nbytes:.2f}x the algorithmic bytes ({nbytes / 1e6:.0f} MB)")
    return lines


def summarize(launches: List[Dict[str, Dict[str, str]]], title: str, command: str, flops: float = 0.0,
              nbytes: float = 0.0, peaks: Optional[Dict] = None) -> str:
    if peaks is None:
        from tridist_b200.utils.roofline import load_peaks
        peaks = load_peaks()
    lines = [f"# ncu summary: {title}", "", "Command (one GPU, after the same command exited 0 without ncu):", "",
             f"    {command}", "",
             "Read with `ncu -i <report> --page raw --csv`; clocks not locked (`--clock-control none`), cold cache, "
             "serialised passes: use the shares and counters, not the duration, as a benchmark.", ""]
    for launch in launches:
        name = launch.get("Kernel Name", {}).get("value", "?")
        lines += [f"## {name[:100]}", "", "| metric | unit | value |", "|---|---|---|"]
        for m in METRICS:
            cell = launch.get(m)
            if cell and cell["value"] != "":
                lines.append(f"| {m} | {cell['unit']} | {cell['value']} |")
        lines.append("")
        lines += derived(launch, flops, nbytes, peaks)
        lines.append("")
    return "\n".join(lines).rstrip("\n") + "\n"


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("report", help=".ncu-rep file, or with --csv the exported raw page")
    ap.add_argument("--csv", action="store_true")
    ap.add_argument("--title", required=True)
    ap.add_argument("--command", required=True, help="the full command that made the report")
    ap.add_argument("--flops", type=float, default=0.0, help="algorithmic FLOPs of one captured launch")
    ap.add_argument("--bytes", type=float, default=0.0, help="algorithmic bytes of one captured launch")
    ap.add_argument("--out", default="")
    args = ap.parse_args()
    if args.csv:
        with open(args.report) as fh:
            text = fh.read()
    else:
        text = subprocess.run(["ncu", "-i", args.report, "--page", "raw", "--csv"], capture_output=True, text=True,
                              check=True).stdout
    launches = read_raw_csv(text)
    if not launches:
        sys.exit("no captured launch found in the report")
    md = summarize(launches, args.title, args.command, args.flops, args.bytes)
    if args.out:
        with open(args.out, "w") as fh:
            fh.write(md)
    print(md)


if __name__ == "__main__":
    main()
