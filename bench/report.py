"""Markdown tables from the recorded benchmark lines (one JSON line of `bench.py` per GPU count).

  python bench/report.py bench/results/bench_1xB200.json bench/results/bench_2xB200.json \\
         bench/results/bench_4xB200.json bench/results/bench_8xB200.json

Per workload and GPU count: fused p50 / cuBLAS+NCCL p50 (speed-up), and the roofline fraction at the
largest GPU count; then the step times with the strong-scaling efficiency relative to the smallest
GPU count present. Files that carry a `note` have it printed under the table.
"""
from __future__ import annotations

import json
import sys
from typing import Dict, List


def load(paths: List[str]) -> Dict[int, Dict]:
    runs = {}
    for p in paths:
        with open(p) as fh:
            text = fh.read().strip()
        line = json.loads(text if text.startswith("{") and "\n{" not in text else text.splitlines()[-1])
        runs[int(line["n_gpus"])] = line
    return dict(sorted(runs.items()))


def tables(runs: Dict[int, Dict]) -> str:
    ns = list(runs)
    names: List[str] = []
    for r in runs.values():
        for k in r.get("ops", {}):
            if k not in names:
                names.append(k)
    head = "| workload | " + " | ".join(f"{n} GPU" + ("s" if n > 1 else "") for n in ns) + f" | of roofline @{ns[-1]} |"
    lines = [head, "|---|" + "---|" * (len(ns) + 1)]
    for name in names:
        cells = []
        for n in ns:
            op = runs[n].get("ops", {}).get(name)
            if not op or op.get("fused_p50_ms") is None:
                cells.append("-")
                continue
            base, sp = op.get("cublas_nccl_p50_ms"), op.get("speedup_vs_cublas_nccl")
            cells.append(f"{op['fused_p50_ms']:.3f}" + (f" / {base:.3f} ({sp:.2f})" if base is not None else ""))
        frac = runs[ns[-1]].get("ops", {}).get(name, {}).get("roofline_frac")
        lines.append(f"| {name} | " + " | ".join(cells) + f" | {frac if frac is not None else '-'} |")
    out = ["Fused p50 ms / cuBLAS+NCCL p50 ms (speed-up):", ""] + lines + [""]
    base_n = ns[0]
    t0 = runs[base_n]["ms_per_step"]
    out += ["| GPUs | ms per step | end to end ms | strong-scaling efficiency | SM MHz (median) | throttle reasons |",
            "|---|---|---|---|---|---|"]
    for n in ns:
        r = runs[n]
        eff = t0 * base_n / (r["ms_per_step"] * n)
        e2e = r.get("e2e", {}).get("value", "-")
        ck = r.get("clocks", {})
        out.append(f"| {n} | {r['ms_per_step']:.3f} | {e2e} | {eff:.2f} | {ck.get('sm_mhz', '-')} | "
                   f"{', '.join(ck.get('reasons', [])) or '-'} |")
    notes = [f"* {n} GPUs: {r['note']}" for n, r in runs.items() if r.get("note")]
    if notes:
        out += [""] + notes
    return "\n".join(out) + "\n"


def main():
    if len(sys.argv) < 2:
        sys.exit(__doc__)
    print(tables(load(sys.argv[1:])))


if __name__ == "__main__":
    main()
