"""Markdown tables from the recorded benchmark lines (one JSON line of `bench.py` per GPU count).

  python bench/report.py bench/results/bench_1xB200.json bench/results/bench_2xB200.json \\
         bench/results/bench_4xB200.json bench/results/bench_8xB200.json

Per workload and GPU count: fused p50 / cuBLAS+NCCL p50 (speed-up), and the roofline fraction at the
largest GPU count; then the step times with the strong-scaling efficiency relative to the smallest
GPU count present. Files that carry a `note` have it printed under the table.

`--override FILE` (repeatable) takes the per-operator cells that FILE holds (a `bench.py --ops ...` line of
the same GPU count) in place of those of the full run and marks them with a dagger: a transport or knob
that was measured separately, in the same call, shows up in the table without touching the recorded lines.

  python bench/report.py bench/results/bench_{1,2,4,8}xB200.json \\
         --override bench/results/bench_4xB200_ag_push.json --override bench/results/bench_8xB200_ag_push.json
"""
from __future__ import annotations

import json
import math
import sys
from typing import Dict, List


def _read(p: str) -> Dict:
    with open(p) as fh:
        text = fh.read().strip()
    return json.loads(text if text.startswith("{") and "\n{" not in text else text.splitlines()[-1])


def load(paths: List[str], overrides: List[str] = ()) -> Dict[int, Dict]:
    runs = {}
    for p in paths:
        line = _read(p)
        runs[int(line["n_gpus"])] = line
    for p in overrides:
        line = _read(p)
        n = int(line["n_gpus"])
        if n not in runs:
            continue
        for name, cell in line.get("ops", {}).items():
            runs[n].setdefault("ops", {})[name] = dict(cell, overridden=True)
        sps = [c["speedup_vs_cublas_nccl"] for c in runs[n]["ops"].values() if "speedup_vs_cublas_nccl" in c]
        if sps:
            runs[n]["vs_baseline"] = round(math.exp(sum(math.log(x) for x in sps) / len(sps)), 3)
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
            cells.append(f"{op['fused_p50_ms']:.3f}" + (f" / {base:.3f} ({sp:.2f})" if base is not None else "")
                         + (" †" if op.get("overridden") else ""))
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
    args = sys.argv[1:]
    overrides = []
    while "--override" in args:
        i = args.index("--override")
        overrides.append(args[i + 1])
        del args[i:i + 2]
    if not args:
        sys.exit(__doc__)
    print(tables(load(args, overrides)))


if __name__ == "__main__":
    main()
