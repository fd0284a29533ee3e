"""Device-side timing helpers (CUDA events, max over ranks, L2 flush, clock sampling).

The reference times with per-iteration event pairs after warm-up and reports
mean / p50 / min (bench/s4_bench.py:59-83); the same scheme is used here, with
the cross-rank maximum taken for every multi-GPU number.
"""
from __future__ import annotations

import statistics
import subprocess
import threading
import time
from typing import Callable, Dict, List, Optional

import torch
import torch.distributed as dist

_flush_buf: Optional[torch.Tensor] = None


def flush_l2(nbytes: int = 256 << 20) -> None:
    """Evict L2 (126 MB on B200) by overwriting a larger buffer."""
    global _flush_buf
    if _flush_buf is None or _flush_buf.numel() < nbytes:
        _flush_buf = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    _flush_buf.zero_()


def max_over_ranks(values: List[float], group=None) -> List[float]:
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return list(values)
    t = torch.tensor(values, dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return t.tolist()


def time_op(fn: Callable[[], None], iters: int = 20, warmup: int = 3, flush: bool = True,
            group=None, barrier: Optional[Callable[[], None]] = None) -> Dict[str, float]:
    """Per-iteration event pairs; returns mean / p50 / min in ms, each the max over ranks."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    # All iterations are enqueued back to back and synchronised once, so that host-side
    # launch latency hides behind the flush / barrier of the same iteration instead of
    # showing up inside the event interval.
    pairs = []
    for _ in range(iters):
        if flush:
            flush_l2()
        if barrier is not None:
            barrier()
        e0 = torch.cuda.Event(enable_timing=True)
        e1 = torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        pairs.append((e0, e1))
    torch.cuda.synchronize()
    times = [a.elapsed_time(b) for a, b in pairs]
    times = max_over_ranks(times, group)
    return {"mean": statistics.fmean(times), "p50": statistics.median(times), "min": min(times),
            "iters": iters}


def time_pair(fn_a: Callable[[], None], fn_b: Callable[[], None], iters: int = 20, warmup: int = 3,
              flush: bool = True, group=None, barrier: Optional[Callable[[], None]] = None):
    """Times two implementations of one operator in alternation (A, B, A, B, ...), each call behind
    its own L2 flush and device barrier: both see the same clocks and power state, which a
    power-capped GPU does not give to two loops run one after the other. Returns the two
    ``time_op``-style dictionaries."""
    for _ in range(warmup):
        fn_a()
        fn_b()
    torch.cuda.synchronize()
    pairs = ([], [])
    for _ in range(iters):
        for which, fn in enumerate((fn_a, fn_b)):
            if flush:
                flush_l2()
            if barrier is not None:
                barrier()
            e0 = torch.cuda.Event(enable_timing=True)
            e1 = torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            pairs[which].append((e0, e1))
    torch.cuda.synchronize()
    out = []
    for which in range(2):
        times = max_over_ranks([a.elapsed_time(b) for a, b in pairs[which]], group)
        out.append({"mean": statistics.fmean(times), "p50": statistics.median(times), "min": min(times),
                    "iters": iters})
    return out[0], out[1]


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region runs (read-only)."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int = 0, period_ms: int = 50):
        self.gpu_index = gpu_index
        self.period_ms = period_ms
        self.lines: List[str] = []
        self.stamps: List[float] = []      # host arrival time of each line (time.monotonic)
        self._proc = None
        self._thr = None

    def start(self) -> None:
        try:
            self._proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-i", str(self.gpu_index), "-lms", str(self.period_ms)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self._proc = None
            return

        def pump():
            for line in self._proc.stdout:
                self.stamps.append(time.monotonic())
                self.lines.append(line.strip())

        self._thr = threading.Thread(target=pump, daemon=True)
        self._thr.start()

    def stop(self, window: Optional[tuple] = None) -> Dict:
        """Stop sampling and summarise. ``window`` = (t0, t1) in ``time.monotonic()`` seconds keeps
        only the samples that arrived inside it (the timed region); if the region was too short to
        catch one, all samples since ``start()`` are used (start the sampler before the warm-up, so
        that these were taken under the same load) and ``"window"`` says so."""
        if self._proc is not None:
            self._proc.terminate()
            try:
                self._proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self._proc.kill()
            if self._thr is not None:
                self._thr.join(timeout=2)
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        lines, where = self.lines, "all samples"
        if window is not None:
            inside = [ln for ln, ts in zip(self.lines, self.stamps) if window[0] <= ts <= window[1] + 0.05]
            if inside:
                lines, where = inside, "timed region"
            else:
                where = "warm-up + timed region (timed region shorter than one sampling period)"
        for line in lines:
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm), "window": where}
