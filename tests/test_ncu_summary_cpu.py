"""bench/ncu_summary.py on a synthetic raw-page CSV (no ncu, no GPU needed)."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

CSV = '''==PROF== banner line that is not CSV
"ID","Kernel Name","gpu__time_duration.sum","dram__bytes_read.sum","dram__bytes_write.sum","sm__pipe_tensor_cycles_active.avg.pct_of_peak_sustained_elapsed"
"","","us","Mbyte","Mbyte","%"
"0","my_kernel(int)","500.0","300.0","100.0","80.5"
"1","my_kernel(int)","250.0","","","40.0"
'''


def test_parse_and_derive():
    from bench.ncu_summary import read_raw_csv, summarize
    launches = read_raw_csv(CSV)
    assert len(launches) == 2
    assert launches[0]["gpu__time_duration.sum"] == {"value": "500.0", "unit": "us"}
    peaks = {"bf16_tflops": 1600.0, "hbm_gbs": 6400.0, "source": "measured"}
    md = summarize(launches, "t", "ncu ... python x.py", flops=4e11, nbytes=2e8, peaks=peaks)
    assert "# ncu summary: t" in md and "    ncu ... python x.py" in md
    assert "| sm__pipe_tensor_cycles_active.avg.pct_of_peak_sustained_elapsed | % | 80.5 |" in md
    # 4e11 FLOP in 500 us = 800 TFLOP/s = 0.50 of 1600; 400 MB in 500 us = 800 GB/s = 0.12 of 6400; 2.00x of 200 MB
    assert "800 TFLOP/s under the profiler = 0.50 of measured" in md
    assert "DRAM traffic 400 MB = 800 GB/s = 0.12 of measured" in md
    assert "2.00x the algorithmic bytes (200 MB)" in md
    # the second launch has no DRAM counters: only the FLOP line is derived for it
    assert md.count("DRAM traffic") == 1 and md.count("TFLOP/s under the profiler") == 2


def test_fallback_wording():
    from bench.ncu_summary import read_raw_csv, summarize
    peaks = {"bf16_tflops": 1590.0, "hbm_gbs": 6650.0, "source": "fallback"}
    md = summarize(read_raw_csv(CSV)[:1], "t", "c", flops=1e11, peaks=peaks)
    assert "of fallback" in md and "of measured" not in md


def test_report_tables_from_recorded_lines(tmp_path):
    import json
    from bench.report import load, tables
    runs = {}
    for n, ms in ((1, 32.0), (8, 8.0)):
        line = {"n_gpus": n, "ms_per_step": ms, "e2e": {"value": 2 * ms}, "clocks": {"sm_mhz": 1400.0, "reasons": []},
                "ops": {"ag_gemm": {"fused_p50_ms": ms / 8, "cublas_nccl_p50_ms": ms / 7, "speedup_vs_cublas_nccl": 8 / 7,
                                    "roofline_frac": 0.7}}}
        p = tmp_path / f"b{n}.json"
        p.write_text("log line\n" + json.dumps(line) + "\n")          # a log with the JSON line last also loads
        runs[n] = str(p)
    md = tables(load(list(runs.values())))
    assert "| ag_gemm | 4.000 / 4.571 (1.14) | 1.000 / 1.143 (1.14) | 0.7 |" in md
    assert "| 8 | 8.000 | 16.0 | 0.50 | 1400.0 | - |" in md           # 32 ms on 1 GPU -> 8 ms on 8: efficiency 0.5
