"""TP-MLP layer benchmark: fused operators against their cuBLAS + NCCL composition.

Counterpart of the reference's bench/s21_bench_tp_mlp_dcu.py: the two layer modes
(``ag_rs``: AG+GEMM -> SwiGLU -> GEMM+RS, ``gemm_ar``: GEMM+AR -> SwiGLU -> GEMM+AR), the
same layer shapes (LLaMA-7B / LLaMA-3.1-70B / LLaMA-3.1-405B / Qwen2-72B) and the same
decode -> prefill sweep of M. Each cell is checked against an fp32 golden assembled from
all ranks' weights, timed (device events, max over ranks, p50) and appended to a JSON
file, one cell at a time (cells already present are skipped).

  python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 bench/bench_tp_mlp.py \
      --models LLaMA-3.1-70B --modes ag_rs,gemm_ar --ms 512,1024,2048,4096,8192 --out bench/results/tp_mlp.json
"""
from __future__ import annotations

import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402
import torch.nn.functional as F  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--models", default="LLaMA-3.1-70B")
    ap.add_argument("--modes", default="ag_rs")
    ap.add_argument("--ms", default="512,1024,2048,4096,8192")
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "fp16"])
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--out", default="")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", str(rank)))
    R = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(local_rank)
    if R > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", rank=rank, world_size=R, device_id=torch.device("cuda", local_rank))

    from tridist_b200.models.tp_mlp import LAYER_CONFIGS, TPMLP, TPMLPConfig
    from tridist_b200.parallel.runtime import init_runtime
    from tridist_b200.utils.timing import time_op

    rt = init_runtime(rank, R)
    dt = torch.bfloat16 if args.dtype == "bf16" else torch.float16
    results = {}
    if args.out and os.path.exists(args.out):
        with open(args.out) as fh:
            results = json.load(fh)

    def t(fn):
        return round(time_op(fn, iters=args.iters, warmup=3, flush=True, barrier=rt.barrier_on_stream)["p50"], 4)

    def gather(x, dim=0):
        if R == 1:
            return x
        parts = [torch.empty_like(x) for _ in range(R)]
        dist.all_gather(parts, x.contiguous())
        return torch.cat(parts, dim)

    for model in args.models.split(","):
        I, K = LAYER_CONFIGS[model]["I"], LAYER_CONFIGS[model]["K"]
        if (I // R) % 128 != 0 or I % R != 0:
            if rank == 0:
                print(f"skip {model}: intermediate/ranks = {I / R} is not 128-aligned", flush=True)
            continue
        i_loc = I // R
        for mode in args.modes.split(","):
            for M in [int(x) for x in args.ms.split(",")]:
                name = f"{mode}/{model}/M{M}/R{R}/{args.dtype}"
                if name in results or M % R != 0 or (mode == "ag_rs" and (M // R) % 128 != 0 and R > 1):
                    continue
                g = torch.Generator(device="cuda")
                g.manual_seed(7300 + rank)
                rnd = lambda *s, sc=1.0: (torch.randn(*s, generator=g, device="cuda") * sc).to(dt)  # noqa: E731
                w_down = rnd(K, i_loc, sc=0.02)
                if mode == "ag_rs":
                    x = rnd(M // R, K)
                    w_gu = rnd(2 * i_loc, K, sc=0.02)
                    # golden: rank-blocked [gate | up] shards, activation per shard
                    x_full = gather(x).float()
                    h = x_full @ w_gu.float().t()
                    part = (F.silu(h[:, :i_loc]) * h[:, i_loc:]) @ w_down.float().t()
                    if R > 1:
                        dist.all_reduce(part)
                    golden = part[rank * (M // R):(rank + 1) * (M // R)]
                    x_buf = torch.empty(M, K, dtype=dt, device="cuda")
                    h_buf = torch.empty(M, 2 * i_loc, dtype=dt, device="cuda")
                    p_buf = torch.empty(M, K, dtype=dt, device="cuda")
                    y_buf = torch.empty(M // R, K, dtype=dt, device="cuda")

                    def torch_e2e():
                        xf = x
                        if R > 1:
                            dist.all_gather_into_tensor(x_buf, x)
                            xf = x_buf
                        torch.matmul(xf, w_gu.t(), out=h_buf)
                        h2 = F.silu(h_buf[:, :i_loc]) * h_buf[:, i_loc:]
                        torch.matmul(h2, w_down.t(), out=p_buf)
                        if R > 1:
                            dist.reduce_scatter_tensor(y_buf, p_buf)
                            return y_buf
                        return p_buf
                else:
                    k_loc = K // R
                    x = rnd(M, k_loc)
                    w_gu = rnd(2 * I, k_loc, sc=0.02)       # global rank-blocked [gate | up] layout, K-sharded
                    h = x.float() @ w_gu.float().t()
                    if R > 1:
                        dist.all_reduce(h)
                    blk = h[:, rank * 2 * i_loc:(rank + 1) * 2 * i_loc]
                    part = (F.silu(blk[:, :i_loc]) * blk[:, i_loc:]) @ w_down.float().t()
                    if R > 1:
                        dist.all_reduce(part)
                    golden = part
                    h_buf = torch.empty(M, 2 * I, dtype=dt, device="cuda")
                    y_buf = torch.empty(M, K, dtype=dt, device="cuda")

                    def torch_e2e():
                        torch.matmul(x, w_gu.t(), out=h_buf)
                        if R > 1:
                            dist.all_reduce(h_buf)
                        b = h_buf[:, rank * 2 * i_loc:(rank + 1) * 2 * i_loc]
                        h2 = F.silu(b[:, :i_loc]) * b[:, i_loc:]
                        torch.matmul(h2, w_down.t(), out=y_buf)
                        if R > 1:
                            dist.all_reduce(y_buf)
                        return y_buf

                cell = {}
                if mode == "gemm_ar" and R * M * 2 * I >= 2 ** 31:
                    if rank == 0:
                        print(f"skip {name}: ranks * M * 2I exceeds the all-reduce context's 2^31 element limit", flush=True)
                    continue
                for fuse in ([True, False] if mode == "ag_rs" else [False]):
                    layer = TPMLP(TPMLPConfig(hidden=K, intermediate=I, max_tokens=M, dtype=dt, mode=mode,
                                              fuse_swiglu=fuse), rank, R, w_gu, w_down)
                    y = layer(x)
                    torch.cuda.synchronize()
                    rt.check()
                    key = "fused_swiglu_in_epilogue" if fuse else "fused"
                    cell[key + "_err"] = round((y.float() - golden).abs().max().item(), 4)
                    cell[key] = t(lambda: layer(x))
                    torch.cuda.synchronize()
                    layer.close()
                    del layer
                cell["torch_err"] = round((torch_e2e().float() - golden).abs().max().item(), 4)
                cell["cublas_nccl"] = t(torch_e2e)
                best = min(v for k, v in cell.items() if k.startswith("fused") and not k.endswith("_err"))
                cell["speedup"] = round(cell["cublas_nccl"] / best, 3)
                results[name] = cell
                if rank == 0:
                    print(name, json.dumps(cell), flush=True)
                    if args.out:
                        os.makedirs(os.path.dirname(os.path.abspath(args.out)), exist_ok=True)
                        with open(args.out, "w") as fh:
                            json.dump(results, fh, indent=1)
                del x, w_gu, w_down
                torch.cuda.empty_cache()
    torch.cuda.synchronize()
    if R > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
