"""Helpers shared by tests and benchmarks: process spawning and seeded inputs.

The input generators follow the discipline of the reference's acceptance tests
(tests/test_ag_gemm.py:76-95, tests/test_moe_a2a.py:54-66): fresh seeded data
every iteration, generated on the CPU so that every rank can rebuild every other
rank's inputs (and hence the expected result) without communication.
"""
from __future__ import annotations

import os
import socket
import traceback
from typing import Callable

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def free_port() -> int:
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _entry(rank: int, world_size: int, backend: str, port: int, fn: Callable, args: tuple, errq,
           pg_timeout_s: float = 1800.0):
    try:
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(port)
        os.environ["RANK"] = str(rank)
        os.environ["WORLD_SIZE"] = str(world_size)
        kwargs = {}
        if backend == "nccl":
            torch.cuda.set_device(rank)
            kwargs["device_id"] = torch.device("cuda", rank)
        import datetime
        dist.init_process_group(backend=backend, rank=rank, world_size=world_size,
                                timeout=datetime.timedelta(seconds=pg_timeout_s), **kwargs)
        fn(rank, world_size, *args)
        dist.barrier()
        dist.destroy_process_group()
    except Exception:  # noqa: BLE001 - forwarded to the parent
        errq.put((rank, traceback.format_exc()))
        raise


def spawn(fn: Callable, world_size: int, backend: str = "gloo", args: tuple = (), timeout: float = 300.0,
          pg_timeout_s: float = 1800.0):
    """Run ``fn(rank, world_size, *args)`` in ``world_size`` processes with an initialised
    process group on 127.0.0.1; raises with the first failing rank's traceback."""
    ctx = mp.get_context("spawn")
    errq = ctx.SimpleQueue()
    port = free_port()
    procs = []
    for r in range(world_size):
        p = ctx.Process(target=_entry, args=(r, world_size, backend, port, fn, args, errq, pg_timeout_s))
        p.start()
        procs.append(p)
    failed = False
    for p in procs:
        p.join(timeout)
        if p.is_alive():
            p.terminate()
            failed = True
        elif p.exitcode != 0:
            failed = True
    if failed:
        msgs = []
        while not errq.empty():
            r, tb = errq.get()
            msgs.append(f"--- rank {r} ---\n{tb}")
        for p in procs:
            if p.is_alive():
                p.terminate()
        raise RuntimeError("spawned ranks failed:\n" + ("\n".join(msgs) if msgs else "(no traceback; timeout?)"))


# ---------------------------------------------------------------------------
# Seeded inputs
# ---------------------------------------------------------------------------
def randn_seeded(shape, seed: int, scale: float = 1.0, dtype=torch.float32, device="cpu") -> torch.Tensor:
    """Seeded normal data. The same (seed, device kind) gives the same values in every process,
    which is what lets each rank rebuild the other ranks' operands for its reference result;
    ``device="cuda"`` generates on the GPU (a long soak would otherwise be bound by the host's
    random-number generation)."""
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    return (torch.randn(shape, generator=g, dtype=torch.float32, device=device) * scale).to(dtype)


def ag_inputs(rank: int, R: int, m_pr: int, K: int, n_pr: int, it: int, dtype, scale=0.02, device="cpu"):
    """Per-rank A shards (seed by source rank and iteration) and this rank's B."""
    a_all = [randn_seeded((m_pr, K), 1000 + 17 * it + s, scale, dtype, device) for s in range(R)]
    b = randn_seeded((n_pr, K), 5000 + 31 * it + rank, scale, dtype, device)
    return a_all, b


def ks_inputs(R: int, M: int, N: int, k_loc: int, it: int, dtype, scale=0.02, device="cpu"):
    """K-sharded operands of every rank (GEMM+RS / GEMM+AR): each source pairs its own B."""
    a_all = [randn_seeded((M, k_loc), 2000 + 13 * it + s, scale, dtype, device) for s in range(R)]
    b_all = [randn_seeded((N, k_loc), 7000 + 29 * it + s, scale, dtype, device) for s in range(R)]
    return a_all, b_all


def moe_inputs(rank: int, T: int, H: int, E: int, topk: int, it: int, dtype, zipf_s: float = 0.0):
    """Tokens, distinct top-k expert ids (uniform or Zipf-skewed) and softmax weights."""
    g = torch.Generator(device="cpu")
    g.manual_seed(9000 + 101 * it + rank)
    tokens = torch.randn((T, H), generator=g, dtype=torch.float32).to(dtype)
    if zipf_s > 0:
        p = 1.0 / torch.arange(1, E + 1, dtype=torch.float64) ** zipf_s
    else:
        p = torch.ones(E, dtype=torch.float64)
    p = (p / p.sum()).expand(T, E)
    idx = torch.multinomial(p, topk, replacement=False, generator=g).to(torch.int32)
    logits = torch.randn((T, topk), generator=g, dtype=torch.float32)
    weights = torch.softmax(logits, dim=-1).contiguous()
    return tokens, idx.contiguous(), weights


def fake_expert(recv_rows: torch.Tensor) -> torch.Tensor:
    """Deterministic stand-in for the expert MLP: ``y = x * 2 + (row % 5)`` (the row-dependent
    term exposes mis-routed rows; kept small for fp16 range, as in tests/test_moe_a2a.py:62-66)."""
    n = recv_rows.shape[0]
    bias = (torch.arange(n, device=recv_rows.device) % 5).to(torch.float32).unsqueeze(1)
    return (recv_rows.float() * 2 + bias).to(recv_rows.dtype)
