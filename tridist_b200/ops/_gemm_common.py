"""Shared host logic of the fused GEMM operators: plan construction and caching.

A *plan* is a pre-built kernel parameter block (TMA descriptors, peer pointers,
tile order) for one (context, tensors, shapes) combination; launching a cached
plan costs one kernel launch and no descriptor encoding.
"""
from __future__ import annotations

from collections import OrderedDict
from typing import Dict, List, Optional

import torch

from ..parallel.runtime import native
from ..utils.config import env_int

OP_PLAIN, OP_AG, OP_RS, OP_AR1, OP_AR2 = 0, 1, 2, 3, 4
EPI_STORE, EPI_SWIGLU = 0, 1
SCHED_NATURAL, SCHED_SEGMENT, SCHED_STRIDED, SCHED_LIST = 0, 1, 2, 3
BM = 128
NUM_SMS_HINT = 148


def is_bf16(dtype: torch.dtype) -> bool:
    if dtype == torch.bfloat16:
        return True
    if dtype == torch.float16:
        return False
    raise TypeError(f"tridist_b200: fused GEMM kernels support fp16 and bf16, got {dtype}")


def choose_bn(M: int, N: int, swiglu: bool = False, K: int = 0) -> int:
    """Output-tile width: 256 unless that leaves most SMs without a tile. A single row block
    (M <= 128) with a long K is the exception: every CTA re-reads the whole A slice of its K
    range, so wider tiles (fewer CTAs per K range, more K slices instead) move a quarter less
    through the L2 fabric, which is what bounds that shape."""
    if swiglu:
        return 256       # gate and up halves are two 128-row TMA boxes of one 256-wide tile
    forced = env_int("TRIDIST_FORCE_BN", 0)
    if forced in (128, 256):
        return forced
    m_tiles = (M + BM - 1) // BM
    if m_tiles == 1 and K >= 8192 and N >= 2048:
        return 256
    width = 128 if swiglu else 256           # output columns covered by a BN=256 tile
    tiles256 = m_tiles * ((N + width - 1) // width)
    return 256 if tiles256 >= NUM_SMS_HINT - 28 else 128


def rotation_order(rank: int, R: int, step: int, own_last: bool) -> List[int]:
    """Segment visiting order.

    own_last=False (all-gather): own rows first, then rank-1, rank-2, ... — the
    order in which shards arrive when every rank pushes to rank+1 first.
    own_last=True (reduce-scatter / all-reduce): rank+1 first, own rows last, so
    that every owner receives its first partial tiles as early as possible.
    """
    if own_last:
        return [(rank + 1 + i) % R for i in range(R)]
    return [(rank - i * step) % R for i in range(R)]


MAX_TICKETS = 1 << 30


def next_round(current: int, what: str = "context") -> int:
    """The next monotonic ticket of a context. Tickets are 32-bit and compared by signed difference;
    a context is refused long before that compare could wrap (the reference asserts a ticket
    ceiling too, gemm_ar_rd.py:78,:422) and has to be created anew."""
    nxt = current + 1
    if nxt >= MAX_TICKETS:
        raise RuntimeError(f"tridist_b200: this {what} has issued {current} tickets; create a new one "
                           f"(tickets are 32-bit and must not wrap)")
    return nxt


_warned = set()


def warn_ignored(where: str, **given) -> None:
    """One warning per (entry point, argument) for a reference argument that has no counterpart in
    the one-kernel design and was given a non-default value."""
    import warnings
    for name, (value, default) in given.items():
        if value != default and (where, name) not in _warned:
            _warned.add((where, name))
            warnings.warn(f"tridist_b200.{where}: {name}={value!r} has no effect here "
                          f"(kept for signature compatibility with the reference)", stacklevel=3)


class PlanCache:
    """Plans of one context, keyed by operand addresses and shapes; least recently used out.

    A plan bakes pointers into tensor maps, so a caller that hands in freshly allocated tensors
    (new addresses) every call misses every time and pays the encoding again. ``hits`` / ``misses`` /
    ``evictions`` make that visible; after ``4 * capacity`` evictions one warning says so."""

    def __init__(self, capacity: int = 64):
        self.capacity = capacity
        self._d: "OrderedDict[tuple, int]" = OrderedDict()
        self.hits = self.misses = self.evictions = 0
        self._warned = False

    def get(self, key: tuple, make) -> int:
        pid = self._d.get(key)
        if pid is not None:
            self._d.move_to_end(key)
            self.hits += 1
            return pid
        self.misses += 1
        pid = make()
        self._d[key] = pid
        if len(self._d) > self.capacity:
            _, old = self._d.popitem(last=False)
            native().gemm_plan_destroy(old)
            self.evictions += 1
            if self.evictions >= 4 * self.capacity and not self._warned:
                self._warned = True
                import warnings
                warnings.warn("tridist_b200: a plan cache keeps evicting (operand addresses change from call to "
                              "call, so tensor maps are re-encoded every time); reuse buffers across calls",
                              stacklevel=3)
        return pid

    def clear(self) -> None:
        C = native()
        for pid in self._d.values():
            C.gemm_plan_destroy(pid)
        self._d.clear()


PROF_SLOTS = ["load_flag_wait", "load_empty_wait", "mma_full_wait", "mma_tmem_wait", "epi_busy", "epi_publish",
              "epi_ticket_wait", "epi_tiles", "comm_total", "kernel", "ar_owner_wait", "ar_owner_work",
              "ar_collect_wait", "ar_collect_copy", "epi_done_at", "ar_owner_done_at",
              # time stamps (since the CTA started) of the last tile each role handled
              "tl_acc_ready", "tl_staged", "tl_stored", "tl_flagged", "tl_own_seen", "tl_own_loaded",
              "tl_own_fenced", "tl_own_flagged", "tl_col_seen", "tl_comm_start", "tl_own_it0", "sk_wait",
              # absolute globaltimer values (ns): CTA entry, roles start, CTA end
              "t_entry", "t_setup", "t_end"]
PROF_WIDTH = 32
_prof_buf: Optional[torch.Tensor] = None


def prof_buffer() -> Optional[torch.Tensor]:
    """Stall-accounting plane of the fused GEMM kernels ([CTA][32] int64 ns sums and stamps), allocated when
    ``TRIDIST_PROF=1``; plans created afterwards write into it."""
    global _prof_buf
    if not env_int("TRIDIST_PROF", 0):
        return None
    if _prof_buf is None:
        _prof_buf = torch.zeros((256, PROF_WIDTH), dtype=torch.int64, device="cuda")
    return _prof_buf


def read_prof(n_ctas: int = 148) -> Dict[str, Dict[str, float]]:
    """Mean and max over CTAs of every accounting slot of the LAST kernel, in microseconds
    (``epi_tiles`` is a count). Call after a synchronisation."""
    if _prof_buf is None:
        return {}
    t = _prof_buf[:n_ctas].cpu().double()
    out = {}
    for i, name in enumerate(PROF_SLOTS):
        col = t[:, i]
        scale = 1.0 if name == "epi_tiles" else 1e-3
        if name.startswith("tl_") or name.endswith("_at"):
            nz = col[col > 0]                     # stamps: only CTAs that had such a tile
            if nz.numel() == 0:
                continue
            out[name] = {"min": round(float(nz.min()) * scale, 2), "mean": round(float(nz.mean()) * scale, 2),
                         "max": round(float(nz.max()) * scale, 2)}
        else:
            out[name] = {"mean": round(float(col.mean()) * scale, 2), "max": round(float(col.max()) * scale, 2)}
    return out


def base_desc(world, rank: int, R: int, a: torch.Tensor, b: torch.Tensor, c_ptr: int, ldc: int,
              M: int, N: int, K: int, bn: int, op: int) -> Dict:
    assert a.stride(1) == 1 and b.stride(1) == 1, "operands must be row-major with unit inner stride"
    d = dict(op=op, epi=EPI_STORE, sched=SCHED_NATURAL, bn=bn, bf16=is_bf16(a.dtype), rank=rank, R=R,
             M=M, N=N, K=K, a=a.data_ptr(), a_rows=a.shape[0], lda=a.stride(0),
             b=b.data_ptr(), b_rows=b.shape[0], ldb=b.stride(0), c=c_ptr, ldc=ldc,
             status_dev=world.status_dev,
             abort_word=world.abort_word_of(rank) if hasattr(world, "abort_word_of") else world.abort_word,
             peer_abort=world.peer_abort_words() if hasattr(world, "peer_abort_words") else [],
             timeout_ns=world.timeout_ns,
             # the grid must fit the device in one wave: its CTAs wait on one another
             check_residency=1 if (env_int("TRIDIST_CHECK_RESIDENCY", 1) and getattr(world, "kind", "") != "emulated") else 0,
             max_ctas=env_int("TRIDIST_MAX_CTAS", 0) or
             (NUM_SMS_HINT // world.num_ranks if getattr(world, "kind", "") == "emulated" else 0),
             poll_ns=env_int("TRIDIST_POLL_NS", 0),
             allow_wide=env_int("TRIDIST_WIDE", 1), allow_splitk=env_int("TRIDIST_SPLITK", 1),
             raster_g=env_int("TRIDIST_RASTER_G", 0),
             l2_ahead=env_int("TRIDIST_L2_AHEAD", 0),
             prof=(prof_buffer().data_ptr() if prof_buffer() is not None else 0),
             # several virtual ranks in one launch keep to single-CTA tiles unless TRIDIST_EMU_PAIR=1
             # asks for CTA pairs there too (a cooperative launch of clusters)
             allow_pair=1 if (env_int("TRIDIST_CTA_PAIR", 1) and
                              (getattr(world, "kind", "") != "emulated" or env_int("TRIDIST_EMU_PAIR", 0))) else 0)
    return d


def tensor_extent_bytes(t: torch.Tensor) -> int:
    """Bytes from the tensor's first element to the end of its storage."""
    return int(t.untyped_storage().nbytes() - t.storage_offset() * t.element_size())


def debug_check(d: Dict, **extents) -> None:
    """With ``TRIDIST_DEBUG=1``: before a plan is created, replay its tile schedule on the host and
    check every ticket index and buffer offset the kernel will compute against the sizes of the
    buffers it is given (a bounds check that cannot fault: nothing is launched). Raises
    ``TriDistError`` with one sentence per violation."""
    if not env_int("TRIDIST_DEBUG", 0):
        return
    bad = native().plan_check(d, {k: int(v) for k, v in extents.items()}, 148)
    if bad:
        from ..parallel.runtime import TriDistError
        raise TriDistError("plan check failed: " + "; ".join(bad))


# ---------------------------------------------------------------------------
# Plain single-GPU GEMM (the R = 1 degenerate of every fused operator and the
# building block of the tile-config sweeps)
# ---------------------------------------------------------------------------
_plain_cache = PlanCache(128)
_plain_world = None


class _PlainWorld:
    """Minimal status plumbing for GEMMs launched outside any context."""

    def __init__(self):
        C = native()
        self.status_host, self.status_dev = C.status_alloc()
        self._abort = torch.zeros(64, dtype=torch.int32, device="cuda")
        self.abort_word = self._abort.data_ptr()
        self.timeout_ns = env_int("TRIDIST_WAIT_TIMEOUT_MS", 4000) * 1_000_000


def plain_world():
    global _plain_world
    if _plain_world is None:
        _plain_world = _PlainWorld()
    return _plain_world


def gemm_nt(a: torch.Tensor, b: torch.Tensor, out: Optional[torch.Tensor] = None,
            bn: Optional[int] = None, swiglu: bool = False, max_ctas: int = 0, probe: int = 0) -> torch.Tensor:
    """``out = a @ b.T`` on the hand-written tcgen05 kernel (fp32 accumulate).

    With ``swiglu=True`` b holds ``[gate; up]`` row blocks (2*I rows) and the
    result is ``silu(a @ gate.T) * (a @ up.T)`` of shape [M, I], computed in the
    GEMM epilogue. ``probe`` = 1 / 2 runs the pipeline probes (tensor-pipe ceiling: resident
    stages re-multiplied without loads; operand-feed ceiling: loads without MMAs); the output
    is then meaningless.
    """
    assert a.is_cuda and b.is_cuda and a.dtype == b.dtype
    M, K = a.shape
    n_rows = b.shape[0]
    N = n_rows // 2 if swiglu else n_rows
    if out is None:
        out = torch.empty((M, N), dtype=a.dtype, device=a.device)
    assert out.stride(1) == 1
    if bn is None:
        bn = choose_bn(M, N, swiglu, K=K)
    w = plain_world()
    key = (a.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, K, a.stride(0), b.stride(0),
           out.stride(0), bn, swiglu, a.dtype, max_ctas, probe)

    def make():
        d = base_desc(w, 0, 1, a, b, out.data_ptr(), out.stride(0), M, N, K, bn, OP_PLAIN)
        if swiglu:
            d["epi"] = EPI_SWIGLU
            d["swiglu_up_row0"] = N
        if max_ctas:
            d["max_ctas"] = max_ctas
        d["probe"] = probe
        debug_check(d, c_bytes=tensor_extent_bytes(out))
        return native().gemm_plan_create(d)

    pid = _plain_cache.get(key, make)
    native().gemm_plan_launch(pid, 1, 0, 0, 0)
    return out
