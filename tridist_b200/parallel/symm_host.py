"""Host-side one-sided API over the symmetric heap.

Counterpart of the reference's DUSHMEM host binding (pydushmem/host.py:93-301 and the
package delegates, pydushmem/__init__.py:45-60): ``malloc / free / ptr / my_pe / n_pes /
putmem / getmem / quiet / fence / barrier_all`` plus the stream helpers of the common
runtime (``set_signal`` / ``wait_signal``, common_ops.py:164-188). Everything is built on
CUDA peer mappings: a put or get is a ``copy_`` between views of two ranks' buffers on the
current stream, a signal is a 4-byte fill of a peer's flag word, a wait is the bounded
device-side spin kernel.
"""
from __future__ import annotations

from typing import Optional

import torch

from .runtime import CpuWorld, SymmBuffer, default_world, init_runtime, native


class SymmHost:
    def __init__(self, world=None):
        self.world = world or default_world()
        if self.world is None:
            raise RuntimeError("initialise the runtime first (init_runtime)")
        if isinstance(self.world, CpuWorld):
            raise RuntimeError("the symmetric heap needs CUDA devices")

    # -- identity -----------------------------------------------------------
    def my_pe(self) -> int:
        return self.world.rank

    def n_pes(self) -> int:
        return self.world.num_ranks

    # -- memory ---------------------------------------------------------------
    def malloc(self, nbytes: int) -> SymmBuffer:
        """Collective; zero-filled (the reference's ``calloc``; ``malloc`` there is unzeroed)."""
        return self.world.alloc(nbytes, self.world.rank)

    calloc = malloc

    def align(self, alignment: int, nbytes: int) -> SymmBuffer:
        """Collective; every symmetric buffer starts on a 256-byte boundary (the reference's
        ``dushmem_align``, pydushmem/host.py:239-249)."""
        if alignment <= 0 or alignment & (alignment - 1) or alignment > 256:
            raise ValueError("alignment must be a power of two up to 256 bytes")
        return self.malloc(nbytes)

    def free(self, buf: SymmBuffer) -> None:
        self.world.free(buf)

    def finalize(self) -> None:
        """Collective: release every symmetric buffer and the process-wide world."""
        global _host
        from .runtime import finalize_runtime
        finalize_runtime()
        _host = None

    def ptr(self, buf: SymmBuffer, pe: int, byte_offset: int = 0) -> int:
        """Address of ``pe``'s copy, valid in this process (the reference's ``dushmem_ptr``)."""
        return buf.peer_ptrs[pe] + byte_offset

    # -- one-sided transfers (stream-ordered on the current stream) --------------
    def putmem(self, dst: SymmBuffer, dst_off: int, src: torch.Tensor, pe: int) -> None:
        n = src.numel() * src.element_size()
        view = dst.tensor(torch.uint8, (n,), dst_off, rank=pe)
        view.copy_(src.contiguous().view(torch.uint8).flatten(), non_blocking=True)

    putmem_nbi = putmem

    def getmem(self, dst: torch.Tensor, src: SymmBuffer, src_off: int, pe: int) -> None:
        n = dst.numel() * dst.element_size()
        view = src.tensor(torch.uint8, (n,), src_off, rank=pe)
        dst.view(torch.uint8).flatten().copy_(view, non_blocking=True)

    getmem_nbi = getmem

    def quiet(self) -> None:
        torch.cuda.current_stream().synchronize()

    fence = quiet

    # -- signals ------------------------------------------------------------------
    def set_signal(self, buf: SymmBuffer, word: int, value: int, pe: int) -> None:
        native().fill_u32(buf.peer_ptrs[pe] + 4 * word, 1, value)

    def wait_signal(self, buf: SymmBuffer, word: int, value: int, timeout_ms: Optional[int] = None) -> None:
        w = self.world
        t = (timeout_ms * 1_000_000) if timeout_ms is not None else w.timeout_ns
        native().wait_flag_test(buf.local_ptr + 4 * word, value, w.status_dev, w.abort_word, t)

    def barrier_all(self) -> None:
        self.world.barrier_on_stream()


_host: Optional[SymmHost] = None


def get_host() -> SymmHost:
    global _host
    if _host is None:
        _host = SymmHost()
    return _host


def init(rank: int, num_ranks: int, comm=None) -> SymmHost:
    init_runtime(rank, num_ranks, comm, device="cuda")
    return get_host()
