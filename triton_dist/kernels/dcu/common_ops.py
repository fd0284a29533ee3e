"""The reference's common runtime names (triton_dist/kernels/dcu/common_ops.py:31-260) on top of
tridist_b200.parallel.runtime, for scripts written against that module.

The fused operators of this library need none of these helpers (their transfers and signals are
issued from inside the kernels); they are kept for the host-driven style of the reference:
stream-ordered peer copies, flag words set and awaited on a stream, and the round barrier.
"""
from typing import Iterable, Tuple

import torch

from tridist_b200.parallel.runtime import default_world, init_runtime, native


def init_dcu(mpi, comm, rank, size, host=None):
    """Process-wide initialisation; ``mpi`` and ``host`` are accepted and ignored, ``comm`` may be a
    torch.distributed process group."""
    return init_runtime(rank, size, comm)


def dcu_state():
    return default_world()


def _stream(stream):
    if stream is None or isinstance(stream, torch.cuda.Stream):
        return stream
    return torch.cuda.ExternalStream(int(stream))


def memcpy_async(dst: int, src: int, nbytes: int, stream_handle=None) -> None:
    """Device-to-device copy between two addresses valid in this process (a peer's buffer included)
    on the given stream (default: the current one)."""
    w = default_world()
    C = native()
    d = C.tensor_from_ptr(int(dst), [int(nbytes)], torch.uint8, w.device)
    s = C.tensor_from_ptr(int(src), [int(nbytes)], torch.uint8, w.device)
    st = _stream(stream_handle)
    if st is None:
        d.copy_(s, non_blocking=True)
    else:
        with torch.cuda.stream(st):
            d.copy_(s, non_blocking=True)


def fan_out_memcpy_async(ops: Iterable[Tuple[int, int, int]]) -> None:
    """``(dst, src, nbytes)`` copies, complete in stream order on the current stream when the next
    operation of that stream runs. The reference spreads them over a pool of side streams
    (common_ops.py:116-158); peer copies here already run at link speed from one stream."""
    for dst, src, nbytes in ops:
        memcpy_async(dst, src, nbytes)


def set_signal(ptr: int, val: int, stream=None, require_i64: bool = False) -> None:
    """Write a 32-bit flag word (own or peer memory) in stream order."""
    st = _stream(stream)
    if st is None:
        native().fill_u32(int(ptr), 1, int(val))
    else:
        with torch.cuda.stream(st):
            native().fill_u32(int(ptr), 1, int(val))


def wait_eq(ptr: int, val: int, stream=None, require_i64: bool = False) -> None:
    """Hold the stream until the flag word reaches ``val`` (tickets are monotonic: the wait is
    "greater or equal"). Bounded: on expiry the world's status block says so and ``check()`` raises."""
    w = default_world()
    st = _stream(stream)
    if st is None:
        native().wait_flag_test(int(ptr), int(val), w.status_dev, w.abort_word, w.timeout_ns)
    else:
        with torch.cuda.stream(st):
            native().wait_flag_test(int(ptr), int(val), w.status_dev, w.abort_word, w.timeout_ns)


class SymmBarrier:
    """Monotonic device-side barrier of all ranks (common_ops.py:212-256): every call of
    ``round_barrier`` is one round, enqueued on the current stream."""

    def __init__(self, n_ranks: int):
        w = default_world()
        if w is None or w.num_ranks != n_ranks:
            raise RuntimeError("initialise the runtime with the same number of ranks first (init_dcu)")
        self.world = w

    def round_barrier(self, my_rank: int = -1) -> None:
        self.world.barrier_on_stream()

    def sync(self) -> None:
        torch.cuda.current_stream().synchronize()


def barrier_all_on_stream(rank=None, num_ranks=None, barrier: "SymmBarrier" = None) -> None:
    (barrier.world if barrier is not None else default_world()).barrier_on_stream()
