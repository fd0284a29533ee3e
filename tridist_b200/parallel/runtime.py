"""Process-level runtime: bootstrap, symmetric heap, barrier and failure status.

Replaces the reference's L1/L2 layers — the DUSHMEM ctypes binding with its MPI
bootstrap (pydushmem/host.py:31-325) and the common runtime ``init_dcu`` /
``SymmBarrier`` / ``memcpy_async`` (triton_dist/kernels/dcu/common_ops.py:31-260)
— with a CUDA-IPC symmetric heap bootstrapped over ``torch.distributed``.

Three kinds of world exist:

* ``ProcessWorld``   one process per GPU; peers are other processes' buffers
                     mapped through CUDA IPC handles (the production mode).
* ``EmulatedWorld``  one process, one GPU, R virtual ranks; every virtual rank's
                     buffers are local and the fused kernels run all ranks in a
                     single launch.  Used to test the cross-rank protocols on a
                     single GPU.
* ``CpuWorld``       no GPU: ranks are gloo processes; ops run the torch oracle.
"""
from __future__ import annotations

import os
import threading
from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import torch
import torch.distributed as dist

from ..utils.config import env_int, env_str

_DTYPE_SIZE = {torch.float16: 2, torch.bfloat16: 2, torch.float32: 4, torch.int32: 4,
               torch.int64: 8, torch.uint8: 1}


class TriDistError(RuntimeError):
    """Raised when a kernel reported a failure through the status plane."""


SITE_NAMES = {
    1: "all-gather chunk ticket", 2: "reduce-scatter tile ticket", 3: "all-reduce tile ticket",
    4: "all-reduce result ticket", 5: "barrier", 6: "MoE metadata", 7: "MoE dispatch completion",
    8: "MoE combine readiness", 9: "split-K partial", 10: "all-gather arrive ticket", 11: "index range check",
    12: "recursive-doubling arrival ticket", 13: "recursive-doubling ack ticket", 16: "pipeline full barrier", 17: "pipeline empty barrier",
    18: "TMEM full barrier", 19: "TMEM empty barrier", 32: "self test",
}
CODE_NAMES = {1: "flag wait timed out", 2: "pipeline barrier wait timed out",
              3: "index out of range", 4: "receive buffer overflow",
              5: "gave up because another rank (or another role of the kernel) raised the abort word"}


def native():
    """The compiled extension; importing it requires the in-tree shared object."""
    from .. import _build
    return _build.load()


def _symm_mem_module():
    """torch's symmetric-memory allocator (import kept in one place so that tests can stand in for it)."""
    import torch.distributed._symmetric_memory as symm_mem
    return symm_mem


# ---------------------------------------------------------------------------
# Symmetric buffers
# ---------------------------------------------------------------------------
@dataclass
class SymmBuffer:
    """A buffer that exists with the same size on every rank.

    ``peer_ptrs[r]`` is rank r's copy as an address valid in *this* process
    (for r == rank it is the local allocation itself).
    """
    nbytes: int
    rank: int
    peer_ptrs: List[int]
    device: int
    _owner: object = field(default=None, repr=False)
    _opened: List[int] = field(default_factory=list, repr=False)
    freed: bool = False

    @property
    def local_ptr(self) -> int:
        return self.peer_ptrs[self.rank]

    def tensor(self, dtype: torch.dtype, shape: Sequence[int], byte_offset: int = 0,
               rank: Optional[int] = None) -> torch.Tensor:
        """A torch view of (part of) one rank's copy; no ownership is taken."""
        n = 1
        for s in shape:
            n *= int(s)
        assert byte_offset + n * _DTYPE_SIZE[dtype] <= self.nbytes, "view exceeds the symmetric buffer"
        base = self.peer_ptrs[self.rank if rank is None else rank]
        return native().tensor_from_ptr(base + byte_offset, [int(s) for s in shape], dtype, self.device)

    def ptrs(self, byte_offset: int = 0) -> List[int]:
        return [p + byte_offset for p in self.peer_ptrs]


@dataclass
class McBuffer(SymmBuffer):
    """A symmetric buffer with an NVSwitch multicast mapping: ``mc_ptr`` addresses all ranks'
    copies at once (``multimem.*`` instructions only)."""
    mc_ptr: int = 0
    _keep: object = field(default=None, repr=False)


class _WorldBase:
    kind = "base"
    rank: int
    num_ranks: int

    def __init__(self):
        self._barrier_ticket = 0
        self._buffers: List[SymmBuffer] = []
        self._mc_buffers: List["McBuffer"] = []
        self.timeout_ms = env_int("TRIDIST_WAIT_TIMEOUT_MS", 4000)

    @property
    def timeout_ns(self) -> int:
        return int(self.timeout_ms) * 1_000_000

    def alloc_multicast(self, nbytes: int):
        """Worlds without an NVSwitch multicast mapping (one process, CPU) have none to give."""
        return None

    def free_multicast(self, buf) -> None:
        return None

    def _alloc_multicast_native(self, nbytes: int) -> Optional["McBuffer"]:
        """Collective. The package's own allocator (cuMemCreate / POSIX descriptors / cuMulticast*,
        ``parallel/vmm.py``); None on every rank when any rank cannot have it."""
        from . import vmm
        ok, why = self.C.vmm_multicast_supported()
        oks = [None] * self.num_ranks
        dist.all_gather_object(oks, "" if ok else (why or "multicast not supported"), group=self.group)
        if any(oks):
            self.multicast_native_unavailable = "; ".join(f"rank {r}: {w}" for r, w in enumerate(oks) if w)
            return None
        try:
            alloc = vmm.alloc_symmetric_multicast(self.C, self.rank, self.num_ranks, self.group, nbytes)
        except RuntimeError as exc:                  # the same on every rank
            self.multicast_native_unavailable = str(exc)
            return None
        buf = McBuffer(nbytes=alloc.nbytes, rank=self.rank, peer_ptrs=list(alloc.peer_ptrs), device=self.device,
                       _owner=self, mc_ptr=alloc.mc_ptr, _keep=alloc)
        self.multicast_allocator = "native"
        self.C.fill_u32(buf.local_ptr, alloc.nbytes // 4, 0)     # driver allocations are not zeroed
        torch.cuda.synchronize()
        dist.barrier(group=self.group)
        self._mc_buffers.append(buf)
        return buf

    def release_multicast(self) -> None:
        return None


class ProcessWorld(_WorldBase):
    """One process per GPU; peers reached through CUDA IPC mappings."""
    kind = "process"

    def __init__(self, rank: int, num_ranks: int, group=None, device: Optional[int] = None):
        super().__init__()
        self.rank, self.num_ranks, self.group = rank, num_ranks, group
        if device is None:
            device = torch.cuda.current_device()
        self.device = device
        torch.cuda.set_device(device)
        self.C = native()
        if num_ranks > 1:
            if not dist.is_initialized():
                raise RuntimeError("tridist_b200: torch.distributed must be initialised for num_ranks > 1")
            devs = [None] * num_ranks
            dist.all_gather_object(devs, int(device), group=group)
            self.peer_devices = devs
            for d in devs:
                if not self.C.enable_peer_access(int(d)):
                    raise RuntimeError(f"tridist_b200: device {device} cannot access peer device {d}")
        else:
            self.peer_devices = [device]
        hp, dp = self.C.status_alloc()
        self.status_host, self.status_dev = hp, dp
        self.abort_buf = self.alloc(256)
        self.abort_word = self.abort_buf.local_ptr
        self.barrier_buf = self.alloc(256)

    def abort_word_of(self, rank: int) -> int:
        """The abort word the kernels of ``rank`` poll (this process runs one rank)."""
        return self.abort_word

    def peer_abort_words(self) -> List[int]:
        """Every rank's abort word as addresses of this process: a kernel that gives up raises all
        of them, so that the peers leave their waits at once."""
        return list(self.abort_buf.peer_ptrs)

    # -- symmetric heap ------------------------------------------------------
    def alloc(self, nbytes: int, rank: Optional[int] = None) -> SymmBuffer:
        """Collective: every rank must call with the same size, in the same order."""
        nbytes = max(256, (int(nbytes) + 255) // 256 * 256)
        local = self.C.symm_alloc(nbytes)
        ptrs = [0] * self.num_ranks
        opened = []
        if self.num_ranks > 1:
            handle = bytes(self.C.symm_export(local))
            handles = [None] * self.num_ranks
            dist.all_gather_object(handles, handle, group=self.group)
            for r, h in enumerate(handles):
                if r == self.rank:
                    ptrs[r] = local
                else:
                    ptrs[r] = self.C.symm_open(h)
                    opened.append(ptrs[r])
            dist.barrier(group=self.group)
        else:
            ptrs[0] = local
        buf = SymmBuffer(nbytes=nbytes, rank=self.rank, peer_ptrs=ptrs, device=self.device,
                         _owner=self, _opened=opened)
        self._buffers.append(buf)
        return buf

    def free(self, buf: SymmBuffer) -> None:
        """Collective: unmaps the peers' copies, then releases the local one."""
        if buf.freed:
            return
        torch.cuda.synchronize()
        if self.num_ranks > 1:
            dist.barrier(group=self.group)
        for p in buf._opened:
            self.C.symm_close(p)
        if self.num_ranks > 1:
            dist.barrier(group=self.group)
        self.C.symm_free(buf.local_ptr)
        buf.freed = True
        if buf in self._buffers:
            self._buffers.remove(buf)

    def alloc_multicast(self, nbytes: int) -> Optional["McBuffer"]:
        """Collective. A symmetric buffer that is also bound to an NVSwitch multicast object, so
        kernels can use ``multimem.ld_reduce`` / ``multimem.st`` on ``mc_ptr`` (in-switch reduction
        and replication). The virtual-memory plumbing (allocation, handle exchange, multicast
        bind) is torch's symmetric-memory allocator; the kernels are this package's own.

        Returns None on every rank when any rank cannot have it: one GPU, ``TRIDIST_NVLS=0``,
        no multicast support in the driver / fabric, or a failed rendezvous."""
        if self.num_ranks < 2 or env_int("TRIDIST_NVLS", 1) == 0:
            return None
        if env_str("TRIDIST_MC_ALLOC", "native") == "native":
            buf = self._alloc_multicast_native(nbytes)
            if buf is not None:
                return buf
            # (every rank took the same branch: the outcome of the native attempt is agreed)
        tensor = handle = None
        mc, ptrs, why = 0, [], ""
        group = self.group if self.group is not None else dist.group.WORLD
        # Agree first, rendezvous second: a rank that cannot even allocate must not leave the
        # others blocked inside the allocator's rendezvous (a different collective).
        symm_mem = None
        try:
            symm_mem = _symm_mem_module()
            nbytes = (int(nbytes) + 255) // 256 * 256
            tensor = symm_mem.empty(nbytes, dtype=torch.uint8, device=torch.device("cuda", self.device))
        except Exception as exc:          # missing API, unsupported driver, out of memory
            why = f"{type(exc).__name__}: {exc}"
        can = [None] * self.num_ranks
        dist.all_gather_object(can, why, group=self.group)
        if any(can):
            self.multicast_unavailable = "; ".join(f"rank {r}: {w}" for r, w in enumerate(can) if w)
            del tensor
            return None
        try:
            handle = symm_mem.rendezvous(tensor, group)
            mc = int(handle.multicast_ptr or 0)
            ptrs = [int(x) for x in handle.buffer_ptrs]
            if mc == 0:
                why = "no multicast address"
            elif len(ptrs) != self.num_ranks or ptrs[self.rank] != tensor.data_ptr():
                mc, why = 0, "unexpected peer pointer table"
        except Exception as exc:          # refused rendezvous (raised on every rank or on none)
            mc, why = 0, f"{type(exc).__name__}: {exc}"
        oks = [None] * self.num_ranks
        dist.all_gather_object(oks, why, group=self.group)
        if any(oks):
            self.multicast_unavailable = "; ".join(f"rank {r}: {w}" for r, w in enumerate(oks) if w)
            del handle, tensor
            return None
        self.multicast_allocator = "torch"
        buf = McBuffer(nbytes=nbytes, rank=self.rank, peer_ptrs=ptrs, device=self.device, _owner=self,
                       mc_ptr=mc, _keep=(tensor, handle))
        self._mc_buffers.append(buf)
        return buf

    def _alloc_multicast_native(self, nbytes: int) -> Optional["McBuffer"]:
        """Collective. The package's own allocator (cuMemCreate / POSIX descriptors / cuMulticast*,
        ``parallel/vmm.py``); None on every rank when any rank cannot have it."""
        from . import vmm
        ok, why = self.C.vmm_multicast_supported()
        oks = [None] * self.num_ranks
        dist.all_gather_object(oks, "" if ok else (why or "multicast not supported"), group=self.group)
        if any(oks):
            self.multicast_native_unavailable = "; ".join(f"rank {r}: {w}" for r, w in enumerate(oks) if w)
            return None
        try:
            alloc = vmm.alloc_symmetric_multicast(self.C, self.rank, self.num_ranks, self.group, nbytes)
        except RuntimeError as exc:                  # the same on every rank
            self.multicast_native_unavailable = str(exc)
            return None
        buf = McBuffer(nbytes=alloc.nbytes, rank=self.rank, peer_ptrs=list(alloc.peer_ptrs), device=self.device,
                       _owner=self, mc_ptr=alloc.mc_ptr, _keep=alloc)
        self.multicast_allocator = "native"
        self.C.fill_u32(buf.local_ptr, alloc.nbytes // 4, 0)     # driver allocations are not zeroed
        torch.cuda.synchronize()
        dist.barrier(group=self.group)
        self._mc_buffers.append(buf)
        return buf

    def release_multicast(self) -> None:
        """Collective: unbind every live multicast buffer (call before a rank leaves, so that no
        rank exits while its memory is still bound to a multicast object the others use)."""
        for buf in list(self._mc_buffers):
            self.free_multicast(buf)

    def free_multicast(self, buf: Optional["McBuffer"]) -> None:
        """Collective: every rank drops its mapping after all of them stopped using it."""
        if buf is None or buf.freed:
            return
        torch.cuda.synchronize()
        dist.barrier(group=self.group)
        from . import vmm
        if isinstance(buf._keep, vmm.VmmAllocation):
            vmm.free_symmetric_multicast(self.C, self.group, buf._keep, self.num_ranks)
        buf._keep = None
        buf.freed = True
        if buf in self._mc_buffers:
            self._mc_buffers.remove(buf)
        dist.barrier(group=self.group)

    # -- synchronisation -----------------------------------------------------
    def barrier_on_stream(self) -> None:
        """Device-side barrier of all ranks, enqueued on the current stream."""
        self._barrier_ticket += 1
        if self.num_ranks == 1:
            return
        self.C.barrier_all(self.barrier_buf.ptrs(), self.rank, self.num_ranks, self._barrier_ticket,
                           self.status_dev, self.abort_word, self.timeout_ns, self.peer_abort_words())

    def host_barrier(self) -> None:
        torch.cuda.synchronize()
        if self.num_ranks > 1:
            dist.barrier(group=self.group)

    # -- failure status ------------------------------------------------------
    def status(self):
        return list(self.C.status_read(self.status_host))

    def check(self, sync: bool = False) -> None:
        """Raise TriDistError if any kernel of this world reported a failure."""
        if sync:
            torch.cuda.synchronize()
        code, rank, site, expected, seen, aux = self.status()
        if code != 0:
            raise TriDistError(
                f"rank {rank}: {CODE_NAMES.get(code, code)} at {SITE_NAMES.get(site, site)} "
                f"(expected {expected}, saw {seen}, aux 0x{aux:x})")

    def clear_status(self) -> None:
        """Forget a reported failure (every rank clears its own record and abort word)."""
        torch.cuda.synchronize()
        self.C.status_clear(self.status_host)
        for r in range(self.num_ranks if self.kind == "emulated" else 1):
            self.C.fill_u32(self.abort_word_of(r if self.kind == "emulated" else self.rank), 1, 0)
        torch.cuda.synchronize()


class EmulatedWorld(_WorldBase):
    """R virtual ranks inside one process on one GPU (single-GPU protocol tests)."""
    kind = "emulated"

    def __init__(self, num_ranks: int, device: Optional[int] = None):
        super().__init__()
        self.rank = 0
        self.num_ranks = num_ranks
        if device is None:
            device = torch.cuda.current_device()
        self.device = device
        self.C = native()
        self._seq = [0] * num_ranks
        self._shared: List[SymmBuffer] = []
        hp, dp = self.C.status_alloc()
        self.status_host, self.status_dev = hp, dp
        self.abort_buf = self.alloc(256)
        self.abort_word = self.abort_buf.peer_ptrs[0]
        self.group = None

    def alloc(self, nbytes: int, rank: Optional[int] = None) -> SymmBuffer:
        """The k-th allocation of every virtual rank names the same set of R buffers,
        as the k-th collective allocation does across processes."""
        nbytes = max(256, (int(nbytes) + 255) // 256 * 256)
        if rank is None:
            ptrs = [self.C.symm_alloc(nbytes) for _ in range(self.num_ranks)]
            buf = SymmBuffer(nbytes=nbytes, rank=0, peer_ptrs=ptrs, device=self.device, _owner=self)
            self._buffers.append(buf)
            return buf
        idx = self._seq[rank]
        self._seq[rank] += 1
        if idx == len(self._shared):
            self._shared.append(self.alloc(nbytes))
        base = self._shared[idx]
        assert base.nbytes == nbytes, "virtual ranks must allocate the same sizes in the same order"
        return self.view(base, rank)

    def abort_word_of(self, rank: int) -> int:
        """Every virtual rank polls its own word, as separate processes would."""
        return self.abort_buf.peer_ptrs[rank]

    def peer_abort_words(self) -> List[int]:
        return list(self.abort_buf.peer_ptrs)

    def view(self, buf: SymmBuffer, rank: int) -> SymmBuffer:
        return SymmBuffer(nbytes=buf.nbytes, rank=rank, peer_ptrs=buf.peer_ptrs, device=buf.device,
                          _owner=self)

    def free(self, buf: SymmBuffer) -> None:
        if buf.freed:
            return
        torch.cuda.synchronize()
        for p in buf.peer_ptrs:
            self.C.symm_free(p)
        buf.freed = True
        if buf in self._buffers:
            self._buffers.remove(buf)

    def barrier_on_stream(self) -> None:   # one stream orders all virtual ranks
        self._barrier_ticket += 1

    def host_barrier(self) -> None:
        torch.cuda.synchronize()

    status = ProcessWorld.status
    check = ProcessWorld.check
    clear_status = ProcessWorld.clear_status


class CpuWorld(_WorldBase):
    """Ranks are CPU processes talking gloo; ops run the torch oracle."""
    kind = "cpu"

    def __init__(self, rank: int, num_ranks: int, group=None):
        super().__init__()
        self.rank, self.num_ranks, self.group = rank, num_ranks, group
        self.device = "cpu"
        if num_ranks > 1 and not dist.is_initialized():
            raise RuntimeError("tridist_b200: torch.distributed (gloo) must be initialised for num_ranks > 1")

    def barrier_on_stream(self) -> None:
        self.host_barrier()

    def host_barrier(self) -> None:
        if self.num_ranks > 1:
            dist.barrier(group=self.group)

    def check(self, sync: bool = False) -> None:
        return None


# ---------------------------------------------------------------------------
# Process-wide default world (the reference keeps one in common_ops._state)
# ---------------------------------------------------------------------------
_lock = threading.Lock()
_default_world: Optional[_WorldBase] = None


def init_runtime(rank: int, num_ranks: int, comm=None, device: Optional[str] = None) -> _WorldBase:
    """Create (once) and return the process-wide world.

    ``comm`` may be a ``torch.distributed`` process group; anything else (such
    as the reference's MPI communicator handle) is ignored and the default
    group is used.  ``device`` is "cuda" or "cpu"; by default CUDA is used when
    available.
    """
    global _default_world
    with _lock:
        if _default_world is not None:
            w = _default_world
            if w.rank != rank or w.num_ranks != num_ranks:
                raise RuntimeError("tridist_b200: runtime already initialised with a different rank/world size")
            return w
        group = comm if isinstance(comm, dist.ProcessGroup) else None
        if device is None:
            device = "cuda" if torch.cuda.is_available() else "cpu"
        if device == "cuda":
            if not dist.is_initialized() and num_ranks > 1:
                _init_process_group("nccl", rank, num_ranks)
            _default_world = ProcessWorld(rank, num_ranks, group)
        else:
            if not dist.is_initialized() and num_ranks > 1:
                _init_process_group("gloo", rank, num_ranks)
            _default_world = CpuWorld(rank, num_ranks, group)
        return _default_world


def _init_process_group(backend: str, rank: int, num_ranks: int) -> None:
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29533")
    kwargs = {}
    if backend == "nccl":
        kwargs["device_id"] = torch.device("cuda", torch.cuda.current_device())
    dist.init_process_group(backend=backend, rank=rank, world_size=num_ranks, **kwargs)


def default_world() -> Optional[_WorldBase]:
    return _default_world


def set_default_world(world: Optional[_WorldBase]) -> None:
    global _default_world
    _default_world = world


def finalize_runtime() -> None:
    """Free every symmetric buffer and forget the default world (collective)."""
    global _default_world
    w = _default_world
    if w is None:
        return
    if isinstance(w, (ProcessWorld, EmulatedWorld)):
        w.release_multicast()
        for buf in list(w._buffers):
            w.free(buf)
        w.C.status_free(w.status_host)
    _default_world = None
