"""Symmetric buffers with an NVSwitch multicast mapping, allocated with the CUDA driver's
virtual-memory calls (native layer: ``csrc/runtime/vmm_heap.cu``).

What the reference gets from its symmetric heap (``malloc`` / ``ptr(addr, pe)``,
pydushmem/host.py:239-264) plus what B200 adds on top: one physical allocation per rank
(``cuMemCreate``), exported as a POSIX file descriptor, imported and mapped by every peer, and
one multicast object (``cuMulticastCreate`` on rank 0, ``cuMulticastAddDevice`` /
``cuMulticastBindMem`` on every rank) whose mapping names all ranks' copies at once: the address
kernels use with ``multimem.ld_reduce`` / ``multimem.st``.

File descriptors cannot travel through ``torch.distributed``; they are passed over Unix-domain
sockets (``SCM_RIGHTS``) whose abstract names the ranks agree on through the process group.
Every step is collective and every socket wait has a limit, so a rank that fails ends the
allocation on all ranks with a reason instead of leaving the others blocked.
"""
from __future__ import annotations

import os
import socket
import threading
import uuid
from dataclasses import dataclass, field
from typing import Dict, List, Optional

import torch.distributed as dist

_SOCKET_TIMEOUT_S = 20.0


def _sock_name(token: str, round_id: int, rank: int) -> str:
    return f"\0tridist-vmm-{token}-{round_id}-{rank}"          # abstract namespace: nothing to unlink


def exchange_fds(rank: int, num_ranks: int, token: str, round_id: int, offer_fd: Optional[int],
                 n_clients: int, fetch_from: List[int]) -> Dict[int, int]:
    """One round of descriptor passing. A rank with ``offer_fd`` serves it to ``n_clients`` peers;
    every rank fetches the descriptor offered by each rank in ``fetch_from``. Returns
    ``{source rank: received descriptor}`` (the caller closes them)."""
    server = None
    thread = None
    errors: List[str] = []
    if offer_fd is not None and n_clients > 0:
        server = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
        server.bind(_sock_name(token, round_id, rank))
        server.listen(num_ranks)
        server.settimeout(_SOCKET_TIMEOUT_S)

        def serve():
            try:
                for _ in range(n_clients):
                    conn, _ = server.accept()
                    with conn:
                        conn.settimeout(_SOCKET_TIMEOUT_S)
                        conn.recv(4)
                        socket.send_fds(conn, [b"fd"], [offer_fd])
            except Exception as exc:   # noqa: BLE001 - reported by the caller
                errors.append(f"serving descriptors: {type(exc).__name__}: {exc}")

        thread = threading.Thread(target=serve, daemon=True)
        thread.start()
    got: Dict[int, int] = {}
    try:
        for src in fetch_from:
            c = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
            c.settimeout(_SOCKET_TIMEOUT_S)
            import time
            deadline = time.monotonic() + _SOCKET_TIMEOUT_S
            while True:
                try:
                    c.connect(_sock_name(token, round_id, src))
                    break
                except (ConnectionRefusedError, FileNotFoundError):
                    if time.monotonic() > deadline:
                        raise TimeoutError(f"rank {src} never offered its descriptor")
                    time.sleep(0.01)
            with c:
                c.sendall(rank.to_bytes(4, "little"))
                _, fds, _, _ = socket.recv_fds(c, 16, 1)
                if len(fds) != 1:
                    raise RuntimeError(f"rank {src} sent {len(fds)} descriptors")
                got[src] = fds[0]
    finally:
        if thread is not None:
            thread.join(_SOCKET_TIMEOUT_S + 5)
        if server is not None:
            server.close()
    if errors:
        for fd in got.values():
            os.close(fd)
        raise RuntimeError("; ".join(errors))
    return got


@dataclass
class VmmAllocation:
    """Driver objects behind one symmetric multicast buffer (kept for the collective teardown)."""
    nbytes: int
    own_handle: int
    peer_handles: Dict[int, int] = field(default_factory=dict)
    peer_ptrs: List[int] = field(default_factory=list)
    mc_handle: int = 0
    mc_ptr: int = 0
    bound: bool = False


def _agree(group, why: str, num_ranks: int) -> List[str]:
    """Every rank's error text (empty = fine) on every rank."""
    out = [None] * num_ranks
    dist.all_gather_object(out, why, group=group)
    return [w or "" for w in out]


def alloc_symmetric_multicast(C, rank: int, num_ranks: int, group, nbytes: int) -> "VmmAllocation":
    """Collective. Raises ``RuntimeError`` (the same on every rank) when any rank fails; nothing stays
    allocated then."""
    tokens = [None] * num_ranks
    dist.all_gather_object(tokens, uuid.uuid4().hex if rank == 0 else None, group=group)
    token = tokens[0]
    alloc: Optional[VmmAllocation] = None
    received: Dict[int, int] = {}
    own_fd = mc_fd = -1
    why = ""
    try:
        gran = int(C.vmm_granularity(True, num_ranks))
        size = (int(nbytes) + gran - 1) // gran * gran
        own = int(C.vmm_create(size))
        alloc = VmmAllocation(nbytes=size, own_handle=own, peer_ptrs=[0] * num_ranks)
        own_fd = int(C.vmm_export_fd(own))
    except Exception as exc:   # noqa: BLE001
        why = f"{type(exc).__name__}: {exc}"
    errs = _agree(group, why, num_ranks)
    if not any(errs):
        try:   # first exchange: every rank offers its allocation to every peer
            received = exchange_fds(rank, num_ranks, token, 1, own_fd, num_ranks - 1,
                                    [r for r in range(num_ranks) if r != rank])
            for src, fd in received.items():
                alloc.peer_handles[src] = int(C.vmm_import_fd(fd))
            for r in range(num_ranks):
                h = alloc.own_handle if r == rank else alloc.peer_handles[r]
                alloc.peer_ptrs[r] = int(C.vmm_map(h, alloc.nbytes))
        except Exception as exc:   # noqa: BLE001
            why = f"{type(exc).__name__}: {exc}"
        errs = _agree(group, why, num_ranks)
    if not any(errs):
        try:   # second exchange: rank 0 creates the multicast object and offers it to the others
            if rank == 0:
                alloc.mc_handle = int(C.vmm_mc_create(alloc.nbytes, num_ranks))
                mc_fd = int(C.vmm_export_fd(alloc.mc_handle))
                exchange_fds(rank, num_ranks, token, 2, mc_fd, num_ranks - 1, [])
            else:
                got = exchange_fds(rank, num_ranks, token, 2, None, 0, [0])
                mc_fd = got[0]
                alloc.mc_handle = int(C.vmm_import_fd(mc_fd))
            C.vmm_mc_add_device(alloc.mc_handle)
        except Exception as exc:   # noqa: BLE001
            why = f"{type(exc).__name__}: {exc}"
        errs = _agree(group, why, num_ranks)          # also: every device is added before anyone binds
    if not any(errs):
        try:
            C.vmm_mc_bind(alloc.mc_handle, alloc.own_handle, alloc.nbytes)
            alloc.bound = True
            alloc.mc_ptr = int(C.vmm_map(alloc.mc_handle, alloc.nbytes))
        except Exception as exc:   # noqa: BLE001
            why = f"{type(exc).__name__}: {exc}"
        errs = _agree(group, why, num_ranks)
    for fd in list(received.values()) + [own_fd, mc_fd]:
        if fd is not None and fd >= 0:
            try:
                os.close(fd)
            except OSError:
                pass
    if any(errs):
        if alloc is not None:
            free_symmetric_multicast(C, group, alloc, num_ranks, collective=False)
        raise RuntimeError("; ".join(f"rank {r}: {e}" for r, e in enumerate(errs) if e))
    return alloc


def free_symmetric_multicast(C, group, alloc: "VmmAllocation", num_ranks: int, collective: bool = True) -> None:
    """Collective (unless ``collective=False``, the clean-up after a failed allocation): every rank
    unmaps and unbinds before any rank releases memory, so that no rank's memory is bound to a
    multicast object the others still use."""
    def barrier():
        if collective and num_ranks > 1:
            dist.barrier(group=group)

    barrier()
    if alloc.mc_ptr:
        C.vmm_unmap(alloc.mc_ptr, alloc.nbytes)
        alloc.mc_ptr = 0
    if alloc.bound:
        C.vmm_mc_unbind(alloc.mc_handle, alloc.nbytes)
        alloc.bound = False
    barrier()
    if alloc.mc_handle:
        C.vmm_release(alloc.mc_handle)
        alloc.mc_handle = 0
    for r, p in enumerate(alloc.peer_ptrs):
        if p:
            C.vmm_unmap(p, alloc.nbytes)
    alloc.peer_ptrs = [0] * len(alloc.peer_ptrs)
    for h in alloc.peer_handles.values():
        C.vmm_release(h)
    alloc.peer_handles = {}
    barrier()
    if alloc.own_handle:
        C.vmm_release(alloc.own_handle)
        alloc.own_handle = 0
