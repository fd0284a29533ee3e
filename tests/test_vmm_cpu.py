"""The virtual-memory / multicast allocator's host logic on CPU processes: descriptors travel over
Unix-domain sockets between gloo ranks, every rank maps every rank's allocation, the multicast
object is created once and bound by all, and the teardown unbinds before anything is released.
The driver is the native layer's in-process stand-in (memfd + mmap), so what one rank writes
through its mapping the others read through theirs."""
import ctypes
import os
import tempfile

from tridist_b200.utils.testing import spawn


def _words(ptr, n):
    return (ctypes.c_uint32 * n).from_address(ptr)


def _alloc_exchange_free(rank, R, outdir):
    import torch.distributed as dist

    from tridist_b200.parallel import vmm
    from tridist_b200.parallel.runtime import native
    C = native()
    C.vmm_use_fake_driver(True)
    alloc = vmm.alloc_symmetric_multicast(C, rank, R, None, 10000)
    assert alloc.nbytes % 4096 == 0 and alloc.nbytes >= 10000
    assert len(alloc.peer_ptrs) == R and all(alloc.peer_ptrs) and alloc.mc_ptr
    mine = _words(alloc.peer_ptrs[rank], 64)
    for i in range(64):
        mine[i] = 1000 * (rank + 1) + i
    dist.barrier()
    for r in range(R):                                   # every rank's copy through MY mapping of it
        theirs = _words(alloc.peer_ptrs[r], 64)
        assert [theirs[i] for i in range(64)] == [1000 * (r + 1) + i for i in range(64)]
    dist.barrier()
    log_alloc = C.vmm_fake_call_log()
    vmm.free_symmetric_multicast(C, None, alloc, R)
    log_free = C.vmm_fake_call_log()
    with open(os.path.join(outdir, f"rank{rank}.txt"), "w") as fh:
        fh.write(",".join(log_alloc) + "|" + ",".join(log_free))


def test_allocation_exchange_and_teardown_order():
    R = 3
    with tempfile.TemporaryDirectory() as d:
        spawn(_alloc_exchange_free, R, args=(d,), timeout=120)
        for r in range(R):
            a, f = open(os.path.join(d, f"rank{r}.txt")).read().split("|")
            a, f = a.split(","), f.split(",")
            assert a[0] == "create" and a.count("import") == (R - 1) + (0 if r == 0 else 1)
            assert a.count("map") == R and a.count("mc_map") + a.count("map") >= R
            assert ("mc_create:%d" % R in a) == (r == 0)
            assert a.index("mc_add_device") < a.index("mc_bind")
            # teardown: the multicast mapping goes and the memory is unbound before any release
            assert f.index("mc_unbind") < min(i for i, x in enumerate(f) if x.endswith("release"))
            assert f[-1] == "release" and f.count("release") == R and f.count("unmap") == R + 1


def _one_rank_fails(rank, R, outdir):
    from tridist_b200.parallel import vmm
    from tridist_b200.parallel.runtime import native
    C = native()
    C.vmm_use_fake_driver(True)

    class Broken:
        def __getattr__(self, name):
            real = getattr(C, name)
            if name == "vmm_map" and rank == 1:
                def boom(*a):
                    raise RuntimeError("cuMemMap failed: out of address space")
                return boom
            return real

    try:
        vmm.alloc_symmetric_multicast(Broken(), rank, R, None, 4096)
        out = "allocated"
    except RuntimeError as exc:
        out = str(exc)
    with open(os.path.join(outdir, f"rank{rank}.txt"), "w") as fh:
        fh.write(out)


def test_a_failing_rank_ends_the_allocation_everywhere():
    with tempfile.TemporaryDirectory() as d:
        spawn(_one_rank_fails, 2, args=(d,), timeout=120)
        texts = [open(os.path.join(d, f"rank{r}.txt")).read() for r in range(2)]
        assert texts[0] == texts[1] and "rank 1" in texts[0] and "cuMemMap failed" in texts[0]
