"""The allocation-free MoE dispatch entry point, called through its exported C symbol.

Some callers may not allocate device memory while they run (everything was given
to a cache or pool at start-up, or an allocation's implicit synchronisation is
not acceptable on their path). For them the library exports
``tdb_moe_local_dispatch_noalloc``: the single-rank dispatch with its scratch in a
fixed array inside the library instead of context-owned tensors. This test calls
it twice in a row through ctypes and checks its outputs against the regular
single-rank dispatch (``moe_dispatch_intra_node_op``), with the tolerance of the
other MoE tests (rows are copied, so they must match exactly).

Collected last on purpose (file name): a run that stops at the first failure has
then already run every other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from tridist_b200.parallel.runtime import native
    C = native()                                   # loads libtorch + the extension first
    lib = ctypes.CDLL(C.__file__)
    fn = lib.tdb_moe_local_dispatch_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                   ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                   ctypes.c_int64, ctypes.c_void_p]
    lib.tdb_noalloc_strerror.restype = ctypes.c_char_p
    lib.tdb_noalloc_strerror.argtypes = [ctypes.c_int]
    return lib, fn


def test_no_alloc_dispatch_matches_regular_entry_point():
    from tridist_b200.ops import create_moe_a2a_intra_node_context, moe_dispatch_intra_node_op
    from tridist_b200.parallel.runtime import ProcessWorld
    from tridist_b200.utils.testing import moe_inputs
    lib, fn = _lib()
    world = ProcessWorld(0, 1)
    dt = torch.float16
    E, H, topk, T = 16, 512, 4, 300
    ctx = create_moe_a2a_intra_node_context(E, H, dt, T, topk, 0, 1, world=world)
    # outputs of the new entry point: allocated here, once, by the caller
    recv = torch.empty((T * topk, H), dtype=dt, device="cuda")
    scatter = torch.empty((T, topk), dtype=torch.int32, device="cuda")
    seg = torch.empty(E, dtype=torch.int32, device="cuda")
    total = torch.empty(1, dtype=torch.int32, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    for call in range(2):                           # two calls in a row share the scratch array
        tokens, idx, _ = [x.cuda() for x in moe_inputs(0, T, H, E, topk, 40 + call, dt, 1.2 if call else 0.0)]
        n_ref = int(moe_dispatch_intra_node_op(tokens, idx, ctx).item())
        torch.cuda.synchronize()
        world.check()
        rc = fn(tokens.data_ptr(), idx.data_ptr(), recv.data_ptr(), scatter.data_ptr(), seg.data_ptr(),
                total.data_ptr(), T, H, topk, E, recv.shape[0], stream)
        assert rc == 0, lib.tdb_noalloc_strerror(rc).decode()
        torch.cuda.synchronize()
        # same segment table and row count as the regular path (R = 1: recv_seg is [1, E])
        assert int(total.item()) == n_ref == T * topk
        assert torch.equal(seg, ctx.recv_seg.flatten())
        # same rows: every (t, j) lands in its expert's segment and carries token t
        sc_new, sc_ref = scatter.long(), ctx.scatter_idx[:T].long()
        assert sorted(sc_new.flatten().tolist()) == list(range(n_ref))
        counts = ctx.recv_counts.flatten().long()
        lo = seg.long()[idx.long()]
        assert bool(((sc_new >= lo) & (sc_new < lo + counts[idx.long()])).all())
        got_new = recv[sc_new.flatten()].view(T, topk, H)
        got_ref = ctx.recv[sc_ref.flatten()].view(T, topk, H)
        assert (got_new.float() - got_ref.float()).abs().max().item() == 0.0
        assert torch.equal(got_new[:, 0], tokens)


def test_no_alloc_dispatch_rejects_oversize():
    lib, fn = _lib()
    dummy = torch.zeros(64, dtype=torch.int32, device="cuda")
    p = dummy.data_ptr()
    rc = fn(p, p, p, p, p, p, 4, 64, 2, 1025, 8, None)            # more experts than the scratch holds
    assert rc == -2 and b"1024" in lib.tdb_noalloc_strerror(rc)
    assert fn(p, p, p, p, p, p, 4, 60, 2, 8, 8, None) == -4       # hidden not a multiple of 8
    assert fn(p, p, p, p, p, p, 4, 64, 2, 8, 7, None) == -5       # recv too small for T * topk rows
    assert fn(p, p, p, p, p, p, 4, 64, 33, 8, 200, None) == -3    # topk too large
    # a view that starts 4 bytes into its buffer: refused here, not a misaligned-address fault on the GPU
    rc = fn(p + 4, p, p, p, p, p, 4, 64, 2, 8, 8, None)
    assert rc == -7 and b"16-byte" in lib.tdb_noalloc_strerror(rc)
    assert fn(p, p, p + 8, p, p, p, 4, 64, 2, 8, 8, None) == -7
