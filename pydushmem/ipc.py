"""The reference's raw IPC pointer list (pydushmem/ipc.py:79-116) on top of the symmetric heap:
one device allocation per rank, every peer's copy mapped into this process, and the table of
peer addresses as an int64 device tensor for kernels that index peers by rank."""
import torch

from tridist_b200.parallel.runtime import default_world


class IpcPtrList:
    def __init__(self, nbytes, mpi=None, comm=None, size=None, rank=None):
        world = default_world()
        if world is None:
            raise RuntimeError("initialise the runtime first (pydushmem.init or init_runtime)")
        if size is not None and size != world.num_ranks:
            raise ValueError("size differs from the initialised world")
        self.world = world
        self.nbytes = int(nbytes)
        self._buf = world.alloc(self.nbytes, world.rank)      # collective
        self.own = self._buf.local_ptr
        self.ptrs = list(self._buf.peer_ptrs)
        self.buffers = torch.tensor(self.ptrs, dtype=torch.int64, device="cuda")

    def free(self):
        """Collective: unmap the peers' copies and release the local one."""
        if self._buf is not None:
            self.world.free(self._buf)
            self._buf = None
            self.own = None
            self.ptrs = []
