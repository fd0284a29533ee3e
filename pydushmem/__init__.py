"""Import-path alias of the reference's host binding package: the one-sided host calls
(``init / malloc / free / ptr / putmem / getmem / quiet / fence / barrier_all / my_pe / n_pes``) map onto
tridist_b200.parallel.symm_host. There is no MPI here: ``host.mpi_init()`` returns placeholders."""
from tridist_b200.parallel.symm_host import SymmHost, get_host, init  # noqa: F401

from . import host  # noqa: F401,E402


def _delegate(name):
    def f(*a, **k):
        return getattr(get_host(), name)(*a, **k)
    f.__name__ = name
    return f


for _n in ("malloc", "calloc", "align", "free", "ptr", "putmem", "putmem_nbi", "getmem", "getmem_nbi", "quiet",
           "fence", "barrier_all", "my_pe", "n_pes", "finalize"):
    globals()[_n] = _delegate(_n)


def get_uniqueid() -> bytes:
    """The reference exchanges a library unique id before ``init`` (pydushmem/__init__.py:22-35); the
    rendezvous here is torch.distributed's, so the id carries no information."""
    return b"tridist_b200"
