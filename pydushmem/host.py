"""Placeholders for the reference's MPI bootstrap calls (pydushmem/host.py:31-61): rank and size come from
the torchrun environment, there is no MPI communicator."""
import os


def mpi_init():
    return None, None


def mpi_comm_rank(mpi=None, comm=None):
    return int(os.environ.get("RANK", "0"))


def mpi_comm_size(mpi=None, comm=None):
    return int(os.environ.get("WORLD_SIZE", "1"))
