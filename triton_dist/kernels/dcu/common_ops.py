"""Alias of the runtime layer: ``init_dcu`` / ``dcu_state`` / ``barrier_all_on_stream`` map onto
tridist_b200.parallel.runtime."""
from tridist_b200.parallel.runtime import default_world, init_runtime


def init_dcu(mpi, comm, rank, num_ranks):
    return init_runtime(rank, num_ranks, comm)


def dcu_state():
    return default_world()


def barrier_all_on_stream(stream=None):
    default_world().barrier_on_stream()
