from .runtime import (CpuWorld, EmulatedWorld, ProcessWorld, SymmBuffer, TriDistError,  # noqa: F401
                      default_world, finalize_runtime, init_runtime, set_default_world)
