from .runtime import (CpuWorld, EmulatedWorld, ProcessWorld, SymmBuffer, TriDistError,  # noqa: F401
                      default_world, finalize_runtime, init_runtime, set_default_world)
from .runtime import McBuffer  # noqa: F401,E402
from .liveness import LivenessBoard, PeerLeft  # noqa: F401,E402
from .predictor import StickyOrderPredictor, infer_straggler  # noqa: F401,E402
from .symm_host import SymmHost  # noqa: F401,E402
