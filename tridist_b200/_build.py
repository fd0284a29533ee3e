"""In-tree build and load of the native extension ``tridist_b200._C``.

The extension is compiled for sm_100a only and the resulting shared object is
kept next to this file, so that a copy of the source tree carries a ready
binary.  A digest of the sources is stored beside it; a stale or missing binary
is rebuilt when a CUDA toolchain is present, and a clear error is raised
otherwise (GPU ops never fall back silently to another implementation).
"""
from __future__ import annotations

import hashlib
import importlib.machinery
import importlib.util
import os
import shutil
import sys
import threading

_PKG_DIR = os.path.dirname(os.path.abspath(__file__))
_CSRC = os.path.join(_PKG_DIR, "csrc")
_SO_NAME = "_C.so"
_DIGEST_NAME = "_C.digest"
_lock = threading.Lock()
_module = None

SOURCES = [
    "bindings.cpp",
    "runtime/symm_heap.cu",
    "runtime/vmm_heap.cu",
    "ops/fused_gemm.cu",
    "ops/elementwise.cu",
    "ops/moe_a2a.cu",
    "ops/rd_exchange.cu",
    "ops/moe_local_noalloc.cu",
]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr",
    "-Xptxas", "-v",
]


def _source_files():
    out = []
    for root, _, files in os.walk(_CSRC):
        for f in sorted(files):
            if f.endswith((".cu", ".cuh", ".cpp", ".h")):
                out.append(os.path.join(root, f))
    return sorted(out)


def source_digest() -> str:
    h = hashlib.sha256()
    for path in _source_files():
        h.update(os.path.relpath(path, _CSRC).encode())
        with open(path, "rb") as fh:
            h.update(fh.read())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def _so_path() -> str:
    return os.path.join(_PKG_DIR, _SO_NAME)


def is_fresh() -> bool:
    so, dg = _so_path(), os.path.join(_PKG_DIR, _DIGEST_NAME)
    if not (os.path.exists(so) and os.path.exists(dg)):
        return False
    with open(dg) as fh:
        return fh.read().strip() == source_digest()


def build(verbose: bool = False) -> str:
    """Compile the extension into this package directory and return the path."""
    import torch  # noqa: F401  (cpp_extension needs torch importable)
    from torch.utils import cpp_extension

    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0a")
    build_dir = os.path.join(_PKG_DIR, "build")
    os.makedirs(build_dir, exist_ok=True)
    sources = [os.path.join(_CSRC, s) for s in SOURCES if os.path.exists(os.path.join(_CSRC, s))]
    cpp_extension.load(
        name="_C",
        sources=sources,
        extra_cflags=["-O3", "-std=c++17"],
        extra_cuda_cflags=NVCC_FLAGS,
        extra_ldflags=["-lcuda"] if False else [],
        build_directory=build_dir,
        verbose=verbose,
        is_python_module=False,
        is_standalone=False,
    )
    built = os.path.join(build_dir, "_C.so")
    shutil.copy2(built, _so_path())
    with open(os.path.join(_PKG_DIR, _DIGEST_NAME), "w") as fh:
        fh.write(source_digest())
    return _so_path()


def load():
    """Return the loaded extension module, building it first if needed."""
    global _module
    with _lock:
        if _module is not None:
            return _module
        if not is_fresh():
            if shutil.which("nvcc") is None and not os.path.exists("/usr/local/cuda/bin/nvcc"):
                if not os.path.exists(_so_path()):
                    raise RuntimeError(
                        "tridist_b200: the native extension is not built and no nvcc is available; "
                        "run `python -c 'import __graft_entry__ as g; g.build()'` on a machine with CUDA 12.9")
            else:
                build()
        import torch  # noqa: F401  (libtorch symbols must be loaded first)
        loader = importlib.machinery.ExtensionFileLoader("tridist_b200._C", _so_path())
        spec = importlib.util.spec_from_file_location("tridist_b200._C", _so_path(), loader=loader)
        mod = importlib.util.module_from_spec(spec)
        loader.exec_module(mod)
        sys.modules["tridist_b200._C"] = mod
        _module = mod
        return mod
