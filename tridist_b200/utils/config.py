"""Environment-variable knobs.

The reference configures itself through constructor keywords, module constants
and environment variables (``TD_PUSH_STREAMS``, ``RD_WAIT_MODE``, ``I1_VERIFY`` ...,
triton_dist/kernels/dcu/common_ops.py:92-97, ag_tr_pred.py:85-170).  The knobs
that still mean something on B200 are read here, under the ``TRIDIST_`` prefix.

TRIDIST_WAIT_TIMEOUT_MS   limit of every in-kernel wait (default 4000)
TRIDIST_MAX_CTAS          cap on the persistent grid of the fused GEMM kernels
TRIDIST_FORCE_BN          128 or 256: override the output-tile width heuristic
TRIDIST_CTA_PAIR          0: never run 256-wide tiles on CTA pairs (2-CTA tcgen05 MMA); default 1
TRIDIST_WIDE              0: never use the 512 x 256 pair tile (two 128-row blocks per CTA); default 1
TRIDIST_SPLITK            0: never cut the tiles of the last, partial round along K; default 1
TRIDIST_RASTER_G          row units per raster group (default: as many as keep a group's A slab within 48 MB)
TRIDIST_L2_AHEAD          k-blocks of L2 look-ahead the operand loads request (default 0 = none: measured slower on every shape tried)
TRIDIST_PUSH_CTAS         CTAs that drive the all-gather push (default: from the shard size and the time the
                          GEMM takes, 34 GB/s per CTA up to the link's 560 GB/s; 0 = all)
TRIDIST_PUSH_SKIP         scheduling rounds the pushing CTAs sit out (default: what their push costs them)
TRIDIST_AG_TICKET_ROWS    rows of a gathered shard covered by one arrival ticket (default 256)
TRIDIST_AG_TRANSPORT      "auto" | "push" | "mc" | "pull": how the all-gather shard travels (auto = push: bulk copies
                          by a few CTAs; mc = multicast stores through the switch; pull = consumers copy)
TRIDIST_RD_TRANSPORT      "rd" (default: panel exchange with XOR partners) | "mesh" (the fused all-reduce kernel)
                          for the gemm_ar_rd entry points; TRIDIST_RD_CTAS = CTAs of the exchange kernel (16)
TRIDIST_RS_MODE           "auto" | "slots" | "nvls": reduce-scatter through peer-written slots or through the
                          switch (multimem.ld_reduce by the owner); auto = nvls wherever a multicast buffer exists
TRIDIST_RS_REDUCE_CTAS    switch-reduced reduce-scatter: CTAs whose communication warps reduce during the mainloop
                          (default 0 = all); TRIDIST_RS_REDUCE_TAIL = last blocks every CTA helps with
TRIDIST_DEBUG             1: before a plan is created, replay its tile schedule on the host and check every
                          ticket index and buffer offset against the buffers' sizes (nothing is launched)
TRIDIST_CHECK_RESIDENCY   0: skip the check at plan creation that the whole grid of a kernel whose CTAs wait on
                          peers can be resident at once (default 1)
TRIDIST_PROF              1: collect per-CTA stall accounting of the fused GEMM kernels
TRIDIST_AR_MODE           "auto" | "one_shot" | "two_shot" | "nvls"
TRIDIST_AR_ONE_SHOT_BYTES size threshold (bytes of one rank's partial) below which
                          the one-shot all-reduce is used (default 4 MiB; peer-store algorithms)
TRIDIST_AR2_ORDER         "interleave" (default: every rank walks the units in the same order) | "own_last"
TRIDIST_NVLS              0: never bind buffers to an NVSwitch multicast object (default 1)
TRIDIST_MC_ALLOC          "native" (default: cuMemCreate / cuMulticast* in csrc/runtime/vmm_heap.cu) | "torch"
                          (torch's symmetric-memory allocator) for the multicast-bound buffers
TRIDIST_NVLS_SELFTEST     0: skip the known-integers check of the switch path at context creation
TRIDIST_AR_NVLS_MIN_BYTES result size from which "auto" uses the switch-reduced all-reduce (default 0)
TRIDIST_POLL_NS           pause between two polls of a cross-rank ticket (default 0: back to back)
TRIDIST_EMU_PAIR          0: emulated multi-rank launches (one GPU) use single CTAs instead of CTA pairs
TRIDIST_VERIFY            1: spot-verify fused AG+GEMM results and repair flagged tiles
TRIDIST_VERIFY_SPOTS      elements recomputed per tile (default 4)
TRIDIST_VERIFY_TOL        relative tolerance of the spot check (default 2e-2)
"""
from __future__ import annotations

import os


def env_int(name: str, default: int) -> int:
    v = os.environ.get(name)
    if v is None or v == "":
        return default
    return int(v)


def env_float(name: str, default: float) -> float:
    v = os.environ.get(name)
    if v is None or v == "":
        return default
    return float(v)


def env_str(name: str, default: str) -> str:
    v = os.environ.get(name)
    return default if v is None or v == "" else v


def env_flag(name: str, default: bool = False) -> bool:
    v = os.environ.get(name)
    if v is None or v == "":
        return default
    return v.lower() not in ("0", "false", "no", "off")
