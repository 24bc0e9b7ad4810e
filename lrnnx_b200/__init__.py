"""lrnnx_b200 — sm_100a (B200) back end for the scan hot path of lrnnx.

The package provides, behind lrnnx's own call surface,
  * ``selective_scan_cuda`` / ``simplified_scan_cuda`` / ``structured_kernels``:
    modules with the ``fwd`` / ``bwd`` functions lrnnx's compiled extensions export,
  * ``lrnnx_b200.ops``: the autograd wrappers (``selective_scan_fn``,
    ``simplified_scan_fn``, ``s5_inner_fn``, ``rglru_scan_fn``, ``s7_scan_fn``,
    ``selective_state_update``, ``cauchy_mult``, ``log_vandermonde_cuda``),
  * ``install()``: registers the three extension modules in ``sys.modules`` under
    the names lrnnx imports, so unmodified lrnnx Python runs on these kernels.

All compute goes through ``lib/liblrnnx_b200.so`` (hand-written CUDA, C ABI in
``include/lrnnx_b200.h``).  There is no CPU or PyTorch fallback.
"""
from __future__ import annotations

import sys

__version__ = "0.1.0"


def install() -> None:
    """Make ``import selective_scan_cuda`` (and the two sibling extension modules
    lrnnx loads at import time: lrnnx/ops/selective_scan.py:11,
    lrnnx/ops/simplified_scan.py:10, csrc/s4/cauchy.py:6) resolve to this package."""
    from . import selective_scan_cuda, simplified_scan_cuda, structured_kernels

    sys.modules["selective_scan_cuda"] = selective_scan_cuda
    sys.modules["simplified_scan_cuda"] = simplified_scan_cuda
    sys.modules["structured_kernels"] = structured_kernels
