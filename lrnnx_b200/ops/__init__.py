"""Autograd wrappers with the names and signatures of ``lrnnx.ops``
(lrnnx/ops/__init__.py:1-25)."""
from .rglru_scan import RGLRUScanFn, rglru_scan_fn
from .s4 import cauchy_mult, log_vandermonde_cuda, log_vandermonde_fast
from .s7_scan import S7ScanFn, s7_scan_fn
from .selective_state_update import selective_state_update
from .selective_scan import SelectiveScanFn, selective_scan_fn
from .simplified_state_update import simplified_state_update
from .simplified_scan import S5InnerFn, SimplifiedScanFn, s5_inner_fn, simplified_scan_fn

__all__ = ["SelectiveScanFn", "selective_scan_fn", "RGLRUScanFn", "rglru_scan_fn", "S7ScanFn", "s7_scan_fn",
           "SimplifiedScanFn", "simplified_scan_fn", "S5InnerFn", "s5_inner_fn",
           "selective_state_update", "simplified_state_update", "cauchy_mult", "log_vandermonde_cuda", "log_vandermonde_fast"]
