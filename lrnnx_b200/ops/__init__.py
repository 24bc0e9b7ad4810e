"""Autograd wrappers with the names and signatures of ``lrnnx.ops``
(lrnnx/ops/__init__.py:1-25)."""
from .rglru_scan import RGLRUScanFn, rglru_scan_fn
from .s7_scan import S7ScanFn, s7_scan_fn
from .selective_scan import SelectiveScanFn, selective_scan_fn

__all__ = ["SelectiveScanFn", "selective_scan_fn", "RGLRUScanFn", "rglru_scan_fn", "S7ScanFn", "s7_scan_fn"]
