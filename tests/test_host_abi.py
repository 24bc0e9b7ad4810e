"""CPU-side checks: the C-ABI library loads, exports every symbol the header declares, the
parsed argument-block layouts agree with the compiled ones, and argument validation rejects
bad calls before anything is launched (no compute calls here; no GPU needed)."""
from __future__ import annotations

import ctypes

import pytest
import torch

from lrnnx_b200 import _lib


def test_library_exports_every_declared_symbol():
    lib = _lib.lib()
    structs, enums, functions = _lib.parse_header()
    assert set(functions) == set(_lib.ENTRY_POINTS)
    for fn in functions:
        assert hasattr(lib, fn), f"{fn} declared in include/lrnnx_b200.h but not exported"
    assert lib.b200_abi_version() >= 1


def test_struct_layouts_match_library():
    lib = _lib.lib()
    structs = _lib.parse_header()[0]
    assert len(structs) >= 6
    for name, st in structs.items():
        assert lib.b200_sizeof(name.encode()) == ctypes.sizeof(st), name
    assert lib.b200_sizeof(b"no_such_struct") == -1


def test_enums_follow_reference_order():
    # csrc/selective_scan/selective_scan.h:14-21 and the Triton map at
    # lrnnx/ops/triton/selective_state_update.py:374-382
    assert [_lib.enum(n) for n in ("B200_DISC_ZOH", "B200_DISC_BILINEAR", "B200_DISC_DIRAC", "B200_DISC_MAMBA",
                                   "B200_DISC_RGLRU", "B200_DISC_S7")] == [0, 1, 2, 3, 4, 5]


def test_null_and_range_checks_return_errors_without_launching():
    lib = _lib.lib()
    a = _lib.struct("b200_selscan_fwd_args")()
    assert lib.b200_selscan_fwd(ctypes.byref(a), None) == _lib.enum("B200_ERR_NULL")
    assert b"non-null" in lib.b200_last_error()
    assert lib.b200_selscan_fwd(None, None) == _lib.enum("B200_ERR_NULL")
    buf = (ctypes.c_float * 64)()
    p = ctypes.addressof(buf)
    a.u = a.delta = a.A = a.B = a.C = a.out = a.x = p
    a.batch = a.dim = a.seqlen = a.n_groups = 1
    a.dstate = 300
    assert lib.b200_selscan_fwd(ctypes.byref(a), None) == _lib.enum("B200_ERR_SHAPE")
    assert b"<= 256" in lib.b200_last_error()
    a.dstate, a.method = 4, 17
    assert lib.b200_selscan_fwd(ctypes.byref(a), None) == _lib.enum("B200_ERR_DTYPE")
    a.method, a.is_complex = _lib.enum("B200_DISC_S7"), 1
    assert lib.b200_selscan_fwd(ctypes.byref(a), None) == _lib.enum("B200_ERR_DTYPE")
    s = _lib.struct("b200_simpscan_args")()
    assert lib.b200_simpscan_fwd(ctypes.byref(s), None) == _lib.enum("B200_ERR_NULL")
    q = _lib.struct("b200_s4_args")()
    assert lib.b200_cauchy_bwd(ctypes.byref(q), None) == _lib.enum("B200_ERR_NULL")
    u = _lib.struct("b200_ssu_args")()
    assert lib.b200_ssu_step(ctypes.byref(u), None) == _lib.enum("B200_ERR_NULL")


def test_scratch_size_query():
    lib = _lib.lib()
    assert lib.b200_s4_bwd_scratch_bytes(0, 1, 1) == 0
    small = lib.b200_s4_bwd_scratch_bytes(4, 2, 17)
    assert small == 4 * 2 * 1 * 2 * 8
    assert lib.b200_s4_bwd_scratch_bytes(4, 2, 1 << 18) > small


def test_python_shims_validate_like_the_reference():
    """Host-side checks mirror the reference's TORCH_CHECKs (selective_scan_cpu.cpp:271-378) and
    fire before any device work, so they can be exercised with CPU tensors."""
    from lrnnx_b200 import selective_scan_cuda, simplified_scan_cuda, structured_kernels
    u = torch.randn(1, 2, 8)
    A = -torch.rand(2, 4)
    with pytest.raises(RuntimeError, match="CUDA"):
        selective_scan_cuda.fwd(u, u, A, A, A, None, None, None, None, False, "mamba")
    with pytest.raises(RuntimeError, match="Discretization method not supported"):
        selective_scan_cuda.fwd(u, u, A, A, A, None, None, None, None, False, "euler")
    with pytest.raises(RuntimeError, match="S7 discretization only supports real"):
        selective_scan_cuda.fwd(u, u, A.to(torch.complex64), A.to(torch.complex64), A.to(torch.complex64), None,
                                None, None, None, False, "s7")
    with pytest.raises(RuntimeError, match="dtype"):
        selective_scan_cuda.fwd(u, u.double(), A, A, A, None, None, None, None, False, "mamba")
    with pytest.raises(RuntimeError, match="complex64"):
        simplified_scan_cuda.fwd(u, u, A, A, A, None, "zoh")
    with pytest.raises(RuntimeError, match="CUDA"):
        structured_kernels.cauchy_mult_sym_fwd(torch.randn(2, 4, dtype=torch.complex64),
                                               torch.randn(8, dtype=torch.complex64),
                                               torch.randn(2, 4, dtype=torch.complex64))


def test_install_registers_extension_modules():
    import sys
    import lrnnx_b200
    saved = {k: sys.modules.get(k) for k in ("selective_scan_cuda", "simplified_scan_cuda", "structured_kernels")}
    try:
        lrnnx_b200.install()
        import selective_scan_cuda, simplified_scan_cuda, structured_kernels  # noqa: F401
        assert selective_scan_cuda.fwd.__module__ == "lrnnx_b200.selective_scan_cuda"
        assert hasattr(simplified_scan_cuda, "bwd") and hasattr(structured_kernels, "vand_log_mult_sym_bwd")
    finally:
        for k, v in saved.items():
            if v is None:
                sys.modules.pop(k, None)
            else:
                sys.modules[k] = v


def test_every_python_module_of_the_package_imports():
    """Import errors in modules that only the GPU tests use must show up without a GPU."""
    import importlib
    import pkgutil

    import lrnnx_b200
    for mod in pkgutil.walk_packages(lrnnx_b200.__path__, "lrnnx_b200."):
        if mod.name.endswith(".build"):
            continue
        importlib.import_module(mod.name)
