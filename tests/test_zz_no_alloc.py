"""b200_cauchy_bwd_static: the Cauchy backward for hosts that cannot give the library any
device memory beyond the call's own tensors (a C program using the ABI without a framework
allocator, or a serving loop with a frozen memory budget).  It must return what
b200_cauchy_bwd returns, call after call, although every call reuses the same built-in
scratch area; and it must refuse problems that do not fit that area.

Collected last on purpose: a failure here cannot hide the result of any other test.
"""
from __future__ import annotations

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _cauchy_bwd(entry, v, z, w, dout, scratch=None, outputs=None, bogus_scratch=False):
    from lrnnx_b200 import _lib
    a = _lib.struct("b200_s4_args")()
    a.batch, a.n, a.seqlen = v.size(0), v.size(1), z.size(0)
    a.v, a.z, a.w, a.dout = v.data_ptr(), z.data_ptr(), w.data_ptr(), dout.data_ptr()
    dv, dw = outputs if outputs is not None else (torch.empty_like(v), torch.empty_like(w))
    a.dv, a.dw = dv.data_ptr(), dw.data_ptr()
    if scratch is not None:
        a.scratch, a.scratch_bytes = scratch.data_ptr(), scratch.numel()
    if bogus_scratch:
        a.scratch, a.scratch_bytes = 0x10, 1     # documented as ignored by the static entry point
    _lib.call(entry, a, torch.cuda.current_stream().cuda_stream)
    return dv, dw


def test_static_scratch_matches_regular_entry_point_twice():
    from lrnnx_b200 import _lib
    lib = _lib.lib()
    g = torch.Generator().manual_seed(2357)
    c = lambda *s: torch.complex(torch.randn(*s, generator=g), torch.randn(*s, generator=g)).cuda()
    # two different problems back to back: the second must not see leftovers of the first
    for batch, n, L in ((16, 32, 20000), (5, 8, 3000)):
        v, w, z, dout = c(batch, n), c(batch, n), c(L), c(batch, L)
        need = lib.b200_s4_bwd_scratch_bytes(batch, n, L)
        scratch = torch.empty(need, dtype=torch.uint8, device="cuda")
        dv_ref, dw_ref = _cauchy_bwd("b200_cauchy_bwd", v, z, w, dout, scratch)
        dv, dw = _cauchy_bwd("b200_cauchy_bwd_static", v, z, w, dout)
        torch.cuda.synchronize()
        # same kernels, same fold order: the tolerance of tests/test_gpu_s4.py is met with room to spare
        torch.testing.assert_close(dv, dv_ref, rtol=2e-4, atol=1e-6)
        torch.testing.assert_close(dw, dw_ref, rtol=2e-4, atol=1e-6)
        # The property in the entry point's name: a further call into preallocated outputs changes
        # neither the device's free memory nor the framework allocator's counters.  The `scratch`
        # field is documented as ignored; a bogus value there must not change the result.
        outputs = (torch.empty_like(v), torch.empty_like(w))
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        stats_before = torch.cuda.memory_stats()
        _cauchy_bwd("b200_cauchy_bwd_static", v, z, w, dout, outputs=outputs, bogus_scratch=True)
        torch.cuda.synchronize()
        stats_after = torch.cuda.memory_stats()
        assert torch.cuda.mem_get_info()[0] == free_before
        for key in ("allocation.all.allocated", "segment.all.allocated", "reserved_bytes.all.current"):
            assert stats_after[key] == stats_before[key], key
        assert torch.equal(outputs[0], dv) and torch.equal(outputs[1], dw)


def test_static_scratch_rejects_oversized_problem():
    from lrnnx_b200 import _lib
    lib = _lib.lib()
    batch, n, L = 4096, 1024, 1 << 20
    assert lib.b200_s4_bwd_scratch_bytes(batch, n, L) > 4 * 1024 * 1024
    a = _lib.struct("b200_s4_args")()
    a.batch, a.n, a.seqlen = batch, n, L
    dummy = torch.zeros(16, device="cuda")
    a.v = a.z = a.w = a.dout = a.dv = a.dw = dummy.data_ptr()   # never dereferenced: the size check comes first
    rc = lib.b200_cauchy_bwd_static(ctypes.byref(a), None)
    assert rc == _lib.enum("B200_ERR_TOO_LARGE")
    assert b"built-in area" in lib.b200_last_error()
