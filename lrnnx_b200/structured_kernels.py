"""Drop-in for lrnnx's compiled ``structured_kernels`` module (S4 kernels).

Same four functions as csrc/s4/cauchy.cpp:93-102 with the checks of
csrc/s4/cauchy.cpp:20-53,64-89: symmetric Cauchy multiply and log-Vandermonde
multiply, forward and backward, on contiguous complex64 CUDA tensors.
"""
from __future__ import annotations

import torch

from . import _lib


def _check(cond: bool, msg: str) -> None:
    if not cond:
        raise RuntimeError(msg)


def _stream(t) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def _args(v, z, w, seqlen):
    a = _lib.struct("b200_s4_args")()
    a.batch, a.n, a.seqlen = v.size(0), v.size(1), seqlen
    a.v, a.w = v.data_ptr(), w.data_ptr()
    a.z = None if z is None else z.data_ptr()
    return a


def _c64(name, t, *shape):
    _check(t.is_cuda, f"{name} must be on CUDA")
    _check(t.dtype == torch.complex64, f"{name} must be complex64")
    _check(tuple(t.shape) == tuple(shape), f"{name} must have shape {tuple(shape)}")
    return t.contiguous()


def _scratch(a, device):
    nbytes = _lib.lib().b200_s4_bwd_scratch_bytes(a.batch, a.n, a.seqlen)
    buf = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=device)
    a.scratch, a.scratch_bytes = buf.data_ptr(), nbytes
    return buf


def cauchy_mult_sym_fwd(v, z, w):
    """v, w (batch, N) complex64 (half spectrum), z (L,) complex64 -> (batch, L) complex64."""
    _check(v.dim() == 2 and z.dim() == 1, "v must be (batch, N) and z (L,)")
    batch, n = v.shape
    L = z.size(0)
    v, z, w = _c64("v", v, batch, n), _c64("z", z, L), _c64("w", w, batch, n)
    with torch.cuda.device(v.device):
        out = torch.empty((batch, L), dtype=v.dtype, device=v.device)
        a = _args(v, z, w, L)
        a.out = out.data_ptr()
        _lib.call("b200_cauchy_fwd", a, _stream(v))
    return out


def cauchy_mult_sym_bwd(v, z, w, dout):
    """-> (dv, dw), each (batch, N) complex64."""
    batch, n = v.shape
    L = z.size(0)
    v, z, w = _c64("v", v, batch, n), _c64("z", z, L), _c64("w", w, batch, n)
    dout = _c64("dout", dout, batch, L)
    with torch.cuda.device(v.device):
        dv, dw = torch.empty_like(v), torch.empty_like(w)
        a = _args(v, z, w, L)
        a.dout, a.dv, a.dw = dout.data_ptr(), dv.data_ptr(), dw.data_ptr()
        keep = _scratch(a, v.device)
        _lib.call("b200_cauchy_bwd", a, _stream(v))
        del keep   # safe: the caching allocator reuses the block in stream order
    return dv, dw


def vand_log_mult_sym_fwd(v, x, L):
    """v, x (batch, N) complex64 -> (batch, L) float32 = 2 Re sum_n v exp(x l)."""
    _check(v.dim() == 2, "v must be (batch, N)")
    batch, n = v.shape
    v, x = _c64("v", v, batch, n), _c64("x", x, batch, n)
    L = int(L)
    with torch.cuda.device(v.device):
        out = torch.empty((batch, L), dtype=torch.float32, device=v.device)
        a = _args(v, None, x, L)
        a.out = out.data_ptr()
        _lib.call("b200_vand_fwd", a, _stream(v))
    return out


def vand_log_mult_sym_bwd(v, x, dout):
    """-> (dv, dx), each (batch, N) complex64."""
    batch, n = v.shape
    v, x = _c64("v", v, batch, n), _c64("x", x, batch, n)
    _check(dout.is_cuda and dout.dtype == torch.float32 and dout.dim() == 2 and dout.size(0) == batch,
           "dout must be a (batch, L) float32 CUDA tensor")
    dout = dout.contiguous()
    L = dout.size(1)
    with torch.cuda.device(v.device):
        dv, dx = torch.empty_like(v), torch.empty_like(x)
        a = _args(v, None, x, L)
        a.dout, a.dv, a.dw = dout.data_ptr(), dv.data_ptr(), dx.data_ptr()
        keep = _scratch(a, v.device)
        _lib.call("b200_vand_bwd", a, _stream(v))
        del keep
    return dv, dx
