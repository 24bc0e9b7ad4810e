"""Drop-in for lrnnx's compiled ``simplified_scan_cuda`` module.

``fwd`` / ``bwd`` keep the signatures bound in csrc/simplified_scan/bindings.cpp:5-8
(declared in csrc/simplified_scan/simplified_scan.h:98-109) and the checks,
allocations and return lists of simplified_scan_fwd / simplified_scan_bwd
(csrc/simplified_scan/simplified_scan_cpu.cpp:160-331).
"""
from __future__ import annotations

import torch

from . import _lib

_METHODS = {"zoh": "B200_DISC_ZOH", "bilinear": "B200_DISC_BILINEAR", "dirac": "B200_DISC_DIRAC"}
CHUNK = 2048


def _check(cond: bool, msg: str) -> None:
    if not cond:
        raise RuntimeError(msg)


def _common(u, delta, A, B, C, deltaA, discretization):
    _check(u.dtype == torch.complex64, "u must be complex64")
    _check(A.dtype == torch.complex64, "A must be complex64")
    _check(delta.dtype == torch.float32, "delta must be float32")
    _check(B.dtype == torch.complex64 and C.dtype == torch.complex64, "B and C must be complex64")
    _check(discretization in _METHODS, "Discretization method not supported")
    for name, t in (("u", u), ("delta", delta), ("A", A), ("B", B), ("C", C)):
        _check(t.is_cuda, f"{name} must be a CUDA tensor")
    _check(u.dim() == 3 and A.dim() == 2, "u must be (batch, dim, seqlen) and A (dim, dstate)")
    _check(u.stride(-1) == 1 or u.size(-1) == 1, "u must be contiguous in the last dimension")
    _check(delta.stride(-1) == 1 or delta.size(-1) == 1, "delta must be contiguous in the last dimension")
    batch, dim, seqlen = u.shape
    dstate = A.size(1)
    _check(dstate <= 256, "simplified_scan only supports state dimension <= 256")
    _check(tuple(delta.shape) == (batch, dim, seqlen), "delta must have shape (batch, dim, seqlen)")
    for name, t in (("A", A), ("B", B), ("C", C)):
        _check(tuple(t.shape) == (dim, dstate), f"{name} must have shape (dim, dstate)")
    if deltaA is not None:
        _check(deltaA.dtype == torch.float32 and deltaA.is_cuda, "deltaA must be a float32 CUDA tensor")
        _check(deltaA.stride(-1) == 1 or deltaA.size(-1) == 1, "deltaA must be contiguous in the last dimension")
        _check(tuple(deltaA.shape) == (batch, dim, seqlen), "deltaA must have shape (batch, dim, seqlen)")
    a = _lib.struct("b200_simpscan_args")()
    a.batch, a.dim, a.seqlen, a.dstate = batch, dim, seqlen, dstate
    a.method = _lib.enum(_METHODS[discretization])
    a.u, a.delta, a.A, a.B, a.C = u.data_ptr(), delta.data_ptr(), A.data_ptr(), B.data_ptr(), C.data_ptr()
    a.deltaA = None if deltaA is None else deltaA.data_ptr()
    a.u_bs, a.u_ds = u.stride(0), u.stride(1)
    a.delta_bs, a.delta_ds = delta.stride(0), delta.stride(1)
    if deltaA is not None:
        a.deltaA_bs, a.deltaA_ds = deltaA.stride(0), deltaA.stride(1)
    a.A_ds, a.A_ns = A.stride(0), A.stride(1)
    a.B_ds, a.B_ns = B.stride(0), B.stride(1)
    a.C_ds, a.C_ns = C.stride(0), C.stride(1)
    return a, (batch, dim, seqlen, dstate)


def _stream(t) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def fwd(u, delta, A, B, C, deltaA_, discretization_method_str):
    """Returns ``[out, x]``: out complex64 like u, x (batch, dim, n_chunks, 2*dstate) complex64."""
    a, (batch, dim, seqlen, dstate) = _common(u, delta, A, B, C, deltaA_, discretization_method_str)
    n_chunks = (seqlen + CHUNK - 1) // CHUNK
    with torch.cuda.device(u.device):
        out = torch.empty_like(u)
        x = torch.empty((batch, dim, n_chunks, 2 * dstate), dtype=torch.complex64, device=u.device)
        a.out, a.x = out.data_ptr(), x.data_ptr()
        a.out_bs, a.out_ds = out.stride(0), out.stride(1)
        _lib.call("b200_simpscan_fwd", a, _stream(u))
    return [out, x]


def bwd(u, delta, A, B, C, deltaA_, dout, x_, discretization_method_str, need_dB_dC=True, out_=None):
    """Returns ``[du, ddelta, dA, dB, dC]`` plus ``ddeltaA`` when deltaA was given
    (simplified_scan_cpu.cpp:328-330).  Two additions to the reference signature, for single-state
    rows: ``need_dB_dC=False`` skips the dB / dC sums and returns None in their place; ``out_``, the
    output of ``fwd`` for the same arguments, lets the kernel take the states from it instead of
    recomputing them (B C must be non-zero)."""
    a, (batch, dim, seqlen, dstate) = _common(u, delta, A, B, C, deltaA_, discretization_method_str)
    _check(dout.dtype == torch.complex64 and dout.is_cuda, "dout must be a complex64 CUDA tensor")
    _check(dout.stride(-1) == 1 or dout.size(-1) == 1, "dout must be contiguous in the last dimension")
    _check(tuple(dout.shape) == (batch, dim, seqlen), "dout must have shape (batch, dim, seqlen)")
    n_chunks = (seqlen + CHUNK - 1) // CHUNK
    if n_chunks > 1:
        _check(x_ is not None, "x is required when seqlen > 2048")
    if x_ is not None:
        _check(x_.dtype == torch.complex64 and x_.is_cuda and x_.is_contiguous(),
               "x must be a contiguous complex64 CUDA tensor")
        _check(tuple(x_.shape) == (batch, dim, n_chunks, 2 * dstate), "x has the wrong shape")
    with torch.cuda.device(u.device):
        du = torch.empty_like(u)
        ddelta = torch.empty_like(delta)
        if A.is_contiguous() and B.is_contiguous() and C.is_contiguous():
            dA, dB, dC = torch.zeros((3,) + tuple(A.shape), dtype=A.dtype, device=A.device).unbind(0)  # one fill
        else:
            dA, dB, dC = torch.zeros_like(A), torch.zeros_like(B), torch.zeros_like(C)
        ddeltaA = torch.empty_like(deltaA_) if deltaA_ is not None else None
        # the kernel addresses dA/dB/dC with the strides of A/B/C
        _check(dA.stride() == A.stride() and dB.stride() == B.stride() and dC.stride() == C.stride(),
               "A, B, C must be dense")
        a.x = None if x_ is None else x_.data_ptr()
        if out_ is not None and dstate == 1:
            _check(out_.dtype == torch.complex64 and out_.is_cuda and tuple(out_.shape) == (batch, dim, seqlen),
                   "out must be a complex64 CUDA tensor of shape (batch, dim, seqlen)")
            _check(out_.stride(-1) == 1 or out_.size(-1) == 1, "out must be contiguous in the last dimension")
            a.out = out_.data_ptr()
            a.out_bs, a.out_ds = out_.stride(0), out_.stride(1)
        a.dout, a.du, a.ddelta = dout.data_ptr(), du.data_ptr(), ddelta.data_ptr()
        a.ddeltaA = None if ddeltaA is None else ddeltaA.data_ptr()
        a.dA = dA.data_ptr()
        if need_dB_dC or dstate != 1:
            a.dB, a.dC = dB.data_ptr(), dC.data_ptr()
        else:
            dB = dC = None
        a.dout_bs, a.dout_ds = dout.stride(0), dout.stride(1)
        a.du_bs, a.du_ds = du.stride(0), du.stride(1)
        a.ddelta_bs, a.ddelta_ds = ddelta.stride(0), ddelta.stride(1)
        if ddeltaA is not None:
            a.ddeltaA_bs, a.ddeltaA_ds = ddeltaA.stride(0), ddeltaA.stride(1)
        _lib.call("b200_simpscan_bwd", a, _stream(u))
    result = [du, ddelta, dA, dB, dC]
    if deltaA_ is not None:
        result.append(ddeltaA)
    return result
