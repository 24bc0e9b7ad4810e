"""S4 kernel wrappers on the sm_100a kernels: ``cauchy_mult`` (csrc/s4/cauchy.py:70-116) and
``log_vandermonde_cuda`` (csrc/s4/vandermonde.py:6-53) with their autograd functions."""
from __future__ import annotations

import torch

from .. import structured_kernels as _sk

_MAX_L = 32 * 1024 * 64 * 1024


class CauchyMultiplySymmetric(torch.autograd.Function):
    @staticmethod
    def forward(ctx, v, z, w):
        batch, N = v.shape
        if N not in [1 << k for k in range(1, 11)]:
            raise NotImplementedError(f"Only support N values in {[1 << k for k in range(1, 11)]}")
        if z.shape[-1] > _MAX_L:
            raise NotImplementedError(f"Only support L values <= {_MAX_L}")
        if not (v.is_cuda and z.is_cuda and w.is_cuda):
            raise NotImplementedError("Only support CUDA tensors")
        ctx.save_for_backward(v, z, w)
        return _sk.cauchy_mult_sym_fwd(v, z, w)

    @staticmethod
    def backward(ctx, dout):
        v, z, w = ctx.saved_tensors
        dv, dw = _sk.cauchy_mult_sym_bwd(v, z, w, dout)
        return dv, None, dw


def cauchy_mult(v, z, w):
    """v, w (..., N) complex64 holding one member of each conjugate pair, z (L,) -> (..., L)."""
    v, w = torch.broadcast_tensors(v, w)
    shape = v.shape
    assert len(z.shape) == 1
    v, w, z = v.contiguous(), w.contiguous(), z.contiguous()
    N = v.size(-1)
    y = CauchyMultiplySymmetric.apply(v.view(-1, N), z, w.view(-1, N))
    return y.view(*shape[:-1], z.size(-1))


class LogVandMultiplySymmetric(torch.autograd.Function):
    @staticmethod
    def forward(ctx, v, x, L):
        batch, N = v.shape
        if N not in [1 << k for k in range(1, 11)]:
            raise NotImplementedError(f"Only support N values in {[1 << k for k in range(1, 11)]}")
        if L > _MAX_L:
            raise NotImplementedError(f"Only support L values <= {_MAX_L}")
        if not (v.is_cuda and x.is_cuda):
            raise NotImplementedError("Only support CUDA tensors")
        ctx.save_for_backward(v, x)
        return _sk.vand_log_mult_sym_fwd(v, x, L)

    @staticmethod
    def backward(ctx, dout):
        v, x = ctx.saved_tensors
        dv, dx = _sk.vand_log_mult_sym_bwd(v, x, dout)
        return dv, dx, None


def log_vandermonde_cuda(v, z, L):
    """v, z (..., N) complex64 -> (..., L) float32 = 2 Re sum_n v exp(z l)."""
    v, z = torch.broadcast_tensors(v, z)
    shape = v.shape
    v, z = v.contiguous(), z.contiguous()
    N = v.size(-1)
    y = LogVandMultiplySymmetric.apply(v.view(-1, N), z.view(-1, N), L)
    return y.view(*shape[:-1], L)


log_vandermonde_fast = LogVandMultiplySymmetric.apply
