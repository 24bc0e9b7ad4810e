"""``rglru_scan_fn`` on the sm_100a kernels (mirrors RGLRUScanFn / rglru_scan_fn,
lrnnx/ops/rglru_scan.py:28-144): the selective-scan kernel with the "rglru"
method, identity B and C, no D / z / bias."""
from __future__ import annotations

import torch

from .. import selective_scan_cuda


class RGLRUScanFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, u, delta, A, return_last_state=False):
        u, delta, A = u.contiguous(), delta.contiguous(), A.contiguous()
        dim, dstate = A.shape
        B = torch.ones(dim, dstate, dtype=u.dtype, device=u.device)
        C = torch.ones(dim, dstate, dtype=u.dtype, device=u.device)
        out, x, *_ = selective_scan_cuda.fwd(u, delta, A, B, C, None, None, None, None, False, "rglru")
        ctx.save_for_backward(u, delta, A, B, C, out, x)
        if return_last_state:
            return out, x[:, :, -1, 1::2]
        return out

    @staticmethod
    def backward(ctx, dout, *args):
        u, delta, A, B, C, out, x = ctx.saved_tensors
        if not dout.is_contiguous():
            dout = dout.contiguous()
        du, ddelta, dA, *_ = selective_scan_cuda.bwd(u, delta, A, B, C, None, None, None, None, dout, x, out, None,
                                                     False, False, "rglru")
        return du, ddelta, dA, None


def rglru_scan_fn(u, delta, A, return_last_state=False):
    """u, delta (batch, dim, L) float32; A (dim, dstate) in (0, 1).  a_t = A**delta_t,
    h_t = a_t h_{t-1} + sqrt(1 - a_t^2) u_t, out = sum over dstate of h."""
    return RGLRUScanFn.apply(u, delta, A, return_last_state)
