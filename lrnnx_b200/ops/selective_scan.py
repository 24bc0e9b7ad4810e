"""``selective_scan_fn`` on the sm_100a kernels.

Mirrors SelectiveScanFn / selective_scan_fn of lrnnx/ops/selective_scan.py:30-197:
same argument order, same contiguity fix-ups, same lifting of 3-D B/C to
(batch, 1, dstate, L), same last-state slice ``x[:, :, -1, 1::2]`` (times B when
B is constant, :87-92), same gradient tuple.
"""
from __future__ import annotations

import torch

from .. import selective_scan_cuda


class SelectiveScanFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, u, delta, A, B, C, D=None, z=None, delta_bias=None, deltaA=None, delta_softplus=False,
                return_last_state=False, discretization=None):
        # The extension takes batch / channel strides as they are (a slice of a wider tensor, such
        # as the x and z halves of a Mamba block's in-projection, is scanned in place); only the
        # sequence dimension has to be dense.  lrnnx's wrapper copies every non-contiguous operand
        # (lrnnx/ops/selective_scan.py:48-62) because its extension assumes more.
        def dense_last(t):
            return t if t is None or t.stride(-1) == 1 or t.size(-1) == 1 else t.contiguous()

        u, delta, z, deltaA = dense_last(u), dense_last(delta), dense_last(z), dense_last(deltaA)
        if D is not None:
            D = D.contiguous()
        if B.dim() >= 3:
            B = dense_last(B)
        if C.dim() >= 3:
            C = dense_last(C)
        ctx.squeeze_B = ctx.squeeze_C = False
        if B.dim() == 3:
            B = B.unsqueeze(1)
            ctx.squeeze_B = True
        if C.dim() == 3:
            C = C.unsqueeze(1)
            ctx.squeeze_C = True
        out, x, *rest = selective_scan_cuda.fwd(u, delta, A, B, C, D, z, delta_bias, deltaA, delta_softplus,
                                                discretization)
        ctx.delta_softplus = delta_softplus
        ctx.has_z = z is not None
        ctx.has_deltaA = deltaA is not None
        ctx.disc_method = discretization
        last_state = x[:, :, -1, 1::2]
        if B.dim() < 3 and return_last_state:
            last_state = last_state * B
        if not ctx.has_z:
            ctx.save_for_backward(u, delta, A, B, C, D, delta_bias, deltaA, x)
            return out if not return_last_state else (out, last_state)
        ctx.save_for_backward(u, delta, A, B, C, D, z, delta_bias, deltaA, x, out)
        out_z = rest[0]
        return out_z if not return_last_state else (out_z, last_state)

    @staticmethod
    def backward(ctx, dout, *args):
        if not ctx.has_z:
            u, delta, A, B, C, D, delta_bias, deltaA, x = ctx.saved_tensors
            z = out = None
        else:
            u, delta, A, B, C, D, z, delta_bias, deltaA, x, out = ctx.saved_tensors
        if dout.stride(-1) != 1:
            dout = dout.contiguous()
        du, ddelta, dA, dB, dC, dD, ddelta_bias, *rest = selective_scan_cuda.bwd(
            u, delta, A, B, C, D, z, delta_bias, deltaA, dout, x, out, None, ctx.delta_softplus, False,
            ctx.disc_method)
        rest = list(rest)
        ddeltaA = rest.pop(0) if ctx.has_deltaA else None
        dz = rest.pop(0) if ctx.has_z else None
        dB = dB.squeeze(1) if ctx.squeeze_B else dB
        dC = dC.squeeze(1) if ctx.squeeze_C else dC
        return (du, ddelta, dA, dB, dC, dD if D is not None else None, dz,
                ddelta_bias if delta_bias is not None else None, ddeltaA, None, None, None)


def selective_scan_fn(u, delta, A, B, C, D=None, z=None, delta_bias=None, deltaA=None, delta_softplus=False,
                      return_last_state=False, discretization="mamba"):
    """If ``return_last_state`` is True returns ``(out, last_state)`` with last_state
    (batch, dim, dstate); the last state carries no gradient (lrnnx/ops/selective_scan.py:180-183)."""
    return SelectiveScanFn.apply(u, delta, A, B, C, D, z, delta_bias, deltaA, delta_softplus, return_last_state,
                                 discretization)
