"""``simplified_scan_fn`` and ``s5_inner_fn`` on the sm_100a kernels.

Mirror SimplifiedScanFn / simplified_scan_fn (lrnnx/ops/simplified_scan.py:14-230) and
S5InnerFn / s5_inner_fn (:343-583): the projections Bu = B u and y = C x (and their data
gradients) run on the tensor-core kernel of ``projection`` where its tiling applies, as complex
einsums (cuBLAS) otherwise, around the diagonal scan kernel, which is called with identity B / C.
The two weight gradients (sums over batch and time) run on its companion kernel.

One deliberate deviation: with ``return_last_state=True`` the reference's CUDA wrapper
slices its output tensor instead of the state (simplified_scan.py:106-110) and returns a
(batch, L/2) tensor; this wrapper returns the final state (batch, P) like
simplified_scan_ref (:329), taken from the kernel's checkpoint tensor.
"""
from __future__ import annotations

import torch

from .. import simplified_scan_cuda
from . import projection

_VALID = ("bilinear", "zoh", "dirac")


def _proj(W, x, conj_transpose=False):
    """W x (or W^H x) per batch: the tensor-core kernel where its tiling applies, einsum otherwise."""
    Wm = W.conj().transpose(0, 1) if conj_transpose else W
    if projection.supported(Wm, x if x.is_contiguous() else x.contiguous()):
        return projection.project(W, x, conj_transpose)
    return torch.einsum("mk,bkn->bmn", Wm, x)


def _wgrad(g, u):
    """sum over batch and time of g u^H: the tensor-core kernel where its tiling applies, einsum otherwise."""
    if projection.grad_supported(g, u):
        return projection.weight_grad(g, u)
    return torch.einsum("bml,bnl->mn", g, u.conj())


def _kernel_A(A):
    return A.unsqueeze(-1) if A.dim() == 1 else A


class SimplifiedScanFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, u, delta, A, B, C, deltaA, discretization, return_last_state=False):
        if u.stride(-1) != 1:
            u = u.contiguous()
        if delta.stride(-1) != 1:
            delta = delta.contiguous()
        if deltaA is not None and deltaA.stride(-1) != 1:
            deltaA = deltaA.contiguous()
        P = A.shape[0]
        A_k = _kernel_A(A).contiguous()
        dstate = A_k.shape[1]
        Bu = _proj(B, u)
        ident = torch.ones(P, dstate, dtype=A.dtype, device=A.device)
        out, xs = simplified_scan_cuda.fwd(Bu, delta, A_k, ident, ident, deltaA, discretization)
        y = _proj(C, out)
        ctx.discretization = discretization
        ctx.has_deltaA = deltaA is not None
        ctx.A_was_1d = A.dim() == 1
        ctx.save_for_backward(u, delta, A_k, B, C, Bu, out, xs, ident, deltaA)
        if return_last_state:
            ctx.mark_non_differentiable(xs)
            return y, xs[:, :, -1, 1::2].squeeze(-1)
        return y

    @staticmethod
    def backward(ctx, dout, *args):
        u, delta, A_k, B, C, Bu, out, xs, ident, deltaA = ctx.saved_tensors
        dx_out = _proj(C, dout, conj_transpose=True)
        dC = _wgrad(dout, out)
        if dx_out.stride(-1) != 1:
            dx_out = dx_out.contiguous()
        res = simplified_scan_cuda.bwd(Bu, delta, A_k, ident, ident, deltaA, dx_out, xs, ctx.discretization,
                                      need_dB_dC=False, out_=out if out.stride(-1) == 1 else None)
        dBu, ddelta, dA = res[0], res[1], res[2]
        ddeltaA = res[5] if ctx.has_deltaA else None
        du = _proj(B, dBu, conj_transpose=True)
        dB = _wgrad(dBu, u)
        if ctx.A_was_1d:
            dA = dA.squeeze(-1)
        return du, ddelta, dA, dB, dC, ddeltaA, None, None


def simplified_scan_fn(u, delta, A, B, C, deltaA=None, return_last_state=False, discretization="bilinear"):
    """u (batch, H, L) complex64; delta, deltaA (batch, P, L) float32; A (P,) or (P, 1) complex64;
    B (P, H), C (H, P) complex64.  Returns y (batch, H, L) complex64 (and the last state (batch, P))."""
    if discretization not in _VALID:
        raise ValueError(f"discretization must be one of {_VALID}, got '{discretization}'")
    return SimplifiedScanFn.apply(u, delta, A, B, C, deltaA, discretization, return_last_state)


class S5InnerFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, u, delta, A, B, C, D, deltaA, discretization, conj_sym):
        if u.stride(-1) != 1:
            u = u.contiguous()
        if delta.stride(-1) != 1:
            delta = delta.contiguous()
        if deltaA is not None and deltaA.stride(-1) != 1:
            deltaA = deltaA.contiguous()
        P = A.shape[0]
        A_k = _kernel_A(A).contiguous()
        dstate = A_k.shape[1]
        Bu = _proj(B, u)
        ident = torch.ones(P, dstate, dtype=A.dtype, device=A.device)
        scan_out, xs = simplified_scan_cuda.fwd(Bu, delta, A_k, ident, ident, deltaA, discretization)
        y_complex = _proj(C, scan_out)
        y_real = 2 * y_complex.real if conj_sym else y_complex.real
        u_real = u.real if u.is_complex() else u
        y = y_real + D.unsqueeze(0).unsqueeze(-1) * u_real
        ctx.discretization, ctx.conj_sym = discretization, conj_sym
        ctx.has_deltaA = deltaA is not None
        ctx.A_was_1d = A.dim() == 1
        ctx.save_for_backward(u, delta, A_k, B, C, D, Bu, scan_out, xs, ident, deltaA)
        return y

    @staticmethod
    def backward(ctx, dout):
        u, delta, A_k, B, C, D, Bu, scan_out, xs, ident, deltaA = ctx.saved_tensors
        u_real = u.real if u.is_complex() else u
        dD = torch.einsum("bhl,bhl->h", dout, u_real)
        du_skip = D.unsqueeze(0).unsqueeze(-1) * dout
        scale = 2.0 if ctx.conj_sym else 1.0
        dy_complex = torch.complex(scale * dout, torch.zeros_like(dout))
        dscan = _proj(C, dy_complex, conj_transpose=True)
        dC = _wgrad(dy_complex, scan_out)
        if dscan.stride(-1) != 1:
            dscan = dscan.contiguous()
        res = simplified_scan_cuda.bwd(Bu, delta, A_k, ident, ident, deltaA, dscan, xs, ctx.discretization,
                                      need_dB_dC=False, out_=scan_out if scan_out.stride(-1) == 1 else None)
        dBu, ddelta, dA = res[0], res[1], res[2]
        ddeltaA = res[5] if ctx.has_deltaA else None
        du_scan = _proj(B, dBu, conj_transpose=True)
        dB = _wgrad(dBu, u) if u.is_complex() else torch.einsum("bpl,bhl->ph", dBu, u.conj())
        if u.is_complex():
            du = du_scan + torch.complex(du_skip, torch.zeros_like(du_skip))
        else:
            du = du_scan.real + du_skip
        if ctx.A_was_1d:
            dA = dA.squeeze(-1)
        return du, ddelta, dA, dB, dC, dD, ddeltaA, None, None


def s5_inner_fn(u, delta, A, B, C, D, deltaA=None, discretization="bilinear", conj_sym=True):
    """(2 if conj_sym else 1) * Re(C x) + D * Re(u), with x the diagonal scan of B u."""
    return S5InnerFn.apply(u, delta, A, B, C, D, deltaA, discretization, conj_sym)
