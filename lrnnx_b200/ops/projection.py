"""Complex projections around the S5 scan on the tensor cores (``b200_cgemm_wx``).

``project(W, x)`` computes ``einsum("mk,bkn->bmn", W, x)`` for complex64 operands, the shape of
Bu = B u, y = C x and of the data gradients du = B^H dBu, dx = C^H dy in lrnnx's
SimplifiedScanFn / S5InnerFn (lrnnx/ops/simplified_scan.py:67,87,136,165,401,419,483-524), with
float32-class accuracy (3xTF32 on tcgen05).  Shapes outside the kernel's tiling (M a multiple of
128, K of 32, N of 64; dense, 16-byte aligned x) are rejected by the C entry point with an error;
``supported`` tells the callers, which keep the einsum for those shapes.
"""
from __future__ import annotations

import torch

from .. import _lib


def supported(W, x) -> bool:
    if not (W.is_cuda and x.is_cuda and W.dtype == torch.complex64 and x.dtype == torch.complex64):
        return False
    if W.dim() != 2 or x.dim() != 3 or x.shape[1] != W.shape[1]:
        return False
    M, K = W.shape
    N = x.shape[2]
    return M % 128 == 0 and K % 32 == 0 and N % 64 == 0 and x.is_contiguous() and x.data_ptr() % 16 == 0


def weight_planes(W, conj_transpose=False):
    """(4, M, K) float32: Re(W) rounded to TF32, the remainder rounded to TF32, and the same for
    Im(W) (one kernel, b200_cgemm_planes).  With ``conj_transpose`` the planes of W^H."""
    if W.is_conj():
        W = W.resolve_conj()
    rows, cols = W.shape
    M, K = (cols, rows) if conj_transpose else (rows, cols)
    a = _lib.struct("b200_cgemm_planes_args")()
    a.M, a.K, a.conj = M, K, int(conj_transpose)
    a.w_rs, a.w_cs = (W.stride(1), W.stride(0)) if conj_transpose else (W.stride(0), W.stride(1))
    with torch.cuda.device(W.device):
        planes = torch.empty((4, M, K), dtype=torch.float32, device=W.device)
        a.w, a.planes = W.data_ptr(), planes.data_ptr()
        _lib.call("b200_cgemm_planes", a, torch.cuda.current_stream(W.device).cuda_stream)
    return planes


def project(W, x, conj_transpose=False):
    """out[b] = W x[b] (or W^H x[b]): W (M, K) (or (K, M)), x (batch, K, N) -> (batch, M, N), complex64."""
    planes = weight_planes(W, conj_transpose)
    _, M, K = planes.shape
    batch, Kx, N = x.shape
    if Kx != K:
        raise RuntimeError(f"project: the weight contracts {K} rows, x has {Kx}")
    if not x.is_contiguous():
        x = x.contiguous()
    a = _lib.struct("b200_cgemm_args")()
    a.batch, a.M, a.K, a.N = batch, M, K, N
    with torch.cuda.device(x.device):
        out = torch.empty((batch, M, N), dtype=torch.complex64, device=x.device)
        a.w_planes, a.x, a.out = planes.data_ptr(), x.data_ptr(), out.data_ptr()
        a.x_bs, a.x_ks = x.stride(0), x.stride(1)
        a.out_bs, a.out_ms = out.stride(0), out.stride(1)
        _lib.call("b200_cgemm_wx", a, torch.cuda.current_stream(x.device).cuda_stream)
    return out


def grad_supported(g, u) -> bool:
    if not (g.is_cuda and u.is_cuda and g.dtype == torch.complex64 and u.dtype == torch.complex64):
        return False
    if g.dim() != 3 or u.dim() != 3 or g.shape[0] != u.shape[0] or g.shape[2] != u.shape[2]:
        return False
    return g.shape[1] % 128 == 0 and u.shape[1] % 128 == 0 and g.shape[2] % 16 == 0


def weight_grad(g, u):
    """einsum("bml,bnl->mn", g, conj(u)) for complex64 g (batch, M, L), u (batch, N, L): the
    gradient of a projection weight, summed over batch and time on the tensor cores."""
    if not g.is_contiguous():
        g = g.contiguous()
    if not u.is_contiguous():
        u = u.contiguous()
    a = _lib.struct("b200_cgemm_grad_args")()
    a.batch, a.M, a.L = g.shape
    a.N = u.shape[1]
    with torch.cuda.device(g.device):
        out = torch.zeros((g.shape[1], u.shape[1]), dtype=torch.complex64, device=g.device)
        a.g, a.u, a.out = g.data_ptr(), u.data_ptr(), out.data_ptr()
        _lib.call("b200_cgemm_grad", a, torch.cuda.current_stream(g.device).cuda_stream)
    return out
