"""``s7_scan_fn`` on the sm_100a kernels (mirrors S7ScanFn / s7_scan_fn,
lrnnx/ops/s7_scan.py:16-181): the input projection Bu and the output projection
C·x stay einsums; the recurrence over the dstate "channels" runs in the
selective-scan kernel with the "s7" method and one state per channel."""
from __future__ import annotations

import torch

from .. import selective_scan_cuda


class S7ScanFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, u, A, B, C, bias=None, return_last_state=False):
        dstate = A.shape[1]
        if not u.is_contiguous():
            u = u.contiguous()
        Bu = torch.einsum("bnhl,bhl->bnl", B.float(), u.float())
        if bias is not None:
            Bu = Bu + bias.float()
        Bu = Bu.contiguous()
        delta = A.contiguous()
        A_k = torch.zeros(dstate, 1, dtype=Bu.dtype, device=Bu.device)
        B_k = torch.ones(dstate, 1, dtype=Bu.dtype, device=Bu.device)
        C_k = torch.ones(dstate, 1, dtype=Bu.dtype, device=Bu.device)
        out_k, x_k, *_ = selective_scan_cuda.fwd(Bu, delta, A_k, B_k, C_k, None, None, None, None, False, "s7")
        y = torch.einsum("bhnl,bnl->bhl", C.float(), out_k.float())
        ctx.save_for_backward(u, B, C, bias, Bu, out_k, x_k, delta, A_k, B_k, C_k)
        if return_last_state:
            return y.to(u.dtype), out_k[:, :, -1]
        return y.to(u.dtype)

    @staticmethod
    def backward(ctx, dout, *args):
        u, B, C, bias, Bu, out_k, x_k, delta, A_k, B_k, C_k = ctx.saved_tensors
        dout = dout.float()
        if dout.stride(-1) != 1:
            dout = dout.contiguous()
        dC = torch.einsum("bhl,bnl->bhnl", dout, out_k.float())
        dout_k = torch.einsum("bhnl,bhl->bnl", C.float(), dout).contiguous()
        dBu, ddelta, *_ = selective_scan_cuda.bwd(Bu, delta, A_k, B_k, C_k, None, None, None, None, dout_k, x_k,
                                                  out_k, None, False, False, "s7")
        dB = torch.einsum("bnl,bhl->bnhl", dBu, u.float())
        du = torch.einsum("bnhl,bnl->bhl", B.float(), dBu)
        return du.to(u.dtype), ddelta, dB, dC, (dBu if bias is not None else None), None


def s7_scan_fn(u, A, B, C, bias=None, return_last_state=False):
    """u (batch, dim, L); A (batch, dstate, L); B (batch, dstate, dim, L); C (batch, dim, dstate, L);
    bias (batch, dstate, L).  a_t = 1 - 1/(A_t^2 + 1/2)."""
    return S7ScanFn.apply(u, A, B, C, bias, return_last_state)
