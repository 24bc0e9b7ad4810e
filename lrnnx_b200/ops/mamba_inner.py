"""``mamba_inner_fn``: the inner part of a Mamba block as ONE autograd node on the sm_100a kernels.

lrnnx ships this function (lrnnx/ops/selective_scan.py:389-784) but its calls into the scan
extension no longer match the extension's signatures (9 / 14 positional arguments against the
11 / 16 that csrc/selective_scan/selective_scan.h:114-136 binds) and it needs the un-vendored
causal_conv1d package, so lrnnx's Mamba never reaches it.  This is a working equivalent with
the same argument list and the semantics of ``mamba_inner_ref`` (:787-850):

    x, z   = xz.chunk(2, dim=1)
    x      = silu(causal_conv1d(x))
    x_dbl  = x_proj(x)             -> (dt_low, B, C)
    delta  = dt_proj.weight @ dt_low
    y      = selective_scan(x, delta, A, B, C, D, z, delta_bias, softplus)
    out    = out_proj(y)

Everything is kept in the (batch, channel, L) layout the scan kernels read, so no tensor is
transposed or copied between the steps: the projections are batched GEMMs with the weight
broadcast over the batch (library GEMMs; the path's own kernels are the convolution and the
scan), B and C are strided views of x_dbl.  The backward recomputes the convolution output and
delta instead of keeping them (they cost one elementwise kernel and one thin GEMM), and writes
dx and dz side by side into one dxz tensor.
"""
from __future__ import annotations

import torch

from .. import _lib, selective_scan_cuda
from .mamba_block import _DT, _conv_args, _stream


def _wb(w, batch):
    """A (rows, cols) weight as a batch-broadcast operand of torch.bmm (no copy)."""
    return w.unsqueeze(0).expand(batch, -1, -1)


def _conv_forward(x, w2, bias):
    a = _conv_args(x, w2, bias, True)
    a.batch, _, a.seqlen = x.shape
    out = torch.empty((x.shape[0], x.shape[1], x.shape[2]), dtype=x.dtype, device=x.device)
    a.x, a.out = x.data_ptr(), out.data_ptr()
    a.x_bs, a.x_ds = x.stride(0), x.stride(1)
    a.out_bs, a.out_ds = out.stride(0), out.stride(1)
    _lib.call("b200_conv1d_fwd", a, _stream(x))
    return out


class MambaInnerFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, xz, conv1d_weight, conv1d_bias, x_proj_weight, delta_proj_weight, out_proj_weight, out_proj_bias,
                A, D, delta_bias, delta_softplus):
        batch, two_d, L = xz.shape
        d = two_d // 2
        N = A.shape[1]
        R = delta_proj_weight.shape[1]
        if xz.stride(-1) != 1:
            xz = xz.contiguous()
        dt = xz.dtype
        w2 = conv1d_weight.reshape(d, -1).to(dt).contiguous()
        cb = None if conv1d_bias is None else conv1d_bias.to(dt).contiguous()
        with torch.cuda.device(xz.device):
            x, z = xz[:, :d], xz[:, d:]
            xc = _conv_forward(x, w2, cb)
            x_dbl = torch.bmm(_wb(x_proj_weight.to(dt), batch), xc)                    # (batch, R + 2N, L)
            delta = torch.bmm(_wb(delta_proj_weight.to(dt), batch), x_dbl[:, :R])       # (batch, d, L)
            Bv, Cv = x_dbl[:, R:R + N].unsqueeze(1), x_dbl[:, R + N:].unsqueeze(1)       # (batch, 1, N, L) views
            out, xs, out_z = selective_scan_cuda.fwd(xc, delta, A, Bv, Cv, D, z, delta_bias, None, delta_softplus, "mamba")
            y = torch.bmm(out_z.transpose(1, 2), _wb(out_proj_weight.to(dt).t(), batch))  # (batch, L, d_model)
            if out_proj_bias is not None:
                y = y + out_proj_bias.to(dt)
        ctx.save_for_backward(xz, w2, cb, x_proj_weight, delta_proj_weight, out_proj_weight, A, D, delta_bias, x_dbl,
                              out, xs, out_z)
        ctx.delta_softplus = delta_softplus
        ctx.meta = (conv1d_weight.shape, conv1d_weight.dtype, None if conv1d_bias is None else conv1d_bias.dtype,
                    out_proj_bias is not None)
        return y

    @staticmethod
    def backward(ctx, dy):
        (xz, w2, cb, x_proj_weight, delta_proj_weight, out_proj_weight, A, D, delta_bias, x_dbl, out, xs,
         out_z) = ctx.saved_tensors
        wshape, wdtype, bdtype, has_out_bias = ctx.meta
        batch, two_d, L = xz.shape
        d = two_d // 2
        N = A.shape[1]
        R = delta_proj_weight.shape[1]
        dt = xz.dtype
        with torch.cuda.device(xz.device):
            x, z = xz[:, :d], xz[:, d:]
            dy = dy.to(dt)
            # out_proj
            dout_z = torch.bmm(_wb(out_proj_weight.to(dt).t(), batch), dy.transpose(1, 2))        # (batch, d, L)
            # weight gradients: batched GEMMs on transposed views (no operand is copied), summed over the batch
            d_out_w = torch.bmm(dy.transpose(1, 2), out_z.transpose(1, 2)).sum(0)
            d_out_b = dy.sum(dim=(0, 1)) if has_out_bias else None
            # recomputed, not stored
            xc = _conv_forward(x, w2, cb)
            delta = torch.bmm(_wb(delta_proj_weight.to(dt), batch), x_dbl[:, :R])
            Bv, Cv = x_dbl[:, R:R + N].unsqueeze(1), x_dbl[:, R + N:].unsqueeze(1)
            dxz = torch.empty_like(xz)
            res = selective_scan_cuda.bwd(xc, delta, A, Bv, Cv, D, z, delta_bias, None, dout_z, xs, out, dxz[:, d:],
                                          ctx.delta_softplus, False, "mamba")
            dxc, ddelta, dA, dB, dC, dD, ddelta_bias = res[:7]
            # dt_proj, x_proj
            dx_dbl = torch.empty_like(x_dbl)
            dx_dbl[:, :R].copy_(torch.bmm(_wb(delta_proj_weight.to(dt).t(), batch), ddelta))
            dx_dbl[:, R:R + N].copy_(dB.squeeze(1))
            dx_dbl[:, R + N:].copy_(dC.squeeze(1))
            d_dt_w = torch.bmm(ddelta, x_dbl[:, :R].transpose(1, 2)).sum(0)
            d_xp_w = torch.bmm(dx_dbl, xc.transpose(1, 2)).sum(0)
            dxc = torch.baddbmm(dxc, _wb(x_proj_weight.to(dt).t(), batch), dx_dbl)
            # convolution
            a = _conv_args(x, w2, cb, True)
            a.batch, _, a.seqlen = x.shape
            dw = torch.zeros(w2.shape, dtype=torch.float32, device=xz.device)
            db = torch.zeros(d, dtype=torch.float32, device=xz.device) if cb is not None else None
            dx = dxz[:, :d]
            a.x, a.dout, a.dx, a.dweight = x.data_ptr(), dxc.data_ptr(), dx.data_ptr(), dw.data_ptr()
            a.dbias = None if db is None else db.data_ptr()
            a.x_bs, a.x_ds = x.stride(0), x.stride(1)
            a.dout_bs, a.dout_ds = dxc.stride(0), dxc.stride(1)
            a.dx_bs, a.dx_ds = dx.stride(0), dx.stride(1)
            _lib.call("b200_conv1d_bwd", a, _stream(xz))
        return (dxz, dw.reshape(wshape).to(wdtype), None if db is None else db.to(bdtype),
                d_xp_w.to(x_proj_weight.dtype), d_dt_w.to(delta_proj_weight.dtype), d_out_w.to(out_proj_weight.dtype),
                d_out_b, dA, dD, ddelta_bias, None)


def mamba_inner_fn(xz, conv1d_weight, conv1d_bias, x_proj_weight, delta_proj_weight, out_proj_weight, out_proj_bias, A,
                   B=None, C=None, D=None, delta_bias=None, B_proj_bias=None, C_proj_bias=None, delta_softplus=True,
                   checkpoint_lvl=1, b_rms_weight=None, c_rms_weight=None, dt_rms_weight=None, b_c_dt_rms_eps=1e-6):
    """xz (batch, 2 d_inner, L); conv1d_weight (d_inner, 1, width); x_proj_weight (dt_rank + 2N, d_inner);
    delta_proj_weight (d_inner, dt_rank); out_proj_weight (d_model, d_inner); A (d_inner, N) real.
    Returns (batch, L, d_model).  Only the input-dependent B / C form that Mamba uses is built."""
    if B is not None or C is not None or B_proj_bias is not None or C_proj_bias is not None:
        raise NotImplementedError("mamba_inner_fn: only input-dependent B and C without projection biases")
    if b_rms_weight is not None or c_rms_weight is not None or dt_rms_weight is not None:
        raise NotImplementedError("mamba_inner_fn: RMS-normalised B / C / dt are not supported")
    if A.is_complex():
        raise NotImplementedError("mamba_inner_fn: real A only")
    if xz.dtype not in _DT:
        raise RuntimeError("mamba_inner_fn: xz must be float32, float16 or bfloat16")
    return MambaInnerFn.apply(xz, conv1d_weight, conv1d_bias, x_proj_weight, delta_proj_weight, out_proj_weight,
                              out_proj_bias, A, D, delta_bias, delta_softplus)
