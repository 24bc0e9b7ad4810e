"""Elementwise companions of the scan inside a Mamba block, on the sm_100a kernels.

``causal_conv1d_fn`` / ``causal_conv1d_update`` take the place of the un-vendored
``causal_conv1d`` package that lrnnx's Mamba looks for (lrnnx/models/ltv/mamba.py:24-27; without
it the layer falls back to nn.Conv1d, :270-279, and to a roll + dot in step(), :394-409).
``rms_norm_fn`` takes the place of the Triton ``rms_norm_fn`` (lrnnx/ops/triton/layer_norm.py:
1028-1058) as the LM blocks call it: optional residual add, ``prenorm`` returning the sum as
well, ``residual_in_fp32``.  Same argument names and return values; no bias, dropout, rowscale
or second input (lrnnx's LM passes none of them for RMSNorm).
"""
from __future__ import annotations

import torch

from .. import _lib

_DT = {torch.float32: "B200_F32", torch.float16: "B200_F16", torch.bfloat16: "B200_BF16"}


def _stream(t):
    return torch.cuda.current_stream(t.device).cuda_stream


def _conv_args(x, weight, bias, silu):
    if x.dtype not in _DT:
        raise RuntimeError("causal_conv1d: x must be float32, float16 or bfloat16")
    if not x.is_cuda:
        raise RuntimeError("causal_conv1d: x must be a CUDA tensor")
    if weight.dim() != 2:
        raise RuntimeError("causal_conv1d: weight must be (dim, width)")
    a = _lib.struct("b200_conv1d_args")()
    a.dim, a.width = weight.shape
    a.dtype = _lib.enum(_DT[x.dtype])
    a.silu = int(bool(silu))
    a.weight = weight.data_ptr()
    a.bias = None if bias is None else bias.data_ptr()
    return a


class CausalConv1dFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, silu):
        if x.stride(-1) != 1:
            x = x.contiguous()
        w = weight.to(x.dtype).contiguous()
        b = None if bias is None else bias.to(x.dtype).contiguous()
        a = _conv_args(x, w, b, silu)
        a.batch, _, a.seqlen = x.shape
        with torch.cuda.device(x.device):
            out = torch.empty_like(x, memory_format=torch.contiguous_format)
            a.x, a.out = x.data_ptr(), out.data_ptr()
            a.x_bs, a.x_ds = x.stride(0), x.stride(1)
            a.out_bs, a.out_ds = out.stride(0), out.stride(1)
            _lib.call("b200_conv1d_fwd", a, _stream(x))
        ctx.save_for_backward(x, w, b)
        ctx.silu = silu
        ctx.wdtype = weight.dtype
        ctx.bdtype = None if bias is None else bias.dtype
        return out

    @staticmethod
    def backward(ctx, dout):
        x, w, b = ctx.saved_tensors
        if dout.stride(-1) != 1:
            dout = dout.contiguous()
        a = _conv_args(x, w, b, ctx.silu)
        a.batch, _, a.seqlen = x.shape
        with torch.cuda.device(x.device):
            dx = torch.empty_like(x, memory_format=torch.contiguous_format)
            dw = torch.zeros(w.shape, dtype=torch.float32, device=x.device)
            db = torch.zeros(w.shape[0], dtype=torch.float32, device=x.device) if b is not None else None
            a.x, a.dout, a.dx, a.dweight = x.data_ptr(), dout.data_ptr(), dx.data_ptr(), dw.data_ptr()
            a.dbias = None if db is None else db.data_ptr()
            a.x_bs, a.x_ds = x.stride(0), x.stride(1)
            a.dout_bs, a.dout_ds = dout.stride(0), dout.stride(1)
            a.dx_bs, a.dx_ds = dx.stride(0), dx.stride(1)
            _lib.call("b200_conv1d_bwd", a, _stream(x))
        return dx, dw.to(ctx.wdtype), (None if db is None else db.to(ctx.bdtype)), None


def causal_conv1d_fn(x, weight, bias=None, activation=None):
    """x (batch, dim, seqlen); weight (dim, width); bias (dim,); activation None, "silu" or "swish".
    out[b, d, t] = act(bias[d] + sum_k weight[d, k] x[b, d, t - (width - 1) + k])."""
    if activation not in (None, "silu", "swish"):
        raise NotImplementedError("activation must be None, silu, or swish")
    return CausalConv1dFn.apply(x, weight, bias, activation is not None)


def causal_conv1d_update(x, conv_state, weight, bias=None, activation=None):
    """One decoding step: x (batch, dim); conv_state (batch, dim, width), shifted and appended in
    place; returns act(bias + sum_k weight[:, k] conv_state[:, :, k]) of shape (batch, dim)."""
    if activation not in (None, "silu", "swish"):
        raise NotImplementedError("activation must be None, silu, or swish")
    if conv_state.dtype != x.dtype or conv_state.stride(-1) != 1:
        raise RuntimeError("causal_conv1d_update: conv_state must have the dtype of x and a dense last dimension")
    w = weight.to(x.dtype).contiguous()
    b = None if bias is None else bias.to(x.dtype).contiguous()
    a = _conv_args(x, w, b, activation is not None)
    a.batch = x.shape[0]
    a.seqlen = 1
    with torch.cuda.device(x.device):
        out = torch.empty_like(x)
        a.x, a.out, a.state = x.data_ptr(), out.data_ptr(), conv_state.data_ptr()
        a.x_bs, a.x_ds = x.stride(0), x.stride(1)
        a.out_bs, a.out_ds = out.stride(0), out.stride(1)
        a.state_bs, a.state_ds = conv_state.stride(0), conv_state.stride(1)
        _lib.call("b200_conv1d_update", a, _stream(x))
    return out


class RMSNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, residual, eps, prenorm, residual_in_fp32):
        shape = x.shape
        x2 = x.reshape(-1, shape[-1])
        if x2.stride(-1) != 1:
            x2 = x2.contiguous()
        res2 = None
        if residual is not None:
            res2 = residual.reshape(-1, shape[-1])
            if res2.stride(-1) != 1:
                res2 = res2.contiguous()
        rdtype = res2.dtype if res2 is not None else (torch.float32 if residual_in_fp32 else x.dtype)
        if x.dtype not in _DT or rdtype not in (x.dtype, torch.float32):
            raise RuntimeError("rms_norm_fn: activations must be float32 / float16 / bfloat16 and the residual "
                               "in the same dtype or float32")
        w = weight.to(x.dtype).contiguous()
        a = _lib.struct("b200_rmsnorm_args")()
        a.rows, a.cols = x2.shape
        a.dtype, a.residual_dtype = _lib.enum(_DT[x.dtype]), _lib.enum(_DT[rdtype])
        a.eps = eps
        with torch.cuda.device(x.device):
            y = torch.empty_like(x2)
            z = torch.empty(x2.shape, dtype=rdtype, device=x.device)     # x + residual: output of prenorm, input of backward
            rstd = torch.empty(x2.shape[0], dtype=torch.float32, device=x.device)
            a.x, a.weight, a.y, a.residual_out, a.rstd = x2.data_ptr(), w.data_ptr(), y.data_ptr(), z.data_ptr(), rstd.data_ptr()
            a.residual = None if res2 is None else res2.data_ptr()
            a.x_rs, a.y_rs, a.residual_out_rs = x2.stride(0), y.stride(0), z.stride(0)
            if res2 is not None:
                a.residual_rs = res2.stride(0)
            _lib.call("b200_rmsnorm_fwd", a, _stream(x))
        ctx.save_for_backward(z, w, rstd)
        ctx.meta = (shape, x.dtype, rdtype, eps, residual is not None, prenorm, weight.dtype)
        y = y.reshape(shape)
        if prenorm:
            return y, z.reshape(shape)
        return y

    @staticmethod
    def backward(ctx, dy, *rest):
        z, w, rstd = ctx.saved_tensors
        shape, xdtype, rdtype, eps, has_residual, prenorm, wdtype = ctx.meta
        dy2 = dy.reshape(-1, shape[-1])
        if dy2.stride(-1) != 1:
            dy2 = dy2.contiguous()
        dres2 = None
        if prenorm and rest and rest[0] is not None:
            dres2 = rest[0].reshape(-1, shape[-1]).to(rdtype)
            if dres2.stride(-1) != 1:
                dres2 = dres2.contiguous()
        a = _lib.struct("b200_rmsnorm_args")()
        a.rows, a.cols = z.shape
        a.dtype, a.residual_dtype = _lib.enum(_DT[xdtype]), _lib.enum(_DT[rdtype])
        a.eps = eps
        with torch.cuda.device(z.device):
            dx = torch.empty(z.shape, dtype=xdtype, device=z.device)
            dres_in = torch.empty(z.shape, dtype=rdtype, device=z.device) if (has_residual and rdtype != xdtype) else None
            dw = torch.zeros(z.shape[1], dtype=torch.float32, device=z.device)
            a.weight, a.residual_out, a.rstd = w.data_ptr(), z.data_ptr(), rstd.data_ptr()
            a.dy, a.dx, a.dweight = dy2.data_ptr(), dx.data_ptr(), dw.data_ptr()
            a.dresidual = None if dres2 is None else dres2.data_ptr()
            a.dresidual_in = None if dres_in is None else dres_in.data_ptr()
            a.residual_out_rs, a.dy_rs, a.dx_rs = z.stride(0), dy2.stride(0), dx.stride(0)
            if dres2 is not None:
                a.dresidual_rs = dres2.stride(0)
            if dres_in is not None:
                a.dresidual_in_rs = dres_in.stride(0)
            _lib.call("b200_rmsnorm_bwd", a, _stream(z))
        dx = dx.reshape(shape)
        dres = None
        if has_residual:
            dres = dres_in.reshape(shape) if dres_in is not None else dx
        return dx, dw.to(wdtype), dres, None, None, None


def rms_norm_fn(x, weight, bias=None, residual=None, eps=1e-6, prenorm=False, residual_in_fp32=False):
    """y = rmsnorm(x + residual) * weight over the last dimension.  With ``prenorm`` returns
    ``(y, x + residual)``; the sum has the dtype of ``residual`` if given, else float32 when
    ``residual_in_fp32``, else the dtype of x."""
    if bias is not None:
        raise NotImplementedError("rms_norm_fn: a bias is not supported (lrnnx's RMSNorm has none)")
    return RMSNormFn.apply(x, weight, residual, eps, prenorm, residual_in_fp32)
