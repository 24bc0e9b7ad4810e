"""``linear_step``: F.linear for the few tokens of a decoding step, on the weight-streaming kernel.

Mamba.step (lrnnx/models/ltv/mamba.py:355-487) applies in_proj, x_proj, dt_proj and out_proj to a
(batch, features) activation; at decoding batch sizes these read each weight once per token and
do almost no arithmetic, so they are bound by how fast the weight streams from HBM.
``b200_skinny_linear`` is built for that case (up to 64 tokens, 16-bit operands).  Measured on B200
at 64 tokens it beats the library GEMM only where the output is narrow — x_proj, 160 features over
K = 4096: 4.7 us against 7.0 us, because the library launches too few thread blocks there — and
loses where the output is wide (in_proj 13 to 17 against 8.2 us, out_proj 9.8 against 8.2 us, LM head
57 to 66 against 37 us): its ``mma.sync`` tiles run on the legacy tensor path, which at 64 tokens is
the limiter before HBM is.  ``linear_step`` therefore takes the kernel for narrow outputs only and
``F.linear`` for everything else.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from .. import _lib
from .mamba_block import _DT, _stream

MAX_FEATURES = 512        # widest output the kernel is used for


def _width_ok(n, k):
    return n <= MAX_FEATURES


def supported(x, weight, bias=None):
    return (x.is_cuda and x.dim() == 2 and x.dtype in (torch.bfloat16, torch.float16) and weight.dtype == x.dtype
            and (bias is None or bias.dtype == x.dtype)
            and 1 <= x.shape[0] <= 64 and _width_ok(weight.shape[0], weight.shape[1]) and weight.shape[1] % 64 == 0 and x.stride(1) == 1 and weight.stride(1) == 1
            and x.stride(0) % 8 == 0 and weight.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0
            and weight.data_ptr() % 16 == 0 and not (torch.is_grad_enabled() and (x.requires_grad or weight.requires_grad)))


def linear_step(x, weight, bias=None):
    """x (tokens, in_features), weight (out_features, in_features), bias (out_features,) or None ->
    (tokens, out_features); the semantics of ``F.linear`` (no gradient through the fast path)."""
    if not supported(x, weight, bias):
        return F.linear(x, weight, bias)
    a = _lib.struct("b200_skinny_linear_args")()
    a.M, a.K = x.shape
    a.N = weight.shape[0]
    a.dtype = _lib.enum(_DT[x.dtype])
    with torch.cuda.device(x.device):
        out = torch.empty(x.shape[0], weight.shape[0], dtype=x.dtype, device=x.device)
        a.x, a.weight, a.out = x.data_ptr(), weight.data_ptr(), out.data_ptr()
        a.bias = None if bias is None else bias.contiguous().data_ptr()
        a.x_rs, a.w_rs, a.out_rs = x.stride(0), weight.stride(0), out.stride(0)
        _lib.call("b200_skinny_linear", a, _stream(x))
    return out
