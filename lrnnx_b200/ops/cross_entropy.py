"""Mean next-token cross-entropy for the LM harness, computed on the logits in their own dtype.

lrnnx has no loss of its own (its LM returns logits, lrnnx/architectures/language_model.py:615-727,
and its training benchmark sums them, benchmarks/benchmark_training.py:33-34).  With a vocabulary
of 50280 the float32 copy of the logits that ``F.cross_entropy(logits.float(), ...)`` makes, and
the passes of log-softmax over it, cost more than any other elementwise step of a training step;
the two kernels here read the logits once each (forward: log-sum-exp and the target logit;
backward: softmax minus one-hot, written in the logits' dtype).
"""
from __future__ import annotations

import torch

from .. import _lib
from .mamba_block import _DT, _stream


class CrossEntropyFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, labels, ignore_index):
        if logits.dim() != 2 or labels.dim() != 1 or labels.shape[0] != logits.shape[0]:
            raise RuntimeError("cross_entropy: logits (rows, classes) and labels (rows,) expected")
        if logits.dtype not in _DT or not logits.is_cuda:
            raise RuntimeError("cross_entropy: logits must be a float32 / float16 / bfloat16 CUDA tensor")
        if logits.stride(-1) != 1:
            logits = logits.contiguous()
        labels = labels.to(torch.int64).contiguous()
        a = _lib.struct("b200_xent_args")()
        a.rows, a.cols = logits.shape
        a.dtype = _lib.enum(_DT[logits.dtype])
        a.ignore_index = ignore_index
        with torch.cuda.device(logits.device):
            lse = torch.empty(logits.shape[0], dtype=torch.float32, device=logits.device)
            loss = torch.empty_like(lse)
            a.logits, a.labels, a.lse, a.loss = logits.data_ptr(), labels.data_ptr(), lse.data_ptr(), loss.data_ptr()
            a.logits_rs = logits.stride(0)
            _lib.call("b200_xent_fwd", a, _stream(logits))
            counted = (labels != ignore_index).sum().clamp(min=1).to(torch.float32)
            out = loss.sum() / counted
        ctx.save_for_backward(logits, labels, lse, counted)
        ctx.ignore_index = ignore_index
        return out

    @staticmethod
    def backward(ctx, grad):
        logits, labels, lse, counted = ctx.saved_tensors
        a = _lib.struct("b200_xent_args")()
        a.rows, a.cols = logits.shape
        a.dtype = _lib.enum(_DT[logits.dtype])
        a.ignore_index = ctx.ignore_index
        with torch.cuda.device(logits.device):
            scale = (grad.to(torch.float32) / counted).reshape(1).contiguous()
            dlogits = torch.empty_like(logits)
            a.logits, a.labels, a.lse = logits.data_ptr(), labels.data_ptr(), lse.data_ptr()
            a.scale, a.dlogits = scale.data_ptr(), dlogits.data_ptr()
            a.logits_rs, a.dlogits_rs = logits.stride(0), dlogits.stride(0)
            _lib.call("b200_xent_bwd", a, _stream(logits))
        return dlogits, None, None


def cross_entropy(logits, labels, ignore_index=-100):
    """Mean over the rows whose label is not ``ignore_index`` of ``logsumexp(logits[r]) -
    logits[r, labels[r]]`` (``F.cross_entropy(logits.float(), labels, ignore_index=...)``), a
    float32 scalar.  logits (rows, classes); labels (rows,) integer."""
    return CrossEntropyFn.apply(logits, labels, ignore_index)
