"""Mamba language-model harness for benchmark configurations 2 (training step) and 4 (decoding).

A host-side mirror of lrnnx's ``LRNNLMHeadModel`` restricted to what those two configurations
use: Mamba mixers, RMSNorm, tied embeddings, no MLP (lrnnx/architectures/language_model.py:
198-511, 514-727; lrnnx/layers/block.py:16-136; lrnnx/models/ltv/mamba.py:66-548).  Modules and
parameters carry lrnnx's names, so a state dict of the reference model loads unchanged
(``dtA_proj``, which only the event mode reads, is accepted and ignored).

What runs where: embedding, the four projections of a block and the LM head are library GEMMs
(torch / cuBLAS: plumbing around the path); residual add + RMSNorm, the causal convolution and
the selective scan (training / prefill) and the convolution update and selective state update
(decoding) are this package's CUDA kernels.  lrnnx has no LM-level generation loop (its
``generate`` drives single mixer layers from a float buffer, lrnnx/utils/generation.py:26-162);
``generate`` here follows that file's pattern at the LM level: warm-up on a side stream,
capture of one decoding step over static buffers, graph replay per token (:121-155, :235-254).
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from .ops.linear_step import linear_step
from .ops.mamba_block import causal_conv1d_fn, causal_conv1d_update, rms_norm_fn
from .ops.mamba_inner import mamba_inner_fn
from .ops.selective_scan import selective_scan_fn
from .ops.selective_state_update import selective_state_update


class RMSNorm(nn.Module):
    def __init__(self, d, eps=1e-5, device=None, dtype=None):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(d, device=device, dtype=dtype))

    def forward(self, x, residual=None, prenorm=False, residual_in_fp32=False):
        return rms_norm_fn(x, self.weight, None, residual=residual, eps=self.eps, prenorm=prenorm,
                           residual_in_fp32=residual_in_fp32)


class _InProjFn(torch.autograd.Function):
    """xz = W hidden^T per batch row, produced directly in the (batch, channel, L) layout the scan
    kernels read.  A plain bmm would do the forward; its autograd hands the input gradient back as
    a transposed view, which the norm backward in front of it then has to copy.  Here the input
    gradient is computed as dxz^T W, i.e. directly in the (batch, L, d_model) layout of ``hidden``."""

    @staticmethod
    def forward(ctx, hidden, weight):
        ctx.save_for_backward(hidden, weight)
        return torch.bmm(weight.unsqueeze(0).expand(hidden.shape[0], -1, -1), hidden.transpose(1, 2))

    @staticmethod
    def backward(ctx, dxz):
        hidden, weight = ctx.saved_tensors
        batch = hidden.shape[0]
        d_hidden = torch.bmm(dxz.transpose(1, 2), weight.unsqueeze(0).expand(batch, -1, -1))
        d_weight = torch.bmm(dxz, hidden).sum(0)
        return d_hidden, d_weight.to(weight.dtype)


class Mamba(nn.Module):
    """The S6 mixer with lrnnx's parameter layout (lrnnx/models/ltv/mamba.py:66-177)."""

    def __init__(self, d_model, d_state=16, d_conv=4, expand=2, dt_rank="auto", dt_min=0.001, dt_max=0.1,
                 dt_init_floor=1e-4, device=None, dtype=None):
        super().__init__()
        kw = dict(device=device, dtype=dtype)
        self.d_model, self.d_state, self.d_conv = d_model, d_state, d_conv
        self.d_inner = expand * d_model
        self.dt_rank = math.ceil(d_model / 16) if dt_rank == "auto" else dt_rank
        self.in_proj = nn.Linear(d_model, 2 * self.d_inner, bias=False, **kw)
        self.conv1d = nn.Conv1d(self.d_inner, self.d_inner, d_conv, groups=self.d_inner, padding=d_conv - 1, **kw)
        self.x_proj = nn.Linear(self.d_inner, self.dt_rank + 2 * d_state, bias=False, **kw)
        self.dt_proj = nn.Linear(self.dt_rank, self.d_inner, bias=True, **kw)
        self.out_proj = nn.Linear(self.d_inner, d_model, bias=False, **kw)
        # dt_proj initialised so that softplus(bias) is log-uniform in [dt_min, dt_max] (mamba.py:135-151)
        std = self.dt_rank ** -0.5
        nn.init.uniform_(self.dt_proj.weight, -std, std)
        dt = torch.exp(torch.rand(self.d_inner) * (math.log(dt_max) - math.log(dt_min)) + math.log(dt_min)).clamp(min=dt_init_floor)
        with torch.no_grad():
            self.dt_proj.bias.copy_(dt + torch.log(-torch.expm1(-dt)))
        self.A_log = nn.Parameter(torch.log(torch.arange(1, d_state + 1, dtype=torch.float32, device=device)
                                            .repeat(self.d_inner, 1)))
        self.D = nn.Parameter(torch.ones(self.d_inner, device=device))

    def _xz(self, hidden):
        """in_proj straight into the (batch, channel, L) layout: W (2d, d_model) @ hidden^T."""
        if torch.is_grad_enabled() and (hidden.requires_grad or self.in_proj.weight.requires_grad):
            return _InProjFn.apply(hidden, self.in_proj.weight)
        batch = hidden.shape[0]
        return torch.bmm(self.in_proj.weight.unsqueeze(0).expand(batch, -1, -1), hidden.transpose(1, 2))

    def forward(self, hidden, cache=None):
        """hidden (batch, L, d_model) -> (batch, L, d_model).  With ``cache`` (a dict with
        "conv_state" (batch, d_inner, d_conv) and "lrnn_state" (batch, d_inner, d_state)) the
        states after the last position are written into it (prefill)."""
        A = -torch.exp(self.A_log.float())
        xz = self._xz(hidden)
        if cache is None:
            return mamba_inner_fn(xz, self.conv1d.weight, self.conv1d.bias, self.x_proj.weight, self.dt_proj.weight,
                                  self.out_proj.weight, None, A, None, None, self.D.float(),
                                  delta_bias=self.dt_proj.bias.float(), delta_softplus=True)
        batch, _, L = xz.shape
        d, N, R = self.d_inner, self.d_state, self.dt_rank
        x, z = xz[:, :d], xz[:, d:]
        if L >= self.d_conv:                               # the last d_conv inputs (a padded copy of x would move all of it)
            cache["conv_state"].copy_(x[..., L - self.d_conv:])
        else:
            cache["conv_state"].copy_(F.pad(x, (self.d_conv - L, 0)))
        xc = causal_conv1d_fn(x, self.conv1d.weight.squeeze(1), self.conv1d.bias, "silu")
        x_dbl = torch.bmm(self.x_proj.weight.unsqueeze(0).expand(batch, -1, -1), xc)
        delta = torch.bmm(self.dt_proj.weight.unsqueeze(0).expand(batch, -1, -1), x_dbl[:, :R])
        y, last = selective_scan_fn(xc, delta, A, x_dbl[:, R:R + N], x_dbl[:, R + N:], self.D.float(), z=z,
                                    delta_bias=self.dt_proj.bias.float(), delta_softplus=True, return_last_state=True)
        cache["lrnn_state"].copy_(last)
        return torch.bmm(y.transpose(1, 2), self.out_proj.weight.t().unsqueeze(0).expand(batch, -1, -1))

    def step(self, hidden, cache):
        """One token: hidden (batch, d_model) -> (batch, d_model); both states advance in place
        (lrnnx/models/ltv/mamba.py:355-487)."""
        d, N, R = self.d_inner, self.d_state, self.dt_rank
        xz = linear_step(hidden, self.in_proj.weight)
        x, z = xz[:, :d], xz[:, d:]
        x = causal_conv1d_update(x, cache["conv_state"], self.conv1d.weight.squeeze(1), self.conv1d.bias, "silu")
        x_db = linear_step(x, self.x_proj.weight)
        dt = linear_step(x_db[:, :R], self.dt_proj.weight)
        y = selective_state_update(cache["lrnn_state"], x, dt, cache["A"], x_db[:, R:R + N], x_db[:, R + N:], cache["D"],
                                   z=z, dt_bias=cache["dt_bias"], dt_softplus=True)
        return linear_step(y, self.out_proj.weight)

    def allocate_inference_cache(self, batch_size, dtype=None, state_dtype=None):
        dev = self.out_proj.weight.device
        dtype = dtype or self.conv1d.weight.dtype
        return {"conv_state": torch.zeros(batch_size, self.d_inner, self.d_conv, device=dev, dtype=dtype),
                "lrnn_state": torch.zeros(batch_size, self.d_inner, self.d_state, device=dev, dtype=state_dtype or dtype),
                # float32 copies of the per-channel parameters, made once instead of once per token
                "A": (-torch.exp(self.A_log.float())).contiguous(), "D": self.D.float().contiguous(),
                "dt_bias": self.dt_proj.bias.float().contiguous()}


class Block(nn.Module):
    def __init__(self, d_model, d_state, eps, device=None, dtype=None, **mixer_kw):
        super().__init__()
        self.norm = RMSNorm(d_model, eps, device=device, dtype=dtype)
        self.mixer = Mamba(d_model, d_state=d_state, device=device, dtype=dtype, **mixer_kw)


class Backbone(nn.Module):
    def __init__(self, d_model, d_state, n_layer, vocab_size, eps, residual_in_fp32, device=None, dtype=None, **mixer_kw):
        super().__init__()
        self.residual_in_fp32 = residual_in_fp32
        self.embedding = nn.Embedding(vocab_size, d_model, device=device, dtype=dtype)
        self.layers = nn.ModuleList([Block(d_model, d_state, eps, device=device, dtype=dtype, **mixer_kw)
                                     for _ in range(n_layer)])
        self.norm_f = RMSNorm(d_model, eps, device=device, dtype=dtype)

    def forward(self, input_ids, caches=None):
        hidden = self.embedding(input_ids)
        residual = None
        for i, layer in enumerate(self.layers):
            normed, residual = layer.norm(hidden, residual, prenorm=True, residual_in_fp32=self.residual_in_fp32)
            hidden = layer.mixer(normed, None if caches is None else caches[i])
        return self.norm_f(hidden, residual)

    def step(self, token_ids, caches):
        hidden = self.embedding(token_ids)
        residual = None
        for i, layer in enumerate(self.layers):
            normed, residual = layer.norm(hidden, residual, prenorm=True, residual_in_fp32=self.residual_in_fp32)
            hidden = layer.mixer.step(normed, caches[i])
        return self.norm_f(hidden, residual)


class MambaLMHeadModel(nn.Module):
    """``LRNNLMHeadModel(mixer_types=["Mamba"] * n_layer, rms_norm=True)`` of lrnnx on this package's kernels."""

    def __init__(self, d_model, n_layer, vocab_size, d_state=16, d_conv=4, expand=2, eps=1e-5, residual_in_fp32=False,
                 device=None, dtype=None):
        super().__init__()
        self.config = dict(d_model=d_model, n_layer=n_layer, vocab_size=vocab_size, d_state=d_state, d_conv=d_conv,
                           expand=expand, eps=eps)
        self.backbone = Backbone(d_model, d_state, n_layer, vocab_size, eps, residual_in_fp32, device=device, dtype=dtype,
                                 d_conv=d_conv, expand=expand)
        self.lm_head = nn.Linear(d_model, vocab_size, bias=False, device=device, dtype=dtype)
        # initialisation of lrnnx's LM (language_model.py:113-166): normal(0.02) embedding, out_proj
        # rescaled by 1/sqrt(n_layer); weights tied (:604-613)
        nn.init.normal_(self.backbone.embedding.weight, std=0.02)
        with torch.no_grad():
            for layer in self.backbone.layers:
                nn.init.kaiming_uniform_(layer.mixer.out_proj.weight, a=math.sqrt(5))
                layer.mixer.out_proj.weight /= math.sqrt(n_layer)
        self.lm_head.weight = self.backbone.embedding.weight
        self._decode_graphs = {}

    def load_state_dict(self, state_dict, strict=True):
        sd = {k: v for k, v in state_dict.items() if "dtA_proj" not in k}
        sd.setdefault("lm_head.weight", sd["backbone.embedding.weight"])
        return super().load_state_dict(sd, strict=strict)

    def forward(self, input_ids, caches=None, num_last_tokens=0):
        hidden = self.backbone(input_ids, caches)
        if num_last_tokens > 0:
            hidden = hidden[:, -num_last_tokens:]
        return self.lm_head(hidden)

    def step(self, token_ids, caches):
        """token_ids (batch,) -> logits (batch, vocab); caches advance in place."""
        return linear_step(self.backbone.step(token_ids, caches), self.lm_head.weight)

    def allocate_inference_cache(self, batch_size, dtype=None, state_dtype=None):
        return [layer.mixer.allocate_inference_cache(batch_size, dtype, state_dtype) for layer in self.backbone.layers]

    def _decode_graph(self, batch, state_dtype):
        """The captured decoding step for this batch size: static state buffers, a static token
        buffer and the graph that advances them by one token.  Built once and kept (the counterpart
        of lrnnx's CUDAGraphStepCache, lrnnx/utils/generation.py:165-290); ``clear_decode_graphs``
        drops it, which is needed after the parameters change because the caches hold float32
        copies of A, D and the step-size bias."""
        dev = self.lm_head.weight.device
        key = (batch, state_dtype, dev)
        entry = self._decode_graphs.get(key)
        if entry is not None:
            return entry
        caches = self.allocate_inference_cache(batch, state_dtype=state_dtype)
        tok_buf = torch.zeros(batch, dtype=torch.long, device=dev)
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):                  # warm-up outside capture; the states it leaves are overwritten by the prefill
            for _ in range(3):
                self.step(tok_buf, caches).argmax(dim=-1)
        torch.cuda.current_stream().wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            nxt = self.step(tok_buf, caches).argmax(dim=-1)
            tok_buf.copy_(nxt)
        entry = {"caches": caches, "tok": tok_buf, "graph": graph}
        self._decode_graphs[key] = entry
        return entry

    def clear_decode_graphs(self):
        self._decode_graphs.clear()

    @torch.no_grad()
    def generate(self, prompt_ids, n_new, use_cuda_graph=True, state_dtype=torch.float32, timings=None):
        """Greedy decoding: prefill ``prompt_ids`` (batch, L) through the scan kernels keeping the
        last states, then ``n_new`` tokens with one decoding step per token, replayed from a
        captured CUDA graph over static buffers (captured at the first call for a batch size and
        reused afterwards).  Returns the (batch, n_new) generated ids."""
        batch = prompt_ids.shape[0]
        dev = prompt_ids.device
        if use_cuda_graph:
            entry = self._decode_graph(batch, state_dtype)
            caches = entry["caches"]
        else:
            caches = self.allocate_inference_cache(batch, state_dtype=state_dtype)
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        ev[0].record()
        logits = self.forward(prompt_ids, caches, num_last_tokens=1)[:, 0]      # writes every state of the caches
        token = logits.argmax(dim=-1)
        out = torch.empty(batch, n_new, dtype=torch.long, device=dev)
        out[:, 0] = token
        ev[1].record()
        if use_cuda_graph:
            tok_buf, graph = entry["tok"], entry["graph"]
            tok_buf.copy_(token)
            for t in range(1, n_new):
                graph.replay()
                out[:, t].copy_(tok_buf)
        else:
            for t in range(1, n_new):
                token = self.step(token, caches).argmax(dim=-1)
                out[:, t] = token
        ev[2].record()
        if timings is not None:
            torch.cuda.synchronize()
            timings["prefill_ms"] = ev[0].elapsed_time(ev[1])
            timings["decode_ms"] = ev[1].elapsed_time(ev[2])
        return out
