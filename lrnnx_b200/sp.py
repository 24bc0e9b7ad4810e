"""Sequence-parallel selective scan (benchmark configuration 3): forward, and the backward that mirrors it.

lrnnx is single-GPU; this is the multi-GPU split its long-sequence case needs.  Rank r owns
the timesteps [r*L/R, (r+1)*L/R).  Because the recurrence h_t = a_t h_{t-1} + b_t is linear,
a slice is summarised by (P_r, h_r) = (product of a over the slice, final state from a zero
start) — exactly the last checkpoint entry the forward kernel already writes
(x[:, :, -1, 0::2], x[:, :, -1, 1::2]).  The ranks all-gather these 2*B*D*N floats, fold the
summaries of the ranks before them (h <- P_j h + h_j) to get the state entering their slice,
and a fix-up kernel adds that state's contribution to the zero-start output.

The backward runs the same exchange from the right.  With g_t the gradient with respect to the
state h_t, a slice [s, e] hands q = a_s g_s to the slice before it, and q = G + P q_next, where
G = sum_t (prod_{k=s..t} a_k) C_t dy_t is the slice's own contribution (``adjoint_summary``, the
transposed map of the fix-up), P the slice's product of a and q_next what arrives from the slice
after it.  The ranks all-gather (P, G), fold the summaries of the ranks after them
(``fold_suffix``), and run the ordinary backward kernel on their slice with the state entering
it (``h_in``) and the gradient arriving at its end (``q_in``).

``fold_prefix``, ``fold_suffix`` and ``exchange_summaries`` are plain tensor / torch.distributed
code and work on CPU tensors with the gloo backend, which is how the exchange logic is tested
without GPUs.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from . import _lib, selective_scan_cuda


def fold_prefix(P_all: torch.Tensor, h_all: torch.Tensor, rank: int):
    """P_all, h_all: (R, batch, dim, dstate) slice summaries in rank order.  Returns
    (p_in, h_in): product of a over all earlier slices and the state entering slice ``rank``."""
    p_in = torch.ones_like(P_all[0])
    h_in = torch.zeros_like(h_all[0])
    for j in range(rank):
        h_in = P_all[j] * h_in + h_all[j]
        p_in = p_in * P_all[j]
    return p_in, h_in


def fold_suffix(P_all: torch.Tensor, G_all: torch.Tensor, rank: int):
    """P_all, G_all: (R, batch, dim, dstate) products and adjoint summaries of the slices in rank
    order.  Returns q_in: the gradient with respect to the state at the end of slice ``rank``."""
    q = torch.zeros_like(G_all[0])
    for j in range(P_all.shape[0] - 1, rank, -1):
        q = G_all[j] + P_all[j] * q
    return q


def exchange_summaries(P: torch.Tensor, h: torch.Tensor, group=None):
    """All-gather the (P, h) summary of every rank; one collective of 2*B*D*N elements per rank."""
    world = dist.get_world_size(group)
    mine = torch.stack([P, h]).contiguous()
    gathered = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(gathered, mine, group=group)
    allp = torch.stack(gathered)          # (R, 2, batch, dim, dstate)
    return allp[:, 0], allp[:, 1]


def apply_fixup(u, delta, A, B, C, D, z, delta_bias, delta_softplus, out, x, out_z, p_in, h_in,
                discretization="mamba"):
    """Run b200_selscan_fixup in place on (out, x, out_z) of a zero-start forward call."""
    a, _ = selective_scan_cuda._common(u, delta, A, B, C, D, z, delta_bias, None, discretization)
    a.delta_softplus = int(bool(delta_softplus))
    a.out, a.x = out.data_ptr(), x.data_ptr()
    a.out_bs, a.out_ds = out.stride(0), out.stride(1)
    if out_z is not None:
        a.out_z = out_z.data_ptr()
        a.out_z_bs, a.out_z_ds = out_z.stride(0), out_z.stride(1)
    q = _lib.struct("b200_selscan_fixup_args")()
    q.f = a
    h_in = h_in.float().contiguous()
    p_in = p_in.float().contiguous()
    q.h_in, q.p_in = h_in.data_ptr(), p_in.data_ptr()
    q.n_segments, q.seg_len = 0, 0
    with torch.cuda.device(u.device):
        _lib.call("b200_selscan_fixup", q, torch.cuda.current_stream(u.device).cuda_stream)


def adjoint_summary(delta, A, C, z, delta_bias, delta_softplus, dout, discretization="mamba"):
    """G (batch, dim, dstate) float32 of this rank's slice (b200_selscan_adjoint_summary)."""
    if C.dim() == 3:
        C = C.unsqueeze(1)
    a, (batch, dim, seqlen, dstate, *_rest) = selective_scan_cuda._common(delta, delta, A, C, C, None, z, delta_bias, None,
                                                                        discretization)
    a.delta_softplus = int(bool(delta_softplus))
    q = _lib.struct("b200_selscan_adjsum_args")()
    q.f = a
    with torch.cuda.device(delta.device):
        G = torch.empty(batch, dim, dstate, dtype=torch.float32, device=delta.device)
        q.dout, q.G = dout.data_ptr(), G.data_ptr()
        q.dout_bs, q.dout_ds = dout.stride(0), dout.stride(1)
        _lib.call("b200_selscan_adjoint_summary", q, torch.cuda.current_stream(delta.device).cuda_stream)
    return G


def sp_selective_scan_fwd(u, delta, A, B, C, D=None, z=None, delta_bias=None, delta_softplus=False, group=None,
                          discretization="mamba", return_context=False):
    """Forward selective scan of a sequence sharded over the ranks of ``group`` (this rank passes
    its slice of u, delta, B, C, z; A, D, delta_bias are replicated).  Returns
    (out or out_z, last_state of this slice with the correct history); with ``return_context`` a
    third value, what the backward of this slice needs: (out, x, P_slice, h_in)."""
    if B.dim() == 3:
        B = B.unsqueeze(1)
    if C.dim() == 3:
        C = C.unsqueeze(1)
    out, x, *rest = selective_scan_cuda.fwd(u, delta, A, B, C, D, z, delta_bias, None, delta_softplus, discretization)
    out_z = rest[0] if rest else None
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    P_slice = x[:, :, -1, 0::2].contiguous()          # before the fix-up turns it into the product from t = 0
    h_in = None
    if world > 1:
        rank = dist.get_rank(group)
        P_all, h_all = exchange_summaries(P_slice, x[:, :, -1, 1::2].contiguous(), group)
        if rank > 0:
            p_in, h_in = fold_prefix(P_all, h_all, rank)
            apply_fixup(u, delta, A, B, C, D, z, delta_bias, delta_softplus, out, x, out_z, p_in, h_in, discretization)
    res = (out_z if out_z is not None else out), x[:, :, -1, 1::2]
    if return_context:
        return res + ((out, x, P_slice, h_in),)
    return res


def sp_selective_scan_bwd(u, delta, A, B, C, D, z, delta_bias, delta_softplus, dout, context, group=None,
                          discretization="mamba"):
    """Backward of ``sp_selective_scan_fwd`` for this rank's slice.  ``dout`` is the gradient of
    the returned output slice, ``context`` the forward's third return value.  Returns
    (du, ddelta, dA, dB, dC, dD, ddelta_bias, dz): the slice's input gradients, and the parameter
    gradients summed over all ranks (one all-reduce of (dim, dstate) + 2 dim floats)."""
    if B.dim() == 3:
        B = B.unsqueeze(1)
    if C.dim() == 3:
        C = C.unsqueeze(1)
    out, x, P_slice, h_in = context
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    q_in = None
    if world > 1:
        rank = dist.get_rank(group)
        G = adjoint_summary(delta, A, C, z, delta_bias, delta_softplus, dout, discretization)
        P_all, G_all = exchange_summaries(P_slice.float(), G, group)
        if rank < world - 1:
            q_in = fold_suffix(P_all, G_all, rank)
    res = selective_scan_cuda.bwd(u, delta, A, B, C, D, z, delta_bias, None, dout, x, out if z is not None else None, None,
                                  delta_softplus, False, discretization, h_in=h_in, q_in=q_in)
    du, ddelta, dA, dB, dC, dD, dbias = res[:7]
    dz = res[7] if z is not None else None
    if world > 1:
        flat = torch.cat([t.reshape(-1).float() for t in (dA, dD, dbias) if t is not None])
        dist.all_reduce(flat, group=group)
        o = 0
        outs = []
        for t in (dA, dD, dbias):
            if t is None:
                outs.append(None)
                continue
            outs.append(flat[o:o + t.numel()].reshape(t.shape).to(t.dtype))
            o += t.numel()
        dA, dD, dbias = outs
    return du, ddelta, dA, dB, dC, dD, dbias, dz


class SPSelectiveScanFn(torch.autograd.Function):
    """``selective_scan_fn`` on a sequence sharded over the ranks of a process group: every rank
    calls it with its slice (and the replicated A, D, delta_bias) and gets its slice of the output;
    ``backward`` returns the slice's input gradients and the full parameter gradients."""

    @staticmethod
    def forward(ctx, u, delta, A, B, C, D, z, delta_bias, delta_softplus, group, discretization):
        y, _last, context = sp_selective_scan_fwd(u, delta, A, B, C, D, z, delta_bias, delta_softplus, group,
                                                  discretization, return_context=True)
        out, x, P_slice, h_in = context
        ctx.save_for_backward(u, delta, A, B, C, D, z, delta_bias, out, x, P_slice, h_in)
        ctx.meta = (delta_softplus, group, discretization)
        return y

    @staticmethod
    def backward(ctx, dy):
        u, delta, A, B, C, D, z, delta_bias, out, x, P_slice, h_in = ctx.saved_tensors
        delta_softplus, group, discretization = ctx.meta
        if dy.stride(-1) != 1:
            dy = dy.contiguous()
        du, ddelta, dA, dB, dC, dD, dbias, dz = sp_selective_scan_bwd(
            u, delta, A, B, C, D, z, delta_bias, delta_softplus, dy, (out, x, P_slice, h_in), group, discretization)
        if B.dim() == 3:
            dB, dC = dB.squeeze(1), dC.squeeze(1)
        return du, ddelta, dA, dB, dC, dD, dz, dbias, None, None, None


def sp_selective_scan_fn(u, delta, A, B, C, D=None, z=None, delta_bias=None, delta_softplus=False, group=None,
                         discretization="mamba"):
    """Differentiable sequence-parallel selective scan (see ``SPSelectiveScanFn``)."""
    return SPSelectiveScanFn.apply(u, delta, A, B, C, D, z, delta_bias, delta_softplus, group, discretization)
