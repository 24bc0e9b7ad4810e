"""Sequence-parallel forward of the selective scan (BASELINE config 3).

lrnnx is single-GPU; this is the multi-GPU split its long-sequence case needs.  Rank r owns
the timesteps [r*L/R, (r+1)*L/R).  Because the recurrence h_t = a_t h_{t-1} + b_t is linear,
a slice is summarised by (P_r, h_r) = (product of a over the slice, final state from a zero
start) — exactly the last checkpoint entry the forward kernel already writes
(x[:, :, -1, 0::2], x[:, :, -1, 1::2]).  The ranks all-gather these 2*B*D*N floats, fold the
summaries of the ranks before them (h <- P_j h + h_j) to get the state entering their slice,
and a fix-up kernel adds that state's contribution to the zero-start output.

``fold_prefix`` and ``exchange_summaries`` are plain tensor / torch.distributed code and work
on CPU tensors with the gloo backend, which is how the exchange logic is tested without GPUs.
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


def sp_selective_scan_fwd(u, delta, A, B, C, D=None, z=None, delta_bias=None, delta_softplus=False, group=None,
                          discretization="mamba"):
    """Forward selective scan of a sequence sharded over the ranks of ``group`` (this rank passes
    its slice of u, delta, B, C, z; A, D, delta_bias are replicated).  Returns
    (out or out_z, last_state of this slice with the correct history)."""
    if B.dim() == 3:
        B = B.unsqueeze(1)
    if C.dim() == 3:
        C = C.unsqueeze(1)
    out, x, *rest = selective_scan_cuda.fwd(u, delta, A, B, C, D, z, delta_bias, None, delta_softplus, discretization)
    out_z = rest[0] if rest else None
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    if world > 1:
        rank = dist.get_rank(group)
        P_all, h_all = exchange_summaries(x[:, :, -1, 0::2].contiguous(), x[:, :, -1, 1::2].contiguous(), group)
        if rank > 0:
            p_in, h_in = fold_prefix(P_all, h_all, rank)
            apply_fixup(u, delta, A, B, C, D, z, delta_bias, delta_softplus, out, x, out_z, p_in, h_in, discretization)
    return (out_z if out_z is not None else out), x[:, :, -1, 1::2]
