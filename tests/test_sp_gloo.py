"""Sequence-parallel exchange logic on CPU ranks (gloo, world size 2 and 3): every rank scans
its slice from a zero state with the CPU oracle, the ranks all-gather their (product, state)
summaries through lrnnx_b200.sp.exchange_summaries, fold them with fold_prefix, apply the
fix-up formula, and the stitched result must equal the unsplit oracle scan.  The backward runs the
mirrored exchange: adjoint summaries all-gathered, folded from the right with fold_suffix, the
slice's gradients taken with the folded gradient applied to its final state; the stitched input
gradients and the all-reduced parameter gradients must equal autograd through the unsplit scan."""
from __future__ import annotations

import os
import sys
from pathlib import Path

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parents[1]


def _inputs(L):
    g = torch.Generator().manual_seed(3)
    b, d, n = 2, 6, 4
    return dict(u=torch.randn(b, d, L, generator=g), delta=torch.randn(b, d, L, generator=g) - 1.0,
                A=-torch.rand(d, n, generator=g) - 0.05, B=torch.randn(b, 1, n, L, generator=g),
                C=torch.randn(b, 1, n, L, generator=g), D=torch.randn(d, generator=g),
                z=torch.randn(b, d, L, generator=g), delta_bias=torch.rand(d, generator=g) - 1.0)


def _worker(rank, world, port, L, q):
    sys.path.insert(0, str(ROOT))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import torch.nn.functional as F
        from lrnnx_b200.sp import exchange_summaries, fold_prefix
        from oracle import scan_oracle as O
        t = _inputs(L)
        lo, hi = rank * L // world, (rank + 1) * L // world
        sl = {k: (v[..., lo:hi] if v.dim() >= 3 else v) for k, v in t.items()}
        # local zero-start scan without gating; the gate is applied after the fix-up
        out, last, x = O.selective_scan_oracle(sl["u"], sl["delta"], sl["A"], sl["B"], sl["C"], sl["D"], None,
                                               sl["delta_bias"], delta_softplus=True, return_last_state=True,
                                               return_checkpoints=True)
        P_all, h_all = exchange_summaries(x[:, :, -1, 0::2].contiguous(), x[:, :, -1, 1::2].contiguous())
        p_in, h_in = fold_prefix(P_all, h_all, rank)
        dl = F.softplus(sl["delta"] + sl["delta_bias"][:, None])
        decay = torch.exp(dl.cumsum(-1).unsqueeze(-1) * sl["A"][None, :, None, :])          # (b, d, l, n)
        Cx = sl["C"].expand(-1, sl["u"].shape[1], -1, -1).permute(0, 1, 3, 2)               # (b, d, l, n)
        out = out + (Cx * decay * h_in.unsqueeze(2)).sum(-1)
        out = out * F.silu(sl["z"])
        last = last + x[:, :, -1, 0::2] * h_in
        q.put((rank, out, last))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,L", [(2, 64), (3, 99)])
def test_sp_fold_matches_unsplit_oracle(world, L):
    from oracle import scan_oracle as O
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + (os.getpid() % 500) + world
    procs = [ctx.Process(target=_worker, args=(r, world, port, L, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = dict()
    for _ in range(world):
        r, out, last = q.get(timeout=120)
        results[r] = (out, last)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    t = _inputs(L)
    ref, ref_last = O.selective_scan_oracle(**t, delta_softplus=True, return_last_state=True)
    got = torch.cat([results[r][0] for r in range(world)], dim=-1)
    torch.testing.assert_close(got, ref, rtol=2e-5, atol=2e-5)
    torch.testing.assert_close(results[world - 1][1], ref_last, rtol=2e-5, atol=2e-5)


def test_fold_prefix_identity_for_rank0():
    from lrnnx_b200.sp import fold_prefix
    P = torch.rand(3, 2, 4, 5)
    h = torch.randn(3, 2, 4, 5)
    p_in, h_in = fold_prefix(P, h, 0)
    assert torch.equal(p_in, torch.ones(2, 4, 5)) and torch.equal(h_in, torch.zeros(2, 4, 5))
    p2, h2 = fold_prefix(P, h, 2)
    torch.testing.assert_close(p2, P[0] * P[1])
    torch.testing.assert_close(h2, P[1] * h[0] + h[1])


def _slice_scan(u, delta, A, B, C, D, z, bias, h0):
    """Differentiable scan of a slice from the state h0 (plain loop; "mamba" discretization)."""
    import torch.nn.functional as F
    dl = F.softplus(delta + bias[:, None])
    h = h0
    ys = []
    for t in range(u.shape[-1]):
        a = torch.exp(dl[:, :, t, None] * A)
        h = a * h + dl[:, :, t, None] * B[:, 0, :, t][:, None, :] * u[:, :, t, None]
        ys.append((h * C[:, 0, :, t][:, None, :]).sum(-1) + D * u[:, :, t])
    return torch.stack(ys, dim=-1) * F.silu(z), h, torch.exp(dl.sum(-1, keepdim=True) * A)


def _bwd_worker(rank, world, port, L, q):
    sys.path.insert(0, str(ROOT))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from lrnnx_b200.sp import exchange_summaries, fold_prefix, fold_suffix
        t = _inputs(L)
        gout = torch.randn(t["u"].shape, generator=torch.Generator().manual_seed(17))
        lo, hi = rank * L // world, (rank + 1) * L // world
        names = ("u", "delta", "B", "C", "z")
        sl = {k: t[k][..., lo:hi].clone().requires_grad_(True) for k in names}
        par = {k: t[k].clone().requires_grad_(True) for k in ("A", "D", "delta_bias")}
        zero = torch.zeros(t["u"].shape[0], t["u"].shape[1], t["A"].shape[1])
        # forward exchange: zero-start summary of the slice, folded from the left
        with torch.no_grad():
            _, h_loc, P_loc = _slice_scan(sl["u"], sl["delta"], par["A"], sl["B"], sl["C"], par["D"], sl["z"],
                                          par["delta_bias"], zero)
        P_all, h_all = exchange_summaries(P_loc.contiguous(), h_loc.contiguous())
        _, h_in = fold_prefix(P_all, h_all, rank)
        # backward exchange: the slice's own adjoint summary is the gradient at its entering state
        h0 = h_in.clone().requires_grad_(True)
        y, h_last, _ = _slice_scan(sl["u"], sl["delta"], par["A"], sl["B"], sl["C"], par["D"], sl["z"],
                                   par["delta_bias"], h0)
        (G,) = torch.autograd.grad((y * gout[..., lo:hi]).sum(), h0, retain_graph=True)
        P_all, G_all = exchange_summaries(P_loc.contiguous(), G.contiguous())
        q_in = fold_suffix(P_all, G_all, rank)
        ((y * gout[..., lo:hi]).sum() + (h_last * q_in).sum()).backward()
        pg = torch.cat([par[k].grad.reshape(-1) for k in ("A", "D", "delta_bias")])
        dist.all_reduce(pg)
        q.put((rank, {k: sl[k].grad for k in names}, pg))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,L", [(2, 48), (3, 75)])
def test_sp_backward_fold_matches_unsplit_autograd(world, L):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29100 + (os.getpid() % 500) + world
    procs = [ctx.Process(target=_bwd_worker, args=(r, world, port, L, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = dict()
    for _ in range(world):
        r, grads, pg = q.get(timeout=180)
        results[r] = (grads, pg)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    t = _inputs(L)
    gout = torch.randn(t["u"].shape, generator=torch.Generator().manual_seed(17))
    leaves = {k: v.clone().requires_grad_(True) for k, v in t.items()}
    zero = torch.zeros(t["u"].shape[0], t["u"].shape[1], t["A"].shape[1])
    y, _, _ = _slice_scan(leaves["u"], leaves["delta"], leaves["A"], leaves["B"], leaves["C"], leaves["D"], leaves["z"],
                          leaves["delta_bias"], zero)
    (y * gout).sum().backward()
    for k in ("u", "delta", "B", "C", "z"):
        got = torch.cat([results[r][0][k] for r in range(world)], dim=-1)
        torch.testing.assert_close(got, leaves[k].grad, rtol=2e-5, atol=2e-5, msg=lambda m: f"d{k}: {m}")
    ref_pg = torch.cat([leaves[k].grad.reshape(-1) for k in ("A", "D", "delta_bias")])
    for r in range(world):
        torch.testing.assert_close(results[r][1], ref_pg, rtol=2e-5, atol=2e-5)


def test_fold_suffix_identity_for_last_rank():
    from lrnnx_b200.sp import fold_suffix
    P = torch.rand(3, 2, 4, 5)
    G = torch.randn(3, 2, 4, 5)
    assert torch.equal(fold_suffix(P, G, 2), torch.zeros(2, 4, 5))
    torch.testing.assert_close(fold_suffix(P, G, 1), G[2])
    torch.testing.assert_close(fold_suffix(P, G, 0), G[1] + P[1] * G[2])
