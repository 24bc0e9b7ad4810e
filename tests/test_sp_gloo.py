"""Sequence-parallel exchange logic on CPU ranks (gloo, world size 2 and 3): every rank scans
its slice from a zero state with the CPU oracle, the ranks all-gather their (product, state)
summaries through lrnnx_b200.sp.exchange_summaries, fold them with fold_prefix, apply the
fix-up formula, and the stitched result must equal the unsplit oracle scan."""
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
