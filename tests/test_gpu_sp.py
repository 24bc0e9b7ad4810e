"""Sequence-parallel fix-up kernel on one GPU: the sequence is cut into R slices that are scanned
one after the other as R emulated ranks (zero-start forward, summary fold on the device,
b200_selscan_fixup), and the stitched output, gated output, checkpoints and last state must
equal the unsplit forward of the same library and the CPU oracle.  The backward is emulated the
same way from the right (adjoint summaries, fold_suffix, b200_selscan_bwd with h_in / q_in) and
must reproduce the gradients of the unsplit backward."""
from __future__ import annotations

import pytest
import torch

from conftest import assert_close
from oracle import scan_oracle as O

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype,rtol,atol", [(torch.float32, 1e-4, 2e-5), (torch.bfloat16, 3e-2, 1e-2)])
@pytest.mark.parametrize("R,L", [(2, 512), (4, 8192), (3, 4104)])
def test_sp_slices_match_unsplit(R, L, dtype, rtol, atol):
    from lrnnx_b200 import selective_scan_cuda
    from lrnnx_b200.sp import apply_fixup, fold_prefix
    g = torch.Generator().manual_seed(L + R)
    b, d, n = 1, 32, 16
    t = dict(u=torch.randn(b, d, L, generator=g).to(dtype), delta=(torch.randn(b, d, L, generator=g) - 2.0).to(dtype),
             A=-torch.rand(d, n, generator=g) * 0.5 - 0.01, B=torch.randn(b, 1, n, L, generator=g).to(dtype),
             C=torch.randn(b, 1, n, L, generator=g).to(dtype), D=torch.randn(d, generator=g),
             z=torch.randn(b, d, L, generator=g).to(dtype), delta_bias=torch.rand(d, generator=g) - 3.0)
    cu = {k: v.cuda() for k, v in t.items()}
    full = selective_scan_cuda.fwd(cu["u"], cu["delta"], cu["A"], cu["B"], cu["C"], cu["D"], cu["z"],
                                   cu["delta_bias"], None, True, "mamba")
    bounds = [(r * L // R) // 8 * 8 for r in range(R)] + [L]
    outs, outzs, Ps, hs, xs = [], [], [], [], []
    for r in range(R):
        lo, hi = bounds[r], bounds[r + 1]
        sl = {k: (v[..., lo:hi].contiguous() if v.dim() >= 3 else v) for k, v in cu.items()}
        out, x, out_z = selective_scan_cuda.fwd(sl["u"], sl["delta"], sl["A"], sl["B"], sl["C"], sl["D"], sl["z"],
                                                sl["delta_bias"], None, True, "mamba")
        Ps.append(x[:, :, -1, 0::2].clone())
        hs.append(x[:, :, -1, 1::2].clone())
        if r > 0:
            p_in, h_in = fold_prefix(torch.stack(Ps), torch.stack(hs), r)
            apply_fixup(sl["u"], sl["delta"], sl["A"], sl["B"], sl["C"], sl["D"], sl["z"], sl["delta_bias"], True,
                        out, x, out_z, p_in, h_in)
        outs.append(out)
        outzs.append(out_z)
        xs.append(x)
    out_sp, outz_sp = torch.cat(outs, -1), torch.cat(outzs, -1)
    assert_close(out_sp.float().cpu(), full[0].float().cpu(), rtol=rtol, atol_scale=atol, name="out vs unsplit")
    assert_close(outz_sp.float().cpu(), full[2].float().cpu(), rtol=rtol, atol_scale=atol, name="out_z vs unsplit")
    assert_close(xs[-1][:, :, -1, 1::2].cpu(), full[1][:, :, -1, 1::2].cpu(), rtol=1e-4, atol_scale=1e-4,
                 name="last state vs unsplit")
    ref = O.selective_scan_oracle(**t, delta_softplus=True)
    assert_close(outz_sp.float().cpu(), ref.float(), rtol=rtol, atol_scale=atol, name="out_z vs oracle")


@pytest.mark.parametrize("dtype,rtol,atol", [(torch.float32, 3e-4, 1e-4), (torch.bfloat16, 3e-2, 1e-2)])
@pytest.mark.parametrize("R,L", [(2, 512), (4, 8192), (3, 4104)])
def test_sp_backward_slices_match_unsplit(R, L, dtype, rtol, atol):
    from lrnnx_b200 import selective_scan_cuda
    from lrnnx_b200.sp import adjoint_summary, apply_fixup, fold_prefix, fold_suffix
    g = torch.Generator().manual_seed(L + 7 * R)
    b, d, n = 2, 32, 16
    t = dict(u=torch.randn(b, d, L, generator=g).to(dtype), delta=(torch.randn(b, d, L, generator=g) - 2.0).to(dtype),
             A=-torch.rand(d, n, generator=g) * 0.5 - 0.01, B=torch.randn(b, 1, n, L, generator=g).to(dtype),
             C=torch.randn(b, 1, n, L, generator=g).to(dtype), D=torch.randn(d, generator=g),
             z=torch.randn(b, d, L, generator=g).to(dtype), delta_bias=torch.rand(d, generator=g) - 3.0)
    cu = {k: v.cuda() for k, v in t.items()}
    gout = torch.randn(b, d, L, generator=g).to(dtype).cuda()
    out, x, _ = selective_scan_cuda.fwd(cu["u"], cu["delta"], cu["A"], cu["B"], cu["C"], cu["D"], cu["z"],
                                        cu["delta_bias"], None, True, "mamba")
    ref = selective_scan_cuda.bwd(cu["u"], cu["delta"], cu["A"], cu["B"], cu["C"], cu["D"], cu["z"], cu["delta_bias"],
                                  None, gout, x, out, None, True, False, "mamba")
    bounds = [(r * L // R) // 8 * 8 for r in range(R)] + [L]
    slices, ctxs, Ps, hs = [], [], [], []
    for r in range(R):                                   # forward, left to right
        lo, hi = bounds[r], bounds[r + 1]
        sl = {k: (v[..., lo:hi].contiguous() if v.dim() >= 3 else v) for k, v in cu.items()}
        o, xs, oz = selective_scan_cuda.fwd(sl["u"], sl["delta"], sl["A"], sl["B"], sl["C"], sl["D"], sl["z"],
                                            sl["delta_bias"], None, True, "mamba")
        Ps.append(xs[:, :, -1, 0::2].clone())
        hs.append(xs[:, :, -1, 1::2].clone())
        h_in = None
        if r > 0:
            p_in, h_in = fold_prefix(torch.stack(Ps), torch.stack(hs), r)
            apply_fixup(sl["u"], sl["delta"], sl["A"], sl["B"], sl["C"], sl["D"], sl["z"], sl["delta_bias"], True,
                        o, xs, oz, p_in, h_in)
        slices.append(sl)
        ctxs.append((o, xs, h_in))
    Gs = [adjoint_summary(sl["delta"], sl["A"], sl["C"], sl["z"], sl["delta_bias"], True,
                          gout[..., bounds[r]:bounds[r + 1]].contiguous()) for r, sl in enumerate(slices)]
    P_all, G_all = torch.stack(Ps).float(), torch.stack(Gs)
    parts = []
    for r in range(R):                                   # every slice's backward is independent of the others now
        sl, (o, xs, h_in) = slices[r], ctxs[r]
        q_in = fold_suffix(P_all, G_all, r) if r < R - 1 else None
        parts.append(selective_scan_cuda.bwd(sl["u"], sl["delta"], sl["A"], sl["B"], sl["C"], sl["D"], sl["z"],
                                             sl["delta_bias"], None, gout[..., bounds[r]:bounds[r + 1]].contiguous(), xs, o,
                                             None, True, False, "mamba", h_in=h_in, q_in=q_in))
    names = ["du", "ddelta", "dA", "dB", "dC", "dD", "ddelta_bias", "dz"]
    for i, name in enumerate(names):
        if name in ("dA", "dD", "ddelta_bias"):
            got = sum(p[i].float() for p in parts)
            tol_r, tol_a = (3e-4, 1e-4) if dtype == torch.float32 else (3e-2, 2e-2)
        else:
            got = torch.cat([p[i].float() for p in parts], dim=-1)
            tol_r, tol_a = rtol, atol
        assert_close(got.cpu(), ref[i].float().cpu(), rtol=tol_r, atol_scale=tol_a, name=f"{name} vs unsplit backward")


def test_adjoint_summary_is_the_transpose_of_the_fixup():
    """<fixup(h), dy> = <h, adjoint_summary(dy)> for random h and dy (both maps are linear)."""
    from lrnnx_b200 import selective_scan_cuda
    from lrnnx_b200.sp import adjoint_summary, apply_fixup
    g = torch.Generator().manual_seed(91)
    b, d, n, L = 2, 16, 16, 777
    mk = lambda *s: torch.randn(*s, generator=g).cuda()
    u, delta = mk(b, d, L), mk(b, d, L) - 2.0
    A = (-torch.rand(d, n, generator=g) * 0.5 - 0.01).cuda()
    B, C = mk(b, 1, n, L), mk(b, 1, n, L)
    bias = (torch.rand(d, generator=g) - 3.0).cuda()
    out, x = selective_scan_cuda.fwd(u, delta, A, B, C, None, None, bias, None, True, "mamba")
    h = mk(b, d, n)
    dy = mk(b, d, L)
    out2, x2 = out.clone(), x.clone()
    apply_fixup(u, delta, A, B, C, None, None, bias, True, out2, x2, None, torch.ones_like(h), h)
    lhs = ((out2 - out).double() * dy.double()).sum().item()
    G = adjoint_summary(delta, A, C, None, bias, True, dy)
    rhs = (h.double() * G.double()).sum().item()
    assert abs(lhs - rhs) <= 1e-4 * max(abs(lhs), abs(rhs), 1.0), (lhs, rhs)


def _nccl_worker(rank, world, port, L, q):
    import os
    import sys
    from pathlib import Path
    sys.path.insert(0, str(Path(__file__).resolve().parents[1]))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from lrnnx_b200.sp import sp_selective_scan_fn
        g = torch.Generator().manual_seed(123)
        b, d, n = 2, 32, 16
        t = dict(u=torch.randn(b, d, L, generator=g), delta=torch.randn(b, d, L, generator=g) - 2.0,
                 A=-torch.rand(d, n, generator=g) * 0.5 - 0.01, B=torch.randn(b, 1, n, L, generator=g),
                 C=torch.randn(b, 1, n, L, generator=g), D=torch.randn(d, generator=g),
                 z=torch.randn(b, d, L, generator=g), delta_bias=torch.rand(d, generator=g) - 3.0)
        gout = torch.randn(b, d, L, generator=g)
        lo, hi = rank * L // world, (rank + 1) * L // world
        dev = torch.device("cuda", rank)
        sl = {k: (v[..., lo:hi].contiguous() if v.dim() >= 3 else v).to(dev).requires_grad_(True) for k, v in t.items()}
        y = sp_selective_scan_fn(sl["u"], sl["delta"], sl["A"], sl["B"], sl["C"], sl["D"], sl["z"], sl["delta_bias"], True)
        y.backward(gout[..., lo:hi].to(dev))
        torch.cuda.synchronize()
        q.put((rank, y.detach().cpu(), {k: v.grad.cpu() for k, v in sl.items()}))
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("L", [4096, 6144])
def test_sp_scan_fn_over_nccl_matches_unsplit(L):
    """sp_selective_scan_fn on two ranks over NCCL (one GPU each): the slices' outputs and input
    gradients, stitched, and the all-reduced parameter gradients equal the unsplit op."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import os
    import torch.multiprocessing as mp
    from lrnnx_b200.ops import selective_scan_fn
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29300 + (os.getpid() % 400)
    procs = [ctx.Process(target=_nccl_worker, args=(r, world, port, L, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = {}
    for _ in range(world):
        r, y, grads = q.get(timeout=300)
        res[r] = (y, grads)
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    g = torch.Generator().manual_seed(123)
    b, d, n = 2, 32, 16
    t = dict(u=torch.randn(b, d, L, generator=g), delta=torch.randn(b, d, L, generator=g) - 2.0,
             A=-torch.rand(d, n, generator=g) * 0.5 - 0.01, B=torch.randn(b, 1, n, L, generator=g),
             C=torch.randn(b, 1, n, L, generator=g), D=torch.randn(d, generator=g),
             z=torch.randn(b, d, L, generator=g), delta_bias=torch.rand(d, generator=g) - 3.0)
    gout = torch.randn(b, d, L, generator=g)
    cu = {k: v.cuda().requires_grad_(True) for k, v in t.items()}
    y = selective_scan_fn(cu["u"], cu["delta"], cu["A"], cu["B"], cu["C"], cu["D"], z=cu["z"], delta_bias=cu["delta_bias"],
                          delta_softplus=True)
    y.backward(gout.cuda())
    assert_close(torch.cat([res[r][0] for r in range(world)], -1), y.detach().cpu(), rtol=1e-4, atol_scale=2e-5, name="out")
    for k in ("u", "delta", "B", "C", "z"):
        got = torch.cat([res[r][1][k] for r in range(world)], -1)
        assert_close(got, cu[k].grad.cpu(), rtol=3e-4, atol_scale=1e-4, name=f"d{k}")
    for k in ("A", "D", "delta_bias"):
        for r in range(world):
            assert_close(res[r][1][k], cu[k].grad.cpu(), rtol=3e-4, atol_scale=1e-4, name=f"d{k} on rank {r}")
