"""Out-of-range reads and run-to-run reproducibility of the CUDA path.

The operands of a call are views into larger buffers whose surroundings are filled with NaN (a
"moat"): a kernel that reads past a row's end, before its start, or into the next row picks up a
NaN that the recurrence carries to the outputs.  The views also start at odd offsets, so the rows
are not 16-byte aligned and the bulk-copy paths must fall back.  Results are compared with the
same call on dense copies of the operands.

State buffers that a call updates in place (``selective_state_update``, ``causal_conv1d_update``)
sit between guard rows whose bit patterns must survive the call.

Forward kernels contain no atomics: a repeated call must reproduce its outputs bit for bit.
"""
from __future__ import annotations

import pytest
import torch

from conftest import assert_close

pytestmark = pytest.mark.gpu


def moat(t, pad=5):
    """A view equal to ``t`` inside a NaN-filled buffer: ``pad`` extra elements on both sides of the
    last dimension and one extra slab on both sides of the first."""
    shape = list(t.shape)
    fill = complex("nan+nanj") if t.is_complex() else float("nan")
    big = torch.full([shape[0] + 2] + shape[1:-1] + [shape[-1] + 2 * pad], fill, dtype=t.dtype, device=t.device)
    view = big[1:-1, ..., pad:pad + shape[-1]]
    view.copy_(t)
    return view


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("L", [37, 256, 300, 2051])
def test_selective_scan_reads_stay_inside_the_rows(L, dtype):
    from lrnnx_b200.ops import selective_scan_fn
    g = torch.Generator().manual_seed(L)
    batch, dim, N = 2, 32, 16
    mk = lambda *s: torch.randn(*s, generator=g).to(dtype).cuda()
    u, delta, z = mk(batch, dim, L), mk(batch, dim, L), mk(batch, dim, L)
    B, C = mk(batch, 1, N, L), mk(batch, 1, N, L)
    A = -torch.rand(dim, N, generator=g).cuda() - 0.5
    D = torch.randn(dim, generator=g).cuda()
    bias = (torch.rand(dim, generator=g) - 3.0).cuda()
    gout = mk(batch, dim, L)

    def run(wrap):
        ins = [wrap(t).detach().requires_grad_(True) for t in (u, delta, B, C, z)]
        Ap, Dp, bp = (t.detach().requires_grad_(True) for t in (A, D, bias))
        y, last = selective_scan_fn(ins[0], ins[1], Ap, ins[2], ins[3], Dp, z=ins[4], delta_bias=bp,
                                    delta_softplus=True, return_last_state=True)
        y.backward(wrap(gout) if wrap is moat else gout)
        return [y.detach(), last] + [t.grad for t in ins] + [Ap.grad, Dp.grad, bp.grad]

    dense = run(lambda t: t.clone())
    guarded = run(moat)
    tol = 2e-4 if dtype == torch.float32 else 3e-2
    for i, (a, b) in enumerate(zip(guarded, dense)):
        assert torch.isfinite(a.float()).all(), f"output {i} picked up a value from outside its operands"
        assert_close(a.float(), b.float(), rtol=tol, atol_scale=tol, name=f"output {i}")


@pytest.mark.parametrize("disc", ["zoh", "bilinear", "dirac"])
@pytest.mark.parametrize("L", [45, 320, 1283])
def test_simplified_scan_reads_stay_inside_the_rows(L, disc):
    from lrnnx_b200 import simplified_scan_cuda as ext
    g = torch.Generator().manual_seed(L)
    batch, P = 2, 24
    cn = lambda *s: torch.complex(torch.randn(*s, generator=g), torch.randn(*s, generator=g)).cuda()
    u, dout = cn(batch, P, L), cn(batch, P, L)
    delta = (0.2 + torch.rand(batch, P, L, generator=g)).cuda()
    A = torch.complex(-0.1 - torch.rand(P, 1, generator=g), torch.randn(P, 1, generator=g)).cuda()
    one = torch.ones(P, 1, dtype=torch.complex64).cuda()

    def run(wrap):
        uu, dd, gg = wrap(u), wrap(delta), wrap(dout)
        out, x = ext.fwd(uu, dd, A, one, one, None, disc)
        res = ext.bwd(uu, dd, A, one, one, None, gg, x, disc)
        return [out] + [r for r in res[:5] if r is not None]

    wrap_moat = lambda t: moat(t, pad=3)

    dense = run(lambda t: t.clone())
    guarded = run(wrap_moat)
    for i, (a, b) in enumerate(zip(guarded, dense)):
        assert torch.isfinite(torch.view_as_real(a) if a.is_complex() else a).all(), f"output {i}"
        assert_close(torch.view_as_real(a) if a.is_complex() else a, torch.view_as_real(b) if b.is_complex() else b,
                     rtol=2e-4, atol_scale=2e-4, name=f"output {i}")


def test_state_update_leaves_guard_rows_alone():
    from lrnnx_b200.ops import selective_state_update
    from lrnnx_b200.ops.mamba_block import causal_conv1d_update
    g = torch.Generator().manual_seed(3)
    batch, dim, N, W = 5, 256, 16, 4
    pattern = torch.arange((batch + 2) * dim * N, dtype=torch.float32).reshape(batch + 2, dim, N).cuda() * 0.5 + 7.0
    big = pattern.clone()
    state = big[1:-1]
    state.copy_(torch.randn(batch, dim, N, generator=g).cuda())
    x, dt = (torch.randn(batch, dim, generator=g).cuda() for _ in range(2))
    A = -torch.rand(dim, N, generator=g).cuda()
    Bm, Cm = (torch.randn(batch, N, generator=g).cuda() for _ in range(2))
    out = selective_state_update(state, x, dt, A, Bm, Cm, dt_softplus=True)
    assert torch.isfinite(out).all()
    assert torch.equal(big[0], pattern[0]) and torch.equal(big[-1], pattern[-1])

    cpat = torch.arange((batch + 2) * dim * W, dtype=torch.float32).reshape(batch + 2, dim, W).cuda() + 0.25
    cbig = cpat.clone()
    cstate = cbig[1:-1]
    cstate.copy_(torch.randn(batch, dim, W, generator=g).cuda())
    w = torch.randn(dim, W, generator=g).cuda()
    y = causal_conv1d_update(x, cstate, w, None, "silu")
    assert torch.isfinite(y).all()
    assert torch.equal(cbig[0], cpat[0]) and torch.equal(cbig[-1], cpat[-1])


def test_forward_kernels_reproduce_bit_for_bit():
    from lrnnx_b200 import selective_scan_cuda, simplified_scan_cuda
    from lrnnx_b200.ops.mamba_block import causal_conv1d_fn, rms_norm_fn
    g = torch.Generator().manual_seed(11)
    batch, dim, N, L = 2, 64, 16, 1000
    mk = lambda *s: torch.randn(*s, generator=g).cuda()
    u, delta, z = mk(batch, dim, L), mk(batch, dim, L), mk(batch, dim, L)
    B, C = mk(batch, 1, N, L), mk(batch, 1, N, L)
    A = -torch.rand(dim, N, generator=g).cuda() - 0.5
    r1 = selective_scan_cuda.fwd(u, delta, A, B, C, None, z, None, None, True, "mamba")
    r2 = selective_scan_cuda.fwd(u, delta, A, B, C, None, z, None, None, True, "mamba")
    for a, b in zip(r1, r2):
        assert torch.equal(a, b)
    cu = torch.complex(mk(batch, dim, L), mk(batch, dim, L))
    Ac = torch.complex(-0.1 - torch.rand(dim, 1, generator=g), torch.randn(dim, 1, generator=g)).cuda()
    one = torch.ones(dim, 1, dtype=torch.complex64).cuda()
    d2 = (0.2 + torch.rand(batch, dim, L, generator=g)).cuda()
    s1 = simplified_scan_cuda.fwd(cu, d2, Ac, one, one, None, "zoh")
    s2 = simplified_scan_cuda.fwd(cu, d2, Ac, one, one, None, "zoh")
    for a, b in zip(s1, s2):
        assert torch.equal(torch.view_as_real(a), torch.view_as_real(b))
    w = mk(dim, 4)
    assert torch.equal(causal_conv1d_fn(u, w, None, "silu"), causal_conv1d_fn(u, w, None, "silu"))
    h = mk(300, 768)
    gw = mk(768)
    assert torch.equal(rms_norm_fn(h, gw, None, residual=h * 0.5), rms_norm_fn(h, gw, None, residual=h * 0.5))
