"""GPU parity of the S4 Cauchy and log-Vandermonde kernels through the C ABI.

Reference side: golden fixtures from lrnnx's cauchy_mult_torch (complex128) and
log_vandermonde_naive, and the complex128 oracle on the sweep of
tests/ops/s4/test_cauchy.py:47-50.  The reference's acceptance rule is relative to pykeops,
which is not available; the rule here is  |x - ref128| <= 1e-4*|ref128| + 1e-4*mean|ref128|
on the output and 2e-4 likewise on gradients (fp32 accumulation over up to 2^18 terms)."""
from __future__ import annotations

import pytest
import torch

from conftest import load_golden
from oracle import scan_oracle as O

pytestmark = pytest.mark.gpu
S4 = load_golden("s4")


def _close(got, want, rtol, name):
    want = want.to(got.dtype)
    tol = rtol * want.abs() + rtol * want.abs().mean()
    bad = (got - want).abs() > tol
    assert not bool(bad.any()), f"{name}: {int(bad.sum())} of {bad.numel()} outside tolerance, " \
                                f"max abs err {float((got - want).abs().max()):.3e}"


@pytest.mark.parametrize("name", sorted(S4))
def test_s4_golden(name):
    from lrnnx_b200.ops import cauchy_mult, log_vandermonde_cuda
    case = S4[name]
    i = case["inputs"]
    if name.startswith("cauchy"):
        v, w = i["v"].cuda().requires_grad_(True), i["w"].cuda().requires_grad_(True)
        out = cauchy_mult(v, i["z"].cuda(), w)
        dv, dw = torch.autograd.grad(out, (v, w), case["gout"].cuda())
        _close(out.detach().cpu(), case["outputs"][0], 1e-4, "out")
        _close(dv.cpu(), case["grads"]["v"], 2e-4, "dv")
        _close(dw.cpu(), case["grads"]["w"], 2e-4, "dw")
    else:
        v, x = i["v"].cuda().requires_grad_(True), i["x"].cuda().requires_grad_(True)
        out = log_vandermonde_cuda(v, x, i["L"])
        dv, dx = torch.autograd.grad(out, (v, x), case["gout"].cuda())
        _close(out.detach().cpu(), case["outputs"][0], 1e-4, "out")
        _close(dv.cpu(), case["grads"]["v"], 2e-4, "dv")
        _close(dx.cpu(), case["grads"]["x"], 2e-4, "dx")


@pytest.mark.parametrize("L", [3, 17, 489, 1024, 1047, 4096, 2 ** 14, 2 ** 18])
@pytest.mark.parametrize("n_half", [2, 16, 128, 1024])
def test_cauchy_sweep(n_half, L):
    from lrnnx_b200.ops import cauchy_mult
    if n_half * L > 2 ** 25:
        pytest.skip("oracle too slow at this size")
    g = torch.Generator().manual_seed(2357)
    batch = 4
    c = lambda *s: torch.complex(torch.randn(*s, generator=g), torch.randn(*s, generator=g))
    v, w = c(batch, n_half), c(batch, n_half)
    z = torch.exp(1j * torch.randn(L, generator=g))
    v64, w64 = v.cdouble().requires_grad_(True), w.cdouble().requires_grad_(True)
    out_c = O.cauchy_oracle(v64, z, w64)
    gout = c(batch, L)
    dv_c, dw_c = torch.autograd.grad(out_c, (v64, w64), gout.cdouble())
    vg, wg = v.cuda().requires_grad_(True), w.cuda().requires_grad_(True)
    out_g = cauchy_mult(vg, z.cuda(), wg)
    dv_g, dw_g = torch.autograd.grad(out_g, (vg, wg), gout.cuda())
    _close(out_g.detach().cpu(), out_c.detach(), 1e-4, "out")
    _close(dv_g.cpu(), dv_c, 2e-4, "dv")
    _close(dw_g.cpu(), dw_c, 2e-4, "dw")


@pytest.mark.parametrize("L", [3, 489, 4096])
@pytest.mark.parametrize("n_half", [2, 32, 128])
def test_vandermonde_sweep(n_half, L):
    from lrnnx_b200.ops import log_vandermonde_cuda
    g = torch.Generator().manual_seed(2357)
    batch = 4
    v = torch.complex(torch.randn(batch, n_half, generator=g), torch.randn(batch, n_half, generator=g))
    # decaying modes with phases that stay exactly representable in fp32 over the whole range
    x = torch.complex(-0.001 * torch.rand(batch, n_half, generator=g),
                      torch.randint(0, 4096, (batch, n_half), generator=g).float() / 4096.0)
    v64, x64 = v.cdouble().requires_grad_(True), x.cdouble().requires_grad_(True)
    out_c = O.vandermonde_oracle(v64, x64, L)
    gout = torch.randn(batch, L, generator=g)
    dv_c, dx_c = torch.autograd.grad(out_c, (v64, x64), gout.double())
    vg, xg = v.cuda().requires_grad_(True), x.cuda().requires_grad_(True)
    out_g = log_vandermonde_cuda(vg, xg, L)
    dv_g, dx_g = torch.autograd.grad(out_g, (vg, xg), gout.cuda())
    _close(out_g.detach().cpu(), out_c.detach(), 2e-4, "out")
    _close(dv_g.cpu(), dv_c, 3e-4, "dv")
    _close(dx_g.cpu(), dx_c, 3e-4, "dx")


def test_cauchy_determinism_and_errors():
    from lrnnx_b200 import structured_kernels as sk
    g = torch.Generator().manual_seed(1)
    c = lambda *s: torch.complex(torch.randn(*s, generator=g), torch.randn(*s, generator=g)).cuda()
    v, w, z, d = c(8, 32), c(8, 32), c(5000), c(8, 5000)
    a = sk.cauchy_mult_sym_bwd(v, z, w, d)
    b = sk.cauchy_mult_sym_bwd(v, z, w, d)
    assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1])     # fixed-order fold: bit-identical
    with pytest.raises(RuntimeError):
        sk.cauchy_mult_sym_fwd(v.cpu(), z, w)
    with pytest.raises(RuntimeError):
        sk.cauchy_mult_sym_fwd(v, z, w[:, :16])
