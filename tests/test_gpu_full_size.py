"""Checks at the full benchmark sizes, where the CPU oracle is too slow, through properties that do
not depend on the size:
  * linearity of the scan in its input (the recurrence is linear in u for fixed delta, A),
  * time-shift consistency: scanning a suffix from a zero state after an all-zero prefix equals
    the suffix of the full scan of the zero-padded input,
  * sequence-split consistency: slices scanned separately and stitched by the summary fold +
    fix-up equal the unsplit scan (config 3 shape),
  * an oracle spot check on a few rows cut out of the full-size problem (rows are independent).
"""
from __future__ import annotations

import math

import pytest
import torch

from conftest import assert_close
from oracle import scan_oracle as O

pytestmark = pytest.mark.gpu


def _cfg1(device="cuda", batch=8, P=256, L=4096, seed=0):
    g = torch.Generator().manual_seed(seed)
    lam = torch.polar(0.9 + 0.099 * torch.rand(P, generator=g), math.pi / 10 * torch.rand(P, generator=g))
    A = torch.log(lam).unsqueeze(-1)
    c = lambda *s: torch.complex(torch.randn(*s, generator=g), torch.randn(*s, generator=g))
    return dict(u=c(batch, P, L).to(device), delta=torch.ones(batch, P, L, device=device), A=A.to(device),
                one=torch.ones(P, 1, dtype=torch.complex64, device=device))


def test_config1_full_size_linearity_and_rows():
    from lrnnx_b200 import simplified_scan_cuda as ext
    t = _cfg1()
    g = torch.Generator().manual_seed(1)
    v = torch.complex(torch.randn(t["u"].shape, generator=g), torch.randn(t["u"].shape, generator=g)).cuda()
    f = lambda u: ext.fwd(u, t["delta"], t["A"], t["one"], t["one"], None, "dirac")[0]
    y1, y2, y12 = f(t["u"]), f(v), f(2.0 * t["u"] - 0.5 * v)
    assert_close(y12, 2.0 * y1 - 0.5 * y2, rtol=1e-4, atol_scale=1e-5, name="linearity in u")
    # backward is linear in dout as well
    x = ext.fwd(t["u"], t["delta"], t["A"], t["one"], t["one"], None, "dirac")[1]
    b = lambda d: ext.bwd(t["u"], t["delta"], t["A"], t["one"], t["one"], None, d, x, "dirac")
    r1, r2, r12 = b(t["u"]), b(v), b(t["u"] + v)
    for name, a1, a2, a12 in zip(("du", "ddelta", "dA"), r1, r2, r12):
        assert_close(a12, a1 + a2, rtol=2e-4, atol_scale=2e-5, name=f"linearity of {name} in dout")
    # oracle on 3 rows of the full-size problem
    rows = [(0, 0), (3, 117), (7, 255)]
    for (bb, pp) in rows:
        yo = O.simplified_kernel_oracle(t["u"][bb:bb + 1, pp:pp + 1].cpu(), t["delta"][bb:bb + 1, pp:pp + 1].cpu(),
                                        t["A"][pp:pp + 1].cpu(), torch.ones(1, 1, dtype=torch.complex64),
                                        torch.ones(1, 1, dtype=torch.complex64), None, "dirac",
                                        compute_dtype=torch.float64)
        assert_close(y1[bb:bb + 1, pp:pp + 1].cpu(), yo, rtol=1e-3, atol_scale=2e-4, name=f"row {bb},{pp}")


def test_config1_full_size_backward_rows_vs_float64():
    """Rows of the full-size backward against float64 autograd through the oracle (rows are
    independent; dA[p] sums the batch, so all 8 rows of one state index are evaluated for it).
    Both backward kernels: recomputing from the checkpoints, and from the forward output."""
    from lrnnx_b200 import simplified_scan_cuda as ext
    t = _cfg1()
    g = torch.Generator().manual_seed(2)
    dout = torch.complex(torch.randn(t["u"].shape, generator=g), torch.randn(t["u"].shape, generator=g)).cuda()
    out, x = ext.fwd(t["u"], t["delta"], t["A"], t["one"], t["one"], None, "dirac")
    cd = torch.complex128
    one = torch.ones(1, 1, dtype=cd)

    def rows64(bs, pp):
        u = t["u"][bs, pp:pp + 1].cpu().to(cd).requires_grad_(True)
        d = t["delta"][bs, pp:pp + 1].cpu().double().requires_grad_(True)
        A = t["A"][pp:pp + 1].cpu().to(cd).requires_grad_(True)
        y = O.simplified_kernel_oracle(u, d, A, one, one, None, "dirac", compute_dtype=torch.float64)
        return torch.autograd.grad(y, [u, d, A], dout[bs, pp:pp + 1].cpu().to(cd))

    for out_arg in (None, out):
        du, ddelta, dA = ext.bwd(t["u"], t["delta"], t["A"], t["one"], t["one"], None, dout, x, "dirac", out_=out_arg)[:3]
        for bb, pp in [(0, 0), (3, 117), (7, 255)]:
            du64, dd64, _ = rows64(slice(bb, bb + 1), pp)
            assert_close(du[bb:bb + 1, pp:pp + 1].cpu(), du64.to(torch.complex64), rtol=1e-3, atol_scale=2e-4,
                         name=f"du row {bb},{pp}")
            assert_close(ddelta[bb:bb + 1, pp:pp + 1].cpu(), dd64.float(), rtol=1e-3, atol_scale=2e-4,
                         name=f"ddelta row {bb},{pp}")
        _, _, dA64 = rows64(slice(0, 8), 117)
        assert_close(dA[117:118].cpu(), dA64.to(torch.complex64), rtol=1e-3, atol_scale=2e-4, name="dA[117]")


def test_config1_full_size_time_shift():
    from lrnnx_b200 import simplified_scan_cuda as ext
    t = _cfg1(batch=2)
    shift = 2048 + 320
    u = t["u"].clone()
    u[..., :shift] = 0
    y_full = ext.fwd(u, t["delta"], t["A"], t["one"], t["one"], None, "dirac")[0]
    y_suffix = ext.fwd(u[..., shift:].contiguous(), t["delta"][..., shift:].contiguous(), t["A"], t["one"], t["one"],
                       None, "dirac")[0]
    assert float(y_full[..., :shift].abs().max()) == 0.0
    assert_close(y_suffix, y_full[..., shift:], rtol=1e-5, atol_scale=1e-6, name="suffix scan")


@pytest.mark.parametrize("R", [2, 8])
def test_config3_full_length_split_consistency(R):
    """B=1, L=131072, N=16, bf16 (D cut to 64 channels to keep the test short): R slices + fold +
    fix-up against the unsplit forward, and an oracle spot check of 2 channels over the first 4096 steps."""
    from lrnnx_b200 import selective_scan_cuda
    from lrnnx_b200.sp import apply_fixup, fold_prefix
    g = torch.Generator().manual_seed(0)
    b, d, n, L = 1, 64, 16, 131072
    dtv = torch.exp(torch.rand(d, generator=g) * (math.log(0.1) - math.log(1e-3)) + math.log(1e-3))
    t = dict(u=torch.randn(b, d, L, generator=g).bfloat16(), delta=torch.randn(b, d, L, generator=g).bfloat16(),
             A=-torch.arange(1, n + 1, dtype=torch.float32).repeat(d, 1), B=torch.randn(b, 1, n, L, generator=g).bfloat16(),
             C=torch.randn(b, 1, n, L, generator=g).bfloat16(), D=torch.ones(d),
             z=torch.randn(b, d, L, generator=g).bfloat16(), delta_bias=dtv + torch.log(-torch.expm1(-dtv)))
    cu = {k: v.cuda() for k, v in t.items()}
    call = lambda s: selective_scan_cuda.fwd(s["u"], s["delta"], s["A"], s["B"], s["C"], s["D"], s["z"],
                                             s["delta_bias"], None, True, "mamba")
    full = call(cu)
    outz, Ps, hs = [], [], []
    for r in range(R):
        lo, hi = r * L // R, (r + 1) * L // R
        sl = {k: (v[..., lo:hi].contiguous() if v.dim() >= 3 else v) for k, v in cu.items()}
        out, x, out_z = call(sl)
        Ps.append(x[:, :, -1, 0::2].clone())
        hs.append(x[:, :, -1, 1::2].clone())
        if r > 0:
            p_in, h_in = fold_prefix(torch.stack(Ps), torch.stack(hs), r)
            apply_fixup(sl["u"], sl["delta"], sl["A"], sl["B"], sl["C"], sl["D"], sl["z"], sl["delta_bias"], True, out,
                        x, out_z, p_in, h_in)
        outz.append(out_z)
    assert_close(torch.cat(outz, -1).float().cpu(), full[2].float().cpu(), rtol=3e-2, atol_scale=1e-2, name="stitched")
    sub = {k: (v[:, :2, :4096] if v.dim() == 3 else (v[..., :4096] if v.dim() == 4 else v[:2])) for k, v in t.items()}
    ref = O.selective_scan_oracle(**sub, delta_softplus=True)
    assert_close(full[2][:, :2, :4096].float().cpu(), ref.float(), rtol=3e-2, atol_scale=1e-2, name="oracle rows")
