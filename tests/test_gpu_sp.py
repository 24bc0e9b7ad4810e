"""Sequence-parallel fix-up kernel on one GPU: the sequence is cut into R slices that are scanned
one after the other as R emulated ranks (zero-start forward, summary fold on the device,
b200_selscan_fixup), and the stitched output, gated output, checkpoints and last state must
equal the unsplit forward of the same library and the CPU oracle."""
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
