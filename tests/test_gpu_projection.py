"""The tensor-core complex projection (tcgen05, 3xTF32) against a complex128 product.

Tolerance: the kernel must be float32-class: its error against the float64 product may not exceed
4x the error of the float32 einsum (cuBLAS cgemm) on the same operands plus 2e-6 of the output
scale; a plain TF32 product would miss this by two orders of magnitude."""
from __future__ import annotations

import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _cn(g, *shape):
    return torch.complex(torch.randn(*shape, generator=g), torch.randn(*shape, generator=g)) / math.sqrt(2)


@pytest.mark.parametrize("batch,M,K,N", [(1, 128, 32, 64), (2, 128, 64, 192), (3, 256, 512, 256), (2, 512, 256, 4096)])
@pytest.mark.parametrize("conj_transpose", [False, True])
def test_projection_matches_float64(batch, M, K, N, conj_transpose):
    from lrnnx_b200 import _lib
    from lrnnx_b200.ops import projection
    g = torch.Generator().manual_seed(M + K + N)
    W = (_cn(g, K, M) if conj_transpose else _cn(g, M, K)) / math.sqrt(K)
    x = _cn(g, batch, K, N)
    Wm = W.conj().transpose(0, 1) if conj_transpose else W
    ref = torch.einsum("mk,bkn->bmn", Wm.to(torch.complex128), x.to(torch.complex128))
    Wg, xg = W.cuda(), x.cuda()
    assert projection.supported(Wg.conj().transpose(0, 1) if conj_transpose else Wg, xg)
    out = projection.project(Wg, xg, conj_transpose)
    torch.cuda.synchronize()
    assert _lib.lib().b200_device_status() == 0
    f32 = torch.einsum("mk,bkn->bmn", Wg.conj().transpose(0, 1) if conj_transpose else Wg, xg)
    scale = float(ref.abs().max())
    err = float((out.cpu().to(torch.complex128) - ref).abs().max())
    err32 = float((f32.cpu().to(torch.complex128) - ref).abs().max())
    assert out.shape == ref.shape and out.dtype == torch.complex64
    assert err <= 4 * err32 + 2e-6 * scale, (err, err32, scale)


def test_unsupported_shapes_are_rejected_by_the_entry_point():
    from lrnnx_b200.ops import projection
    g = torch.Generator().manual_seed(0)
    W, x = _cn(g, 96, 32).cuda(), _cn(g, 1, 32, 64).cuda()
    assert not projection.supported(W, x)
    with pytest.raises(RuntimeError, match="multiple of"):
        projection.project(W, x)


def test_simplified_scan_uses_the_projection_kernel_and_matches_the_oracle():
    """simplified_scan_fn at a shape inside the projection kernel's tiling (P=128, H=128, L=2048):
    output and gradients against the float32 oracle with the float64-adjudicated rule."""
    from lrnnx_b200.ops import simplified_scan_fn
    from oracle import scan_oracle as O
    g = torch.Generator().manual_seed(3)
    batch, P, H, L = 2, 128, 128, 2048
    lam = torch.polar(0.9 + 0.09 * torch.rand(P, generator=g), math.pi / 10 * torch.rand(P, generator=g))
    t = [_cn(g, batch, H, L), 0.5 + torch.rand(batch, P, L, generator=g), torch.log(lam), _cn(g, P, H) / math.sqrt(H),
         _cn(g, H, P) / math.sqrt(P)]
    gout = _cn(g, batch, H, L)

    def oracle(dtype):
        cd = torch.complex64 if dtype == torch.float32 else torch.complex128
        lv = [(v.to(cd) if v.is_complex() else v.to(dtype)).clone().requires_grad_(True) for v in t]
        y = O.simplified_scan_oracle(*lv, discretization="zoh", compute_dtype=dtype)
        return y.detach(), torch.autograd.grad(y, lv, gout.to(cd))

    y32, g32 = oracle(torch.float32)
    y64, g64 = oracle(torch.float64)
    lv = [v.cuda().requires_grad_(True) for v in t]
    y = simplified_scan_fn(*lv, discretization="zoh")
    gg = torch.autograd.grad(y, lv, gout.cuda())
    for name, a, b32, b64 in zip(("y", "du", "ddelta", "dA", "dB", "dC"), (y.detach(),) + gg, (y32,) + g32, (y64,) + g64):
        wide = torch.complex128 if b64.is_complex() else torch.float64
        scale = float(b64.abs().max())
        e_ref = float((b32.to(wide) - b64).abs().max())
        e_gpu = float((a.cpu().to(wide) - b64).abs().max())
        assert e_gpu <= 4 * e_ref + 1e-5 * scale, (name, e_gpu, e_ref, scale)


@pytest.mark.parametrize("batch,M,N,L", [(1, 128, 128, 16), (2, 128, 256, 208), (3, 256, 128, 2048), (8, 512, 256, 4096)])
def test_weight_gradient_matches_float64(batch, M, N, L):
    """sum over batch and time of g u^H (the gradient of a projection weight) on the tensor cores."""
    from lrnnx_b200 import _lib
    from lrnnx_b200.ops import projection
    g = torch.Generator().manual_seed(M + N + L)
    G, U = _cn(g, batch, M, L), _cn(g, batch, N, L)
    Gg, Ug = G.cuda(), U.cuda()
    assert projection.grad_supported(Gg, Ug)
    out = projection.weight_grad(Gg, Ug)
    torch.cuda.synchronize()
    assert _lib.lib().b200_device_status() == 0
    f32 = torch.einsum("bml,bnl->mn", Gg, Ug.conj())
    if batch * M * N * L <= 3 * 256 * 128 * 2048:
        ref = torch.einsum("bml,bnl->mn", G.to(torch.complex128), U.to(torch.complex128).conj())
    else:       # the float64 product of the large case on the GPU
        ref = torch.einsum("bml,bnl->mn", Gg.to(torch.complex128), Ug.to(torch.complex128).conj()).cpu()
    scale = float(ref.abs().max())
    err = float((out.cpu().to(torch.complex128) - ref).abs().max())
    err32 = float((f32.cpu().to(torch.complex128) - ref).abs().max())
    assert out.shape == (M, N) and out.dtype == torch.complex64
    assert err <= 4 * err32 + 2e-6 * scale, (err, err32, scale)
