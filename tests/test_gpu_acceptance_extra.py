"""Acceptance cases beyond the reference's own sweeps: large state dimensions, non-contiguous
batch / channel strides, tensors larger than 2^31 bytes (64-bit offsets; the reference's uint32
strides would wrap, csrc/selective_scan/selective_scan.h:26), batch-sharded gradients against the
unsharded ones, the deltaA == delta identity of the S5 scan
(tests/ops/s5/test_simplified_scan_async.py:238-326) and the S5 decode step against the scan."""
from __future__ import annotations

import math

import pytest
import torch

from conftest import assert_close
from oracle import scan_oracle as O
from test_gpu_selective_scan import _make_inputs, _oracle_vs_gpu, _to_cuda

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("N", [128, 256])
def test_large_state_dimension(N):
    t, g = _make_inputs(2, 4, N, 300, seed=N, groups=1)
    _oracle_vs_gpu(t, g, "mamba", 1e-4, 2e-5, 3e-4, 1e-4)


@pytest.mark.parametrize("dtype,dim,N", [(torch.float32, 6, 8), (torch.bfloat16, 32, 16), (torch.float32, 32, 16)])
def test_noncontiguous_batch_and_channel_strides(dtype, dim, N):
    """u, delta, z and the upstream gradient are views into larger tensors (padded batch and
    channel strides, unit stride along time); results must equal those of packed copies.  The
    16-channel cases run on the throughput kernels, the other on the coverage kernels."""
    from lrnnx_b200.ops import selective_scan_fn
    batch, L = 2, 520
    t, g = _make_inputs(batch, dim, N, L, seed=7, dtype=dtype)
    gpu = _to_cuda(t)
    padded = {}
    for k in ("u", "delta", "z"):
        big = torch.zeros(batch + 1, dim + 16, L + 24, dtype=dtype, device="cuda")
        big[1:, 8 : 8 + dim, 8 : 8 + L] = gpu[k].detach()
        padded[k] = big[1:, 8 : 8 + dim, 8 : 8 + L].requires_grad_(True)
        assert not padded[k].is_contiguous() and padded[k].stride(-1) == 1
    kw = dict(delta_softplus=True, discretization="mamba")
    packed = selective_scan_fn(**gpu, **kw)
    other = {k: (padded[k] if k in padded else v) for k, v in gpu.items()}
    strided = selective_scan_fn(**other, **kw)
    tol = dict(rtol=0, atol=0) if dtype == torch.float32 else dict(rtol=1e-2, atol=1e-2)
    torch.testing.assert_close(strided, packed, **tol)
    gout = torch.randn(packed.shape, generator=g).to(dtype).cuda()
    names = ["u", "delta", "z", "A", "D"]
    g_packed = torch.autograd.grad(packed, [gpu[k] for k in names], gout)
    g_strided = torch.autograd.grad(strided, [other[k] for k in names], gout)
    for k, a, b in zip(names, g_strided, g_packed):
        assert_close(a.float().cpu(), b.float().cpu(), rtol=1e-3 if dtype == torch.float32 else 3e-2,
                     atol_scale=1e-4 if dtype == torch.float32 else 1e-2, name=f"d{k}")


def test_offsets_beyond_2g_bytes():
    """A bf16 activation tensor of 2.2 GB: the rows past the 2^31-byte mark must be addressed with
    64-bit offsets.  The last 16 channels (one thread block of the throughput kernel, all of them
    beyond the mark) are compared with the oracle run on those channels alone; forward and the
    per-channel gradients."""
    from lrnnx_b200 import selective_scan_cuda
    free, _ = torch.cuda.mem_get_info()
    if free < 40 * 2**30:
        pytest.skip("needs 40 GB of free device memory")
    L, N, dim = 4096, 16, 2**18 + 32           # dim * L * 2 bytes = 2.2e9 > 2^31
    gen = torch.Generator(device="cuda").manual_seed(3)
    rb = lambda *s: torch.randn(*s, generator=gen, device="cuda", dtype=torch.bfloat16)
    u, delta, z, dout = rb(1, dim, L), rb(1, dim, L), rb(1, dim, L), rb(1, dim, L)
    assert u.numel() * 2 > 2**31
    B, C = rb(1, 1, N, L), rb(1, 1, N, L)
    A = -torch.rand(dim, N, generator=gen, device="cuda") * 2 - 0.05
    D = torch.randn(dim, generator=gen, device="cuda")
    bias = torch.rand(dim, generator=gen, device="cuda") - 4.0
    out, x, out_z = selective_scan_cuda.fwd(u, delta, A, B, C, D, z, bias, None, True, "mamba")
    res = selective_scan_cuda.bwd(u, delta, A, B, C, D, z, bias, None, dout, x, out, None, True, False, "mamba")
    du, ddelta = res[0], res[1]
    sl = slice(dim - 16, dim)
    cpu = dict(u=u[:, sl].cpu(), delta=delta[:, sl].cpu(), A=A[sl].cpu(), B=B.cpu(), C=C.cpu(), D=D[sl].cpu(),
               z=z[:, sl].cpu(), delta_bias=bias[sl].cpu())
    leaves = {k: v.clone().requires_grad_(True) for k, v in cpu.items()}
    ref = O.selective_scan_oracle(**leaves, delta_softplus=True, discretization="mamba")
    assert_close(out_z[:, sl].float().cpu(), ref.detach().float(), rtol=3e-2, atol_scale=1e-2, name="out")
    gu, gd = torch.autograd.grad(ref, [leaves["u"], leaves["delta"]], dout[:, sl].cpu())
    assert_close(du[:, sl].float().cpu(), gu.float(), rtol=3e-2, atol_scale=1e-2, name="du")
    assert_close(ddelta[:, sl].float().cpu(), gd.float(), rtol=3e-2, atol_scale=1e-2, name="ddelta")


@pytest.mark.parametrize("dtype,dim", [(torch.float32, 6), (torch.bfloat16, 32)])
def test_batch_sharded_gradients_match_unsharded(dtype, dim):
    """Data parallel by batch shards: the parameter gradients of the shards add up to those of
    the whole batch, the per-sample gradients concatenate."""
    from lrnnx_b200.ops import selective_scan_fn
    t, g = _make_inputs(4, dim, 16, 300 if dim == 6 else 512, seed=11, dtype=dtype)
    kw = dict(delta_softplus=True, discretization="mamba")
    gout = torch.randn(t["u"].shape, generator=g).to(dtype).cuda()
    per_sample, params = ("u", "delta", "B", "C", "z"), ("A", "D", "delta_bias")

    def grads(rows):
        gpu = _to_cuda({k: (v[rows] if k in per_sample else v) for k, v in t.items()})
        out = selective_scan_fn(**gpu, **kw)
        names = per_sample + params
        return dict(zip(names, torch.autograd.grad(out, [gpu[k] for k in names], gout[rows])))

    whole, lo, hi = grads(slice(0, 4)), grads(slice(0, 2)), grads(slice(2, 4))
    f32 = dtype == torch.float32
    for k in params:
        assert_close((lo[k] + hi[k]).float().cpu(), whole[k].float().cpu(), rtol=1e-4 if f32 else 2e-2,
                     atol_scale=2e-5 if f32 else 1e-2, name=f"d{k}")
    for k in per_sample:   # dB / dC are sums over channels by atomics: equal up to summation order
        assert_close(torch.cat([lo[k], hi[k]]).float().cpu(), whole[k].float().cpu(), rtol=1e-5 if f32 else 2e-2,
                     atol_scale=1e-6 if f32 else 1e-2, name=f"d{k}")


@pytest.mark.parametrize("disc", ["bilinear", "zoh", "dirac"])
def test_s5_deltaA_equal_to_delta_is_the_identity(disc):
    from lrnnx_b200.ops import simplified_scan_fn
    g = torch.Generator().manual_seed(5)
    c = lambda *s: torch.complex(torch.randn(*s, generator=g), torch.randn(*s, generator=g))
    b, H, P, L = 2, 12, 7, 2600
    u, Bm, Cm = c(b, H, L).cuda(), (c(P, H) / math.sqrt(H)).cuda(), (c(H, P) / math.sqrt(P)).cuda()
    A = torch.complex(-0.5 * torch.rand(P, generator=g) - 0.02, math.pi * torch.rand(P, generator=g)).cuda()
    delta = (0.1 * torch.rand(b, P, L, generator=g) + 0.01).cuda()
    gout = c(b, H, L).cuda()
    d1 = delta.clone().requires_grad_(True)
    y1 = simplified_scan_fn(u, d1, A, Bm, Cm, discretization=disc)
    d2, dA2 = delta.clone().requires_grad_(True), delta.clone().requires_grad_(True)
    y2 = simplified_scan_fn(u, d2, A, Bm, Cm, deltaA=dA2, discretization=disc)
    assert_close(y2.detach().cpu(), y1.detach().cpu(), rtol=1e-5, atol_scale=1e-6, name="y")
    (g1,) = torch.autograd.grad(y1, [d1], gout)
    g2 = torch.autograd.grad(y2, [d2, dA2], gout, allow_unused=True)
    total = sum(x for x in g2 if x is not None)
    assert_close(total.cpu(), g1.cpu(), rtol=3e-4, atol_scale=1e-4, name="ddelta + ddeltaA")


@pytest.mark.parametrize("disc", ["bilinear", "zoh", "dirac"])
def test_s5_step_equals_scan(disc):
    """L calls of simplified_state_update from a zero state reproduce s5_inner_fn over the same
    tokens (tests/models/test_ltv/test_s5.py step-vs-forward check, reduced to the two ops)."""
    from lrnnx_b200.ops import s5_inner_fn, simplified_state_update
    g = torch.Generator().manual_seed(9)
    c = lambda *s: torch.complex(torch.randn(*s, generator=g), torch.randn(*s, generator=g))
    b, H, P, L = 3, 40, 24, 200
    x = torch.randn(b, H, L, generator=g).cuda()
    Bm, Cm = (c(P, H) / math.sqrt(H)).cuda(), (c(H, P) / math.sqrt(P)).cuda()
    A = torch.complex(-0.5 * torch.rand(P, generator=g) - 0.02, math.pi * torch.rand(P, generator=g)).cuda()
    delta = (0.1 * torch.rand(b, P, L, generator=g) + 0.01).cuda()
    y = s5_inner_fn(x.to(torch.complex64), delta, A, Bm, Cm, torch.zeros(H, device="cuda"), discretization=disc,
                    conj_sym=True)
    state = torch.zeros(b, P, dtype=torch.complex64, device="cuda")
    ys = [simplified_state_update(state, x[:, :, t].contiguous(), delta[:, :, t].contiguous(), A, Bm, Cm,
                                  discretization=disc, conj_sym=True) for t in range(L)]
    assert_close(torch.stack(ys, dim=-1).cpu(), y.cpu(), rtol=2e-4, atol_scale=2e-5, name="outputs")
