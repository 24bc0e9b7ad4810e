"""GPU parity of the simplified (S5) scan through the C ABI.

Reference side: golden fixtures from lrnnx's simplified_scan_ref / s5_inner_ref and the CPU
oracle on seeded CPU-generated inputs.  fp32/complex64 tolerance rtol 1e-4 (3e-4 for
gradients) with an absolute floor of 2e-5 (1e-4) times the reference tensor's largest
magnitude.
"""
from __future__ import annotations

import math

import pytest
import torch

from conftest import assert_close, load_golden
from oracle import scan_oracle as O

pytestmark = pytest.mark.gpu
RTOL, ATOL, GRTOL, GATOL = 1e-4, 2e-5, 3e-4, 1e-4

SIMP = load_golden("simplified_scan")


def _cuda_leaves(inputs):
    out = {}
    for k, v in inputs.items():
        if torch.is_tensor(v):
            v = v.cuda().requires_grad_(True)
        out[k] = v
    return out


@pytest.mark.parametrize("name", sorted(SIMP))
def test_simplified_golden(name):
    from lrnnx_b200.ops import s5_inner_fn, simplified_scan_fn
    case = SIMP[name]
    leaves = _cuda_leaves(case["inputs"])
    fn = simplified_scan_fn if name.startswith("scan_") else s5_inner_fn
    res = fn(**leaves, **case["kwargs"])
    res = res if isinstance(res, tuple) else (res,)
    for i, (got, want) in enumerate(zip(res, case["outputs"])):
        assert got.shape == want.shape and got.dtype == want.dtype
        assert_close(got.detach().cpu(), want, rtol=RTOL, atol_scale=ATOL, name=f"output{i}")
    names = [k for k, g in case["grads"].items() if g is not None]
    grads = torch.autograd.grad(res[0], [leaves[k] for k in names], case["gout"].cuda())
    for k, g in zip(names, grads):
        assert_close(g.cpu(), case["grads"][k], rtol=GRTOL, atol_scale=GATOL, name=f"d{k}")


def _kernel_inputs(batch, P, L, S, seed, with_dA):
    g = torch.Generator().manual_seed(seed)
    c = lambda *s: torch.complex(torch.randn(*s, generator=g), torch.randn(*s, generator=g))
    A = torch.complex(-0.5 * torch.rand(P, S, generator=g) - 0.02, math.pi * torch.rand(P, S, generator=g))
    return dict(u=c(batch, P, L), delta=0.1 * torch.rand(batch, P, L, generator=g) + 0.01, A=A,
                deltaA=(0.1 * torch.rand(batch, P, L, generator=g) + 0.01) if with_dA else None), g, c


@pytest.mark.parametrize("disc", ["bilinear", "zoh", "dirac"])
@pytest.mark.parametrize("L,with_dA", [(1, False), (7, True), (320, False), (321, True), (1000, False),
                                       (2048, False), (2050, True), (3072, True), (4096, False), (4097, False),
                                       (6403, False)])
def test_kernel_vs_oracle(disc, L, with_dA):
    """fwd/bwd of the raw kernel entry points (identity B/C, dstate 1) against the oracle; ragged
    lengths exercise the 320-step stage, the 2048-step chunk and the unaligned (plain-load) paths;
    lengths that are multiples of 32 take the swizzled tensor-copy path of the backward."""
    from lrnnx_b200 import simplified_scan_cuda
    batch, P, S = 2, 5, 1
    t, g, c = _kernel_inputs(batch, P, L, S, seed=L, with_dA=with_dA)
    one = torch.ones(P, S, dtype=torch.complex64)
    cpu = {k: (v.clone().requires_grad_(True) if torch.is_tensor(v) else v) for k, v in t.items()}
    out_c, x_c = O.simplified_kernel_oracle(cpu["u"], cpu["delta"], cpu["A"], one, one, cpu["deltaA"], disc,
                                            return_checkpoints=True)
    cu = {k: (v.cuda() if torch.is_tensor(v) else v) for k, v in t.items()}
    out_g, x_g = simplified_scan_cuda.fwd(cu["u"], cu["delta"], cu["A"], one.cuda(), one.cuda(), cu["deltaA"], disc)
    assert_close(out_g.cpu(), out_c.detach(), rtol=RTOL, atol_scale=ATOL, name="out")
    assert x_g.shape == x_c.shape
    assert_close(x_g.cpu()[..., 1::2], x_c.detach()[..., 1::2], rtol=RTOL, atol_scale=ATOL, name="x state")
    assert_close(x_g.cpu()[..., 0::2], x_c.detach()[..., 0::2], rtol=2e-3, atol_scale=1e-6, name="x product")
    gout = c(batch, P, L)
    names = [k for k in ("u", "delta", "A", "deltaA") if cpu[k] is not None]
    gc = torch.autograd.grad(out_c, [cpu[k] for k in names], gout, allow_unused=True)
    # both backward kernels: the one that recomputes the states from the checkpoints, and the one
    # that takes them from the forward output
    for out_arg in (None, out_g):
        res = simplified_scan_cuda.bwd(cu["u"], cu["delta"], cu["A"], one.cuda(), one.cuda(), cu["deltaA"],
                                       gout.cuda(), x_g, disc, out_=out_arg)
        got = dict(u=res[0], delta=res[1], A=res[2])
        if with_dA:
            got["deltaA"] = res[5]
        for k, want in zip(names, gc):
            if want is None:
                assert float(got[k].abs().max()) == 0.0
                continue
            assert_close(got[k].cpu(), want, rtol=GRTOL, atol_scale=GATOL, name=f"d{k}")


@pytest.mark.parametrize("disc", ["bilinear", "zoh", "dirac"])
@pytest.mark.parametrize("L,with_dA", [(700, False), (4097, True)])
def test_kernel_constant_step(disc, L, with_dA):
    """Rows whose step size does not change over time take the kernels' single-coefficient path;
    rows 0-2 are constant over the whole row, row 3 over its first half only, row 4 never.
    Also checks the need_dB_dC=False variant of the backward entry point."""
    from lrnnx_b200 import simplified_scan_cuda
    batch, P, S = 2, 5, 1
    t, g, c = _kernel_inputs(batch, P, L, S, seed=100 + L, with_dA=with_dA)
    for k in ("delta", "deltaA"):
        if t[k] is not None:
            t[k][:, :3, :] = t[k][:, :3, :1]
            t[k][:, 3, : L // 2] = t[k][:, 3, :1]
    one = torch.ones(P, S, dtype=torch.complex64)
    cpu = {k: (v.clone().requires_grad_(True) if torch.is_tensor(v) else v) for k, v in t.items()}
    out_c = O.simplified_kernel_oracle(cpu["u"], cpu["delta"], cpu["A"], one, one, cpu["deltaA"], disc)
    cu = {k: (v.cuda() if torch.is_tensor(v) else v) for k, v in t.items()}
    out_g, x_g = simplified_scan_cuda.fwd(cu["u"], cu["delta"], cu["A"], one.cuda(), one.cuda(), cu["deltaA"], disc)
    assert_close(out_g.cpu(), out_c.detach(), rtol=RTOL, atol_scale=ATOL, name="out")
    gout = c(batch, P, L)
    names = [k for k in ("u", "delta", "A", "deltaA") if cpu[k] is not None]
    gc = torch.autograd.grad(out_c, [cpu[k] for k in names], gout, allow_unused=True)
    for need, out_arg in ((True, None), (False, None), (True, out_g), (False, out_g)):
        res = simplified_scan_cuda.bwd(cu["u"], cu["delta"], cu["A"], one.cuda(), one.cuda(), cu["deltaA"],
                                       gout.cuda(), x_g, disc, need_dB_dC=need, out_=out_arg)
        assert (res[3] is None) == (not need) and (res[4] is None) == (not need)
        got = dict(u=res[0], delta=res[1], A=res[2])
        if with_dA:
            got["deltaA"] = res[5]
        for k, want in zip(names, gc):
            if want is None:
                assert float(got[k].abs().max()) == 0.0
                continue
            assert_close(got[k].cpu(), want, rtol=GRTOL, atol_scale=GATOL, name=f"d{k}")


def test_multi_state_kernel():
    """dstate > 1 with non-trivial B/C on the forward (out = sum_s h_s B_s C_s)."""
    from lrnnx_b200 import simplified_scan_cuda
    batch, P, L, S = 2, 3, 700, 4
    t, g, c = _kernel_inputs(batch, P, L, S, seed=9, with_dA=False)
    B, C = c(P, S), c(P, S)
    out_c = O.simplified_kernel_oracle(t["u"], t["delta"], t["A"], B, C, None, "zoh")
    out_g, _ = simplified_scan_cuda.fwd(t["u"].cuda(), t["delta"].cuda(), t["A"].cuda(), B.cuda(), C.cuda(), None, "zoh")
    assert_close(out_g.cpu(), out_c, rtol=RTOL, atol_scale=ATOL, name="out")
    # backward with identity B/C and several states
    one = torch.ones(P, S, dtype=torch.complex64)
    cpu = {k: v.clone().requires_grad_(True) for k, v in t.items() if v is not None}
    oc = O.simplified_kernel_oracle(cpu["u"], cpu["delta"], cpu["A"], one, one, None, "bilinear")
    gout = c(batch, P, L)
    gc = torch.autograd.grad(oc, [cpu["u"], cpu["delta"], cpu["A"]], gout)
    _, x = simplified_scan_cuda.fwd(t["u"].cuda(), t["delta"].cuda(), t["A"].cuda(), one.cuda(), one.cuda(), None,
                                    "bilinear")
    res = simplified_scan_cuda.bwd(t["u"].cuda(), t["delta"].cuda(), t["A"].cuda(), one.cuda(), one.cuda(), None,
                                   gout.cuda(), x, "bilinear")
    for name, got, want in zip(("du", "ddelta", "dA"), res[:3], gc):
        assert_close(got.cpu(), want, rtol=GRTOL, atol_scale=GATOL, name=name)


def test_config1_recurrence_shape_slice():
    """benchmark configuration 1 recurrence x_k = Lambda x_{k-1} + (B u)_k through simplified_scan_fn with
    A = log Lambda, delta = 1, "dirac"; a (2, 64, 4096) slice of the (8, 256/512, 4096) shape.

    |Lambda| reaches 0.999, i.e. a memory of ~1000 steps through which every rounding of the
    discrete A is amplified, so two correct fp32 evaluations differ by more than 1e-4.  The check
    is therefore made against the float64 oracle: the kernel's error must not exceed 3x the
    error of the fp32 oracle (the reference's own arithmetic) plus 1e-5 of the tensor scale,
    for the output and for every gradient; the fp32 outputs must also agree to rtol 1e-3."""
    from lrnnx_b200.ops import simplified_scan_fn
    g = torch.Generator().manual_seed(0)
    batch, P, H, L = 2, 64, 96, 4096
    lam = torch.polar(0.9 + 0.099 * torch.rand(P, generator=g), math.pi / 10 * torch.rand(P, generator=g))
    A = torch.log(lam)
    cn = lambda *s: torch.complex(torch.randn(*s, generator=g), torch.randn(*s, generator=g)) / math.sqrt(2)
    B, C = cn(P, H) / math.sqrt(H), cn(H, P) / math.sqrt(P)
    u = torch.randn(batch, L, H, generator=g).transpose(1, 2).to(torch.complex64)
    delta = torch.ones(batch, P, L)
    gout = cn(batch, H, L)

    def oracle(dtype):
        leaves = [t.clone().requires_grad_(True) for t in (u, delta, A, B, C)]
        y = O.simplified_scan_oracle(*leaves, discretization="dirac", compute_dtype=dtype)
        return y.detach(), torch.autograd.grad(y, leaves, gout)

    y32, g32 = oracle(torch.float32)
    cd = torch.complex128
    l64 = [t.clone().requires_grad_(True) for t in (u.to(cd), delta.double(), A.to(cd), B.to(cd), C.to(cd))]
    y64 = O.simplified_scan_oracle(*l64, discretization="dirac", compute_dtype=torch.float64)
    g64 = torch.autograd.grad(y64, l64, gout.to(cd))
    y64 = y64.detach()
    cl = [t.cuda().requires_grad_(True) for t in (u, delta, A, B, C)]
    y_g = simplified_scan_fn(*cl, discretization="dirac")
    scale = float(y64.abs().max())
    err_ref = float((y32.to(cd) - y64).abs().max())
    err_gpu = float((y_g.detach().cpu().to(cd) - y64).abs().max())
    assert err_gpu <= 3 * err_ref + 1e-5 * scale, (err_gpu, err_ref, scale)
    assert_close(y_g.detach().cpu(), y32, rtol=1e-3, atol_scale=2e-4, name="y")
    gg = torch.autograd.grad(y_g, cl, gout.cuda())
    # the gradients get the same float64-adjudicated rule as the output
    for name, a, b32, b64 in zip(("du", "ddelta", "dA", "dB", "dC"), gg, g32, g64):
        wide = torch.complex128 if b64.is_complex() else torch.float64
        gscale = float(b64.abs().max())
        e_ref = float((b32.to(wide) - b64).abs().max())
        e_gpu = float((a.cpu().to(wide) - b64).abs().max())
        assert e_gpu <= 3 * e_ref + 1e-5 * gscale, (name, e_gpu, e_ref, gscale)


def test_device_status_clean():
    from lrnnx_b200 import _lib
    assert _lib.lib().b200_device_status() == 0


@pytest.mark.parametrize("disc", ["bilinear", "zoh", "dirac"])
@pytest.mark.parametrize("with_dA", [False, True])
def test_single_state_backward_with_nontrivial_B_C(disc, with_dA):
    """dstate == 1 with random complex B and C.  The forward output is sum_s h B C; the backward
    kernel of lrnnx seeds the adjoint with dout conj(C) and treats B as 1 inside the recurrence
    (simplified_scan_backward.cuh:213,237), which the oracle's simplified_kernel_grads_oracle
    restates.  Both backward kernels here (recomputing the states from the checkpoints, and taking
    them from the forward output as h = out / (B C)) must give those gradients."""
    from lrnnx_b200 import simplified_scan_cuda
    batch, P, L, S = 2, 6, 2600, 1
    t, g, c = _kernel_inputs(batch, P, L, S, seed=77 + with_dA, with_dA=with_dA)
    B, C = c(P, S) + 0.5, c(P, S) - 0.5
    out_c = O.simplified_kernel_oracle(t["u"], t["delta"], t["A"], B, C, t["deltaA"], disc)
    gout = c(batch, P, L)
    want = O.simplified_kernel_grads_oracle(t["u"], t["delta"], t["A"], C, gout, t["deltaA"], disc)
    cu = {k: (v.cuda() if torch.is_tensor(v) else v) for k, v in t.items()}
    Bg, Cg = B.cuda(), C.cuda()
    out_g, x_g = simplified_scan_cuda.fwd(cu["u"], cu["delta"], cu["A"], Bg, Cg, cu["deltaA"], disc)
    assert_close(out_g.cpu(), out_c, rtol=RTOL, atol_scale=ATOL, name="out")
    names = ["du", "ddelta", "dA", "dB", "dC"] + (["ddeltaA"] if with_dA else [])
    results = []
    for out_arg in (None, out_g):
        res = simplified_scan_cuda.bwd(cu["u"], cu["delta"], cu["A"], Bg, Cg, cu["deltaA"], gout.cuda(), x_g, disc,
                                       out_=out_arg)
        results.append(res)
        for name, got, w in zip(names, res, want):
            if w is None:
                assert float(got.abs().max()) == 0.0, name
                continue
            assert_close(got.cpu(), w, rtol=GRTOL, atol_scale=GATOL,
                         name=f"{name} (out_={'given' if out_arg is not None else 'None'})")
    for name, a, b in zip(names, *results):
        assert_close(a.cpu(), b.cpu(), rtol=GRTOL, atol_scale=GATOL, name=f"{name}: the two backward kernels")
