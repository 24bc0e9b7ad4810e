"""Pins the CPU oracle (oracle/scan_oracle.py) against outputs and gradients recorded from the
lrnnx reference's own *_ref functions (tests/golden/*.pt, made by tests/golden/make_golden.py)."""
from __future__ import annotations

import pytest
import torch

from conftest import assert_close, load_golden
from oracle import scan_oracle as O

RTOL = 2e-5   # oracle and reference are both fp32 on CPU; differences are summation order only


def _leaves(inputs):
    return {k: (v.clone().requires_grad_(True) if torch.is_tensor(v) and (v.is_floating_point() or v.is_complex())
                else v) for k, v in inputs.items()}


def _check_grads(out, leaves, case, rtol=RTOL):
    names = [k for k, g in case["grads"].items() if g is not None]
    grads = torch.autograd.grad(out, [leaves[k] for k in names], case["gout"])
    for k, g in zip(names, grads):
        assert_close(g, case["grads"][k], rtol=rtol * 5, atol_scale=2e-5, name=f"d{k}")


SEL = load_golden("selective_scan")


@pytest.mark.parametrize("name", sorted(SEL))
def test_selective_scan_oracle(name):
    case = SEL[name]
    leaves = _leaves(case["inputs"])
    out, last = O.selective_scan_oracle(**leaves, **case["kwargs"])
    assert out.shape == case["outputs"][0].shape and out.dtype == case["outputs"][0].dtype
    assert_close(out, case["outputs"][0], rtol=RTOL, name="out")
    assert_close(last, case["outputs"][1], rtol=RTOL, name="last_state")
    _check_grads(out, leaves, case)


RS = load_golden("rglru_s7")


@pytest.mark.parametrize("name", sorted(RS))
def test_rglru_s7_oracle(name):
    case = RS[name]
    leaves = _leaves(case["inputs"])
    fn = O.rglru_scan_oracle if name.startswith("rglru") else O.s7_scan_oracle
    out, last = fn(**leaves, **case["kwargs"])
    assert_close(out, case["outputs"][0], rtol=RTOL, name="out")
    assert_close(last, case["outputs"][1], rtol=RTOL, name="last_state")
    _check_grads(out, leaves, case)


SIMP = load_golden("simplified_scan")


@pytest.mark.parametrize("name", sorted(SIMP))
def test_simplified_scan_oracle(name):
    case = SIMP[name]
    leaves = _leaves(case["inputs"])
    if name.startswith("scan_"):
        out, last = O.simplified_scan_oracle(**leaves, **case["kwargs"])
        assert_close(last, case["outputs"][1], rtol=RTOL, name="last_state")
    else:
        out = O.s5_inner_oracle(**leaves, **case["kwargs"])
    assert_close(out, case["outputs"][0], rtol=RTOL, name="out")
    _check_grads(out, leaves, case)


SSU = load_golden("state_update")


@pytest.mark.parametrize("name", sorted(SSU))
def test_state_update_oracle(name):
    case = SSU[name]
    t = {k: (v.clone() if torch.is_tensor(v) else v) for k, v in case["inputs"].items()}
    state = t.pop("state")
    out = O.selective_state_update_oracle(state, **t, **case["kwargs"])
    assert_close(out, case["outputs"][0], rtol=RTOL, name="out")
    assert_close(state, case["outputs"][1], rtol=RTOL, name="state")


S4 = load_golden("s4")


@pytest.mark.parametrize("name", sorted(S4))
def test_s4_oracle(name):
    case = S4[name]
    i = case["inputs"]
    if name.startswith("cauchy"):
        v = i["v"].cdouble().requires_grad_(True)
        w = i["w"].cdouble().requires_grad_(True)
        out = O.cauchy_oracle(v, i["z"], w)
        dv, dw = torch.autograd.grad(out, (v, w), case["gout"].cdouble())
        assert_close(out.cfloat(), case["outputs"][0], rtol=1e-5, name="out")
        assert_close(dv.cfloat(), case["grads"]["v"], rtol=1e-5, name="dv")
        assert_close(dw.cfloat(), case["grads"]["w"], rtol=1e-5, name="dw")
    else:
        v = i["v"].cdouble().requires_grad_(True)
        x = i["x"].cdouble().requires_grad_(True)
        out = O.vandermonde_oracle(v, x, i["L"])
        dv, dx = torch.autograd.grad(out, (v, x), case["gout"].double())
        assert_close(out.float(), case["outputs"][0], rtol=1e-5, name="out")
        assert_close(dv.cfloat(), case["grads"]["v"], rtol=1e-5, name="dv")
        assert_close(dx.cfloat(), case["grads"]["x"], rtol=1e-5, name="dx")


def test_checkpoint_layout():
    """x[..., 2n+1] of the last chunk is the final state (lrnnx/ops/selective_scan.py:87) and
    x[..., 2n] the running product of the discrete A."""
    g = torch.Generator().manual_seed(5)
    b, d, n, L = 1, 2, 3, 2050
    u, delta = torch.randn(b, d, L, generator=g), 0.1 * torch.rand(b, d, L, generator=g)
    A = -torch.rand(d, n, generator=g)
    B, C = torch.randn(b, n, L, generator=g), torch.randn(b, n, L, generator=g)
    out, last, x = O.selective_scan_oracle(u, delta, A, B, C, return_last_state=True, return_checkpoints=True)
    assert x.shape == (b, d, 2, 2 * n)
    torch.testing.assert_close(x[:, :, -1, 1::2], last)
    prod = torch.exp(delta.sum(-1)[..., None] * A)
    torch.testing.assert_close(x[:, :, -1, 0::2], prod, rtol=1e-4, atol=1e-30)


S5STEP = load_golden("s5_step")


@pytest.mark.parametrize("name", sorted(S5STEP))
def test_s5_step_oracle(name):
    case = S5STEP[name]
    t = {k: (v.clone() if torch.is_tensor(v) else v) for k, v in case["inputs"].items()}
    state = t.pop("state")
    out = O.simplified_state_update_oracle(state, **t, **case["kwargs"])
    assert_close(out, case["outputs"][0], rtol=RTOL, name="out")
    assert_close(state, case["outputs"][1], rtol=RTOL, name="state")
