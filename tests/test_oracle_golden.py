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


# ----------------------------------------------------------------------------- Mamba LM (configs 2 and 4 harness)
LM = load_golden("mamba_lm")


@pytest.mark.parametrize("name", sorted(LM))
def test_mamba_lm_oracle_matches_reference_model(name):
    """The oracle's restatement of LRNNLMHeadModel (Mamba mixers, RMSNorm) against the logits,
    parameter gradients and step() logits recorded from lrnnx's own model."""
    import torch.nn.functional as F
    case = LM[name]
    cfg = case["config"]
    sd = {k: v.clone().requires_grad_(True) for k, v in case["state_dict"].items()}
    sd["lm_head.weight"] = sd["backbone.embedding.weight"]          # tied (language_model.py:573,604-613)
    ids = case["input_ids"]
    logits = O.mamba_lm_oracle(sd, ids, cfg["n_layer"], cfg["eps"])
    torch.testing.assert_close(logits, case["logits"], rtol=RTOL, atol=1e-5)
    loss = F.cross_entropy(logits[:, :-1].reshape(-1, cfg["vocab_size"]), ids[:, 1:].reshape(-1))
    torch.testing.assert_close(loss, case["loss"], rtol=RTOL, atol=1e-6)
    names = [k for k, g in case["grads"].items() if g is not None and k != "lm_head.weight"]
    grads = torch.autograd.grad(loss, [sd[k] for k in names])
    for k, g in zip(names, grads):
        want = case["grads"][k]
        torch.testing.assert_close(g, want, rtol=1e-4, atol=1e-6 + 1e-5 * float(want.abs().max()), msg=lambda m: f"{k}: {m}")
    # step by step from zero states, and prefill + continue
    sd = {k: v.detach() for k, v in sd.items()}
    batch, L = ids.shape
    d_inner = cfg["expand"] * cfg["d_model"]
    states = [(torch.zeros(batch, d_inner, cfg["d_conv"]), torch.zeros(batch, d_inner, cfg["d_state"]))
              for _ in range(cfg["n_layer"])]
    for t in range(L):
        lg = O.mamba_lm_step_oracle(sd, ids[:, t], states, cfg["n_layer"], cfg["eps"])
        torch.testing.assert_close(lg, case["step_logits"][:, t], rtol=1e-4, atol=1e-5)
    cut = L // 2
    lg, states = O.mamba_lm_prefill_oracle(sd, ids[:, :cut], cfg["n_layer"], cfg["eps"])
    torch.testing.assert_close(lg, case["logits"][:, cut - 1], rtol=1e-4, atol=1e-5)
    for t in range(cut, L):
        lg = O.mamba_lm_step_oracle(sd, ids[:, t], states, cfg["n_layer"], cfg["eps"])
        torch.testing.assert_close(lg, case["logits"][:, t], rtol=1e-4, atol=2e-5)
