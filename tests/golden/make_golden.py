"""Generate the golden fixtures in this directory from the lrnnx reference.

Run where the lrnnx source tree is available:
    LRNNX_REF=/path/to/lrnnx python tests/golden/make_golden.py
It imports the reference's own pure-PyTorch functions on CPU (the three compiled
extension modules lrnnx imports at module top are replaced by empty stand-ins,
they are not needed by the *_ref functions), evaluates them on small seeded
inputs, back-propagates a seeded upstream gradient through them, and stores
inputs, outputs and gradients as ``<family>.pt`` (a dict of cases).  The
fixtures pin oracle/scan_oracle.py (tests/test_oracle_golden.py) and are the
reference side of the GPU parity tests (tests/test_gpu_*.py).
"""
from __future__ import annotations

import math
import os
import sys
import types
from pathlib import Path

import torch

REF = os.environ.get("LRNNX_REF")
if not REF:
    raise SystemExit("set LRNNX_REF to the root of the lrnnx source tree")
for name in ("selective_scan_cuda", "simplified_scan_cuda", "structured_kernels"):
    m = types.ModuleType(name)
    for attr in ("fwd", "bwd", "cauchy_mult_sym_fwd", "cauchy_mult_sym_bwd", "vand_log_mult_sym_fwd",
                 "vand_log_mult_sym_bwd"):
        setattr(m, attr, None)
    sys.modules[name] = m
sys.path.insert(0, REF)

from lrnnx.ops.selective_scan import selective_scan_ref  # noqa: E402
from lrnnx.ops.rglru_scan import rglru_scan_ref  # noqa: E402
from lrnnx.ops.s7_scan import s7_scan_ref  # noqa: E402
from lrnnx.ops.simplified_scan import simplified_scan_ref, s5_inner_ref  # noqa: E402
from lrnnx.ops.triton.selective_state_update import selective_state_update_ref  # noqa: E402
from lrnnx.ops.triton.simplified_state_update import simplified_state_update_ref  # noqa: E402
from lrnnx.ops.s4_utils import log_vandermonde_naive  # noqa: E402
from csrc.s4.cauchy import cauchy_mult_torch  # noqa: E402

OUT = Path(__file__).resolve().parent


def gen(seed):
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)
    return g


def randn(g, *shape, dtype=torch.float32):
    if dtype.is_complex:
        return torch.complex(torch.randn(*shape, generator=g), torch.randn(*shape, generator=g)).to(dtype)
    return torch.randn(*shape, generator=g, dtype=dtype)


def rand(g, *shape):
    return torch.rand(*shape, generator=g)


def run_with_grads(fn, tensors: dict, kwargs: dict, g, n_out=1):
    """Evaluate fn(**tensors, **kwargs); backprop a seeded gradient through the first output."""
    leaves = {k: (v.clone().requires_grad_(True) if v is not None and (v.is_floating_point() or v.is_complex())
                  else v) for k, v in tensors.items()}
    res = fn(**leaves, **kwargs)
    outs = res if isinstance(res, tuple) else (res,)
    gout = randn(g, *outs[0].shape, dtype=outs[0].dtype)
    wanted = [(k, v) for k, v in leaves.items() if v is not None and v.requires_grad]
    grads = torch.autograd.grad(outs[0], [v for _, v in wanted], gout, allow_unused=True)
    return {
        "inputs": {k: (None if v is None else v.detach().clone()) for k, v in tensors.items()},
        "kwargs": kwargs,
        "outputs": [o.detach().clone() for o in outs],
        "gout": gout,
        "grads": {k: (None if gr is None else gr.detach().clone()) for (k, _), gr in zip(wanted, grads)},
    }


def selective_cases():
    cases = {}
    batch, dim, N = 2, 4, 8
    for disc in ("mamba", "zoh", "bilinear", "dirac"):
        for var_B in (True, False):
            for var_C in (True, False):
                for L in (37, 300):
                    if L == 300 and not (var_B and var_C):
                        continue
                    g = gen(0)
                    A = -0.5 * rand(g, dim, N) - 0.05
                    t = dict(
                        u=randn(g, batch, dim, L), delta=0.5 * rand(g, batch, dim, L), A=A,
                        B=randn(g, batch, N, L) if var_B else randn(g, dim, N),
                        C=randn(g, batch, N, L) if var_C else randn(g, dim, N),
                        D=randn(g, dim), z=randn(g, batch, dim, L), delta_bias=0.5 * rand(g, dim))
                    kw = dict(delta_softplus=True, return_last_state=True, discretization=disc)
                    cases[f"{disc}_vB{int(var_B)}_vC{int(var_C)}_L{L}"] = run_with_grads(selective_scan_ref, t, kw, g)
    # grouped B/C, no z, no softplus
    g = gen(1)
    batch, dim, N, L, G = 2, 8, 4, 45, 2
    t = dict(u=randn(g, batch, dim, L), delta=0.5 * rand(g, batch, dim, L), A=-rand(g, dim, N) - 0.1,
             B=randn(g, batch, G, N, L), C=randn(g, batch, G, N, L), D=None, z=None, delta_bias=None)
    cases["mamba_groups2"] = run_with_grads(
        selective_scan_ref, t, dict(delta_softplus=False, return_last_state=True, discretization="mamba"), g)
    # deltaA ("event" mode), all four methods
    for disc in ("mamba", "zoh", "bilinear", "dirac"):
        g = gen(2)
        batch, dim, N, L = 2, 4, 8, 53
        t = dict(u=randn(g, batch, dim, L), delta=0.5 * rand(g, batch, dim, L), A=-rand(g, dim, N) - 0.1,
                 B=randn(g, batch, N, L), C=randn(g, batch, N, L), D=randn(g, dim), z=randn(g, batch, dim, L),
                 delta_bias=0.1 * randn(g, dim), deltaA=0.5 * rand(g, batch, dim, L))
        cases[f"{disc}_deltaA"] = run_with_grads(
            selective_scan_ref, t, dict(delta_softplus=True, return_last_state=True, discretization=disc), g)
    # complex A; constant and variable B/C (tests/ops/mamba/test_selective_scan.py:241-389 uses constant)
    for disc in ("mamba", "zoh", "bilinear", "dirac"):
        for var in (False, True):
            g = gen(42)
            batch, dim, N, L = 2, 4, 8, 41
            A = torch.complex(-0.5 * rand(g, dim, N) - 0.05, 2.0 * rand(g, dim, N)).to(torch.complex64)
            t = dict(u=randn(g, batch, dim, L), delta=0.3 * rand(g, batch, dim, L) + 0.01, A=A,
                     B=randn(g, batch, 1, N, 2 * L) if var else randn(g, dim, N, dtype=torch.complex64),
                     C=randn(g, batch, 1, N, 2 * L) if var else randn(g, dim, N, dtype=torch.complex64),
                     D=randn(g, dim), z=None, delta_bias=None)
            cases[f"complex_{disc}_var{int(var)}"] = run_with_grads(
                selective_scan_ref, t, dict(delta_softplus=False, return_last_state=True, discretization=disc), g)
    return cases


def rglru_s7_cases():
    cases = {}
    for N in (1, 3):
        g = gen(7)
        batch, dim, L = 2, 8, 61
        t = dict(u=randn(g, batch, dim, L), delta=8.0 * torch.sigmoid(randn(g, batch, dim, L)),
                 A=0.9 + 0.099 * rand(g, dim, N))
        cases[f"rglru_N{N}"] = run_with_grads(rglru_scan_ref, t, dict(return_last_state=True), g)
    for use_bias in (False, True):
        g = gen(8)
        batch, H, N, L = 2, 8, 16, 47
        t = dict(u=randn(g, batch, H, L), A=randn(g, batch, N, L), B=randn(g, batch, N, H, L) / math.sqrt(H),
                 C=randn(g, batch, H, N, L) / math.sqrt(N), bias=randn(g, batch, N, L) if use_bias else None)
        cases[f"s7_bias{int(use_bias)}"] = run_with_grads(s7_scan_ref, t, dict(return_last_state=True), g)
    return cases


def simplified_cases():
    cases = {}
    for disc in ("bilinear", "zoh", "dirac"):
        for use_dA in (False, True):
            g = gen(42)
            batch, H, P, L = 2, 8, 16, 67
            A = torch.complex(-0.5 * rand(g, P) - 0.05, math.pi * rand(g, P)).to(torch.complex64)
            t = dict(u=randn(g, batch, H, L, dtype=torch.complex64), delta=0.1 * rand(g, batch, P, L) + 0.01, A=A,
                     B=randn(g, P, H, dtype=torch.complex64) / math.sqrt(H),
                     C=randn(g, H, P, dtype=torch.complex64) / math.sqrt(P),
                     deltaA=(0.1 * rand(g, batch, P, L) + 0.01) if use_dA else None)
            cases[f"scan_{disc}_dA{int(use_dA)}"] = run_with_grads(
                simplified_scan_ref, t, dict(return_last_state=True, discretization=disc), g)
    for conj_sym in (True, False):
        g = gen(43)
        batch, H, P, L = 2, 8, 16, 33
        A = torch.complex(-0.5 * rand(g, P) - 0.05, math.pi * rand(g, P)).to(torch.complex64)
        t = dict(u=randn(g, batch, H, L, dtype=torch.complex64), delta=0.1 * rand(g, batch, P, L) + 0.01, A=A,
                 B=randn(g, P, H, dtype=torch.complex64) / math.sqrt(H),
                 C=randn(g, H, P, dtype=torch.complex64) / math.sqrt(P), D=randn(g, H))
        cases[f"inner_conj{int(conj_sym)}"] = run_with_grads(
            s5_inner_ref, t, dict(discretization="zoh", conj_sym=conj_sym), g)
    return cases


def state_update_cases():
    cases = {}
    for disc in ("mamba", "zoh", "bilinear", "dirac", "rglru", "s7"):
        for use_dA in (False, True):
            if use_dA and disc == "s7":
                continue   # the reference's Triton kernel and its _ref disagree there; not pinned
            g = gen(3)
            # the reference's _ref only broadcasts for "s7" when dstate == 1 (the S7 mixer's case)
            batch, dim, N = 3, 20, (1 if disc == "s7" else 8)
            A = (0.9 + 0.099 * rand(g, dim, N)) if disc == "rglru" else (-rand(g, dim, N) - 0.1)
            t = dict(state=randn(g, batch, dim, N), x=randn(g, batch, dim), dt=randn(g, batch, dim), A=A,
                     B=randn(g, batch, N), C=randn(g, batch, N), D=randn(g, dim), z=randn(g, batch, dim),
                     dt_bias=0.3 * randn(g, dim), deltaA=rand(g, batch, dim) if use_dA else None)
            state = t["state"].clone()
            out = selective_state_update_ref(state, *[t[k] for k in ("x", "dt", "A", "B", "C")], D=t["D"], z=t["z"],
                                             dt_bias=t["dt_bias"], dt_softplus=True, deltaA=t["deltaA"],
                                             discretization=disc)
            cases[f"{disc}_dA{int(use_dA)}"] = {"inputs": t, "kwargs": dict(dt_softplus=True, discretization=disc),
                                                "outputs": [out, state]}
    # heads + groups
    g = gen(4)
    batch, nheads, hd, N, ng = 2, 4, 16, 8, 2
    t = dict(state=randn(g, batch, nheads, hd, N), x=randn(g, batch, nheads, hd), dt=randn(g, batch, nheads, hd),
             A=-rand(g, nheads, hd, N) - 0.1, B=randn(g, batch, ng, N), C=randn(g, batch, ng, N),
             D=randn(g, nheads, hd), z=randn(g, batch, nheads, hd), dt_bias=0.3 * randn(g, nheads, hd), deltaA=None)
    state = t["state"].clone()
    out = selective_state_update_ref(state, *[t[k] for k in ("x", "dt", "A", "B", "C")], D=t["D"], z=t["z"],
                                     dt_bias=t["dt_bias"], dt_softplus=True, discretization="mamba")
    cases["heads_groups"] = {"inputs": t, "kwargs": dict(dt_softplus=True, discretization="mamba"),
                             "outputs": [out, state]}
    return cases


def s5_step_cases():
    cases = {}
    for disc in ("bilinear", "zoh", "dirac"):
        for use_dA, conj_sym, dt_1d in ((False, True, False), (True, False, False), (False, True, True)):
            g = gen(11)
            batch, P, H = 3, 24, 40
            A = torch.complex(-0.5 * rand(g, P) - 0.05, math.pi * rand(g, P)).to(torch.complex64)
            t = dict(state=randn(g, batch, P, dtype=torch.complex64), x=randn(g, batch, H),
                     dt=(0.1 * rand(g, P) + 0.01) if dt_1d else (0.1 * rand(g, batch, P) + 0.01), A=A,
                     B=randn(g, P, H, dtype=torch.complex64) / math.sqrt(H),
                     C=randn(g, H, P, dtype=torch.complex64) / math.sqrt(P), D=randn(g, H, H) / math.sqrt(H),
                     deltaA=(0.1 * rand(g, batch, P) + 0.01) if use_dA else None)
            state = t["state"].clone()
            out = simplified_state_update_ref(state, t["x"], t["dt"], t["A"], t["B"], t["C"], t["D"], t["deltaA"],
                                              discretization=disc, conj_sym=conj_sym)
            cases[f"{disc}_dA{int(use_dA)}_cs{int(conj_sym)}_1d{int(dt_1d)}"] = {
                "inputs": t, "kwargs": dict(discretization=disc, conj_sym=conj_sym), "outputs": [out, state]}
    return cases


def s4_cases():
    cases = {}
    for n_half, L in ((2, 3), (8, 17), (32, 129)):
        g = gen(2357)
        batch = 4
        v = randn(g, batch, n_half, dtype=torch.complex64)
        w = randn(g, batch, n_half, dtype=torch.complex64)
        z = torch.exp(1j * randn(g, L))
        vf = torch.cat([v, v.conj()], -1).cdouble().requires_grad_(True)
        wf = torch.cat([w, w.conj()], -1).cdouble().requires_grad_(True)
        out = cauchy_mult_torch(vf, z.cdouble(), wf, symmetric=True)
        gout = randn(g, *out.shape, dtype=torch.complex64)
        dv, dw = torch.autograd.grad(out, (vf, wf), gout.cdouble())
        # gradient w.r.t. the half spectrum = first half + conj(second half)
        # (tests/ops/s4/test_cauchy.py:42-44 grad_to_half_grad)
        half = lambda d: d[:, :n_half] + d[:, n_half:].conj()
        cases[f"cauchy_n{n_half}_L{L}"] = {"inputs": dict(v=v, z=z, w=w), "outputs": [out.detach().cfloat()],
                                           "gout": gout, "grads": dict(v=half(dv).cfloat(), w=half(dw).cfloat())}
        x = (0.001 * rand(g, batch, n_half) + 1j * rand(g, batch, n_half)).to(torch.complex64)
        vv = v.cdouble().requires_grad_(True)
        xx = x.cdouble().requires_grad_(True)
        outv = log_vandermonde_naive(vv, xx, L)
        goutv = randn(g, *outv.shape)
        dvv, dxx = torch.autograd.grad(outv, (vv, xx), goutv.double())
        cases[f"vand_n{n_half}_L{L}"] = {"inputs": dict(v=v, x=x, L=L), "outputs": [outv.detach().float()],
                                         "gout": goutv, "grads": dict(v=dvv.cfloat(), x=dxx.cfloat())}
    return cases


def mamba_lm_cases():
    """lrnnx's own LRNNLMHeadModel with Mamba mixers, run on CPU: the layer's selective_scan_fn and
    selective_state_update are rebound to the reference's *_ref functions (same signatures) and
    RMSNorm.forward to rms_norm_ref, fused_add_norm off (the Triton kernels need a GPU).  Stored:
    the weights, token ids, the logits of forward(), the gradients of the shifted cross-entropy
    loss for every parameter, and the logits of step() fed the same tokens one by one."""
    import torch.nn.functional as F
    import lrnnx.models.ltv.mamba as M
    import lrnnx.ops.triton.layer_norm as LN
    from lrnnx.architectures.language_model import LRNNLMHeadModel
    M.selective_scan_fn = selective_scan_ref
    M.selective_state_update = selective_state_update_ref
    LN.RMSNorm.forward = lambda self, x, residual=None, prenorm=False, residual_in_fp32=False: LN.rms_norm_ref(
        x, self.weight, None, residual=residual, eps=self.eps, prenorm=prenorm)
    cases = {}
    for name, (d_model, n_layer, vocab, batch, L) in {"small": (64, 2, 96, 2, 40), "wide": (128, 3, 160, 3, 24)}.items():
        torch.manual_seed(5)
        model = LRNNLMHeadModel(d_model=d_model, d_state=16, n_layer=n_layer, vocab_size=vocab,
                                mixer_types=["Mamba"] * n_layer, mixer_kwargs={"Mamba": {"discretization": "mamba"}},
                                rms_norm=True, fused_add_norm=False)
        # the zero-initialised biases and the unit norm weights are moved off their trivial values
        g = gen(11)
        with torch.no_grad():
            for k, prm in model.named_parameters():
                if k.endswith("norm.weight") or k.endswith("norm_f.weight"):
                    prm.add_(0.1 * randn(g, *prm.shape))
                if k.endswith("conv1d.bias"):
                    prm.add_(0.1 * randn(g, *prm.shape))
        ids = torch.randint(0, vocab, (batch, L), generator=g)
        logits = model(ids).logits
        loss = F.cross_entropy(logits[:, :-1].reshape(-1, vocab), ids[:, 1:].reshape(-1))
        names = [k for k, _ in model.named_parameters()]
        grads = torch.autograd.grad(loss, [prm for _, prm in model.named_parameters()], allow_unused=True)
        caches = model.allocate_inference_cache(batch, L)
        step_logits = []
        with torch.no_grad():
            for t in range(L):
                step_logits.append(model.step(ids[:, t:t + 1], caches).logits[:, 0])
        cases[name] = {
            "config": dict(d_model=d_model, n_layer=n_layer, vocab_size=vocab, d_state=16, d_conv=4, expand=2, eps=1e-5),
            "state_dict": {k: v.detach().clone() for k, v in model.state_dict().items() if "dtA_proj" not in k},
            "input_ids": ids, "logits": logits.detach().clone(), "loss": loss.detach().clone(),
            "grads": {k: (None if gr is None else gr.detach().clone()) for k, gr in zip(names, grads) if "dtA_proj" not in k},
            "step_logits": torch.stack(step_logits, dim=1),
        }
    return cases


def main():
    torch.set_num_threads(4)
    only = set(sys.argv[1:])
    for name, fn in (("selective_scan", selective_cases), ("rglru_s7", rglru_s7_cases),
                     ("simplified_scan", simplified_cases), ("state_update", state_update_cases),
                     ("s5_step", s5_step_cases), ("s4", s4_cases), ("mamba_lm", mamba_lm_cases)):
        if only and name not in only:
            continue
        cases = fn()
        path = OUT / f"{name}.pt"
        torch.save(cases, path)
        print(f"{path.name}: {len(cases)} cases, {path.stat().st_size / 1024:.0f} KiB")


if __name__ == "__main__":
    main()
