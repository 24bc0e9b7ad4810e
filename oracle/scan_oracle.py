"""CPU oracle for the lrnnx scan hot path.  TEST INFRASTRUCTURE ONLY.

This module restates, in plain PyTorch on CPU tensors, the algorithms of the
reference implementation for the path this repository accelerates.  It exists
to CHECK the CUDA kernels (tests/, the smoke test, and the CPU-baseline leg of
bench.py); nothing in the product package imports it and it is never a
fallback.  Parity status: PINNED — every function here is compared, in
tests/test_oracle_golden.py, with outputs and gradients of the reference's own
functions (selective_scan_ref, rglru_scan_ref, s7_scan_ref, simplified_scan_ref,
s5_inner_ref, selective_state_update_ref, cauchy_mult_torch,
log_vandermonde_naive) recorded in tests/golden/ by tests/golden/make_golden.py.

Each function cites the lrnnx file and lines it follows.  The recurrences are
evaluated step by step with the discrete coefficients computed per timestep
(nothing of shape (batch, dim, L, dstate) is materialised), so long sequences
can be checked on channel slices.  All functions are differentiable by
autograd, which is how reference gradients are obtained (the reference's tests
do the same through its *_ref functions).
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

CHUNK = 2048  # checkpoint spacing of the kernels' x tensor (selective_scan_cpu.cpp:380)


def _expand_groups(M, dim):
    """(batch, G, N, L) -> (batch, dim, N, L) by repeating each group dim/G times."""
    if M.dim() == 3:
        M = M.unsqueeze(1)
    g = M.shape[1]
    return M.repeat_interleave(dim // g, dim=1)


def _discretize(method, A, delta_t, deltaA_t, compute_k=True):
    """Discrete transition a_t and input coefficient k_t for one timestep.

    A: (dim, N); delta_t, deltaA_t: (batch, dim).  Returns a, k of shape
    (batch, dim, N).  Formulas: lrnnx/ops/selective_scan.py:249-319 (mamba, zoh,
    bilinear, dirac), csrc/selective_scan/selective_scan.cuh:287-302 (s7, rglru;
    same as lrnnx/ops/s7_scan.py:216-217 and lrnnx/ops/rglru_scan.py:172-182).
    """
    d = delta_t.unsqueeze(-1)
    dA = deltaA_t.unsqueeze(-1)
    one = torch.ones((), dtype=A.dtype)
    if method == "mamba":
        return torch.exp(dA * A), d.to(A.dtype) * one
    if method == "dirac":
        return torch.exp(dA * A), torch.ones_like(dA * A)
    if method == "zoh":
        x = d * A
        k = (torch.expm1(x) if not A.is_complex() else torch.exp(x) - one) / A
        return torch.exp(dA * A), k
    if method == "bilinear":
        vA = 0.5 * dA * A
        return (one + vA) / (one - vA), d / (one - 0.5 * d * A)
    if method == "s7":
        a = 1.0 - 1.0 / (d * d + 0.5)
        return a.expand(*a.shape[:-1], A.shape[-1]), torch.ones_like(d * A)
    if method == "rglru":
        a = torch.exp(d * torch.log(A))
        return a, torch.sqrt(1.0 - a * a)
    raise ValueError(f"Unknown discretization method: {method}")


def selective_scan_oracle(u, delta, A, B, C, D=None, z=None, delta_bias=None, deltaA=None, delta_softplus=False,
                          return_last_state=False, discretization="mamba", compute_dtype=torch.float32,
                          return_checkpoints=False):
    """Restatement of selective_scan_ref (lrnnx/ops/selective_scan.py:200-360) extended
    with the "s7" and "rglru" methods of the CUDA kernel.

    u, delta, z, deltaA: (batch, dim, L); A: (dim, N) real or complex; B, C:
    (dim, N), (batch, N, L) or (batch, G, N, L) (last dim 2L interleaved re/im
    when A is complex); D, delta_bias: (dim,).  ``compute_dtype`` float64 gives a
    high-precision variant of the same arithmetic.  With ``return_checkpoints``
    the kernels' x tensor (batch, dim, ceil(L/2048), 2N) is returned as a third
    value: x[..., 2n] = running product of a, x[..., 2n+1] = state (without the
    constant B factor, csrc/selective_scan/selective_scan.cuh:216-220,331-334).
    """
    dtype_in = u.dtype
    rdt = compute_dtype
    cdt = torch.complex64 if rdt == torch.float32 else torch.complex128
    is_cplx = A.is_complex()
    wdt = cdt if is_cplx else rdt
    uf = u.to(rdt)
    dl = delta.to(rdt)
    if delta_bias is not None:
        dl = dl + delta_bias.to(rdt)[:, None]
    if delta_softplus:
        dl = F.softplus(dl)
    dlA = deltaA.to(rdt) if deltaA is not None else dl
    batch, dim, L = u.shape
    N = A.shape[1]
    Aw = A.to(wdt)
    var_B, var_C = B.dim() >= 3, C.dim() >= 3

    def prep(M, var):
        if not var:
            return M.to(wdt)
        M = M.to(rdt)
        if is_cplx:
            M = torch.view_as_complex(M.reshape(*M.shape[:-1], L, 2).contiguous())
        return _expand_groups(M, dim)   # (batch, dim, N, L)

    Bw, Cw = prep(B, var_B), prep(C, var_C)
    ignore_B = discretization == "rglru"

    h = torch.zeros(batch, dim, N, dtype=wdt)          # state without a constant B
    prod = torch.ones(batch, dim, N, dtype=wdt)
    ys, ckpt = [], []
    # per-timestep views taken once (unbind has a single stacked backward; indexing inside the
    # loop would materialise a full-size zero tensor per step under autograd)
    dl_t, dlA_t, u_t = dl.unbind(-1), dlA.unbind(-1), uf.unbind(-1)
    B_t = Bw.unbind(-1) if var_B else None
    C_t = Cw.unbind(-1) if var_C else None
    for t in range(L):
        a, k = _discretize(discretization, Aw, dl_t[t], dlA_t[t])
        beta = k * u_t[t].unsqueeze(-1)
        if var_B and not ignore_B:
            beta = beta * B_t[t]
        h = a * h + beta
        if return_checkpoints:
            prod = prod * a
        cfac = C_t[t] if var_C else Cw
        if not var_B:
            cfac = cfac * Bw
        y = (h * cfac).sum(-1)
        ys.append(2 * y.real if is_cplx else y)
        if return_checkpoints and ((t + 1) % CHUNK == 0 or t == L - 1):
            ckpt.append(torch.stack([prod, h], dim=-1).reshape(batch, dim, 2 * N))
    y = torch.stack(ys, dim=2)
    out = y if D is None else y + uf * D.to(rdt)[:, None]
    if z is not None:
        out = out * F.silu(z.to(rdt))
    out = out.to(dtype_in)
    last_state = h if var_B else h * Bw    # the reference's state includes B (selective_scan.py:88-92,346)
    res = (out,)
    if return_last_state:
        res += (last_state,)
    if return_checkpoints:
        res += (torch.stack(ckpt, dim=2),)
    return res[0] if len(res) == 1 else res


def rglru_scan_oracle(u, delta, A, return_last_state=False, compute_dtype=torch.float32):
    """rglru_scan_ref (lrnnx/ops/rglru_scan.py:147-203): a = A^delta, b = sqrt(1-a^2) u, y = sum_n h."""
    ones = torch.ones_like(A)
    return selective_scan_oracle(u, delta, A, ones, ones, discretization="rglru",
                                 return_last_state=return_last_state, compute_dtype=compute_dtype)


def s7_scan_oracle(u, A, B, C, bias=None, return_last_state=False, compute_dtype=torch.float32):
    """s7_scan_ref (lrnnx/ops/s7_scan.py:183-233).  u (b, h, L); A (b, n, L); B (b, n, h, L);
    C (b, h, n, L); bias (b, n, L).  The scan runs over the n "channels" with one state each."""
    rdt = compute_dtype
    Bu = torch.einsum("bnhl,bhl->bnl", B.to(rdt), u.to(rdt))
    if bias is not None:
        Bu = Bu + bias.to(rdt)
    n = A.shape[1]
    one = torch.ones(n, 1, dtype=rdt)
    xs = selective_scan_oracle(Bu, A.to(rdt), torch.zeros(n, 1, dtype=rdt), one, one, discretization="s7",
                               compute_dtype=rdt)
    y = torch.einsum("bhnl,bnl->bhl", C.to(rdt), xs).to(u.dtype)
    return (y, xs[:, :, -1]) if return_last_state else y


def simplified_kernel_oracle(u, delta, A, B, C, deltaA=None, discretization="bilinear", compute_dtype=torch.float32,
                             return_checkpoints=False):
    """The simplified-scan KERNEL (csrc/simplified_scan/simplified_scan.cuh:85-262): complex u
    (batch, P, L), real delta, complex A/B/C (P, S).  h = a h + k u (B is not part of the
    recurrence), out = sum_s h * (B*C)."""
    cdt = torch.complex64 if compute_dtype == torch.float32 else torch.complex128
    uc, dl = u.to(cdt), delta.to(compute_dtype)
    dlA = deltaA.to(compute_dtype) if deltaA is not None else dl
    Aw, BC = A.to(cdt), (B * C).to(cdt)
    batch, P, L = u.shape
    S = A.shape[1]
    h = torch.zeros(batch, P, S, dtype=cdt)
    prod = torch.ones(batch, P, S, dtype=cdt)
    outs, ckpt = [], []
    for t in range(L):
        a, k = _discretize(discretization, Aw, dl[:, :, t], dlA[:, :, t])
        h = a * h + k * uc[:, :, t].unsqueeze(-1)
        outs.append((h * BC).sum(-1))
        if return_checkpoints:
            prod = prod * a
            if (t + 1) % CHUNK == 0 or t == L - 1:
                ckpt.append(torch.stack([prod, h], dim=-1).reshape(batch, P, 2 * S))
    out = torch.stack(outs, dim=2).to(u.dtype)
    return (out, torch.stack(ckpt, dim=2)) if return_checkpoints else out


def simplified_kernel_grads_oracle(u, delta, A, C, dout, deltaA=None, discretization="bilinear",
                                  compute_dtype=torch.float32):
    """Gradients as the simplified-scan backward KERNEL of lrnnx defines them
    (csrc/simplified_scan/simplified_scan_backward.cuh:213,237,296,315,380): the adjoint is seeded
    with dout * conj(C) and B enters the recurrence as the constant 1 ("B_term = one"), i.e. the
    gradients of  out' = sum_s C_s h_s,  h = a h + k * Bp * u  at Bp = 1, with dB := d out'/d Bp.
    For B = 1 (the only way lrnnx calls the kernel) this is the gradient of the forward output;
    for other B the forward multiplies the output by B as well and the two differ.
    Returns (du, ddelta, dA, dB, dC, ddeltaA or None)."""
    cdt = torch.complex64 if compute_dtype == torch.float32 else torch.complex128
    leaves = [u.detach().to(cdt).requires_grad_(True), delta.detach().to(compute_dtype).requires_grad_(True),
              A.detach().to(cdt).requires_grad_(True), torch.ones_like(A, dtype=cdt).requires_grad_(True),
              C.detach().to(cdt).requires_grad_(True)]
    if deltaA is not None:
        leaves.append(deltaA.detach().to(compute_dtype).requires_grad_(True))
    uc, dl, Aw, Bp, Cw = leaves[:5]
    dlA = leaves[5] if deltaA is not None else dl
    batch, P, L = u.shape
    h = torch.zeros(batch, P, A.shape[1], dtype=cdt)
    outs = []
    dl_t, dlA_t, u_t = dl.unbind(-1), dlA.unbind(-1), uc.unbind(-1)
    for t in range(L):
        a, k = _discretize(discretization, Aw, dl_t[t], dlA_t[t])
        h = a * h + k * Bp * u_t[t].unsqueeze(-1)
        outs.append((h * Cw).sum(-1))
    out = torch.stack(outs, dim=2)
    grads = torch.autograd.grad(out, leaves, dout.to(cdt), allow_unused=True)
    return tuple(grads) + ((None,) if deltaA is None else ())


def simplified_scan_oracle(u, delta, A, B, C, deltaA=None, return_last_state=False, discretization="bilinear",
                           compute_dtype=torch.float32):
    """simplified_scan_ref (lrnnx/ops/simplified_scan.py:233-340): u (batch, H, L) complex,
    delta (batch, P, L) real, A (P,) complex, B (P, H), C (H, P).  Bu = B u; x_t = a_t x_{t-1} + k_t Bu_t;
    y = C x."""
    cdt = torch.complex64 if compute_dtype == torch.float32 else torch.complex128
    A2 = (A if A.dim() == 2 else A.unsqueeze(-1)).to(cdt)
    Bu = torch.einsum("ph,bhl->bpl", B.to(cdt), u.to(cdt))
    one = torch.ones_like(A2)
    xs = simplified_kernel_oracle(Bu, delta, A2, one, one, deltaA, discretization, compute_dtype)
    y = torch.einsum("hp,bpl->bhl", C.to(cdt), xs).to(u.dtype)
    return (y, xs[:, :, -1]) if return_last_state else y


def s5_inner_oracle(u, delta, A, B, C, D, deltaA=None, discretization="bilinear", conj_sym=True,
                    compute_dtype=torch.float32):
    """s5_inner_ref (lrnnx/ops/simplified_scan.py:586-640): (2 if conj_sym else 1) * Re(y) + D * Re(u)."""
    y = simplified_scan_oracle(u, delta, A, B, C, deltaA, False, discretization, compute_dtype)
    yr = 2 * y.real if conj_sym else y.real
    ur = u.real if u.is_complex() else u
    return yr + D[None, :, None] * ur


def selective_state_update_oracle(state, x, dt, A, B, C, D=None, z=None, dt_bias=None, dt_softplus=False,
                                  deltaA=None, discretization="mamba"):
    """selective_state_update_ref (lrnnx/ops/triton/selective_state_update.py:479-599).
    Updates ``state`` in place and returns out.  Accepts the 3-D and the 4-D (heads) forms."""
    has_heads = state.dim() > 3
    if state.dim() == 3:
        state = state.unsqueeze(1)
    lift = lambda t: t if t is None or t.dim() == 3 else t.unsqueeze(1)    # (batch, dim) -> (batch, 1, dim)
    x, dt = lift(x), lift(dt)
    A = A if A.dim() == 3 else A.unsqueeze(0)
    B = B if B.dim() == 3 else B.unsqueeze(1)
    C = C if C.dim() == 3 else C.unsqueeze(1)
    D = D if D is None or D.dim() == 2 else D.unsqueeze(0)
    z = lift(z)
    dt_bias = dt_bias if dt_bias is None or dt_bias.dim() == 2 else dt_bias.unsqueeze(0)
    deltaA = lift(deltaA)
    batch, nheads, dim, dstate = state.shape
    ngroups = B.shape[1]
    dtv = dt + dt_bias if dt_bias is not None else dt
    dtv = F.softplus(dtv) if dt_softplus else dtv
    method = discretization.lower()
    d1 = dtv.unsqueeze(-1)
    dA1 = deltaA.unsqueeze(-1) if deltaA is not None else d1
    if method == "rglru":
        a = A ** dA1
    elif method == "s7":
        a = 1.0 - 1.0 / (d1 * d1 + 0.5)
    else:
        a = torch.exp(dA1 * A)      # also for "bilinear" (selective_state_update.py:555-562)
    Bh = B.repeat_interleave(nheads // ngroups, dim=1).unsqueeze(2)    # (batch, nheads, 1, dstate)
    Ch = C.repeat_interleave(nheads // ngroups, dim=1)
    if method == "zoh":
        bbar = Bh * (torch.exp(d1 * A) - 1.0) / A
    elif method == "bilinear":
        bbar = Bh * (1.0 / (1.0 - 0.5 * d1 * A)) * d1
    elif method in ("dirac", "s7"):
        bbar = Bh.expand_as(a * Bh)
    elif method == "rglru":
        bbar = Bh * torch.sqrt(1.0 - a * a)
    else:
        bbar = d1 * Bh
    state.copy_(state * a + bbar * x.unsqueeze(-1))
    out = torch.einsum("bhdn,bhn->bhd", state.to(Ch.dtype), Ch)
    if D is not None:
        out = out + (x * D).to(out.dtype)
    out = (out if z is None else out * F.silu(z)).to(x.dtype)
    return out if has_heads else out.squeeze(1)


def simplified_state_update_oracle(state, x, dt, A, B, C, D=None, deltaA=None, discretization="bilinear",
                                   conj_sym=True):
    """simplified_state_update_ref (lrnnx/ops/triton/simplified_state_update.py:404-469): one S5 step.
    state (batch, P) complex, updated in place; x (batch, H) real; dt, deltaA (batch, P) or (P,);
    A (P,), B (P, H), C (H, P) complex; D (H, H) real.  Returns y (batch, H) real."""
    batch, P = state.shape
    dtb = dt if dt.dim() == 2 else dt.unsqueeze(0).expand(batch, -1)
    dA = dtb if deltaA is None else (deltaA if deltaA.dim() == 2 else deltaA.unsqueeze(0).expand(batch, -1))
    a, k = _discretize(discretization.lower(), A.unsqueeze(-1), dtb, dA)      # (batch, P, 1)
    Bu = torch.einsum("ph,bh->bp", B, x.to(B.dtype))
    state.copy_(a.squeeze(-1) * state + k.squeeze(-1) * Bu)
    y = torch.einsum("hp,bp->bh", C, state).real
    if conj_sym:
        y = 2.0 * y
    if D is not None:
        y = y + x @ D.T
    return y


def cauchy_oracle(v, z, w, compute_dtype=torch.complex128):
    """cauchy_mult_torch(..., symmetric=True) restricted to the half spectrum
    (csrc/s4/cauchy.py:26-49; kernel csrc/s4/cauchy_cuda.cu:68-79): v, w (batch, n) hold one
    member of each conjugate pair; out[b,l] = sum_n v/(z_l-w) + conj(v)/(z_l-conj(w))."""
    vv, ww, zz = v.to(compute_dtype).unsqueeze(1), w.to(compute_dtype).unsqueeze(1), z.to(compute_dtype)[:, None]
    return (vv / (zz - ww) + vv.conj() / (zz - ww.conj())).sum(-1)


def vandermonde_oracle(v, x, L, compute_dtype=torch.complex128):
    """log_vandermonde_naive (lrnnx/ops/s4_utils.py:131-141; kernel csrc/s4/cauchy_cuda.cu:211-260):
    out[b,l] = 2 Re sum_n v_n exp(x_n l)."""
    vv, xx = v.to(compute_dtype), x.to(compute_dtype)
    ar = torch.arange(L, dtype=xx.real.dtype)
    return 2 * torch.einsum("bn,bnl->bl", vv, torch.exp(xx.unsqueeze(-1) * ar)).real


# ----------------------------------------------------------------------------- Mamba block and LM
def causal_conv1d_oracle(x, weight, bias=None, activation=None):
    """The depthwise causal convolution of lrnnx's Mamba without the causal_conv1d package
    (lrnnx/models/ltv/mamba.py:270-279): nn.Conv1d(groups=dim, padding=width-1) cut to the input
    length, then SiLU.  x (batch, dim, L); weight (dim, width); bias (dim,)."""
    L = x.shape[-1]
    y = F.conv1d(x, weight.unsqueeze(1), bias, padding=weight.shape[-1] - 1, groups=weight.shape[0])[..., :L]
    return F.silu(y) if activation in ("silu", "swish") else y


def causal_conv1d_update_oracle(x, conv_state, weight, bias=None, activation=None):
    """The convolution step of Mamba.step (lrnnx/models/ltv/mamba.py:394-409): roll the state,
    append x, dot with the weights.  x (batch, dim); conv_state (batch, dim, width), in place."""
    conv_state.copy_(torch.roll(conv_state, shifts=-1, dims=-1))
    conv_state[:, :, -1] = x
    y = torch.sum(conv_state * weight, dim=-1)
    if bias is not None:
        y = y + bias
    return (F.silu(y) if activation in ("silu", "swish") else y).to(x.dtype)


def rms_norm_oracle(x, weight, residual=None, eps=1e-6, prenorm=False):
    """rms_norm_ref without bias, dropout and rowscale (lrnnx/ops/triton/layer_norm.py:84-134)."""
    dtype = x.dtype
    if residual is not None:
        x = (x + residual).to(x.dtype)
    rstd = 1 / torch.sqrt(x.square().mean(dim=-1, keepdim=True) + eps)
    out = (x * rstd * weight).to(dtype)
    return (out, x) if prenorm else out


def mamba_mixer_oracle(p, hidden, return_states=False):
    """Mamba.forward in its plain mode (lrnnx/models/ltv/mamba.py:227-353): in_proj, causal
    conv + SiLU, x_proj -> (dt, B, C), dt_proj, selective scan with D skip, z gate, dt bias and
    softplus, out_proj.  ``p`` maps the parameter names of lrnnx's Mamba ("in_proj.weight",
    "conv1d.weight" (dim, 1, width), "conv1d.bias", "x_proj.weight", "dt_proj.weight",
    "dt_proj.bias", "A_log", "D", "out_proj.weight") to tensors.  hidden (batch, L, d_model).
    With ``return_states`` also returns (conv_state, ssm_state) as the layer caches them."""
    batch, L, _ = hidden.shape
    d_inner, dt_rank = p["dt_proj.weight"].shape
    N = p["A_log"].shape[1]
    width = p["conv1d.weight"].shape[-1]
    xz = (hidden @ p["in_proj.weight"].t()).transpose(1, 2)          # (batch, 2 d_inner, L)
    x, z = xz.chunk(2, dim=1)
    conv_state = F.pad(x, (width - L, 0))
    x = causal_conv1d_oracle(x, p["conv1d.weight"].squeeze(1), p["conv1d.bias"], "silu")
    x_dbl = x.transpose(1, 2) @ p["x_proj.weight"].t()               # (batch, L, dt_rank + 2N)
    dt = (x_dbl[..., :dt_rank] @ p["dt_proj.weight"].t()).transpose(1, 2)
    Bm = x_dbl[..., dt_rank:dt_rank + N].transpose(1, 2).contiguous()
    Cm = x_dbl[..., dt_rank + N:].transpose(1, 2).contiguous()
    A = -torch.exp(p["A_log"].float())
    y, last = selective_scan_oracle(x, dt, A, Bm, Cm, p["D"].float(), z=z, delta_bias=p["dt_proj.bias"].float(),
                                    delta_softplus=True, return_last_state=True, discretization="mamba")
    out = y.transpose(1, 2) @ p["out_proj.weight"].t()
    return (out, conv_state, last) if return_states else out


def mamba_mixer_step_oracle(p, hidden, conv_state, ssm_state):
    """Mamba.step (lrnnx/models/ltv/mamba.py:355-487): hidden (batch, d_model); both states are
    updated in place."""
    d_inner, dt_rank = p["dt_proj.weight"].shape
    N = p["A_log"].shape[1]
    xz = hidden @ p["in_proj.weight"].t()
    x, z = xz.chunk(2, dim=-1)
    x = causal_conv1d_update_oracle(x, conv_state, p["conv1d.weight"].squeeze(1), p["conv1d.bias"], "silu")
    x_db = x @ p["x_proj.weight"].t()
    dt = x_db[:, :dt_rank] @ p["dt_proj.weight"].t()
    A = -torch.exp(p["A_log"].float())
    y = selective_state_update_oracle(ssm_state, x, dt, A, x_db[:, dt_rank:dt_rank + N], x_db[:, dt_rank + N:],
                                      p["D"], z=z, dt_bias=p["dt_proj.bias"], dt_softplus=True)
    return y @ p["out_proj.weight"].t()


def _layer_params(sd, i):
    pre = f"backbone.layers.{i}.mixer."
    return {k[len(pre):]: v for k, v in sd.items() if k.startswith(pre)}


def mamba_lm_oracle(sd, input_ids, n_layer, eps=1e-5):
    """LRNNLMHeadModel.forward with Mamba mixers and RMSNorm, residuals in the activation dtype
    (lrnnx/architectures/language_model.py:453-511,683-727; lrnnx/layers/block.py:60-103):
    embedding, per layer residual add -> norm -> mixer, final add + norm, tied lm_head.
    ``sd`` is a state dict with lrnnx's parameter names.  Returns the logits (batch, L, vocab)."""
    hidden = F.embedding(input_ids, sd["backbone.embedding.weight"])
    residual = None
    for i in range(n_layer):
        normed, residual = rms_norm_oracle(hidden, sd[f"backbone.layers.{i}.norm.weight"], residual, eps, prenorm=True)
        hidden = mamba_mixer_oracle(_layer_params(sd, i), normed)
    hidden = rms_norm_oracle(hidden, sd["backbone.norm_f.weight"], residual, eps)
    return hidden @ sd["lm_head.weight"].t()


def mamba_lm_prefill_oracle(sd, input_ids, n_layer, eps=1e-5):
    """The same forward keeping, per layer, the states a decoder continues from.  Returns
    (logits of the last position, [(conv_state, ssm_state)] per layer)."""
    hidden = F.embedding(input_ids, sd["backbone.embedding.weight"])
    residual, states = None, []
    for i in range(n_layer):
        normed, residual = rms_norm_oracle(hidden, sd[f"backbone.layers.{i}.norm.weight"], residual, eps, prenorm=True)
        hidden, cs, ss = mamba_mixer_oracle(_layer_params(sd, i), normed, return_states=True)
        states.append((cs.clone(), ss.clone()))
    hidden = rms_norm_oracle(hidden[:, -1], sd["backbone.norm_f.weight"], residual[:, -1], eps)
    return hidden @ sd["lm_head.weight"].t(), states


def mamba_lm_step_oracle(sd, token_ids, states, n_layer, eps=1e-5):
    """LRNNModel.step + lm_head (lrnnx/architectures/language_model.py:344-451,653-681) for
    token ids (batch,); ``states`` is updated in place.  Returns logits (batch, vocab)."""
    hidden = F.embedding(token_ids, sd["backbone.embedding.weight"])
    residual = None
    for i in range(n_layer):
        normed, residual = rms_norm_oracle(hidden, sd[f"backbone.layers.{i}.norm.weight"], residual, eps, prenorm=True)
        hidden = mamba_mixer_step_oracle(_layer_params(sd, i), normed, states[i][0], states[i][1])
    hidden = rms_norm_oracle(hidden, sd["backbone.norm_f.weight"], residual, eps)
    return hidden @ sd["lm_head.weight"].t()
