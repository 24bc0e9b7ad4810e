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
