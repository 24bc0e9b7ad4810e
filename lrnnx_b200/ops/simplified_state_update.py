"""``simplified_state_update`` (one S5 decode step) on the sm_100a kernel; same signature,
assertions and in-place state update as lrnnx/ops/triton/simplified_state_update.py:254-401."""
from __future__ import annotations

import torch

from .. import _lib

_METHODS = {"zoh": "B200_DISC_ZOH", "bilinear": "B200_DISC_BILINEAR", "dirac": "B200_DISC_DIRAC"}


def simplified_state_update(state, x, dt, A, B, C, D=None, deltaA=None, discretization="bilinear", conj_sym=True):
    """state (batch, P) complex64, modified in place; x (batch, H) float32; dt, deltaA (batch, P) or (P,)
    float32; A (P,), B (P, H), C (H, P) complex64; D (H, H) float32 or None.  Returns (batch, H) float32."""
    assert state.is_complex(), "state must be complex64"
    assert A.is_complex(), "A must be complex64"
    assert B.is_complex(), "B must be complex64"
    assert C.is_complex(), "C must be complex64"
    assert not x.is_complex(), "x must be real (float32)"
    batch, P = state.shape
    H = x.shape[1]
    assert x.shape == (batch, H)
    assert A.shape == (P,)
    assert B.shape == (P, H)
    assert C.shape == (H, P)
    if D is not None:
        assert D.shape == (H, H)
    if discretization.lower() not in _METHODS:
        raise ValueError(f"Unknown discretization: {discretization}")
    for name, t in (("state", state), ("x", x), ("dt", dt), ("A", A), ("B", B), ("C", C)):
        if not t.is_cuda:
            raise RuntimeError(f"{name} must be a CUDA tensor")
    if state.dtype != torch.complex64 or x.dtype != torch.float32 or dt.dtype != torch.float32:
        raise RuntimeError("state must be complex64 and x, dt float32")
    if state.stride(1) != 1:
        raise RuntimeError("state must be contiguous in its last dimension")
    x = x if x.stride(1) == 1 else x.contiguous()

    def rows(t, name):
        if t.dim() == 1:
            assert t.shape == (P,), f"{name} must be (P,) or (batch, P)"
            return t.contiguous(), 0
        assert t.shape == (batch, P), f"{name} must be (P,) or (batch, P)"
        t = t if t.stride(1) == 1 else t.contiguous()
        return t, t.stride(0)

    dt, dt_bs = rows(dt, "dt")
    a = _lib.struct("b200_s5_step_args")()
    a.batch, a.P, a.H = batch, P, H
    a.method = _lib.enum(_METHODS[discretization.lower()])
    a.conj_sym = int(bool(conj_sym))
    A, B, C = A.contiguous(), B.contiguous(), C.contiguous()
    keep = [dt, A, B, C, x]
    with torch.cuda.device(x.device):
        out = torch.empty((batch, H), dtype=torch.float32, device=x.device)
        a.state, a.x, a.dt, a.A, a.B, a.C, a.out = (state.data_ptr(), x.data_ptr(), dt.data_ptr(), A.data_ptr(),
                                                    B.data_ptr(), C.data_ptr(), out.data_ptr())
        a.state_bs, a.x_bs, a.dt_bs, a.out_bs = state.stride(0), x.stride(0), dt_bs, out.stride(0)
        if deltaA is not None:
            deltaA, dA_bs = rows(deltaA.float(), "deltaA")
            keep.append(deltaA)
            a.deltaA, a.deltaA_bs = deltaA.data_ptr(), dA_bs
        if D is not None:
            D = D.float().contiguous()
            keep.append(D)
            a.D = D.data_ptr()
        _lib.call("b200_s5_step", a, torch.cuda.current_stream(x.device).cuda_stream)
    return out
