"""``selective_state_update`` on the sm_100a kernel.

Same signature, shape handling and in-place state update as
lrnnx/ops/triton/selective_state_update.py:300-476; arbitrary strides
(including stride-0 broadcasts, the "tied head dim" case of :409-414) and
``state_batch_indices`` are passed through to the kernel.  The call allocates
only ``out`` (through the PyTorch caching allocator, so it is legal inside
``torch.cuda.graph`` capture) and launches on the current stream.
"""
from __future__ import annotations

import torch

from .. import _lib

_DT = {torch.float32: "B200_F32", torch.float16: "B200_F16", torch.bfloat16: "B200_BF16"}
_METHODS = {"zoh": "B200_DISC_ZOH", "bilinear": "B200_DISC_BILINEAR", "dirac": "B200_DISC_DIRAC",
            "mamba": "B200_DISC_MAMBA", "rglru": "B200_DISC_RGLRU", "s7": "B200_DISC_S7"}


def _dt(t, name):
    if t.dtype not in _DT:
        raise RuntimeError(f"{name} must be float32, float16 or bfloat16")
    return _lib.enum(_DT[t.dtype])


def selective_state_update(state, x, dt, A, B, C, D=None, z=None, dt_bias=None, dt_softplus=False, deltaA=None,
                           state_batch_indices=None, discretization="mamba"):
    """state (batch, dim, dstate) or (batch, nheads, dim, dstate), updated in place;
    x, dt, z, deltaA (batch, dim) or (batch, nheads, dim); A (dim, dstate) or (nheads, dim, dstate);
    B, C (batch, dstate) or (batch, ngroups, dstate); D, dt_bias (dim,) or (nheads, dim).
    Returns out with the shape and dtype of x."""
    has_heads = state.dim() > 3
    if state.dim() == 3:
        state = state.unsqueeze(1)
    if x.dim() == 2:
        x = x.unsqueeze(1)
    if dt.dim() == 2:
        dt = dt.unsqueeze(1)
    if A.dim() == 2:
        A = A.unsqueeze(0)
    if B.dim() == 2:
        B = B.unsqueeze(1)
    if C.dim() == 2:
        C = C.unsqueeze(1)
    if D is not None and D.dim() == 1:
        D = D.unsqueeze(0)
    if z is not None and z.dim() == 2:
        z = z.unsqueeze(1)
    if dt_bias is not None and dt_bias.dim() == 1:
        dt_bias = dt_bias.unsqueeze(0)
    if deltaA is not None and deltaA.dim() == 2:
        deltaA = deltaA.unsqueeze(1)
    _, nheads, dim, dstate = state.shape
    batch = x.shape[0]
    assert x.shape == (batch, nheads, dim)
    assert dt.shape == x.shape
    assert A.shape == (nheads, dim, dstate)
    ngroups = B.shape[1]
    assert nheads % ngroups == 0, "nheads must be divisible by ngroups"
    assert B.shape == (batch, ngroups, dstate)
    assert C.shape == B.shape
    if D is not None:
        assert D.shape == (nheads, dim)
    if z is not None:
        assert z.shape == x.shape
    if dt_bias is not None:
        assert dt_bias.shape == (nheads, dim)
    if deltaA is not None:
        assert deltaA.shape == (batch, nheads, dim)
    if state_batch_indices is not None:
        assert state_batch_indices.shape == (batch,)
        if state_batch_indices.dtype != torch.int32 or not state_batch_indices.is_contiguous():
            raise RuntimeError("state_batch_indices must be a contiguous int32 tensor")
    for name, t in (("state", state), ("x", x), ("dt", dt), ("A", A), ("B", B), ("C", C)):
        if not t.is_cuda:
            raise RuntimeError(f"{name} must be a CUDA tensor")
    if B.dtype != C.dtype:
        raise RuntimeError("B and C must have the same dtype")

    a = _lib.struct("b200_ssu_args")()
    a.batch, a.nheads, a.dim, a.dstate, a.ngroups = batch, nheads, dim, dstate, ngroups
    a.state_dtype, a.x_dtype, a.dt_dtype = _dt(state, "state"), _dt(x, "x"), _dt(dt, "dt")
    a.A_dtype, a.bc_dtype = _dt(A, "A"), _dt(B, "B")
    a.dt_softplus = int(bool(dt_softplus))
    a.method = _lib.enum(_METHODS.get(discretization.lower(), "B200_DISC_MAMBA"))
    with torch.cuda.device(x.device):
        out = torch.empty_like(x)
        a.state, a.x, a.dt, a.A, a.B, a.C, a.out = (state.data_ptr(), x.data_ptr(), dt.data_ptr(), A.data_ptr(),
                                                    B.data_ptr(), C.data_ptr(), out.data_ptr())
        a.state_bs, a.state_hs, a.state_ds, a.state_ns = state.stride()
        a.x_bs, a.x_hs, a.x_ds = x.stride()
        a.dt_bs, a.dt_hs, a.dt_ds = dt.stride()
        a.A_hs, a.A_ds, a.A_ns = A.stride()
        a.B_bs, a.B_gs, a.B_ns = B.stride()
        a.C_bs, a.C_gs, a.C_ns = C.stride()
        a.out_bs, a.out_hs, a.out_ds = out.stride()
        if D is not None:
            a.D, a.D_dtype = D.data_ptr(), _dt(D, "D")
            a.D_hs, a.D_ds = D.stride()
        if z is not None:
            a.z, a.z_dtype = z.data_ptr(), _dt(z, "z")
            a.z_bs, a.z_hs, a.z_ds = z.stride()
        if dt_bias is not None:
            a.dt_bias, a.dt_bias_dtype = dt_bias.data_ptr(), _dt(dt_bias, "dt_bias")
            a.dt_bias_hs, a.dt_bias_ds = dt_bias.stride()
        if deltaA is not None:
            a.deltaA, a.deltaA_dtype = deltaA.data_ptr(), _dt(deltaA, "deltaA")
            a.deltaA_bs, a.deltaA_hs, a.deltaA_ds = deltaA.stride()
        if state_batch_indices is not None:
            a.state_batch_indices = state_batch_indices.data_ptr()
        _lib.call("b200_ssu_step", a, torch.cuda.current_stream(x.device).cuda_stream)
    return out if has_heads else out.squeeze(1)
