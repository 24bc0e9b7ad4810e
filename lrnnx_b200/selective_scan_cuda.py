"""Drop-in for lrnnx's compiled ``selective_scan_cuda`` module.

``fwd`` / ``bwd`` keep the positional signatures bound in
csrc/selective_scan/bindings.cpp:5-8 (declared in
csrc/selective_scan/selective_scan.h:114-136) and reproduce the checks,
allocations and return lists of selective_scan_fwd / selective_scan_bwd
(csrc/selective_scan/selective_scan_cpu.cpp:263-632).  A failed check raises
``RuntimeError`` like the reference's ``TORCH_CHECK``.  Unlike the reference
(selective_scan_cpu.cpp:404,612) fp16 / bf16 activations are accepted; the
recurrence state is always fp32.
"""
from __future__ import annotations

import ctypes

import torch

from . import _lib

_METHODS = {
    "zoh": "B200_DISC_ZOH",
    "bilinear": "B200_DISC_BILINEAR",
    "dirac": "B200_DISC_DIRAC",
    "mamba": "B200_DISC_MAMBA",
    "s7": "B200_DISC_S7",
    "rglru": "B200_DISC_RGLRU",
}
_DTYPES = {torch.float32: "B200_F32", torch.float16: "B200_F16", torch.bfloat16: "B200_BF16"}
CHUNK = 2048


def _check(cond: bool, msg: str) -> None:
    if not cond:
        raise RuntimeError(msg)


def _ptr(t):
    return None if t is None else t.data_ptr()


def _shape(t, *shape, name: str) -> None:
    _check(tuple(t.shape) == tuple(shape), f"{name} must have shape {tuple(shape)}, got {tuple(t.shape)}")


def _common(u, delta, A, B, C, D, z, delta_bias, deltaA, discretization):
    """Validation shared by fwd and bwd; returns the partially filled argument block."""
    _check(u.dtype in _DTYPES, "u must be float32, float16 or bfloat16")
    _check(A.dtype in (torch.float32, torch.complex64), "A must be float32 or complex64")
    _check(discretization in _METHODS, "Discretization method not supported")
    is_complex = A.dtype == torch.complex64
    if discretization == "s7":
        _check(not is_complex, "S7 discretization only supports real (float) weights, not complex")
    if discretization == "rglru":
        _check(not is_complex, "RGLRU discretization only supports real (float) weights, not complex")
    var_B, var_C = B.dim() >= 3, C.dim() >= 3
    _check(delta.dtype == u.dtype, "delta must have the dtype of u")
    _check(B.dtype == (u.dtype if var_B else A.dtype), "B has the wrong dtype")
    _check(C.dtype == (u.dtype if var_C else A.dtype), "C has the wrong dtype")
    for name, t in (("u", u), ("delta", delta), ("A", A), ("B", B), ("C", C)):
        _check(t.is_cuda, f"{name} must be a CUDA tensor")
    _check(u.dim() == 3, "u must be (batch, dim, seqlen)")
    _check(u.stride(-1) == 1 or u.size(-1) == 1, "u must be contiguous in the last dimension")
    _check(delta.stride(-1) == 1 or delta.size(-1) == 1, "delta must be contiguous in the last dimension")
    batch, dim, seqlen = u.shape
    _check(A.dim() == 2, "A must be (dim, dstate)")
    dstate = A.size(1)
    n_groups = B.size(1) if var_B else 1
    _check(dstate <= 256, "selective_scan only supports state dimension <= 256")
    _shape(delta, batch, dim, seqlen, name="delta")
    _shape(A, dim, dstate, name="A")
    lb = seqlen * 2 if is_complex else seqlen
    if var_B:
        _shape(B, batch, n_groups, dstate, lb, name="B")
        _check(B.stride(-1) == 1 or B.size(-1) == 1, "B must be contiguous in the last dimension")
    else:
        _shape(B, dim, dstate, name="B")
    if var_C:
        _shape(C, batch, C.size(1), dstate, lb, name="C")
        _check(C.size(1) == n_groups or not var_B, "B and C must have the same number of groups")
        _check(C.stride(-1) == 1 or C.size(-1) == 1, "C must be contiguous in the last dimension")
        if not var_B:
            n_groups = C.size(1)
    else:
        _shape(C, dim, dstate, name="C")
    _check(dim % n_groups == 0, "dim must be a multiple of the number of groups")
    for name, t in (("D", D), ("delta_bias", delta_bias)):
        if t is not None:
            _check(t.dtype == torch.float32, f"{name} must be float32")
            _check(t.is_cuda, f"{name} must be a CUDA tensor")
            _check(t.stride(-1) == 1 or t.size(-1) == 1, f"{name} must be contiguous")
            _shape(t, dim, name=name)
    for name, t in (("deltaA", deltaA), ("z", z)):
        if t is not None:
            _check(t.dtype == u.dtype, f"{name} must have the dtype of u")
            _check(t.is_cuda, f"{name} must be a CUDA tensor")
            _check(t.stride(-1) == 1 or t.size(-1) == 1, f"{name} must be contiguous in the last dimension")
            _shape(t, batch, dim, seqlen, name=name)

    a = _lib.struct("b200_selscan_fwd_args")()
    a.batch, a.dim, a.seqlen, a.dstate, a.n_groups = batch, dim, seqlen, dstate, n_groups
    a.dtype = _lib.enum(_DTYPES[u.dtype])
    a.is_complex = int(is_complex)
    a.var_B, a.var_C = int(var_B), int(var_C)
    a.method = _lib.enum(_METHODS[discretization])
    a.u, a.delta, a.A, a.B, a.C = u.data_ptr(), delta.data_ptr(), A.data_ptr(), B.data_ptr(), C.data_ptr()
    a.D, a.z, a.delta_bias, a.deltaA = _ptr(D), _ptr(z), _ptr(delta_bias), _ptr(deltaA)
    a.u_bs, a.u_ds = u.stride(0), u.stride(1)
    a.delta_bs, a.delta_ds = delta.stride(0), delta.stride(1)
    if z is not None:
        a.z_bs, a.z_ds = z.stride(0), z.stride(1)
    if deltaA is not None:
        a.deltaA_bs, a.deltaA_ds = deltaA.stride(0), deltaA.stride(1)
    a.A_ds, a.A_ns = A.stride(0), A.stride(1)
    if var_B:
        a.B_bs, a.B_gs, a.B_ns = B.stride(0), B.stride(1), B.stride(2)
    else:
        a.B_bs, a.B_gs, a.B_ns = 0, B.stride(0), B.stride(1)
    if var_C:
        a.C_bs, a.C_gs, a.C_ns = C.stride(0), C.stride(1), C.stride(2)
    else:
        a.C_bs, a.C_gs, a.C_ns = 0, C.stride(0), C.stride(1)
    return a, (batch, dim, seqlen, dstate, n_groups, is_complex, var_B, var_C)


def _stream(t) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


_SM_COUNT = {}


def _segments_for(u, batch, dim, seqlen, dstate, n_groups, is_complex, var_B, var_C, deltaA, method):
    """Number of sequence segments for the forward call: > 1 only for long rows that would leave
    most of the GPU idle (few (batch, channel-tile) thread blocks), on the shape class of the
    throughput kernel.  Segments are scanned concurrently from zero states and stitched by the
    summary fold + fix-up that the multi-GPU sequence-parallel path uses."""
    if is_complex or method != "mamba" or not (var_B and var_C) or deltaA is not None or dstate != 16:
        return 1
    if dim % 16 or (dim // n_groups) % 16 or seqlen % 8 or seqlen < 4 * CHUNK:
        return 1
    idx = u.device.index if u.device.index is not None else torch.cuda.current_device()
    if idx not in _SM_COUNT:
        _SM_COUNT[idx] = torch.cuda.get_device_properties(idx).multi_processor_count
    slots = 8 * _SM_COUNT[idx]     # resident 16-channel warp tiles of the streaming kernel
    ctas = batch * dim // 16
    if ctas >= 4 * slots:
        return 1
    # pick the segment count whose thread blocks fill whole waves best (ties: fewer segments)
    best, best_eff = 1, 0.0
    for want in range(1, 17):
        seg_len = -(-(-(-seqlen // want)) // CHUNK) * CHUNK
        if want > 1 and seg_len < 2 * CHUNK:
            break
        S = -(-seqlen // seg_len)
        waves = ctas * S / slots
        # below one wave more segments simply mean more of the GPU in use; above, whole waves count.
        # Every extra segment also costs a fix-up pass over its first steps: demand a clear gain.
        eff = waves if waves <= 1.0 else waves / -(-waves // 1)
        if eff > best_eff * 1.10 + 1e-9:
            best, best_eff = S, eff
    return best


# Stage states: the throughput kernels pass the state at every stage boundary from the forward to
# the backward call (which then skips recomputing them).  They live behind the checkpoints in x's
# own allocation, so the reference's fwd / bwd signatures stay as they are.  bwd() recognises an x
# made by fwd() through a registry of weak references to the storages fwd() allocated (a copy, a
# user-built x or a recycled address never matches) and falls back to recomputation otherwise.
_STAGE_REGISTRY = {}     # storage impl pointer -> (weak reference to the storage, stage length)


def _stage_numel(batch, dim, seqlen, dstate, stage_len):
    return batch * dim * (-(-seqlen // stage_len)) * dstate


def _register_stage_storage(x, stage_len):
    from torch.multiprocessing.reductions import StorageWeakRef
    if len(_STAGE_REGISTRY) > 256:
        for key in [k for k, (ref, _) in _STAGE_REGISTRY.items() if ref.expired()]:
            del _STAGE_REGISTRY[key]
    st = x.untyped_storage()
    _STAGE_REGISTRY[st._cdata] = (StorageWeakRef(st), stage_len)


def _stage_states_of(x_, batch, dim, seqlen, dstate):
    """(device address, stage length) of the stage states behind the checkpoints of an x made by
    fwd(), else (None, 0)."""
    if x_ is None or x_.dtype != torch.float32 or x_.storage_offset() != 0 or not x_.is_contiguous():
        return None, 0
    st = x_.untyped_storage()
    entry = _STAGE_REGISTRY.get(st._cdata)
    if entry is None or entry[0].expired():
        return None, 0
    stage_len = entry[1]
    if st.nbytes() != (x_.numel() + _stage_numel(batch, dim, seqlen, dstate, stage_len)) * 4:
        return None, 0
    return x_.data_ptr() + x_.numel() * 4, stage_len


def _stitch_segments(a, x, S, seqlen, u):
    """Fold the zero-start summaries of the segments (one kernel) and run the fix-up kernel on segments >= 1."""
    seg_len = -(-(-(-seqlen // S)) // CHUNK) * CHUNK
    batch, dim, _, two_n = x.shape
    h_in = torch.empty((S, batch, dim, two_n // 2), dtype=torch.float32, device=x.device)
    p_in = torch.empty_like(h_in)
    q = _lib.struct("b200_selscan_fixup_args")()
    a.l_segments = 0
    q.f = a
    q.h_in, q.p_in = h_in.data_ptr(), p_in.data_ptr()
    q.n_segments, q.seg_len = S, seg_len
    _lib.call("b200_selscan_fold", q, _stream(u))
    _lib.call("b200_selscan_fixup", q, _stream(u))


def fwd(u, delta, A, B, C, D_, z_, delta_bias_, deltaA_, delta_softplus, discretization_method_str):
    """Returns ``[out, x]`` or ``[out, x, out_z]`` (selective_scan_cpu.cpp:418-420)."""
    a, (batch, dim, seqlen, dstate, n_groups, is_complex, var_B, var_C) = _common(
        u, delta, A, B, C, D_, z_, delta_bias_, deltaA_, discretization_method_str)
    n_chunks = (seqlen + CHUNK - 1) // CHUNK
    with torch.cuda.device(u.device):
        out = torch.empty_like(delta)
        x = torch.empty((batch, dim, n_chunks, dstate * 2), dtype=A.dtype, device=u.device)
        out_z = torch.empty_like(z_) if z_ is not None else None
        a.delta_softplus = int(bool(delta_softplus))
        a.out, a.x, a.out_z = out.data_ptr(), x.data_ptr(), _ptr(out_z)
        a.out_bs, a.out_ds = out.stride(0), out.stride(1)
        if out_z is not None:
            a.out_z_bs, a.out_z_ds = out_z.stride(0), out_z.stride(1)
        S = _segments_for(u, batch, dim, seqlen, dstate, n_groups, is_complex, var_B, var_C, deltaA_,
                          discretization_method_str)
        stage_len = _lib.lib().b200_selscan_stage_states(ctypes.byref(a)) if S <= 1 else 0
        if stage_len > 0:
            x_numel = x.numel()
            flat = torch.empty(x_numel + _stage_numel(batch, dim, seqlen, dstate, stage_len), dtype=x.dtype,
                               device=u.device)
            x = flat[:x_numel].view(batch, dim, n_chunks, dstate * 2)
            _register_stage_storage(x, stage_len)
            a.x = x.data_ptr()
            a.stage_h = x.data_ptr() + x_numel * x.element_size()
            a.stage_len = stage_len
        if S > 1:
            a.l_segments = S
            try:
                _lib.call("b200_selscan_fwd", a, _stream(u))
            except RuntimeError as e:
                if "l_segments" not in str(e):
                    raise
                S, a.l_segments = 1, 0       # operands not aligned for the throughput kernel
                _lib.call("b200_selscan_fwd", a, _stream(u))
            if S > 1:
                _stitch_segments(a, x, S, seqlen, u)
        else:
            _lib.call("b200_selscan_fwd", a, _stream(u))
    return [out, x] if out_z is None else [out, x, out_z]


def bwd(u, delta, A, B, C, D_, z_, delta_bias_, deltaA_, dout, x_, out_, dz_, delta_softplus, recompute_out_z,
        discretization_method_str, h_in=None, q_in=None):
    """Returns ``[du, ddelta, dA, dB, dC, dD, ddelta_bias, (ddeltaA), (dz), (out_z)]``
    (selective_scan_cpu.cpp:627-631); dD / ddelta_bias are None when D / delta_bias are.
    Two additions to the reference signature, for a slice of a sequence-parallel scan (real A):
    ``h_in`` (batch, dim, dstate) float32, the state entering the first step, with ``x_`` holding
    the checkpoints corrected for it; ``q_in``, same shape, the gradient with respect to the state
    after the last step."""
    f, (batch, dim, seqlen, dstate, n_groups, is_complex, var_B, var_C) = _common(
        u, delta, A, B, C, D_, z_, delta_bias_, deltaA_, discretization_method_str)
    _check(dout.dtype == u.dtype, "dout must have the dtype of u")
    _check(dout.is_cuda, "dout must be a CUDA tensor")
    _check(dout.stride(-1) == 1 or dout.size(-1) == 1, "dout must be contiguous in the last dimension")
    _shape(dout, batch, dim, seqlen, name="dout")
    has_z = z_ is not None
    n_chunks = (seqlen + CHUNK - 1) // CHUNK
    with torch.cuda.device(u.device):
        out = dz = out_z = None
        if has_z:
            _check(out_ is not None, "out is required when z is given")
            out = out_
            _check(out.dtype == u.dtype and out.is_cuda, "out must be a CUDA tensor with the dtype of u")
            _check(out.stride(-1) == 1 or out.size(-1) == 1, "out must be contiguous in the last dimension")
            _shape(out, batch, dim, seqlen, name="out")
            if dz_ is not None:
                dz = dz_
                _check(dz.dtype == u.dtype and dz.is_cuda, "dz must be a CUDA tensor with the dtype of u")
                _check(dz.stride(-1) == 1 or dz.size(-1) == 1, "dz must be contiguous in the last dimension")
                _shape(dz, batch, dim, seqlen, name="dz")
            else:
                dz = torch.empty_like(z_)
            if recompute_out_z:
                out_z = torch.empty_like(out)
        if n_chunks > 1:
            _check(x_ is not None, "x is required when seqlen > 2048")
        if x_ is not None:
            _check(x_.dtype == A.dtype and x_.is_cuda and x_.is_contiguous(), "x must be a contiguous CUDA tensor in A's dtype")
            _shape(x_, batch, dim, n_chunks, 2 * dstate, name="x")
        du = torch.empty_like(u)
        ddelta = torch.empty_like(delta)
        dA = torch.zeros_like(A)
        dB = torch.zeros_like(B) if not var_B else torch.zeros_like(B, dtype=torch.float32)
        dC = torch.zeros_like(C) if not var_C else torch.zeros_like(C, dtype=torch.float32)
        dD = torch.zeros_like(D_) if D_ is not None else None
        ddelta_bias = torch.zeros_like(delta_bias_) if delta_bias_ is not None else None
        ddeltaA = torch.empty_like(deltaA_) if deltaA_ is not None else None

        q = _lib.struct("b200_selscan_bwd_args")()
        f.delta_softplus = int(bool(delta_softplus))
        f.x = _ptr(x_)
        f.stage_h, f.stage_len = _stage_states_of(x_, batch, dim, seqlen, dstate)
        f.out = _ptr(out)
        if out is not None:
            f.out_bs, f.out_ds = out.stride(0), out.stride(1)
        f.out_z = _ptr(out_z)
        if out_z is not None:
            f.out_z_bs, f.out_z_ds = out_z.stride(0), out_z.stride(1)
        q.f = f
        q.dout, q.du, q.ddelta = dout.data_ptr(), du.data_ptr(), ddelta.data_ptr()
        q.ddeltaA, q.dz = _ptr(ddeltaA), _ptr(dz)
        q.dA, q.dB, q.dC = dA.data_ptr(), dB.data_ptr(), dC.data_ptr()
        q.dD, q.ddelta_bias = _ptr(dD), _ptr(ddelta_bias)
        if h_in is not None or q_in is not None:
            _check(not is_complex, "h_in / q_in need a real A")
            keep = []
            for name, t in (("h_in", h_in), ("q_in", q_in)):
                if t is None:
                    continue
                _check(t.is_cuda and tuple(t.shape) == (batch, dim, dstate), f"{name} must be a CUDA tensor (batch, dim, dstate)")
                t = t.to(torch.float32).contiguous()
                keep.append(t)
                setattr(q, name, t.data_ptr())
            if h_in is not None:
                f.stage_h, f.stage_len = None, 0      # stage states of a zero-start forward do not apply
                q.f = f
        q.dout_bs, q.dout_ds = dout.stride(0), dout.stride(1)
        q.du_bs, q.du_ds = du.stride(0), du.stride(1)
        q.ddelta_bs, q.ddelta_ds = ddelta.stride(0), ddelta.stride(1)
        if ddeltaA is not None:
            q.ddeltaA_bs, q.ddeltaA_ds = ddeltaA.stride(0), ddeltaA.stride(1)
        if dz is not None:
            q.dz_bs, q.dz_ds = dz.stride(0), dz.stride(1)
        q.dA_ds, q.dA_ns = dA.stride(0), dA.stride(1)
        if var_B:
            q.dB_bs, q.dB_gs, q.dB_ns = dB.stride(0), dB.stride(1), dB.stride(2)
        else:
            q.dB_bs, q.dB_gs, q.dB_ns = 0, dB.stride(0), dB.stride(1)
        if var_C:
            q.dC_bs, q.dC_gs, q.dC_ns = dC.stride(0), dC.stride(1), dC.stride(2)
        else:
            q.dC_bs, q.dC_gs, q.dC_ns = 0, dC.stride(0), dC.stride(1)
        _lib.call("b200_selscan_bwd", q, _stream(u))
        result = [du, ddelta, dA, dB.to(B.dtype), dC.to(C.dtype), dD, ddelta_bias]
        if deltaA_ is not None:
            result.append(ddeltaA)
        if has_z:
            result.append(dz)
        if recompute_out_z:
            result.append(out_z)
    return result
