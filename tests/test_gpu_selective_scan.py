"""GPU parity of the selective scan (forward + backward) through the C ABI.

Reference side: the golden fixtures recorded from lrnnx's selective_scan_ref /
rglru_scan_ref / s7_scan_ref, and the CPU oracle on seeded CPU-generated inputs.
Tolerance: rtol 1e-4 for fp32 activations, 3e-2 for bf16/fp16 activations
(the acceptance tolerance of the benchmark specification), with an absolute floor of 1e-5 (fp32) / 1e-2 (16-bit)
times the largest reference magnitude of the tensor being compared.
"""
from __future__ import annotations

import pytest
import torch

from conftest import assert_close, load_golden
from oracle import scan_oracle as O

pytestmark = pytest.mark.gpu

RTOL32, ATOL32 = 1e-4, 2e-5
GRAD_RTOL32, GRAD_ATOL32 = 3e-4, 1e-4


def _to_cuda(inputs, requires_grad=True):
    out = {}
    for k, v in inputs.items():
        if torch.is_tensor(v):
            v = v.cuda()
            if requires_grad and (v.is_floating_point() or v.is_complex()):
                v.requires_grad_(True)
        out[k] = v
    return out


def _run_case(fn, case, rtol=RTOL32, atol=ATOL32, grtol=GRAD_RTOL32, gatol=GRAD_ATOL32):
    leaves = _to_cuda(case["inputs"])
    res = fn(**leaves, **case["kwargs"])
    res = res if isinstance(res, tuple) else (res,)
    for i, (got, want) in enumerate(zip(res, case["outputs"])):
        assert got.shape == want.shape and got.dtype == want.dtype
        assert_close(got.detach().cpu(), want, rtol=rtol, atol_scale=atol, name=f"output{i}")
    names = [k for k, g in case["grads"].items() if g is not None]
    grads = torch.autograd.grad(res[0], [leaves[k] for k in names], case["gout"].cuda())
    for k, g in zip(names, grads):
        want = case["grads"][k]
        assert g.shape == want.shape and g.dtype == want.dtype
        assert_close(g.cpu(), want, rtol=grtol, atol_scale=gatol, name=f"d{k}")


SEL = load_golden("selective_scan")
RS = load_golden("rglru_s7")


@pytest.mark.parametrize("name", sorted(SEL))
def test_selective_scan_golden(name):
    from lrnnx_b200.ops import selective_scan_fn
    _run_case(selective_scan_fn, SEL[name])


@pytest.mark.parametrize("name", sorted(RS))
def test_rglru_s7_golden(name):
    from lrnnx_b200.ops import rglru_scan_fn, s7_scan_fn
    _run_case(rglru_scan_fn if name.startswith("rglru") else s7_scan_fn, RS[name])


def _make_inputs(batch, dim, N, L, seed, dtype=torch.float32, groups=1, with_z=True, with_deltaA=False):
    g = torch.Generator().manual_seed(seed)
    A = -torch.rand(dim, N, generator=g) * 2 - 0.05
    t = dict(
        u=torch.randn(batch, dim, L, generator=g).to(dtype),
        delta=torch.randn(batch, dim, L, generator=g).to(dtype),
        A=A,
        B=torch.randn(batch, groups, N, L, generator=g).to(dtype),
        C=torch.randn(batch, groups, N, L, generator=g).to(dtype),
        D=torch.randn(dim, generator=g),
        z=torch.randn(batch, dim, L, generator=g).to(dtype) if with_z else None,
        delta_bias=torch.rand(dim, generator=g) - 4.0,
        deltaA=(0.3 * torch.rand(batch, dim, L, generator=g)).to(dtype) if with_deltaA else None,
    )
    return t, g


def _oracle_vs_gpu(t, g, disc, rtol, atol, grtol, gatol, check_x=True):
    from lrnnx_b200.ops import selective_scan_fn
    kw = dict(delta_softplus=True, return_last_state=True, discretization=disc)
    cpu = {k: (v.clone().requires_grad_(True) if torch.is_tensor(v) else v) for k, v in t.items()}
    out_c, last_c = O.selective_scan_oracle(**cpu, **kw)
    gpu = _to_cuda(t)
    out_g, last_g = selective_scan_fn(**gpu, **kw)
    assert out_g.dtype == t["u"].dtype and out_g.shape == out_c.shape
    assert_close(out_g.detach().float().cpu(), out_c.detach().float(), rtol=rtol, atol_scale=atol, name="out")
    assert_close(last_g.detach().cpu(), last_c.detach(), rtol=rtol, atol_scale=atol, name="last_state")
    gout = torch.randn(out_c.shape, generator=g).to(out_c.dtype)
    names = [k for k, v in cpu.items() if torch.is_tensor(v)]
    gc = torch.autograd.grad(out_c, [cpu[k] for k in names], gout, allow_unused=True)
    gg = torch.autograd.grad(out_g, [gpu[k] for k in names], gout.cuda(), allow_unused=True)
    for k, a, b in zip(names, gg, gc):
        if b is None:      # input does not enter the result (e.g. delta under "dirac" with deltaA)
            assert a is None or float(a.abs().max()) == 0.0, f"d{k} must be zero"
            continue
        assert a.dtype == b.dtype and a.shape == b.shape
        assert_close(a.float().cpu(), b.float(), rtol=grtol, atol_scale=gatol, name=f"d{k}")


@pytest.mark.parametrize("L", [1, 8, 255, 257, 372, 1134, 2048, 2049, 4100])
def test_seqlen_sweep_fp32(L):
    """Ragged lengths around the 256-step stage and the 2048-step checkpoint chunk
    (sweep of tests/ops/mamba/test_selective_scan.py:15 plus the boundaries)."""
    t, g = _make_inputs(2, 4, 8, L, seed=L)
    _oracle_vs_gpu(t, g, "mamba", RTOL32, ATOL32, GRAD_RTOL32, GRAD_ATOL32)


@pytest.mark.parametrize("disc", ["mamba", "zoh", "bilinear", "dirac"])
@pytest.mark.parametrize("N", [1, 16, 64])
def test_dstate_methods_fp32(disc, N):
    t, g = _make_inputs(2, 6, N, 300, seed=N, groups=2, with_deltaA=(N == 16))
    _oracle_vs_gpu(t, g, disc, RTOL32, ATOL32, GRAD_RTOL32, GRAD_ATOL32)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_half_precision_inputs(dtype):
    """16-bit activations with fp32 state; the oracle up-casts internally like
    selective_scan_ref (lrnnx/ops/selective_scan.py:221-245)."""
    t, g = _make_inputs(2, 8, 16, 600, seed=11, dtype=dtype)
    _oracle_vs_gpu(t, g, "mamba", 3e-2, 1e-2, 3e-2, 2e-2)


def test_config0_shape():
    """benchmark configuration 0: B=2, D=256, L=512, N=16, A = -[1..N], D = 1, dt-style bias."""
    import math
    g = torch.Generator().manual_seed(0)
    batch, dim, L, N = 2, 256, 512, 16
    dt = torch.exp(torch.rand(dim, generator=g) * (math.log(0.1) - math.log(1e-3)) + math.log(1e-3))
    t = dict(u=torch.randn(batch, dim, L, generator=g), delta=torch.randn(batch, dim, L, generator=g),
             A=-torch.arange(1, N + 1, dtype=torch.float32).repeat(dim, 1),
             B=torch.randn(batch, N, L, generator=g), C=torch.randn(batch, N, L, generator=g),
             D=torch.ones(dim), z=torch.randn(batch, dim, L, generator=g),
             delta_bias=dt + torch.log(-torch.expm1(-dt)), deltaA=None)
    _oracle_vs_gpu(t, g, "mamba", RTOL32, ATOL32, GRAD_RTOL32, GRAD_ATOL32)


def test_checkpoints_match_oracle():
    from lrnnx_b200 import selective_scan_cuda
    t, g = _make_inputs(1, 3, 4, 4500, seed=3, with_z=False)
    _, _, x_c = O.selective_scan_oracle(**t, delta_softplus=True, return_last_state=True, return_checkpoints=True)
    cu = {k: (v.cuda() if torch.is_tensor(v) else v) for k, v in t.items()}
    out, x = selective_scan_cuda.fwd(cu["u"], cu["delta"], cu["A"], cu["B"], cu["C"], cu["D"], None,
                                     cu["delta_bias"], None, True, "mamba")
    assert x.shape == (1, 3, 3, 8)
    assert_close(x.cpu()[..., 1::2], x_c[..., 1::2], rtol=RTOL32, atol_scale=ATOL32, name="x state")
    assert_close(x.cpu()[..., 0::2], x_c[..., 0::2], rtol=1e-3, atol_scale=1e-6, name="x product")


def test_argument_errors():
    from lrnnx_b200 import selective_scan_cuda
    u = torch.randn(1, 2, 8, device="cuda")
    A = -torch.rand(2, 300, device="cuda")
    B = torch.randn(2, 300, device="cuda")
    with pytest.raises(RuntimeError, match="state dimension <= 256"):
        selective_scan_cuda.fwd(u, u, A, B, B, None, None, None, None, False, "mamba")
    A = -torch.rand(2, 4, device="cuda")
    B = torch.randn(2, 4, device="cuda")
    with pytest.raises(RuntimeError, match="Discretization method not supported"):
        selective_scan_cuda.fwd(u, u, A, B, B, None, None, None, None, False, "euler")
    with pytest.raises(RuntimeError):
        selective_scan_cuda.fwd(u.cpu(), u, A, B, B, None, None, None, None, False, "mamba")


@pytest.fixture(params=["stream", "lanescan"])
def kernel_family(request, monkeypatch):
    """Runs a test once on each throughput-kernel family: the library picks the streaming kernels
    (one warp per 16 channels, serial in time) when a problem has at least
    LRNNX_B200_SL_MIN_WARPS warps of work and the lane-scan kernels otherwise."""
    monkeypatch.setenv("LRNNX_B200_SL_MIN_WARPS", "1" if request.param == "stream" else "1000000000")
    return request.param


@pytest.mark.parametrize("L", [8, 40, 264, 2048, 2312, 4104])
@pytest.mark.parametrize("dtype,groups", [(torch.float32, 1), (torch.float32, 2), (torch.bfloat16, 1),
                                          (torch.float16, 2)])
def test_throughput_kernel_shape_class(L, dtype, groups, kernel_family):
    """Shapes served by the packed-fp32 throughput kernels (real A, mamba, variable B/C, dstate 16,
    channel count a multiple of 16 per group, L a multiple of 8): one and several stages, a ragged
    last stage, and a 2048-step checkpoint boundary; on both kernel families."""
    t, g = _make_inputs(2, 32 * groups, 16, L, seed=L, dtype=dtype, groups=groups)
    if dtype == torch.float32:
        _oracle_vs_gpu(t, g, "mamba", RTOL32, ATOL32, GRAD_RTOL32, GRAD_ATOL32)
    else:
        _oracle_vs_gpu(t, g, "mamba", 3e-2, 1e-2, 3e-2, 2e-2)


@pytest.mark.parametrize("with_z,with_D,with_bias,softplus", [(False, True, True, True), (True, False, False, False),
                                                             (False, False, True, False)])
def test_throughput_kernel_optional_operands(with_z, with_D, with_bias, softplus, kernel_family):
    """z, D, delta_bias absent and delta_softplus off, on both kernel families."""
    from lrnnx_b200.ops import selective_scan_fn
    t, g = _make_inputs(2, 32, 16, 296, seed=5, with_z=with_z)
    if not with_D:
        t["D"] = None
    if not with_bias:
        t["delta_bias"] = None
    if not softplus:       # raw step sizes must be positive then
        t["delta"] = 0.5 * torch.rand(t["delta"].shape, generator=g)
        if with_bias:
            t["delta_bias"] = 0.1 * torch.rand(t["delta_bias"].shape, generator=g)
    kw = dict(delta_softplus=softplus, return_last_state=True, discretization="mamba")
    cpu = {k: (v.clone().requires_grad_(True) if torch.is_tensor(v) else v) for k, v in t.items()}
    out_c, last_c = O.selective_scan_oracle(**cpu, **kw)
    gpu = _to_cuda(t)
    out_g, last_g = selective_scan_fn(**gpu, **kw)
    assert_close(out_g.detach().cpu(), out_c.detach(), rtol=RTOL32, atol_scale=ATOL32, name="out")
    assert_close(last_g.detach().cpu(), last_c.detach(), rtol=RTOL32, atol_scale=ATOL32, name="last_state")
    gout = torch.randn(out_c.shape, generator=g)
    names = [k for k, v in cpu.items() if torch.is_tensor(v)]
    gc = torch.autograd.grad(out_c, [cpu[k] for k in names], gout)
    gg = torch.autograd.grad(out_g, [gpu[k] for k in names], gout.cuda())
    for k, a, b in zip(names, gg, gc):
        assert_close(a.cpu(), b, rtol=GRAD_RTOL32, atol_scale=GRAD_ATOL32, name=f"d{k}")


def test_streaming_kernel_many_tiles():
    """Enough rows that the library picks the streaming kernels by itself (at least two warps of
    work per SM): 4 x 1280 channels in 2 groups, two stages plus a ragged one."""
    t, g = _make_inputs(4, 1280, 16, 72, seed=12, groups=2)
    _oracle_vs_gpu(t, g, "mamba", RTOL32, ATOL32, GRAD_RTOL32, GRAD_ATOL32)


def test_throughput_kernel_checkpoints(kernel_family):
    from lrnnx_b200 import selective_scan_cuda
    t, g = _make_inputs(1, 16, 16, 4360, seed=8, with_z=False)
    _, _, x_c = O.selective_scan_oracle(**t, delta_softplus=True, return_last_state=True, return_checkpoints=True)
    cu = {k: (v.cuda() if torch.is_tensor(v) else v) for k, v in t.items()}
    out, x = selective_scan_cuda.fwd(cu["u"], cu["delta"], cu["A"], cu["B"], cu["C"], cu["D"], None,
                                     cu["delta_bias"], None, True, "mamba")
    assert x.shape == x_c.shape == (1, 16, 3, 32)
    assert_close(x.cpu()[..., 1::2], x_c[..., 1::2], rtol=RTOL32, atol_scale=ATOL32, name="x state")
    assert_close(x.cpu()[..., 0::2], x_c[..., 0::2], rtol=1e-3, atol_scale=1e-6, name="x product")


@pytest.mark.parametrize("dtype,L", [(torch.float32, 4360), (torch.bfloat16, 2048), (torch.bfloat16, 520)])
def test_backward_with_and_without_saved_stage_states(dtype, L, kernel_family):
    """The forward call of the throughput kernels leaves the state at every stage boundary
    behind the checkpoints of x; the backward call uses them when it is handed that x and
    recomputes them when it is handed a copy, or a tensor of the same size that did not come from
    fwd().  All must give the same gradients."""
    from lrnnx_b200 import selective_scan_cuda as ext
    t, g = _make_inputs(2, 16, 16, L, seed=31, dtype=dtype)
    cu = {k: (v.cuda() if torch.is_tensor(v) else v) for k, v in t.items()}
    args = (cu["u"], cu["delta"], cu["A"], cu["B"], cu["C"], cu["D"], cu["z"], cu["delta_bias"], None)
    out, x, out_z = ext.fwd(*args, True, "mamba")
    ptr, stage_len = ext._stage_states_of(x, 2, 16, L, 16)
    assert ptr is not None and stage_len == (32 if kernel_family == "stream" else 256)
    assert ext._stage_states_of(x.clone(), 2, 16, L, 16) == (None, 0)
    # a caller-built x whose allocation happens to have the same size is not mistaken for one made by fwd()
    fake = torch.empty(x.untyped_storage().nbytes() // 4, device="cuda")[: x.numel()].view_as(x).copy_(x)
    assert ext._stage_states_of(fake, 2, 16, L, 16) == (None, 0)
    dout = torch.randn(out.shape, generator=g).to(dtype).cuda()
    with_states = ext.bwd(*args, dout, x, out, None, True, False, "mamba")
    recomputed = ext.bwd(*args, dout, fake, out, None, True, False, "mamba")
    f32 = dtype == torch.float32
    for i, (a, b) in enumerate(zip(with_states, recomputed)):
        if a is None:
            assert b is None
            continue
        assert_close(a.float().cpu(), b.float().cpu(), rtol=2e-5 if f32 else 2e-2, atol_scale=2e-6 if f32 else 1e-2,
                     name=f"gradient {i}")


def test_long_row_segmented_forward_matches_oracle():
    """Few rows and a long sequence: the forward is cut into concurrently scanned segments and
    stitched (l_segments > 1 + fix-up); compare with the oracle and check the checkpoints."""
    from lrnnx_b200 import selective_scan_cuda
    t, g = _make_inputs(1, 16, 16, 5 * 2048 + 264, seed=21)
    assert selective_scan_cuda._segments_for(t["u"].cuda(), 1, 16, t["u"].shape[-1], 16, 1, False, True, True, None,
                                             "mamba") > 1
    out_c, last_c, x_c = O.selective_scan_oracle(**t, delta_softplus=True, return_last_state=True,
                                                 return_checkpoints=True)
    cu = {k: (v.cuda() if torch.is_tensor(v) else v) for k, v in t.items()}
    out, x, out_z = selective_scan_cuda.fwd(cu["u"], cu["delta"], cu["A"], cu["B"], cu["C"], cu["D"], cu["z"],
                                            cu["delta_bias"], None, True, "mamba")
    assert_close(out_z.cpu(), out_c, rtol=RTOL32, atol_scale=ATOL32, name="out_z")
    assert_close(x.cpu()[..., 1::2], x_c[..., 1::2], rtol=RTOL32, atol_scale=ATOL32, name="x state")
    assert_close(x.cpu()[..., 0::2], x_c[..., 0::2], rtol=1e-3, atol_scale=1e-6, name="x product")
