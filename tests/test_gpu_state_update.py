"""GPU parity of the one-token selective_state_update through the C ABI: golden fixtures from
lrnnx's selective_state_update_ref plus oracle comparisons on the reference test's shapes
(tests/ops/mamba/test_selective_state_update.py:16-28,80-98,174-188,352-361).
Tolerance: rtol 1e-4 / atol 1e-5*scale in fp32 (reference test: rtol 3e-4, atol 1e-3);
3e-2 / 1e-2*scale with 16-bit tensors."""
from __future__ import annotations

import pytest
import torch

from conftest import assert_close, load_golden
from oracle import scan_oracle as O

pytestmark = pytest.mark.gpu
SSU = load_golden("state_update")


@pytest.mark.parametrize("name", sorted(SSU))
def test_state_update_golden(name):
    from lrnnx_b200.ops import selective_state_update
    case = SSU[name]
    t = {k: (v.cuda() if torch.is_tensor(v) else v) for k, v in case["inputs"].items()}
    state = t.pop("state").clone()
    out = selective_state_update(state, **t, **case["kwargs"])
    assert_close(out.cpu(), case["outputs"][0], rtol=1e-4, atol_scale=1e-5, name="out")
    assert_close(state.cpu(), case["outputs"][1], rtol=1e-4, atol_scale=1e-5, name="state")


def _inputs(batch, dim, N, seed, itype=torch.float32, stype=torch.float32, heads=None, ngroups=1):
    g = torch.Generator().manual_seed(seed)
    hd = (heads, dim // heads) if heads else (dim,)
    bg = (batch, ngroups, N) if heads else (batch, N)
    r = lambda *s: torch.randn(*s, generator=g)
    return dict(state=r(batch, *hd, N).to(stype), x=r(batch, *hd).to(itype), dt=r(batch, *hd).to(itype),
                A=-torch.rand(*hd, N, generator=g) - 0.5, B=r(*bg).to(itype), C=r(*bg).to(itype),
                D=r(*hd), z=r(batch, *hd).to(itype), dt_bias=torch.rand(*hd, generator=g) - 4.0)


@pytest.mark.parametrize("dim", [2048, 2064, 4096])
@pytest.mark.parametrize("N", [16, 32, 64])
@pytest.mark.parametrize("has_z", [False, True])
def test_state_update_shapes(dim, N, has_z):
    from lrnnx_b200.ops import selective_state_update
    t = _inputs(2, dim, N, seed=dim + N)
    if not has_z:
        t["z"] = None
    cpu_state = t["state"].clone()
    args = {k: v for k, v in t.items() if k != "state"}
    out_c = O.selective_state_update_oracle(cpu_state, **args, dt_softplus=True)
    st = t["state"].cuda()
    out_g = selective_state_update(st, **{k: (v.cuda() if torch.is_tensor(v) else v) for k, v in args.items()},
                                   dt_softplus=True)
    assert_close(out_g.cpu(), out_c, rtol=1e-4, atol_scale=1e-5, name="out")
    assert_close(st.cpu(), cpu_state, rtol=1e-4, atol_scale=1e-5, name="state")


@pytest.mark.parametrize("ngroups", [1, 2, 4])
@pytest.mark.parametrize("tie_hdim", [False, True])
def test_state_update_heads(ngroups, tie_hdim):
    """Heads with grouped B/C; with tie_hdim A, dt and dt_bias are stride-0 broadcasts over the
    head dimension (lrnnx/ops/triton/selective_state_update.py:409-414)."""
    from lrnnx_b200.ops import selective_state_update
    batch, nheads, hd, N = 2, 32, 64, 16
    t = _inputs(batch, nheads * hd, N, seed=ngroups, heads=nheads, ngroups=ngroups)
    if tie_hdim:
        g = torch.Generator().manual_seed(99)
        t["A"] = (-torch.rand(nheads, generator=g) - 0.5)[:, None, None].expand(nheads, hd, N)
        t["dt"] = torch.randn(batch, nheads, generator=g)[:, :, None].expand(batch, nheads, hd)
        t["dt_bias"] = (torch.rand(nheads, generator=g) - 4.0)[:, None].expand(nheads, hd)
    cpu_state = t["state"].clone()
    args = {k: v for k, v in t.items() if k != "state"}
    out_c = O.selective_state_update_oracle(cpu_state, **args, dt_softplus=True)
    st = t["state"].cuda()
    cu = {}
    for k, v in args.items():
        if torch.is_tensor(v):
            base = v.cuda() if v.is_contiguous() else None
            if base is None:   # rebuild the broadcast view on the GPU so the strides stay 0
                if k == "A":
                    base = v[:, 0, 0].contiguous().cuda()[:, None, None].expand(nheads, hd, N)
                elif k == "dt":
                    base = v[:, :, 0].contiguous().cuda()[:, :, None].expand(batch, nheads, hd)
                else:
                    base = v[:, 0].contiguous().cuda()[:, None].expand(nheads, hd)
            v = base
        cu[k] = v
    out_g = selective_state_update(st, **cu, dt_softplus=True)
    assert_close(out_g.cpu(), out_c, rtol=1e-4, atol_scale=1e-5, name="out")
    assert_close(st.cpu(), cpu_state, rtol=1e-4, atol_scale=1e-5, name="state")


def test_state_batch_indices_and_bf16():
    """Indirect state rows (state_batch_indices) with bf16 activations and bf16 state."""
    from lrnnx_b200.ops import selective_state_update
    batch, dim, N, pool = 4, 512, 16, 9
    t = _inputs(batch, dim, N, seed=5, itype=torch.bfloat16, stype=torch.bfloat16)
    g = torch.Generator().manual_seed(6)
    big = torch.randn(pool, dim, N, generator=g).to(torch.bfloat16)
    idx = torch.tensor([7, 2, 5, 0], dtype=torch.int32)
    args = {k: v for k, v in t.items() if k != "state"}
    ref_state = big[idx.long()].clone()
    out_c = O.selective_state_update_oracle(ref_state, **args, dt_softplus=True)
    big_g = big.cuda()
    out_g = selective_state_update(big_g, **{k: v.cuda() for k, v in args.items()}, dt_softplus=True,
                                   state_batch_indices=idx.cuda())
    assert out_g.dtype == torch.bfloat16
    assert_close(out_g.float().cpu(), out_c.float(), rtol=3e-2, atol_scale=1e-2, name="out")
    assert_close(big_g.cpu()[idx.long()].float(), ref_state.float(), rtol=3e-2, atol_scale=1e-2, name="state")
    untouched = [i for i in range(pool) if i not in idx.tolist()]
    assert torch.equal(big_g.cpu()[untouched], big[untouched])


@pytest.mark.parametrize("stype,itype,N", [(torch.float32, torch.float32, 8), (torch.float32, torch.bfloat16, 16),
                                           (torch.bfloat16, torch.bfloat16, 16), (torch.float16, torch.float16, 32)])
@pytest.mark.parametrize("method,heads,with_dA", [("mamba", None, False), ("zoh", 3, True), ("bilinear", None, False),
                                                  ("dirac", 3, False), ("rglru", None, True), ("s7", None, False)])
def test_state_update_tile_pipeline(stype, itype, N, method, heads, with_dA):
    """Dense operands with dim a multiple of 128 take the bulk-copy tile pipeline; enough tiles
    (batch 5 x 3 heads x 3 tiles, or 5 x 6) that the persistent CTAs wrap around their 3-slot
    ring, with optional z / D / dt_bias / deltaA, every discretization and indirect state rows."""
    from lrnnx_b200.ops import selective_state_update
    batch, hd = 5, 384
    dim = hd * (heads or 2)
    t = _inputs(batch, dim, N, seed=N + len(method), itype=itype, stype=stype, heads=heads, ngroups=1)
    g = torch.Generator().manual_seed(17)
    if method == "rglru":
        t["A"] = torch.rand(t["A"].shape, generator=g) * 0.5 + 0.4      # A ** deltaA needs A > 0
    if with_dA:
        t["deltaA"] = (torch.rand(t["x"].shape, generator=g) * 0.5 + 0.05).to(itype)
    if method in ("bilinear", "s7"):
        t["z"] = None
    pool = batch + 2
    big = torch.randn(pool, *t["state"].shape[1:], generator=g).to(stype)
    idx = torch.tensor([6, 0, 3, 1, 4], dtype=torch.int32)
    args = {k: v for k, v in t.items() if k != "state"}
    ref_state = big[idx.long()].clone()
    out_c = O.selective_state_update_oracle(ref_state, **args, dt_softplus=True, discretization=method)
    big_g = big.cuda()
    out_g = selective_state_update(big_g, **{k: (v.cuda() if torch.is_tensor(v) else v) for k, v in args.items()},
                                   dt_softplus=True, discretization=method, state_batch_indices=idx.cuda())
    lo = stype != torch.float32 or itype != torch.float32
    rtol, atol = (3e-2, 1e-2) if lo else (1e-4, 1e-5)
    assert_close(out_g.float().cpu(), out_c.float(), rtol=rtol, atol_scale=atol, name="out")
    assert_close(big_g.cpu()[idx.long()].float(), ref_state.float(), rtol=rtol, atol_scale=atol, name="state")
    untouched = [i for i in range(pool) if i not in idx.tolist()]
    assert torch.equal(big_g.cpu()[untouched], big[untouched])
    from lrnnx_b200 import _lib
    assert _lib.lib().b200_device_status() == 0


def test_state_update_in_cuda_graph():
    """The step is capturable: static buffers, launch on the capturing stream, output allocated by
    the caching allocator (pattern of lrnnx/utils/generation.py:143-155)."""
    from lrnnx_b200.ops import selective_state_update
    t = {k: v.cuda() for k, v in _inputs(4, 256, 16, seed=1).items()}
    state0 = t["state"].clone()
    args = {k: v for k, v in t.items() if k != "state"}
    ref = state0.clone()
    outs_ref = [selective_state_update(ref, **args, dt_softplus=True).clone() for _ in range(3)]
    static_state = state0.clone()
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        warm = state0.clone()
        for _ in range(2):
            selective_state_update(warm, **args, dt_softplus=True)
    torch.cuda.current_stream().wait_stream(s)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        y = selective_state_update(static_state, **args, dt_softplus=True)
    static_state.copy_(state0)
    for k in range(3):
        graph.replay()
        torch.testing.assert_close(y, outs_ref[k], rtol=0, atol=0)
    torch.testing.assert_close(static_state, ref, rtol=0, atol=0)


S5STEP = load_golden("s5_step")


@pytest.mark.parametrize("name", sorted(S5STEP))
def test_s5_step_golden(name):
    from lrnnx_b200.ops import simplified_state_update
    case = S5STEP[name]
    t = {k: (v.cuda() if torch.is_tensor(v) else v) for k, v in case["inputs"].items()}
    state = t.pop("state").clone()
    out = simplified_state_update(state, **t, **case["kwargs"])
    assert out.dtype == torch.float32
    assert_close(out.cpu(), case["outputs"][0], rtol=1e-4, atol_scale=1e-5, name="out")
    assert_close(state.cpu(), case["outputs"][1], rtol=1e-4, atol_scale=1e-5, name="state")


@pytest.mark.parametrize("H,P", [(256, 16), (272, 32), (512, 64)])
def test_s5_step_shapes(H, P):
    """Shapes of tests/ops/s5/test_simplified_state_update.py (H in {256, 272, 512}, P in {16, 32, 64})."""
    import math
    from lrnnx_b200.ops import simplified_state_update
    g = torch.Generator().manual_seed(H + P)
    c = lambda *s: torch.complex(torch.randn(*s, generator=g), torch.randn(*s, generator=g))
    batch = 5
    t = dict(x=torch.randn(batch, H, generator=g), dt=0.1 * torch.rand(batch, P, generator=g) + 0.01,
             A=torch.complex(-0.5 * torch.rand(P, generator=g) - 0.05, math.pi * torch.rand(P, generator=g)),
             B=c(P, H) / math.sqrt(H), C=c(H, P) / math.sqrt(P), D=torch.randn(H, H, generator=g) / math.sqrt(H))
    state = c(batch, P)
    ref_state = state.clone()
    out_c = O.simplified_state_update_oracle(ref_state, **t, discretization="zoh")
    st = state.cuda()
    out_g = simplified_state_update(st, **{k: v.cuda() for k, v in t.items()}, discretization="zoh")
    assert_close(out_g.cpu(), out_c, rtol=1e-4, atol_scale=2e-5, name="out")
    assert_close(st.cpu(), ref_state, rtol=1e-4, atol_scale=1e-5, name="state")


def test_s7_with_deltaA_is_refused():
    """lrnnx's Triton kernel and its selective_state_update_ref disagree on "s7" + deltaA
    (selective_state_update.py:168-176 against :551-553); the combination is rejected."""
    from lrnnx_b200.ops import selective_state_update
    t = _inputs(2, 128, 16, seed=1, itype=torch.float32, stype=torch.float32, heads=None, ngroups=1)
    args = {k: (v.cuda() if torch.is_tensor(v) else v) for k, v in t.items() if k != "state"}
    state = t["state"].cuda()
    before = state.clone()
    with pytest.raises(RuntimeError, match="deltaA is not defined for the s7"):
        selective_state_update(state, **args, deltaA=torch.rand_like(args["x"]), discretization="s7")
    assert torch.equal(state, before)
