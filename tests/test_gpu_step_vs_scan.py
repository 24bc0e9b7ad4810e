"""Decode steps reproduce the parallel scan (the reference's per-model "step == parallel forward"
tests, tests/models/test_ltv/test_mamba.py:51-86, reduced to the two ops this library owns):
L calls of selective_state_update on a zero state give the outputs and the final state of one
selective_scan_fn call over the same L tokens."""
from __future__ import annotations

import pytest
import torch

from conftest import assert_close

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("disc", ["mamba", "zoh", "dirac"])
@pytest.mark.parametrize("L", [16, 300])
def test_step_equals_parallel_scan(disc, L):
    from lrnnx_b200.ops import selective_scan_fn, selective_state_update
    g = torch.Generator().manual_seed(L)
    b, d, n = 3, 64, 16
    r = lambda *s: torch.randn(*s, generator=g).cuda()
    u, delta, z = r(b, d, L), r(b, d, L), r(b, d, L)
    A = (-torch.rand(d, n, generator=g) - 0.2).cuda()
    B, C = r(b, n, L), r(b, n, L)
    D, bias = r(d), (torch.rand(d, generator=g) - 3.0).cuda()
    y, last = selective_scan_fn(u, delta, A, B, C, D, z, bias, delta_softplus=True, return_last_state=True,
                                discretization=disc)
    state = torch.zeros(b, d, n, device="cuda")
    ys = []
    for t in range(L):
        ys.append(selective_state_update(state, u[:, :, t].contiguous(), delta[:, :, t].contiguous(), A,
                                         B[:, :, t].contiguous(), C[:, :, t].contiguous(), D, z[:, :, t].contiguous(),
                                         bias, dt_softplus=True, discretization=disc))
    y_steps = torch.stack(ys, dim=-1)
    assert_close(y_steps, y, rtol=2e-4, atol_scale=2e-5, name="outputs")
    assert_close(state, last, rtol=2e-4, atol_scale=2e-5, name="final state")
