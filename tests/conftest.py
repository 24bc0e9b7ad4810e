"""Shared pytest configuration.

Markers: ``gpu`` — needs a CUDA device (parity tests proper; they call through the C ABI).
Everything else runs on CPU.
"""
from __future__ import annotations

import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

GOLDEN = ROOT / "tests" / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: test needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def load_golden(name: str) -> dict:
    return torch.load(GOLDEN / f"{name}.pt", map_location="cpu", weights_only=False)


def assert_close(actual, expected, rtol, atol_scale=1e-5, name=""):
    """|a - e| <= atol + rtol*|e| with atol = atol_scale * max|e| (so near-zero entries of a
    tensor are judged against the tensor's own scale)."""
    expected = expected.to(actual.device)
    atol = atol_scale * float(expected.abs().max()) + 1e-30
    torch.testing.assert_close(actual, expected.to(actual.dtype), rtol=rtol, atol=atol, msg=lambda m: f"{name}: {m}")
