"""Shared test plumbing: import paths, the ``gpu`` marker, fixtures loader, input recipes."""

from __future__ import annotations

import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
for p in (ROOT / "ml-cross-entropy_b200", ROOT):
    if str(p) not in sys.path:
        sys.path.insert(0, str(p))

GOLDEN_DIR = Path(__file__).resolve().parent / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def golden_names() -> list[str]:
    return sorted(p.stem for p in GOLDEN_DIR.glob("*.pt"))


def load_golden(name: str) -> dict:
    return torch.load(GOLDEN_DIR / f"{name}.pt", weights_only=False)


def planted_inputs(N, V, D, dtype, device, seed=0, bias=False, ignored=0.0):
    """Input recipe of the reference's numeric tests (tests/test_cce_loss_forward.py:66-88):
    e ~ N(0,1)/sqrt(D), c ~ N(0,1) with the first min(N,V)/2 rows of c copied from e (peaked
    softmax), bias ~ 0.02 N(0,1), uniform labels, a fraction of them set to ignore_index."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    e = (torch.randn(N, D, generator=g) / D**0.5).to(dtype)
    c = torch.randn(V, D, generator=g).to(dtype)
    h = min(N, V) // 2
    c[:h] = e[:h]
    b = (torch.randn(V, generator=g) * 0.02).to(dtype) if bias else None
    t = torch.randint(0, V, (N,), generator=g)
    if ignored:
        t[torch.randperm(N, generator=g)[: int(ignored * N)]] = -100
    mv = lambda x: None if x is None else x.to(device)
    return mv(e), mv(c), mv(b), mv(t)
