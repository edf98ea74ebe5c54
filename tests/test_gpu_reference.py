"""Parity with the UNMODIFIED reference running on the same GPU.

The reference package (Triton kernels and its materialised-logits ``torch_compile`` path) is
imported from ``baseline/_ref`` beside this repository's package (``baseline/reference_loader.py``)
and both are run on the benchmark's own seeded tensors.  Skipped when the reference is not
installed in the checkout.  Tolerances are the project's: loss 1e-3 relative, log-sum-exp 2e-3
absolute, gradients cosine >= 0.9999 and max error <= 1e-2 of max|reference|.  The filtered
default (``impl="cce"``) is held to the reference's own filter: element by element it may be no
further from the exact gradient than the reference's ``cce`` is, plus the same 1e-2 allowance.
"""

from __future__ import annotations

import os

import pytest
import torch

import bench
from conftest import planted_inputs

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(scope="module")
def ref():
    from baseline.reference_loader import load_reference, reference_available

    ok, why = reference_available()
    if not ok:
        pytest.skip(why)
    for var, path in (("CXX", "/usr/bin/g++"), ("CC", "/usr/bin/gcc")):  # a host compiler inductor can use
        if os.path.exists(path):
            os.environ[var] = path
    return load_reference()


def _run(fn, e, c, bias, targets, **kw):
    for t in (e, c, bias):
        if t is not None:
            t.grad = None
    loss, lse = fn(e, c, targets, bias=bias, return_lse=True, **kw)
    loss.backward()
    out = dict(loss=loss.detach().float(), lse=lse.detach().float(), de=e.grad.float(), dc=c.grad.float())
    if bias is not None:
        out["dbias"] = bias.grad.float()
    e.grad = c.grad = None
    return out


def _check_exact(got, want, what):
    assert abs(got["loss"].item() - want["loss"].item()) <= 1e-3 * abs(want["loss"].item()), what
    assert (got["lse"] - want["lse"]).abs().max().item() <= 2e-3, what
    for k in ("de", "dc", "dbias"):
        if k not in want:
            continue
        g, w = got[k], want[k]
        scale = w.abs().max().item()
        err = (g - w).abs().max().item()
        assert err <= 1e-2 * scale, f"{what} {k}: max error {err:.3e} against scale {scale:.3e}"
        cos = torch.nn.functional.cosine_similarity(g.flatten(), w.flatten(), dim=0).item()
        assert cos >= 0.9999, f"{what} {k}: cosine {cos}"


def _check_filtered(ours, ref_filtered, ref_exact, what):
    """|ours - exact| <= |reference's filtered - exact| + 1e-2 max|exact|, element-wise."""
    assert abs(ours["loss"].item() - ref_exact["loss"].item()) <= 1e-3 * abs(ref_exact["loss"].item()), what
    assert (ours["lse"] - ref_exact["lse"]).abs().max().item() <= 2e-3, what
    for k in ("de", "dc"):
        w = ref_exact[k]
        scale = w.abs().max().item()
        excess = (ours[k] - w).abs() - (ref_filtered[k] - w).abs() - 1e-2 * scale
        assert excess.max().item() <= 0, f"{what} {k}: exceeds the reference's own filter error by {excess.max().item():.3e}"


def test_gemma2_2b_head_against_the_reference_on_this_gpu(ref):
    """Benchmark configuration 1 (8192 x 2304 x 256000, bf16, 5 % ignored labels), every element of
    loss, log-sum-exp, dE and dC."""
    from cut_cross_entropy import linear_cross_entropy

    cfg = bench.CONFIGS["gemma2-2b-head"]
    e, c, bias, targets = bench.make_inputs(cfg, DEV)
    e.requires_grad_(True)
    c.requires_grad_(True)

    ref_exact = _run(ref.linear_cross_entropy, e, c, bias, targets, impl="cce_exact")
    ours_exact = _run(linear_cross_entropy, e, c, bias, targets, impl="cce_exact")
    _check_exact(ours_exact, ref_exact, "cce_exact against the reference's cce_exact")
    del ours_exact["lse"]

    try:
        ref_tc = _run(ref.linear_cross_entropy, e, c, bias, targets, impl="torch_compile")
    except Exception as ex:  # inductor needs a working host toolchain on the box
        ref_tc = None
        print(f"reference torch_compile path unavailable here: {type(ex).__name__}: {str(ex)[:200]}")
    if ref_tc is not None:
        ours = _run(linear_cross_entropy, e, c, bias, targets, impl="cce_exact")
        _check_exact(ours, ref_tc, "cce_exact against the reference's torch_compile")
        del ref_tc, ours

    ref_cce = _run(ref.linear_cross_entropy, e, c, bias, targets, impl="cce")
    for impl in ("cce", "cce_kahan"):
        ours_cce = _run(linear_cross_entropy, e, c, bias, targets, impl=impl)
        _check_filtered(ours_cce, ref_cce, ref_exact, f"{impl} against the reference's filter")


@pytest.mark.parametrize("softcap,has_bias", [(None, False), (30.0, True)])
def test_peaked_inputs_against_the_reference_on_this_gpu(ref, softcap, has_bias):
    """The reference's own test recipe (half of the rows have one dominant logit), mid size."""
    from cut_cross_entropy import linear_cross_entropy

    e, c, bias, targets = planted_inputs(2048, 16384, 512, torch.bfloat16, DEV, seed=3, bias=has_bias, ignored=0.1)
    e.requires_grad_(True)
    c.requires_grad_(True)
    if bias is not None:
        bias = bias.float().requires_grad_(True)
    kw = dict(softcap=softcap)
    ref_exact = _run(ref.linear_cross_entropy, e, c, bias, targets, impl="cce_exact", **kw)
    ours_exact = _run(linear_cross_entropy, e, c, bias, targets, impl="cce_exact", **kw)
    _check_exact(ours_exact, ref_exact, "cce_exact against the reference's cce_exact")
    ref_cce = _run(ref.linear_cross_entropy, e, c, bias, targets, impl="cce", **kw)
    ours_cce = _run(linear_cross_entropy, e, c, bias, targets, impl="cce", **kw)
    _check_filtered(ours_cce, ref_cce, ref_exact, "cce against the reference's filter")
