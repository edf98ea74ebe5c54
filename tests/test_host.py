"""CPU tests: host-side logic of the package and the shape of the C-ABI library.
No kernel is launched here."""

from __future__ import annotations

import ctypes
import re
from pathlib import Path

import pytest
import torch

from oracle import cce_oracle as O

ROOT = Path(__file__).resolve().parent.parent


def test_library_loads_and_exports_every_declared_symbol():
    from cut_cross_entropy import _build, _native

    _build.build()
    header = (ROOT / "include" / "cce_b200.h").read_text()
    declared = set(re.findall(r"\b(cce_b200_[a-z_0-9]+)\s*\(", header))
    assert declared, "no declarations found in the header"
    L = _native.lib()
    for name in sorted(declared):
        assert hasattr(L, name), f"{name} declared in include/cce_b200.h but not exported"
    assert declared == set(_native.EXPORTS)
    assert L.cce_b200_version() >= 1
    assert L.cce_b200_strerror(0) == b"ok" and b"workspace" in L.cce_b200_strerror(-3)
    assert L.cce_b200_launch_count() >= 0


def test_ctypes_structs_match_the_header_layout():
    from cut_cross_entropy import _native

    # 4 pointers, 6 int64, 4 int32, 1 float -> 100 bytes, padded to 8-byte alignment
    assert ctypes.sizeof(_native.Operands) == 104
    assert _native.BackwardArgs.op.offset == 0 and _native.BackwardArgs.lse.offset == 104
    # no GPU here: argument checks must reject, not crash
    L = _native.lib()
    op = _native.Operands()
    assert L.cce_b200_lse_workspace_bytes(op) == 0
    assert L.cce_b200_lse_forward(op, None, None, None, 0, None) == -1
    assert L.cce_b200_backward(None, None, 0, None) == -1


def test_presets():
    from cut_cross_entropy.cce_utils import CCEPreset, CCEPresets, LinearCrossEntropyImpl

    user = CCEPreset(filter_eps=1e-3, accum_e_fp32=False, accum_c_fp32=False, filter_e_grad=False, filter_c_grad=True)
    assert CCEPresets.build_for_impl("cce", user) == user
    for name in ("cce_exact", "cce_kahan_full", "cce_kahan_full_c_full_e"):
        o = CCEPresets.build_for_impl(name, user)
        assert o["filter_eps"] is None and o["accum_e_fp32"] and o["accum_c_fp32"]
    o = CCEPresets.build_for_impl("cce_kahan_full_c", user)
    assert (o["filter_eps"], o["filter_c_grad"], o["filter_e_grad"]) == ("auto", False, True)
    o = CCEPresets.build_for_impl("cce_kahan_full_e", user)
    assert (o["filter_eps"], o["filter_c_grad"], o["filter_e_grad"]) == ("auto", True, False)
    o = CCEPresets.build_for_impl("cce_kahan", user)
    assert o["filter_eps"] == 1e-3 and o["accum_e_fp32"] and o["accum_c_fp32"] and not o["filter_e_grad"]
    with pytest.raises(ValueError):
        CCEPresets.build_for_impl("torch_compile", user)
    assert {m.name.lower() for m in LinearCrossEntropyImpl} - {"torch_compile"} == CCEPresets.names
    assert user["filter_eps"] == 1e-3  # the caller's dict is not modified


@pytest.mark.parametrize("shift", [0, 1, 3])
@pytest.mark.parametrize("frac", [0.0, 0.3])
def test_flat_valids_against_oracle(shift, frac):
    from cut_cross_entropy.utils import _build_flat_valids, handle_reduction_none

    g = torch.Generator().manual_seed(shift)
    t = torch.randint(0, 50, (3, 11), generator=g)
    if frac:
        t[torch.rand(3, 11, generator=g) < frac] = -100
    got = _build_flat_valids(t, -100, shift)
    want = O.flat_valids(t, -100, shift)
    if shift == 0 and frac == 0.0:
        assert got is None
    else:
        assert got.dtype == (torch.int32 if shift == 0 else torch.int64)
        assert torch.equal(got.long(), want)
        vals = torch.arange(1.0, want.numel() + 1)
        assert torch.equal(handle_reduction_none(t.shape, got, shift, vals), O.scatter_none(t.shape, want, shift, vals))


def test_eps_and_z_loss_known_answers():
    from cut_cross_entropy.utils import _handle_eps, compute_z_loss

    assert _handle_eps("auto", torch.bfloat16) == 2.0**-12
    assert _handle_eps("auto", torch.float16) == 2.0**-15
    assert _handle_eps(None, torch.float16) is None and _handle_eps(0.5, torch.float16) == 0.5
    with pytest.raises(RuntimeError):
        _handle_eps("big", torch.float16)
    lse = torch.arange(1, 11, dtype=torch.float64)
    assert compute_z_loss(lse, reduction="sum").item() == pytest.approx(385.0)
    targets = torch.full((10,), -100)
    targets[3], targets[5] = 1, 2
    assert compute_z_loss(lse, targets, reduction="mean").item() == pytest.approx((16.0 + 36.0) / 2)
    assert compute_z_loss(lse[:9], targets, shift=1, reduction="sum").item() == pytest.approx(9.0 + 25.0)
    with pytest.raises(ValueError):
        compute_z_loss(lse, reduction="max")


def test_public_api_validation_and_no_cpu_path():
    from cut_cross_entropy import VocabParallelOptions, linear_cross_entropy

    e, c, t = torch.randn(4, 8, 16).bfloat16(), torch.randn(32, 16).bfloat16(), torch.randint(0, 32, (4, 8))
    with pytest.raises(ValueError, match="Shift must be"):
        linear_cross_entropy(e, c, t, shift=8)
    with pytest.raises(ValueError, match="Bias has"):
        linear_cross_entropy(e, c, t, bias=torch.zeros(31))
    with pytest.raises(ValueError, match="Expected c.size"):
        linear_cross_entropy(e, c, t, vocab_parallel_options=VocabParallelOptions(0, 16))
    with pytest.raises(NotImplementedError):
        linear_cross_entropy(e, c, t, impl="torch_compile")
    # CPU tensors: the backend refuses instead of falling back
    with pytest.raises(RuntimeError, match="no CPU path"):
        linear_cross_entropy(e, c, t)


def test_partition():
    from cut_cross_entropy.vocab_parallel import partition_n_into_range

    for n, w in ((10, 3), (262144, 8), (5, 8)):
        for r in range(w):
            assert partition_n_into_range(n, r, w) == O.partition_n_into_range(n, r, w)
