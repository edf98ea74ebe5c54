"""Pins the CPU oracle: against fixtures produced by the reference's own code, and against the
known answers held by the reference's tests."""

from __future__ import annotations

import pytest
import torch
from conftest import golden_names, load_golden

from oracle import cce_oracle as O


@pytest.mark.parametrize("name", golden_names())
def test_oracle_matches_reference_fixture(name):
    g = load_golden(name)
    o = g["opts"]
    shift, reduction, softcap = o.get("shift", 0), o.get("reduction", "mean"), o.get("softcap")
    loss, lse = O.linear_cross_entropy(
        g["e"], g["c"], g["targets"], g["bias"], softcap=softcap, reduction=reduction, shift=shift, return_lse=True
    )
    # the fixture was computed in float32 by the reference; the oracle works in float64
    torch.testing.assert_close(loss.float(), g["loss"], rtol=2e-6, atol=2e-6)
    torch.testing.assert_close(lse.float(), g["lse"], rtol=2e-6, atol=2e-6)

    # same scalar objective as the generator: sum of the returned loss (+ z-loss term)
    d_loss = torch.ones_like(g["loss"], dtype=torch.float64)
    d_lse = None
    if o.get("z_loss"):
        t = g["targets"][..., shift:] if shift else g["targets"]
        keep = (t != -100).double()
        d_lse = g["z_coef"] * 2.0 * lse * keep / keep.sum()
    de, dc, db = O.linear_cross_entropy_grads(
        g["e"], g["c"], g["targets"], g["bias"], softcap=softcap, reduction=reduction, shift=shift,
        d_loss=d_loss, d_lse=d_lse,
    )
    torch.testing.assert_close(de.float(), g["de"], rtol=1e-4, atol=2e-6)
    torch.testing.assert_close(dc.float(), g["dc"], rtol=1e-4, atol=2e-6)
    if g["dbias"] is not None:
        torch.testing.assert_close(db.float(), g["dbias"], rtol=1e-4, atol=2e-6)
    if o.get("z_loss"):
        z = O.compute_z_loss(lse, g["targets"], shift)
        torch.testing.assert_close(z.float(), g["z_loss"], rtol=1e-5, atol=1e-6)


def test_z_loss_known_answers():
    # closed forms held by the reference's tests/test_compute_z_loss.py:39-44
    lse = torch.arange(1, 11, dtype=torch.float64)
    assert O.compute_z_loss(lse, reduction="sum").item() == pytest.approx(385.0)
    assert O.compute_z_loss(lse, reduction="mean").item() == pytest.approx(38.5)
    targets = torch.full((10,), -100)
    targets[3] = 1
    targets[5] = 2
    assert O.compute_z_loss(lse, targets, reduction="sum").item() == pytest.approx(4.0**2 + 6.0**2)
    assert O.compute_z_loss(lse, targets, reduction="mean").item() == pytest.approx((4.0**2 + 6.0**2) / 2)
    # with a shift the labels are read `shift` positions later
    lse9 = torch.arange(1, 10, dtype=torch.float64)
    assert O.compute_z_loss(lse9, targets, shift=1, reduction="sum").item() == pytest.approx(3.0**2 + 5.0**2)


@pytest.mark.parametrize("n,world", [(10, 3), (262144, 8), (7, 8), (1000, 1)])
def test_partition_known_answers(n, world):
    # property held by the reference's tests/test_vocab_parallel.py:153-165
    prev = 0
    sizes = []
    for r in range(world):
        s, t = O.partition_n_into_range(n, r, world)
        assert s == prev and t >= s
        sizes.append(t - s)
        prev = t
    assert prev == n
    assert max(sizes) - min(sizes) <= 1 and sizes == sorted(sizes, reverse=True)


def test_flat_valids_loop_and_vector_forms_agree():
    g = torch.Generator().manual_seed(3)
    t = torch.randint(0, 50, (3, 17), generator=g)
    t[torch.rand(3, 17, generator=g) < 0.3] = -100
    for shift in (0, 1, 4):
        assert torch.equal(O.flat_valids(t, -100, shift), O._flat_valids_fast(t, -100, shift))


@pytest.mark.parametrize("world", [2, 4])
def test_vocab_parallel_restatement_equals_unsharded(world):
    g = load_golden("bias_softcap")
    lse, nll = O.vocab_parallel_forward(g["e"], g["c"], g["targets"], world, g["bias"], softcap=20.0)
    v = O._flat_valids_fast(g["targets"], -100, 0)
    torch.testing.assert_close(lse.float(), g["lse"].reshape(-1)[v], rtol=2e-6, atol=2e-6)
    torch.testing.assert_close(nll.mean().float(), g["loss"], rtol=2e-6, atol=2e-6)
    # gradients: shard r's dC equals the slice of the full dC, the dE partials add up
    de_sum = 0
    for r in range(world):
        s, t = O.partition_n_into_range(g["c"].size(0), r, world)
        de, dc, db = O.linear_cross_entropy_grads(
            g["e"], g["c"][s:t], g["targets"], g["bias"][s:t], softcap=20.0, vocab_start=s, lse_override=lse
        )
        torch.testing.assert_close(dc.float(), g["dc"][s:t], rtol=1e-4, atol=2e-6)
        torch.testing.assert_close(db.float(), g["dbias"][s:t], rtol=1e-4, atol=2e-6)
        de_sum = de_sum + de
    torch.testing.assert_close(de_sum.float(), g["de"], rtol=1e-4, atol=2e-6)
