"""Vocabulary ordering of the filtered backward, and the forward by-products it needs.

Reference behaviour: ``cut_cross_entropy/cce.py:43-45,171-174`` (argsort of the mean logit),
``cce_lse_forward.py:95-97`` (the mean logit), ``cce_backward.py:154-155`` (tiles follow the order).
"""

from __future__ import annotations

import math

import pytest
import torch

from conftest import planted_inputs

pytestmark = pytest.mark.gpu
DEV = "cuda"
LOG2E = 1.4426950408889634


def _scattered_hot(N, V, D, hot, seed=0, gain=8.0, bias=False):
    """Near-uniform softmax except for `hot` vocabulary entries at random positions that have a
    large logit for every row (the case where natural vocabulary order defeats the tile filter)."""
    g = torch.Generator().manual_seed(seed)
    u = torch.randn(D, generator=g)
    u /= u.norm()
    e = (torch.randn(N, D, generator=g) + 4.0 * u).bfloat16()
    c = torch.randn(V, D, generator=g) * 0.02
    idx = torch.randperm(V, generator=g)[:hot]
    c[idx] += u * (gain / 4.0)
    c = c.bfloat16()
    t = torch.randint(0, V, (N,), generator=g)
    t[torch.randperm(N, generator=g)[: N // 10]] = -100
    b = (torch.randn(V, generator=g) * 0.02).float() if bias else None
    mv = lambda x: None if x is None else x.to(DEV)
    return mv(e), mv(c), mv(b), mv(t)


def _logits(e, c, bias, softcap):
    x = e.float() @ c.float().T
    if bias is not None:
        x = x + bias.float()
    if softcap is not None:
        x = torch.tanh(x / softcap) * softcap
    return x


def _decode_keys(k: torch.Tensor) -> torch.Tensor:
    k = k.to(torch.int32)
    return torch.where(k >= 0, k, k ^ 0x7FFFFFFF).view(torch.float32)


@pytest.mark.parametrize("softcap", [None, 20.0])
@pytest.mark.parametrize("has_bias", [False, True])
@pytest.mark.parametrize("shape", [(256, 512, 128), (252, 507, 123), (700, 2500, 192)])
def test_forward_by_products_for_the_ordering(shape, has_bias, softcap):
    from cut_cross_entropy.cce_lse_forward import cce_lse_forward_kernel

    N, V, D = shape
    e, c, bias, t = planted_inputs(N, V, D, torch.bfloat16, DEV, bias=has_bias)
    valids = torch.arange(0, N, 3, device=DEV, dtype=torch.int32)
    for rows in (None, valids):
        lse, logit_avg, col_max = cce_lse_forward_kernel(e, c, bias, rows, softcap, return_logit_avg=True,
                                                         return_col_max=True)
        er = e if rows is None else e[rows.long()]
        x = _logits(er, c, bias, softcap)
        torch.testing.assert_close(lse, torch.logsumexp(x, -1), rtol=1e-5, atol=2e-5)
        # largest logit of every column over the rows, in log2 units
        torch.testing.assert_close(_decode_keys(col_max), x.max(0).values * LOG2E, rtol=1e-5, atol=1e-4)
        # the integer keys sort like the maxima
        assert torch.equal(torch.argsort(col_max, stable=True), torch.argsort(_decode_keys(col_max), stable=True))
        # mean logit: exact without soft-capping, the cap of the mean with it
        mean_uncapped = _logits(er, c, bias, None).mean(0)
        want = mean_uncapped if softcap is None else torch.tanh(mean_uncapped / softcap) * softcap
        torch.testing.assert_close(logit_avg, want, rtol=1e-4, atol=1e-4)


def _exact_and_droppable(e, c, bias, t, softcap, eps):
    """float32 gradients of the mean loss, and the element-wise mass the filter may drop."""
    keep = (t != -100).nonzero().squeeze(1)
    x = _logits(e[keep], c, bias, softcap)
    lse = torch.logsumexp(x, -1)
    p = torch.exp(x - lse[:, None])
    ds = p.clone()
    ds[torch.arange(keep.numel(), device=DEV), t[keep]] -= 1
    ds /= keep.numel()
    small = p < eps
    small[torch.arange(keep.numel(), device=DEV), t[keep]] = False
    if softcap is not None:
        ds = ds * (1 - (x / softcap) ** 2)
    de = torch.zeros(e.shape, device=DEV)
    de[keep] = ds @ c.float()
    dc = ds.T @ e[keep].float()
    slack_e = torch.zeros(e.shape, device=DEV)
    slack_e[keep] = (ds.abs() * small) @ c.float().abs()
    slack_c = (ds.abs() * small).T @ e[keep].float().abs()
    return de, dc, slack_e, slack_c


@pytest.mark.parametrize("mode", ["max", "mean"])
@pytest.mark.parametrize("softcap,has_bias", [(None, False), (30.0, True)])
def test_ordered_backward_stays_within_the_filter_bound_and_recomputes_fewer_tiles(mode, softcap, has_bias):
    from cut_cross_entropy import _native, linear_cross_entropy
    from cut_cross_entropy import cce as cce_mod

    N, V, D, hot = 1024, 131072, 128, 1024
    e, c, bias, t = _scattered_hot(N, V, D, hot, bias=has_bias)
    e.requires_grad_(True)
    c.requires_grad_(True)
    eps = 2.0**-12
    de_x, dc_x, slack_e, slack_c = _exact_and_droppable(e.detach(), c.detach(), bias, t, softcap, eps)
    L = _native.lib()
    counts = torch.zeros(3, dtype=torch.int32, device=DEV)
    survival = {}
    grads = {}
    for name in ("off", mode):
        prev = cce_mod.set_vocab_ordering(name)
        try:
            e.grad = c.grad = None
            counts.zero_()
            L.cce_b200_profile_tile_counts(counts.data_ptr())
            loss = linear_cross_entropy(e, c, t, bias=bias, softcap=softcap, impl="cce")
            loss.backward()
            torch.cuda.synchronize()
        finally:
            L.cce_b200_profile_tile_counts(None)
            cce_mod.set_vocab_ordering(prev)
        n_act, n_all, _ = counts.tolist()
        assert n_all == math.ceil(int((t != -100).sum()) / 128) * (V // 256)
        survival[name] = n_act / n_all
        grads[name] = (e.grad.float().clone(), c.grad.float().clone())
        for got, want, slack, what in ((grads[name][0], de_x, slack_e, "dE"), (grads[name][1], dc_x, slack_c, "dC")):
            excess = (got - want).abs() - 1e-2 * want.abs().max() - slack
            assert excess.max().item() <= 0, f"{what} with ordering {name}: beyond the filter bound by {excess.max().item():.3e}"
    # 1024 hot entries touch ~86 % of the 512 tiles of 256 in natural order; sorted, they fill four
    assert survival["off"] > 0.6, survival
    assert survival[mode] < 0.5 * survival["off"], survival


@pytest.mark.parametrize("mode", ["max", "mean"])
@pytest.mark.parametrize("name", ["multi_band", "odd_shapes", "shift2_none_zloss"])
def test_golden_fixtures_with_a_vocabulary_order(name, mode):
    """The reference-made fixtures again, with the backward walking a sorted vocabulary (and, for the
    largest one, a tile pool that needs several passes)."""
    import os

    from cut_cross_entropy import cce as cce_mod
    from test_gpu_loss import test_golden_fixtures

    prev = cce_mod.set_vocab_ordering(mode)
    if name == "multi_band":
        os.environ["CCE_B200_GBUF_MB"] = "1"
    try:
        test_golden_fixtures(name, "cce")
    finally:
        cce_mod.set_vocab_ordering(prev)
        os.environ.pop("CCE_B200_GBUF_MB", None)
