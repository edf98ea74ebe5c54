"""Parity and size-independent properties at the full sizes of the benchmark configurations.

The CPU oracle would need minutes at these sizes, so the yardstick here is a plain PyTorch float32
computation on the GPU, in row chunks (the inputs are bf16, so their products are exact in
float32 and in TF32): log-sum-exp and loss for every row, dE for a sample of rows, dC for a
sample of classifier rows (label rows included).  Tolerances are the project's: loss 1e-3
relative, lse 2e-3 absolute, gradients cosine >= 0.9999 and max error <= 1e-2 of max|ref|.
"""

from __future__ import annotations

import os

import pytest
import torch

import bench

pytestmark = pytest.mark.gpu
DEV = "cuda"
IGNORE = -100


def _ref_forward(e2, c, bias, softcap, rows, chunk=4096):
    """float32 logits statistics for the listed rows: lse [len(rows)]."""
    out = []
    cf = c.float()
    for r0 in range(0, rows.numel(), chunk):
        x = e2[rows[r0 : r0 + chunk]].float() @ cf.T
        if bias is not None:
            x += bias.float()
        if softcap is not None:
            x = torch.tanh(x / softcap) * softcap
        out.append(torch.logsumexp(x, -1))
        del x
    return torch.cat(out)


def _run(cfg_name, impl=None):
    from cut_cross_entropy import linear_cross_entropy
    from cut_cross_entropy.utils import compute_z_loss

    cfg = bench.CONFIGS[cfg_name]
    e, c, bias, targets = bench.make_inputs(cfg, DEV)
    e.requires_grad_(True)
    c.requires_grad_(True)
    if bias is not None:
        bias.requires_grad_(True)
    kw = dict(cfg["kw"])
    if impl:
        kw["impl"] = impl
    loss, lse = linear_cross_entropy(e, c, targets, bias=bias, return_lse=True, **kw)
    total = loss
    z = cfg.get("z_loss")
    if z:
        total = total + z * compute_z_loss(lse, targets, kw.get("shift", 0))
    total.backward()
    return cfg, kw, e, c, bias, targets, loss.detach(), lse.detach()


def _check_grad(got, want, what, slack=None, rel=1e-2, min_cos=0.9999):
    """|got - want| <= rel * max|want| (+ slack, the element-wise bound on what the gradient filter
    is allowed to drop) and, when nothing is filtered, cosine similarity >= min_cos."""
    got, want = got.float(), want.float()
    scale = want.abs().max().item()
    excess = (got - want).abs() - rel * scale
    if slack is not None:
        excess = excess - slack
    assert excess.max().item() <= 0, f"{what}: error exceeds the allowance by {excess.max().item():.3e} (scale {scale:.3e})"
    if slack is None:
        cos = torch.nn.functional.cosine_similarity(got.flatten(), want.flatten(), dim=0).item()
        assert cos >= min_cos, f"{what}: cosine {cos}"


@pytest.mark.parametrize("cfg_name", ["gemma2-2b-head", "llama3-8b-head-shift", "gemma2-9b-head-softcap-zloss",
                                      "qwen25-7b-head-long-kahan", "vocab-parallel-head"])  # fmt: skip
def test_full_size_against_float32(cfg_name):
    torch.backends.cuda.matmul.allow_tf32 = True  # exact for bf16-valued operands
    cfg, kw, e, c, bias, targets, loss, lse = _run(cfg_name)
    shift, softcap, reduction = kw.get("shift", 0), kw.get("softcap"), kw.get("reduction", "mean")
    D = e.size(-1)
    e2 = e.detach().reshape(-1, D)
    tflat = targets.reshape(-1)
    seq = targets.size(-1)
    all_rows = torch.arange(tflat.numel(), device=DEV).view(targets.shape)[..., : seq - shift].reshape(-1)
    labels = tflat[all_rows + shift]
    keep = labels != IGNORE
    rows, labels = all_rows[keep], labels[keep]
    B = rows.numel()

    # forward: every row
    ref_lse = _ref_forward(e2, c.detach(), None if bias is None else bias.detach(), softcap, rows)
    tgt = (e2[rows].float() * c.detach()[labels].float()).sum(-1)
    if bias is not None:
        tgt = tgt + bias.detach()[labels].float()
    if softcap is not None:
        tgt = torch.tanh(tgt / softcap) * softcap
    nll = ref_lse - tgt
    ref_loss = nll.mean() if reduction == "mean" else nll.sum()
    assert abs(loss.item() - ref_loss.item()) <= 1e-3 * abs(ref_loss.item())
    lse_flat = lse.reshape(-1)  # positions: label positions; rows map to (row + shift) minus the dropped columns
    lse_full = torch.zeros(tflat.numel(), device=DEV)
    lse_view = lse_full.view(targets.shape)
    lse_view[..., shift:] = lse
    got_lse = lse_full[rows + shift]
    assert (got_lse - ref_lse).abs().max().item() <= 2e-3
    assert lse_flat.numel() == all_rows.numel()

    # upstream weights of this objective
    g = torch.full((B,), 1.0 / B if reduction == "mean" else 1.0, device=DEV)
    dl = torch.zeros(B, device=DEV)
    if cfg.get("z_loss"):
        dl = cfg["z_loss"] * 2.0 * ref_lse / B

    torch.backends.cuda.matmul.allow_tf32 = False
    gen = torch.Generator(device=DEV).manual_seed(0)
    # dE for a sample of rows
    pick = torch.randperm(B, device=DEV, generator=gen)[:192]
    x = e2[rows[pick]].float() @ c.detach().float().T
    if bias is not None:
        x += bias.detach().float()
    if softcap is not None:
        x = torch.tanh(x / softcap) * softcap
    prob = torch.exp(x - ref_lse[pick, None])
    ds = prob * (g[pick] + dl[pick])[:, None]
    ds[torch.arange(pick.numel(), device=DEV), labels[pick]] -= g[pick]
    if softcap is not None:
        ds = ds * (1 - (x / softcap) ** 2)
    # The filtered variants may drop any entry whose |softmax - onehot| < eps (never the label's):
    # the sum of |entry * c| over those entries bounds the difference from the exact gradient.
    # With these near-uniform synthetic softmaxes (every probability ~ 1/V << eps) that is almost
    # the whole non-label part of dE, so the allowance is not small here; on the exact variants it is 0.
    eps = 2.0**-12
    filt_e = kw["impl"] in ("cce", "cce_kahan", "cce_kahan_full_c")
    filt_c = kw["impl"] in ("cce", "cce_kahan", "cce_kahan_full_e")
    slack = None
    if filt_e:
        droppable = ds.abs() * (prob < eps)
        droppable[torch.arange(pick.numel(), device=DEV), labels[pick]] = 0
        slack = droppable @ c.detach().float().abs()
    _check_grad(e.grad.reshape(-1, D)[rows[pick]], ds @ c.detach().float(), "dE (sampled rows)", slack)
    del x, ds, prob

    # dC (and dBias) for a sample of classifier rows: some that are labels, some arbitrary
    cols = torch.cat([labels[pick[:64]], torch.randint(0, c.size(0), (192,), device=DEV, generator=gen)]).unique()
    acc = torch.zeros(cols.numel(), D, device=DEV)
    accb = torch.zeros(cols.numel(), device=DEV)
    slack_c = torch.zeros(cols.numel(), D, device=DEV) if filt_c else None
    for r0 in range(0, B, 8192):
        rr = rows[r0 : r0 + 8192]
        x = e2[rr].float() @ c.detach()[cols].float().T
        if bias is not None:
            x += bias.detach()[cols].float()
        if softcap is not None:
            x = torch.tanh(x / softcap) * softcap
        prob = torch.exp(x - ref_lse[r0 : r0 + 8192, None])
        ds = prob * (g[r0 : r0 + 8192] + dl[r0 : r0 + 8192])[:, None]
        hit = labels[r0 : r0 + 8192, None] == cols[None, :]
        ds -= hit * g[r0 : r0 + 8192, None]
        if softcap is not None:
            ds = ds * (1 - (x / softcap) ** 2)
        acc += ds.T @ e2[rr].float()
        accb += ds.sum(0)
        if filt_c:
            slack_c += (ds.abs() * ((prob < eps) & ~hit)).T @ e2[rr].float().abs()
    _check_grad(c.grad[cols], acc, "dC (sampled classifier rows)", slack_c)
    if bias is not None:
        _check_grad(bias.grad[cols], accb, "dBias (sampled)")


def test_full_size_properties():
    """Size-independent checks at the Gemma-2-2B head size: linearity in the upstream gradient,
    mean = sum / count, independence of the chunking of the vocabulary, agreement of the unfiltered
    products of the half-filtered variants with the exact one."""
    from cut_cross_entropy import linear_cross_entropy

    cfg = bench.CONFIGS["gemma2-2b-head"]
    e, c, _, targets = bench.make_inputs(cfg, DEV)
    e.requires_grad_(True)
    c.requires_grad_(True)
    n_valid = int((targets != IGNORE).sum())

    def grads(impl, scale=1.0, reduction="mean"):
        e.grad = c.grad = None
        loss = linear_cross_entropy(e, c, targets, impl=impl, reduction=reduction)
        (loss * scale).backward()
        return loss.detach(), e.grad.clone(), c.grad.clone()

    l1, de1, dc1 = grads("cce_exact")
    l2, de2, dc2 = grads("cce_exact", scale=2.0)
    torch.testing.assert_close(de2.float(), 2 * de1.float(), rtol=0, atol=0)
    torch.testing.assert_close(dc2.float(), 2 * dc1.float(), rtol=0, atol=0)
    ls, des, dcs = grads("cce_exact", reduction="sum")
    torch.testing.assert_close(ls / n_valid, l1, rtol=1e-6, atol=0)
    _check_grad(des / n_valid, de1, "dE sum/count vs mean")

    # a smaller logit-gradient buffer means more, narrower vocabulary chunks: dC is the same numbers,
    # dE differs only by the order of its fp32 partial sums
    os.environ["CCE_B200_GBUF_MB"] = "96"
    try:
        l3, de3, dc3 = grads("cce_exact")
    finally:
        del os.environ["CCE_B200_GBUF_MB"]
    torch.testing.assert_close(l3, l1, rtol=0, atol=0)
    torch.testing.assert_close(dc3, dc1, rtol=0, atol=0)
    _check_grad(de3, de1, "dE under a different chunking")

    # Half-filtered variants: the product that is NOT filtered must match the exact one at the stated
    # tolerances.  (What a filtered product may differ by is bounded by the reference's own filter on
    # the same GPU and tensors in tests/test_gpu_reference.py, and by the element-wise droppable mass
    # in test_full_size_against_float32.)
    for impl in ("cce_kahan_full_c", "cce_kahan_full_e"):
        lf, def_, dcf = grads(impl)
        torch.testing.assert_close(lf, l1, rtol=0, atol=0)
        if impl == "cce_kahan_full_e":
            _check_grad(def_, de1, f"dE {impl} vs exact")
        else:
            _check_grad(dcf, dc1, f"dC {impl} vs exact")
    # the fully filtered variant must give identical results with a tile pool too small for one pass
    lf, de_a, dc_a = grads("cce")
    os.environ["CCE_B200_GBUF_MB"] = "64"
    try:
        lf2, de_b, dc_b = grads("cce")
    finally:
        del os.environ["CCE_B200_GBUF_MB"]
    torch.testing.assert_close(dc_b, dc_a, rtol=0, atol=0)
    _check_grad(de_b, de_a, "dE with a small tile pool")


@pytest.mark.parametrize("cfg_name,world", [("gemma2-2b-head", 4), ("gemma2-2b-head", 8), ("vocab-parallel-head", 8)])
def test_full_size_vocabulary_shards_on_one_gpu(cfg_name, world):
    """The per-rank work of `bench.py --gpus N` (Gemma-2-2B head, and the 32768 x 4096 x 262144
    vocab-parallel head split 8 ways), shard after shard on one GPU, with the block-list backward each rank runs (per-shard tile maxima, global lse):
    the shards' log-sum-exps merge to the unsharded one, each shard's dC is the matching slice of
    the unsharded dC bit for bit (the same tiles, the same order of row blocks), and the fp32 dE
    partial sums add up to the unsharded dE within its bf16 rounding."""
    from cut_cross_entropy.cce_backward import cce_backward_kernel
    from cut_cross_entropy.cce_lse_forward import cce_lse_forward_kernel
    from cut_cross_entropy.utils import TensorInfo, _build_flat_valids
    from cut_cross_entropy.vocab_parallel import partition_n_into_range

    cfg = bench.CONFIGS[cfg_name]
    e, c, _, targets = bench.make_inputs(cfg, DEV)
    t = targets.flatten()
    valids = _build_flat_valids(targets, IGNORE, 0)  # None when no label is ignored
    B, V = (e.size(0) if valids is None else valids.numel()), c.size(0)
    info = TensorInfo(torch.bfloat16, True)
    do = torch.ones((), device=DEV)
    eps = 2.0**-12

    def bwd(cs, lse, tile_max, start):
        return cce_backward_kernel(do=do, dlse=None, e=e, e_info=info, c=cs, c_info=info, bias=None, bias_info=None,
                                   lse=lse, valids=valids, softcap=None, filter_eps=eps, targets=t,
                                   grad_scale=1.0 / B, vocab_start=start, reduce_e_grad=False,
                                   tile_max=tile_max)  # fmt: skip

    lse_full, tm_full = cce_lse_forward_kernel(e, c, None, valids, return_tile_max=True)
    de_full, dc_full, _ = bwd(c, lse_full, tm_full, 0)

    parts = []
    for r in range(world):
        s0, s1 = partition_n_into_range(V, r, world)
        cs = c[s0:s1].contiguous()
        lse_r, tm_r = cce_lse_forward_kernel(e, cs, None, valids, return_tile_max=True)
        parts.append((s0, s1, cs, lse_r, tm_r))
    lse = torch.logsumexp(torch.stack([p[3] for p in parts]), 0)
    torch.testing.assert_close(lse, lse_full, rtol=0, atol=1e-5)

    de_sum = torch.zeros(de_full.shape, dtype=torch.float32, device=DEV)
    for s0, s1, cs, _, tm_r in parts:
        de, dc, _ = bwd(cs, lse_full, tm_r, s0)
        if s0 % 256 == 0:  # the shard's 256-column tiles are tiles of the unsharded problem
            torch.testing.assert_close(dc, dc_full[s0:s1], rtol=0, atol=0)
        else:
            _check_grad(dc, dc_full[s0:s1], f"dC of shard [{s0}, {s1})")
        de_sum += de.float()
        del de, dc
    _check_grad(de_sum, de_full, "sum of the shards' dE")
