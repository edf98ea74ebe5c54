"""CPU oracle for the linear-cross-entropy path.  TEST INFRASTRUCTURE ONLY.

This file restates, in plain torch-on-CPU arithmetic (float64 by default), what the
reference computes on the path ``cut_cross_entropy.linear_cross_entropy`` forward +
backward.  It exists to check the CUDA kernels.  Nothing in the shipped package
imports it: only ``tests/``, ``__graft_entry__.smoke()`` and the CPU-baseline /
reference legs of ``bench.py`` may use it, and only as the checker or as the timed
CPU baseline, never as a compute path of the product.

Pinning.  The reference stores no golden vectors; its tests hold two kinds of known
answers (z-loss closed forms, ``tests/test_compute_z_loss.py:39-44``; the partition
rule, ``tests/test_vocab_parallel.py:153-165``) and otherwise compare against plain
PyTorch.  This oracle is pinned by
  (a) those known answers, and
  (b) fixtures under ``tests/golden/`` produced by running the reference's own
      ``impl="torch_compile"`` code (``cut_cross_entropy/torch_compile.py:18-117``)
      in the build container (script: ``tests/golden/make_golden.py``),
both checked by ``tests/test_oracle.py``.

Each function names the reference lines it follows.
"""

from __future__ import annotations

import math

import torch

IGNORE_INDEX = -100


# --------------------------------------------------------------------------- host helpers
def partition_n_into_range(n: int, rank: int, world_size: int) -> tuple[int, int]:
    """vocab_parallel/utils.py:9-13 — contiguous split, remainder to the low ranks."""
    q, r = divmod(n, world_size)
    start = rank * q + min(rank, r)
    stop = start + q + (1 if rank < r else 0)
    return start, stop


def handle_eps(filter_eps, dtype: torch.dtype):
    """utils.py:17-25 — ``"auto"`` is eps(dtype)/32."""
    if filter_eps is None:
        return None
    if isinstance(filter_eps, float):
        return filter_eps
    if filter_eps == "auto":
        return torch.finfo(dtype).eps / 32
    raise RuntimeError(f"Unknown eps {filter_eps=}")


def flat_valids(targets: torch.Tensor, ignore_index: int, shift: int) -> torch.Tensor:
    """utils.py:28-49 — rows r of the flattened ``e`` whose label ``targets.flatten()[r + shift]``
    is not ignored.  Always returns an int64 tensor (the reference returns ``None`` when
    shift == 0 and nothing is ignored, which is the identity list)."""
    targets = targets.contiguous()
    seq = targets.size(-1)
    flat = targets.reshape(-1)
    out = []
    for r in range(flat.numel()):
        pos_in_seq = r % seq
        if pos_in_seq + shift >= seq:
            continue
        if int(flat[r + shift]) != ignore_index:
            out.append(r)
    return torch.tensor(out, dtype=torch.int64)


def _flat_valids_fast(targets: torch.Tensor, ignore_index: int, shift: int) -> torch.Tensor:
    """Vectorised form of :func:`flat_valids` for large inputs (same definition)."""
    targets = targets.contiguous()
    seq = targets.size(-1)
    rows = torch.arange(targets.numel()).view(targets.shape)[..., : seq - shift]
    keep = targets[..., shift:] != ignore_index
    return rows[keep]


def scatter_none(batch_shape, valids: torch.Tensor, shift: int, values: torch.Tensor) -> torch.Tensor:
    """utils.py:52-61 — per-valid-row values placed at the label position, zeros elsewhere."""
    full = values.new_zeros((math.prod(batch_shape),))
    full[valids + shift] = values
    return full.view(*batch_shape)


def compute_z_loss(lse, targets=None, shift=0, ignore_index=IGNORE_INDEX, reduction="mean"):
    """utils.py:64-102 — ``lse**2``; ignored positions give 0 and the mean is over kept ones."""
    z = lse.pow(2)
    if targets is not None:
        shift = int(shift)
        if shift:
            targets = targets[..., shift:]
        keep = targets != ignore_index
        z = torch.where(keep, z, torch.zeros_like(z))
        if reduction == "mean":
            z = z * (z.numel() / keep.sum().to(z.dtype))
    if reduction == "mean":
        return z.mean()
    if reduction == "sum":
        return z.sum()
    if reduction == "none":
        return z
    raise ValueError(reduction)


# --------------------------------------------------------------------------- kernels, restated
def _logits(e_rows, c, bias, softcap, work_dtype):
    """cce_lse_forward.py:65-93 / torch_compile.py:29-35 — e.c^T, + bias, then tanh soft-cap."""
    x = e_rows.to(work_dtype) @ c.to(work_dtype).T
    if bias is not None:
        x = x + bias.to(work_dtype)
    if softcap is not None:
        x = torch.tanh(x / softcap) * softcap
    return x


def lse_forward(e, c, bias=None, valids=None, softcap=None, work_dtype=torch.float64, row_chunk=2048):
    """cce_lse_forward.py:99-117 — log-sum-exp over the vocabulary for each listed row of ``e``."""
    rows = e if valids is None else e[valids.long()]
    out = []
    for r0 in range(0, rows.size(0), row_chunk):
        out.append(torch.logsumexp(_logits(rows[r0 : r0 + row_chunk], c, bias, softcap, work_dtype), dim=-1))
    return torch.cat(out) if out else rows.new_zeros((0,), dtype=work_dtype)


def indexed_neg_dot(e, c, inds, bias=None, shift=0, valids=None, softcap=None, work_dtype=torch.float64,
                    vocab_start=0):
    """indexed_dot.py:52-85,150-151 — minus the (soft-capped) logit of each row's own label;
    0 where the label lies outside this shard (cce.py:130-133)."""
    n = e.size(0)
    rows = torch.arange(n) if valids is None else valids.long()
    t = inds.reshape(-1)[rows + shift].long() - vocab_start
    own = (t >= 0) & (t < c.size(0))
    ts = torch.where(own, t, torch.zeros_like(t))
    dot = (e[rows].to(work_dtype) * c[ts].to(work_dtype)).sum(-1)
    if bias is not None:
        dot = dot + bias[ts].to(work_dtype)
    if softcap is not None:
        dot = torch.tanh(dot / softcap) * softcap
    return torch.where(own, -dot, torch.zeros_like(dot))


def linear_cross_entropy(e, c, targets, bias=None, ignore_index=IGNORE_INDEX, softcap=None, reduction="mean",
                         shift=0, return_lse=False, work_dtype=torch.float64):
    """linear_cross_entropy.py:103-198 with cce.py:78-160 — loss (and lse) of the whole path.

    ``e`` is ``(..., D)``, ``targets`` is ``(...)``.  Returns tensors in ``work_dtype`` with the
    reference's shapes: scalar loss, or ``(..., T - shift)`` for ``reduction="none"`` and for lse.
    """
    shift = int(shift)
    batch_shape = tuple(targets.shape)
    valids = _flat_valids_fast(targets, ignore_index, shift)
    e2 = e.reshape(-1, e.size(-1))
    lse = lse_forward(e2, c, bias, valids, softcap, work_dtype)
    nll = lse + indexed_neg_dot(e2, c, targets, bias, shift, valids, softcap, work_dtype)
    if reduction == "mean":
        loss = nll.mean()
    elif reduction == "sum":
        loss = nll.sum()
    elif reduction == "none":
        loss = scatter_none(batch_shape, valids, shift, nll)
        if shift:
            loss = loss[..., shift:]
    else:
        raise ValueError(f"Unknown reduction {reduction}")
    if not return_lse:
        return loss
    lse_full = scatter_none(batch_shape, valids, shift, lse)
    if shift:
        lse_full = lse_full[..., shift:]
    return loss, lse_full


def linear_cross_entropy_grads(e, c, targets, bias=None, ignore_index=IGNORE_INDEX, softcap=None,
                               reduction="mean", shift=0, d_loss=None, d_lse=None, work_dtype=torch.float64,
                               vocab_start=0, lse_override=None, row_chunk=1024):
    """cce_backward.py:182-256 — closed-form gradients, no autograd.

    For each valid row i with label t and upstream weights g_i (of the loss) and l_i (of lse):
        dS[i, v] = softmax[i, v] * (g_i + l_i) - [v == t] * g_i        (cce_backward.py:196-248)
        dS *= 1 - (capped/softcap)^2  when soft-capping                 (tl_utils.py:31-34)
        dE[i] = dS[i] @ c,  dC = dS^T @ e,  dBias = colsum(dS)          (cce_backward.py:253-310)
    ``g_i = grad_scale * d_loss`` with grad_scale = 1/B for mean (cce.py:177-186).  ``d_loss`` is a
    scalar, or for ``reduction="none"`` has the shape of the returned loss; ``d_lse`` has the shape
    of the returned lse.  ``vocab_start`` / ``lse_override`` restate one vocab-parallel rank
    (cce.py:193-205): labels outside the shard never match, and the softmax uses the global lse.
    Returns (dE like e, dC like c, dBias or None) in ``work_dtype``.
    """
    shift = int(shift)
    batch_shape = tuple(targets.shape)
    n_total = math.prod(batch_shape)
    valids = _flat_valids_fast(targets, ignore_index, shift)
    B = valids.numel()
    D = e.size(-1)
    e2 = e.reshape(-1, D)
    flat_t = targets.reshape(-1)

    def full_len(x):  # gradient given in the shape of a returned tensor -> one value per flat position
        if x is None:
            return None
        x = x.to(work_dtype)
        if x.numel() == 1:
            return x.reshape(())
        if shift:
            pad = x.new_zeros(batch_shape)
            pad[..., shift:] = x
            x = pad
        return x.reshape(-1)

    d_loss = torch.ones((), dtype=work_dtype) if d_loss is None else full_len(d_loss)
    d_lse_f = full_len(d_lse)
    grad_scale = 1.0 / max(B, 1) if reduction == "mean" else 1.0

    lse = lse_override if lse_override is not None else lse_forward(e2, c, bias, valids, softcap, work_dtype)
    dE = torch.zeros(n_total, D, dtype=work_dtype)
    dC = torch.zeros(c.shape, dtype=work_dtype)
    dB = torch.zeros(c.size(0), dtype=work_dtype) if bias is not None else None
    cw = c.to(work_dtype)
    for r0 in range(0, B, row_chunk):
        rows = valids[r0 : r0 + row_chunk]
        x = _logits(e2[rows], c, bias, softcap, work_dtype)
        p = torch.exp(x - lse[r0 : r0 + row_chunk].to(work_dtype)[:, None])
        t = flat_t[rows + shift].long() - vocab_start
        own = (t >= 0) & (t < c.size(0))
        g = grad_scale * (d_loss if d_loss.dim() == 0 else d_loss[rows + shift])
        g = g.expand(rows.numel()) if g.dim() == 0 else g
        l = torch.zeros_like(g) if d_lse_f is None else (d_lse_f.expand(n_total)[rows + shift] if d_lse_f.dim() == 0 else d_lse_f[rows + shift])
        ds = p * (g + l)[:, None]
        idx = torch.nonzero(own).squeeze(1)
        ds[idx, t[idx]] -= g[idx]
        if softcap is not None:
            ds = ds * (1 - (x / softcap) ** 2)
        dE[rows] = ds @ cw
        dC += ds.T @ e2[rows].to(work_dtype)
        if dB is not None:
            dB += ds.sum(0)
    return dE.view(*e.shape), dC, dB


# --------------------------------------------------------------------------- vocab parallelism
def vocab_parallel_forward(e, c, targets, world_size, bias=None, softcap=None, shift=0,
                           ignore_index=IGNORE_INDEX, work_dtype=torch.float64):
    """vocab_parallel/utils.py:47-65 with cce.py:94-137 — per-shard lse and correct logit,
    merged as max + log(sum exp(lse_r - max)) and a plain sum.  Returns (lse, nll) per valid row."""
    valids = _flat_valids_fast(targets, ignore_index, int(shift))
    e2 = e.reshape(-1, e.size(-1))
    lses, dots = [], []
    for r in range(world_size):
        s, t = partition_n_into_range(c.size(0), r, world_size)
        b = bias[s:t] if bias is not None else None
        lses.append(lse_forward(e2, c[s:t], b, valids, softcap, work_dtype))
        dots.append(indexed_neg_dot(e2, c[s:t], targets, b, int(shift), valids, softcap, work_dtype, vocab_start=s))
    stack = torch.stack(lses)
    mx = stack.max(0).values
    lse = mx + torch.log(torch.exp(stack - mx).sum(0))
    return lse, lse + torch.stack(dots).sum(0)
