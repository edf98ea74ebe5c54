"""Vocabulary parallelism: each rank holds a contiguous slice of the classifier rows.

Reference behaviour followed here: ``cut_cross_entropy/vocab_parallel/utils.py:9-76``.
The reference merges the per-rank statistics with three small all-reduces (max,
sum of exponentials, correct logit); here the two per-token vectors travel
together in ONE all-gather and are merged locally, which is the same arithmetic
with one exchange instead of three.  ``dE`` is summed across ranks in fp32, as in
the reference (``utils.py:68-76``).
"""

from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist


def partition_n_into_range(n: int, rank: int, world_size: int) -> tuple[int, int]:
    """Contiguous ``[start, stop)`` slice of ``range(n)`` for ``rank``; the first
    ``n % world_size`` ranks get one extra element."""
    base, extra = divmod(n, world_size)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


@dataclass
class VocabParallelOptions:
    """Configure vocab-parallel loss computation.

    :param start: first vocabulary index held by this rank.
    :param stop: one past the last vocabulary index held by this rank.
    :param group: process group that spans the vocabulary shards.
    :param reduce_e_grad: sum the gradient of ``e`` over the group (usually wanted;
        switch off if the surrounding framework reduces it itself).
    """

    start: int
    stop: int
    group: "dist.ProcessGroup | None" = None
    reduce_e_grad: bool = True

    @classmethod
    def from_vocab(
        cls, vocab_size: int, group: "dist.ProcessGroup | None" = None, reduce_e_grad: bool = True
    ) -> "VocabParallelOptions":
        start, stop = partition_n_into_range(vocab_size, dist.get_rank(group), dist.get_world_size(group))
        return cls(start, stop, group, reduce_e_grad)


def vp_gather_stats(local: torch.Tensor, pg: "dist.ProcessGroup | None") -> torch.Tensor:
    """All-gather of the ranks' ``[2, B]`` float32 blocks (local log-sum-exp, minus the local
    correct-token logit) into ``[world, 2, B]``: the forward's one exchange, merged afterwards by
    the tail kernel (``cce_b200_loss_tail``)."""
    world = dist.get_world_size(pg)
    assert local.dim() == 2 and local.size(0) == 2 and local.dtype == torch.float32
    local = local.contiguous()
    out = local.new_empty((world, 2, local.size(1)))
    dist.all_gather_into_tensor(out.view(world * 2, local.size(1)), local, group=pg)
    return out


def vp_merge_forward(
    local_lse: torch.Tensor, local_neg_dot: torch.Tensor, pg: "dist.ProcessGroup | None"
) -> tuple[torch.Tensor, torch.Tensor]:
    """Merge per-rank ``(lse, -correct_logit)`` vectors into their global values.

    One all-gather of a ``[2, B]`` float32 block per rank; then
    ``lse = logsumexp_r(lse_r)`` and ``neg_dot = sum_r neg_dot_r`` (only the rank
    that owns a label contributes a non-zero correct logit).  Equivalent to
    ``vp_reduce_lse`` + ``vp_reduce_correct_logit`` of the reference.
    """
    world = dist.get_world_size(pg)
    mine = torch.stack((local_lse.float(), local_neg_dot.float())).contiguous()
    flat = mine.new_empty((world * 2, mine.size(1)))  # rank r fills rows 2r, 2r+1
    dist.all_gather_into_tensor(flat, mine, group=pg)
    gathered = flat.view(world, 2, mine.size(1))
    lse = torch.logsumexp(gathered[:, 0], dim=0)
    neg_dot = gathered[:, 1].sum(dim=0)
    return lse, neg_dot


def vp_reduce_e_grad_cast(
    e_grad_f32: torch.Tensor, out_dtype: torch.dtype, pg: "dist.ProcessGroup | None"
) -> torch.Tensor:
    """Sum of the partial ``dE`` over the group in fp32, returned in ``out_dtype``: a reduce-scatter
    of the fp32 partial sums, a cast of this rank's slice, and an all-gather of the 16-bit slices.
    Same arithmetic as an fp32 all-reduce followed by the cast (reference
    ``vocab_parallel/utils.py:68-76``) with a quarter less traffic, since the second half of the
    exchange moves 2-byte values."""
    assert e_grad_f32.dtype == torch.float32 and e_grad_f32.is_contiguous()
    world = dist.get_world_size(pg)
    flat = e_grad_f32.view(-1)
    n = flat.numel()
    per = -(-n // world)
    if per * world != n:  # pad to a multiple of the group size
        padded = flat.new_zeros(per * world)
        padded[:n] = flat
        flat = padded
    mine = flat.new_empty(per)
    dist.reduce_scatter_tensor(mine, flat, group=pg)
    mine_lp = mine.to(out_dtype)
    out = mine_lp.new_empty(per * world)
    dist.all_gather_into_tensor(out, mine_lp, group=pg)
    return out[:n].view(e_grad_f32.shape)


def vp_reduce_e_grad_(e_grad_f32: torch.Tensor, pg: "dist.ProcessGroup | None") -> torch.Tensor:
    """In-place fp32 sum of the partial ``dE`` over the group."""
    assert e_grad_f32.dtype == torch.float32
    dist.all_reduce(e_grad_f32, group=pg)
    return e_grad_f32


# ---- the reference's own helper names (cut_cross_entropy/vocab_parallel/utils.py:47-103), kept for
# callers that import them; the loss path above needs one exchange where these take three.
def vp_reduce_lse(vp_lse: torch.Tensor, pg: "dist.ProcessGroup | None") -> torch.Tensor:
    """Global log-sum-exp from per-rank ones: max all-reduce, then sum all-reduce of the rescaled terms."""
    lse_max = vp_lse.clone()
    dist.all_reduce(lse_max, op=dist.ReduceOp.MAX, group=pg)
    scaled = (vp_lse - lse_max).exp()
    dist.all_reduce(scaled, group=pg)
    return lse_max + scaled.log()


def vp_reduce_correct_logit(
    vp_correct_logit: torch.Tensor, pg: "dist.ProcessGroup | None", dtype: torch.dtype | None = None
) -> torch.Tensor:
    """Sum over the ranks of the correct-token logit (zero on ranks that do not own the label)."""
    out = vp_correct_logit.to(dtype=dtype, copy=True)
    dist.all_reduce(out, group=pg)
    return out


def vp_reduce_e_grad(e_grad: torch.Tensor, pg: "dist.ProcessGroup | None") -> torch.Tensor:
    """Sum of the partial ``dE`` over the ranks, accumulated in float32, returned in ``e_grad``'s dtype."""
    return vp_reduce_e_grad_(e_grad.to(dtype=torch.float32, copy=True), pg).type_as(e_grad)


class _ReduceEGradHook(torch.autograd.Function):
    @staticmethod
    def forward(ctx, e: torch.Tensor, pg: "dist.ProcessGroup | None" = None) -> torch.Tensor:
        ctx.pg = pg
        return e

    @staticmethod
    def backward(ctx, e_grad: torch.Tensor) -> tuple[torch.Tensor, None]:
        return vp_reduce_e_grad(e_grad, ctx.pg), None


def vp_reduce_e_grad_hook(e: torch.Tensor, vocab_parallel_options: VocabParallelOptions) -> torch.Tensor:
    """Identity in the forward pass; sums the gradient of ``e`` over the group in the backward pass
    (when ``reduce_e_grad`` is set)."""
    if vocab_parallel_options.reduce_e_grad:
        return _ReduceEGradHook.apply(e, vocab_parallel_options.group)
    return e
