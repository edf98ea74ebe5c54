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


def vp_reduce_e_grad_(e_grad_f32: torch.Tensor, pg: "dist.ProcessGroup | None") -> torch.Tensor:
    """In-place fp32 sum of the partial ``dE`` over the group."""
    assert e_grad_f32.dtype == torch.float32
    dist.all_reduce(e_grad_f32, group=pg)
    return e_grad_f32
