"""Tail of the forward pass: from per-row statistics to the returned loss (and log-sum-exp).

One launch of ``cce_b200_loss_tail`` does what the reference spreads over several PyTorch
operations: the merge of the per-rank statistics under vocab parallelism
(``cut_cross_entropy/vocab_parallel/utils.py:47-65``), ``nll = lse - correct_logit`` and its
mean/sum (``cut_cross_entropy/cce.py:139-160``), and the scatter back to the batch shape for
``reduction="none"`` and ``return_lse`` (``cut_cross_entropy/utils.py:52-61``).
"""

from __future__ import annotations

import torch

from . import _native

_REDUCTION_CODE = {"mean": 0, "sum": 1, "none": 2}


def loss_tail_kernel(
    stats: torch.Tensor,
    valids: torch.Tensor | None,
    shift: int,
    batch_shape: torch.Size,
    reduction: str,
    return_lse: bool,
    want_lse_rows: bool,
    n_rows_dev: torch.Tensor | None = None,
) -> tuple[torch.Tensor, torch.Tensor | None, torch.Tensor | None]:
    """``stats`` is ``[world, 2, B]`` float32: per vocabulary shard the log-sum-exp of every valid
    row and minus its correct-token logit (``world = 1`` without vocab parallelism).

    Returns ``(loss, lse_out, lse_rows)``: the reduced loss (a scalar, or ``batch_shape`` for
    ``"none"`` with zeros where no row lands), the log-sum-exp scattered to ``batch_shape`` (only
    with ``return_lse``), and the merged log-sum-exp per valid row (only with ``want_lse_rows``).
    With ``n_rows_dev`` (the row count on the device) ``B`` is only the pitch of ``stats``."""
    if reduction not in _REDUCTION_CODE:
        raise ValueError(f"Unknown reduction {reduction}")
    assert stats.dim() == 3 and stats.size(1) == 2 and stats.dtype == torch.float32 and stats.is_contiguous()
    world, _, n_rows = stats.shape
    n_total = batch_shape.numel()
    dev = stats.device
    loss = torch.empty(batch_shape if reduction == "none" else (), dtype=torch.float32, device=dev)
    lse_out = torch.empty(batch_shape, dtype=torch.float32, device=dev) if return_lse else None
    lse_rows = torch.empty((n_rows,), dtype=torch.float32, device=dev) if want_lse_rows else None
    with torch.cuda.device(dev):
        rc = _native.lib().cce_b200_loss_tail(
            stats.data_ptr(), world, n_rows, _native._ptr(valids),
            _native.IDX_I64 if (valids is not None and valids.dtype == torch.int64) else _native.IDX_I32,
            int(shift), n_total, _REDUCTION_CODE[reduction], _native._ptr(lse_rows), loss.data_ptr(),
            _native._ptr(lse_out), None, _native._ptr(n_rows_dev), _native.stream_ptr(dev),
        )  # fmt: skip
    _native.check(rc, "cce_b200_loss_tail")
    return loss, lse_out, lse_rows
