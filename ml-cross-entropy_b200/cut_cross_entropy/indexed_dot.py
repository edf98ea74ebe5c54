"""Negated correct-token logit: a gather-dot over rows of ``e`` and rows of ``c``.

Same call as the reference launcher ``indexed_neg_dot_forward_kernel``
(``cut_cross_entropy/indexed_dot.py:102-158``); the work is done by
``cce_b200_indexed_neg_dot``.  One extra keyword, ``vocab_start``, lets a
vocab-parallel rank pass global labels and get 0 for labels it does not own.
"""

from __future__ import annotations

import torch

from . import _native


def indexed_neg_dot_forward_kernel(
    e: torch.Tensor,
    c: torch.Tensor,
    inds: torch.Tensor,
    bias: torch.Tensor | None = None,
    shift: int = 0,
    valids: torch.Tensor | None = None,
    softcap: float | None = None,
    out_dtype: torch.dtype | None = None,
    vocab_start: int = 0,
    out: torch.Tensor | None = None,
    n_rows_dev: torch.Tensor | None = None,
) -> torch.Tensor:
    """``out[i] = -softcap(e[r] @ c[t] + bias[t])`` with ``r = valids[i]``, ``t = inds[r + shift] - vocab_start``.

    ``out`` (float32, contiguous, one element per row) is written in place and returned when given;
    ``n_rows_dev`` as in :func:`cut_cross_entropy.cce_lse_forward.cce_lse_forward_kernel`."""
    assert inds.ndim == 1 and e.ndim == 2 and c.ndim == 2
    assert inds.size(0) == e.size(0)
    assert c.size(1) == e.size(1)
    if e.stride(1) != 1:
        e = e.contiguous()
    if c.stride(1) != 1:
        c = c.contiguous()
    inds = inds.contiguous()
    if inds.dtype != torch.int64:
        inds = inds.long()
    if bias is not None:
        bias = bias.contiguous()
    if valids is not None:
        valids = valids.contiguous()

    op = _native.make_operands(e, c, bias, valids, softcap, n_rows_dev)
    if out is not None:
        assert out.dtype == torch.float32 and out.is_contiguous() and out.numel() == op.n_rows
        out_dtype = torch.float32
    else:
        out = torch.empty((op.n_rows,), dtype=torch.float32, device=e.device)
    with torch.cuda.device(e.device):
        rc = _native.lib().cce_b200_indexed_neg_dot(
            op, inds.data_ptr(), int(shift), int(vocab_start), out.data_ptr(), _native.stream_ptr(e.device)
        )
    _native.check(rc, "cce_b200_indexed_neg_dot")
    if out_dtype is None:
        out_dtype = e.dtype
    return out.to(out_dtype)
