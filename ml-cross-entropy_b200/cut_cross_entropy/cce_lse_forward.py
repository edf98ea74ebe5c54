"""Log-sum-exp of the (never materialised) logits, on the B200 tensor-core pipeline.

Same call as the reference launcher ``cce_lse_forward_kernel``
(``cut_cross_entropy/cce_lse_forward.py:163-237``); the work is done by
``cce_b200_lse_forward`` in ``libcce_b200.so``.
"""

from __future__ import annotations

import torch

from . import _native
from .utils import PendingValidRows


def cce_lse_forward_kernel(
    e: torch.Tensor,
    c: torch.Tensor,
    bias: torch.Tensor | None = None,
    valids: torch.Tensor | PendingValidRows | None = None,
    softcap: float | None = None,
    return_logit_avg: bool = False,
    return_tile_max: bool = False,
    stats_flat: torch.Tensor | None = None,
    return_col_max: bool = False,
    n_rows_dev: torch.Tensor | None = None,
    return_packed_e: bool = False,
) -> tuple[torch.Tensor, ...] | torch.Tensor:
    """``lse[i] = logsumexp_v(softcap(e[valids[i]] @ c[v] + bias[v]))`` as float32 ``[B]``.

    ``return_logit_avg`` also returns the reference's vocabulary-ordering key (its
    ``cce_lse_forward.py:95-97``), float32 ``[V]``: the mean over the valid rows of each column's
    logit, computed as ``softcap(mean(e) @ c.T + bias)`` by ``cce_b200_logit_avg`` (with
    soft-capping that is the cap of the mean rather than the mean of the capped values: the same
    ordering).

    ``valids`` may be a :class:`~cut_cross_entropy.utils.PendingValidRows` (a row list the GPU is
    still writing): buffers are then sized for all rows and the operand description is prepared
    before the list's length is waited for, so the launch follows the wait at once.

    ``stats_flat`` (float32, at least as many elements as there can be rows) receives the result in
    its first ``B`` elements instead of a fresh tensor: the forward pass keeps the log-sum-exp and the
    correct-token logit side by side for its tail kernel.

    ``return_tile_max`` asks for this backend's own by-product instead: the largest logit (in
    log2 units) of every (32-row group, 256-column tile) block, which lets the filtered
    backward skip recomputing tiles that cannot hold a value above the filter threshold.
    ``return_col_max`` adds the largest logit of every vocabulary entry over all rows (int32 keys
    ``[V]``, see ``cce_b200_lse_forward_ex``), which a backward with a vocabulary order needs.

    ``n_rows_dev`` (one int64 on the device) is the length of ``valids`` when the host never read it:
    ``valids`` is then the whole list buffer, the result has one slot per entry of that buffer and
    only the first ``n_rows_dev`` are written.

    ``return_packed_e`` adds the staged copy of ``e`` the kernel made in its workspace (the valid
    rows gathered into a dense matrix; ``None`` when it read ``e`` in place), which the backward
    launcher accepts so that it need not gather the same rows again.

    Returns ``lse`` alone, or a tuple ``(lse[, logit_avg][, tile_max][, col_max][, packed_e])`` of what
    was asked for.
    """
    assert e.shape[1] == c.shape[1], "Incompatible dimensions"
    assert e.is_contiguous(), "Matrix A must be contiguous"
    if bias is not None:
        assert bias.ndim == 1 and c.shape[0] == bias.shape[0]
        bias = bias.contiguous()
    if c.stride(1) != 1:
        c = c.contiguous()
    pending = valids if isinstance(valids, PendingValidRows) else None
    if pending is not None:
        valids = pending.rows  # the whole buffer: an upper bound of the list, for sizing
    if valids is not None:
        assert valids.ndim == 1
        valids = valids.contiguous()

    op = _native.make_operands(e, c, bias, valids, softcap, n_rows_dev)
    if stats_flat is not None:
        assert stats_flat.dtype == torch.float32 and stats_flat.is_contiguous() and stats_flat.numel() >= op.n_rows
        lse = stats_flat[: op.n_rows]
    else:
        lse = torch.empty((op.n_rows,), dtype=torch.float32, device=e.device)
    L = _native.lib()
    tile_max = None
    if return_tile_max:
        tile_max = torch.empty((L.cce_b200_tile_max_elems(op),), dtype=torch.float32, device=e.device)
    ws = _native.workspace(L.cce_b200_lse_workspace_bytes(op), e.device)
    stream = _native.stream_ptr(e.device)
    if pending is not None:  # now wait for the list and shrink everything to its true length
        rows = pending.resolve()
        op.n_rows = e.size(0) if rows is None else rows.numel()
        op.valids = _native._ptr(rows)
        lse = lse[: op.n_rows]
        if tile_max is not None:
            tile_max = tile_max[: L.cce_b200_tile_max_elems(op)]
        need = L.cce_b200_lse_workspace_bytes(op)  # not monotonic in n_rows (the band split changes)
        if need > ws.numel():
            ws = _native.workspace(need, e.device)
    col_max = torch.empty((op.V,), dtype=torch.int32, device=e.device) if return_col_max else None
    with torch.cuda.device(e.device):
        rc = L.cce_b200_lse_forward_ex(
            op, lse.data_ptr(), _native._ptr(tile_max), _native._ptr(col_max), ws.data_ptr(), ws.numel(), stream
        )
        _native.check(rc, "cce_b200_lse_forward")
        logit_avg = None
        if return_logit_avg:
            logit_avg = torch.empty((op.V,), dtype=torch.float32, device=e.device)
            ws2 = _native.workspace(L.cce_b200_logit_avg_workspace_bytes(op), e.device)
            rc = L.cce_b200_logit_avg(op, logit_avg.data_ptr(), ws2.data_ptr(), ws2.numel(), stream)
            _native.check(rc, "cce_b200_logit_avg")
    _native.finish(ws, "cce_b200_lse_forward")
    packed_e = None
    if return_packed_e:
        import ctypes

        off, pitch = ctypes.c_size_t(0), ctypes.c_int64(0)
        if L.cce_b200_lse_packed_e(op, ctypes.byref(off), ctypes.byref(pitch)) == 1 and op.n_rows > 0:
            nbytes = op.n_rows * pitch.value * 2
            packed_e = ws[off.value : off.value + nbytes].view(torch.int16).view(op.n_rows, pitch.value)
    extras = [x for x, want in ((logit_avg, return_logit_avg), (tile_max, return_tile_max),
                                (col_max, return_col_max), (packed_e, return_packed_e)) if want]  # fmt: skip
    return (lse, *extras) if extras else lse
