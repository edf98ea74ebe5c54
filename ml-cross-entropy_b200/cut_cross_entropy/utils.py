"""Small host-side helpers of the loss path.

Reference behaviour followed here: ``cut_cross_entropy/utils.py:12-120``
(softcapping, filter-eps resolution, valid-row list, scatter for
``reduction="none"``, z-loss).
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from .constants import IGNORE_INDEX


def softcapping(logits: torch.Tensor, softcap: float) -> torch.Tensor:
    """tanh soft-capping, ``softcap * tanh(logits / softcap)`` (reference utils.py:12-14)."""
    return torch.tanh(logits / softcap) * softcap


def _handle_eps(filter_eps: float | str | None, dtype: torch.dtype) -> float | None:
    """Resolve the gradient-filter threshold (reference utils.py:17-25).

    ``"auto"`` is 1/32 of the machine epsilon of ``dtype``: 2**-12 for bf16,
    2**-15 for fp16.
    """
    if filter_eps is None:
        return None
    if isinstance(filter_eps, float):
        return filter_eps
    if filter_eps == "auto":
        return torch.finfo(dtype).eps / 32
    raise RuntimeError(f"Unknown eps {filter_eps=}")


_UNRESOLVED = object()


class PendingValidRows:
    """A list of valid rows that the GPU is still writing: the kernels are enqueued, the length
    of the list has not been read back.  :meth:`resolve` reads it (the one host synchronisation of
    the forward pass) and returns what ``_build_flat_valids`` returns."""

    def __init__(self, rows: torch.Tensor, count: torch.Tensor, done: "torch.cuda.Event | None", n_total: int,
                 shift: int, count_dev: torch.Tensor | None = None):
        self.rows, self.count, self.done, self.n_total, self.shift = rows, count, done, n_total, shift
        # the list's length in device memory, for a caller that never reads it (then `count`/`done` are unused)
        self.count_dev = count_dev
        self._resolved: torch.Tensor | None | object = _UNRESOLVED

    def __del__(self):
        # The length is written by a kernel into pinned host memory that PyTorch's host allocator
        # knows nothing about being in use: if this object goes away before the kernel has run (an
        # exception between the launch and resolve()), wait for it, so that the block cannot be
        # handed to somebody else and then overwritten.
        try:
            if self.count_dev is None and self.done is not None and self._resolved is _UNRESOLVED:
                self.done.synchronize()
        except Exception:
            pass

    def resolve(self) -> torch.Tensor | None:
        if self._resolved is _UNRESOLVED and self.count_dev is not None:
            n = int(self.count_dev.item())  # synchronises; the sync-free path never calls this
            self._resolved = None if (self.shift == 0 and n == self.n_total) else self.rows[:n]
        if self._resolved is _UNRESOLVED:
            # The kernel wrote the length straight into pinned host memory: waiting for the event
            # is all it takes, no device-to-host copy that could queue behind a bulk download.
            self.done.synchronize()
            n = int(self.count[0])
            self._resolved = None if (self.shift == 0 and n == self.n_total) else self.rows[:n]
        return self._resolved


def launch_flat_valids(
    targets: torch.Tensor, ignore_index: int, shift: int, count_on_device: bool = False
) -> PendingValidRows:
    """Enqueue ``cce_b200_valid_rows`` on the current stream for CUDA ``targets`` of shape
    ``[..., seq_len]``; host work that does not need the list can follow before ``resolve()``.
    With ``count_on_device`` the length of the list is written to device memory (``count_dev``) and
    nothing is prepared for reading it back: the kernels of the loss take it from there."""
    from . import _native

    flat = targets.reshape(-1)
    if flat.dtype != torch.int64:
        flat = flat.long()
    flat = flat.contiguous()
    n_total = flat.numel()
    seq = targets.size(-1) if targets.dim() > 0 else 1
    L = _native.lib()
    rows = torch.empty((n_total,), dtype=torch.int32 if shift == 0 else torch.int64, device=targets.device)
    if count_on_device:
        count = torch.empty((1,), dtype=torch.int64, device=targets.device)
    else:
        count = torch.empty((1,), dtype=torch.int64, pin_memory=True)  # device-writable through unified addressing
    ws = _native.workspace(L.cce_b200_valid_rows_workspace_bytes(n_total), targets.device)
    with torch.cuda.device(targets.device):
        rc = L.cce_b200_valid_rows(
            flat.data_ptr(), n_total, max(seq, 1), shift, ignore_index, rows.data_ptr(),
            _native.IDX_I32 if shift == 0 else _native.IDX_I64, count.data_ptr(), ws.data_ptr(), ws.numel(),
            _native.stream_ptr(targets.device),
        )  # fmt: skip
    _native.check(rc, "cce_b200_valid_rows")
    if count_on_device:
        return PendingValidRows(rows, count, None, n_total, shift, count_dev=count)
    done = torch.cuda.Event()
    done.record(torch.cuda.current_stream(targets.device))
    return PendingValidRows(rows, count, done, n_total, shift)


def _build_flat_valids(targets: torch.Tensor, ignore_index: int, shift: int) -> torch.Tensor | None:
    """Rows of the flattened ``e`` that enter the loss (reference utils.py:28-49).

    Row ``r`` of ``e`` is paired with label ``targets.flatten()[r + shift]``.
    Without a shift the result is ``None`` when no label is ignored, else int32
    row numbers; with a shift it is always an int64 tensor (rows whose label
    would fall past the end of their sequence are never listed).  Reading the
    length of the list synchronises the stream, as the ``nonzero`` of the
    reference does.  CUDA labels go through ``cce_b200_valid_rows``; the
    PyTorch expressions below serve labels in host memory.
    """
    if targets.is_cuda:
        return launch_flat_valids(targets, ignore_index, shift).resolve()
    if shift == 0:
        keep = (targets.reshape(-1) != ignore_index).nonzero().squeeze(1)
        if keep.numel() == targets.numel():
            return None
        return keep.to(torch.int32)
    seq = targets.size(-1)
    rows = torch.arange(targets.numel(), device=targets.device).view(targets.shape)[..., : seq - shift]
    keep = targets[..., shift:] != ignore_index
    return rows[keep]


def handle_reduction_none(
    batch_shape: torch.Size, valids: torch.Tensor | None, shift: int, loss: torch.Tensor
) -> torch.Tensor:
    """Scatter per-valid-row values back to ``batch_shape`` with zeros elsewhere
    (reference utils.py:52-61).  With a shift the value of row ``r`` lands at the
    position of its label, ``r + shift``."""
    if valids is None:
        return loss.view(batch_shape)
    full = loss.new_zeros((batch_shape.numel(),))
    full[(valids + shift).long() if shift != 0 else valids.long()] = loss
    return full.view(batch_shape)


def compute_z_loss(
    lse: torch.Tensor,
    targets: torch.Tensor | None = None,
    shift: bool | int = False,
    ignore_index: int = IGNORE_INDEX,
    reduction: str = "mean",
) -> torch.Tensor:
    """z-loss ``lse**2`` (reference utils.py:64-102).

    Given ``targets``, positions whose label is ``ignore_index`` contribute zero
    and the mean is taken over the kept positions only.
    """
    z = lse.pow(2)
    if targets is not None:
        shift = int(shift)
        if shift != 0:
            targets = targets[..., shift:]
        keep = targets != ignore_index
        z = torch.where(keep, z, torch.zeros((), dtype=z.dtype, device=z.device))
        if reduction == "mean":
            z = z * (z.numel() / keep.count_nonzero().to(z.dtype))
    if reduction == "mean":
        return z.mean()
    if reduction == "sum":
        return z.sum()
    if reduction == "none":
        return z
    raise ValueError(f"Invalid reduction: {reduction}")


@dataclass
class TensorInfo:
    dtype: torch.dtype
    requires_grad: bool
