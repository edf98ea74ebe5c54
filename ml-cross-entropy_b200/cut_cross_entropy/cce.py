"""Autograd glue of the Cut Cross-Entropy loss on the B200 backend.

Follows ``cut_cross_entropy/cce.py:26-319`` of the reference: the same
parameters, saved tensors, reductions and gradient scaling; the three kernel
launchers it calls are this package's C-ABI wrappers.
"""

from __future__ import annotations

import os
from dataclasses import dataclass
from typing import cast

import torch
import torch.amp

from .cce_backward import cce_backward_kernel
from .cce_loss_tail import loss_tail_kernel
from .cce_lse_forward import cce_lse_forward_kernel
from .constants import IGNORE_INDEX
from .indexed_dot import indexed_neg_dot_forward_kernel
from .utils import PendingValidRows, TensorInfo, _handle_eps, launch_flat_valids
from .vocab_parallel.utils import VocabParallelOptions, vp_gather_stats


# Vocabulary ordering of the filtered backward (reference cce.py:43-45,171-174): "off" = tiles are
# formed in natural vocabulary order; "max" = sorted by each entry's largest logit over the batch
# (the quantity this backend's tile bound uses); "mean" = sorted by the mean logit, the reference's
# key.  It pays when the entries with large probabilities are scattered over the vocabulary; it
# costs a reordered copy of the classifier per backward, so it is off unless asked for
# (set_vocab_ordering, or CCE_B200_VOCAB_ORDER in the environment).
_VOCAB_ORDERING = os.environ.get("CCE_B200_VOCAB_ORDER", "off").lower()
if _VOCAB_ORDERING in ("", "0", "false"):
    _VOCAB_ORDERING = "off"
elif _VOCAB_ORDERING in ("1", "true", "on"):
    _VOCAB_ORDERING = "max"


def set_vocab_ordering(mode: bool | str) -> str:
    """Choose how the filtered backward orders the vocabulary (``"off"``, ``"max"``, ``"mean"``;
    ``True`` = ``"max"``, ``False`` = ``"off"``).  Returns the previous setting."""
    global _VOCAB_ORDERING
    if isinstance(mode, bool):
        mode = "max" if mode else "off"
    if mode not in ("off", "max", "mean"):
        raise ValueError(f"unknown vocabulary ordering {mode!r}")
    prev, _VOCAB_ORDERING = _VOCAB_ORDERING, mode
    return prev


# Whether the forward pass reads the number of valid rows back to the host (one stream
# synchronisation per call, as the reference's `nonzero` does, reference utils.py:28-49), or
# leaves it on the device: launches and buffers are then sized for every row, the kernels take the
# real count from device memory, and the host never waits for the GPU.  CCE_B200_SYNC_FREE=0 in
# the environment, or set_sync_free(False), selects the read-back.
_SYNC_FREE = os.environ.get("CCE_B200_SYNC_FREE", "1").lower() not in ("0", "false", "off", "")


def set_sync_free(on: bool) -> bool:
    """Keep the valid-row count on the device (``True``) or read it back in the forward pass
    (``False``).  Returns the previous setting."""
    global _SYNC_FREE
    prev, _SYNC_FREE = _SYNC_FREE, bool(on)
    return prev


def sort_logit_avg(logit_avg: torch.Tensor) -> torch.Tensor:
    """Vocabulary order from a per-entry key, hottest entries first (reference cce.py:43-45; there
    ascending, which clusters the same entries at the other end)."""
    return torch.argsort(logit_avg, descending=True).to(torch.int32)


@dataclass
class CCEParams:
    targets: torch.Tensor
    valids: torch.Tensor | None
    softcap: float | None
    reduction: str
    filter_eps: float | None
    shift: int
    batch_shape: torch.Size
    accum_e_fp32: bool
    accum_c_fp32: bool
    filter_e_grad: bool
    filter_c_grad: bool
    vocab_parallel_options: VocabParallelOptions | None
    return_lse: bool
    # the valid-row list while the GPU is still writing it; forward() turns it into `valids`
    pending_valids: PendingValidRows | None = None
    # length of `valids` on the device when the host never read it (then `valids` is the whole buffer)
    n_rows_dev: torch.Tensor | None = None


class LinearCrossEntropyFunction(torch.autograd.Function):
    @staticmethod
    @torch.amp.custom_fwd(device_type="cuda")
    def forward(
        ctx,
        e: torch.Tensor,
        c: torch.Tensor,
        bias: torch.Tensor | None,
        params: CCEParams,
    ) -> tuple[torch.Tensor, torch.Tensor | None]:
        e_info = TensorInfo(e.dtype, e.requires_grad)
        c_info = TensorInfo(c.dtype, c.requires_grad)
        bias_info = TensorInfo(bias.dtype, bias.requires_grad) if bias is not None else None

        if torch.is_autocast_enabled("cuda"):
            amp_dtype = torch.get_autocast_dtype("cuda")
            e, c = e.to(dtype=amp_dtype), c.to(dtype=amp_dtype)
            if bias is not None:
                bias = bias.to(dtype=amp_dtype)

        vp = params.vocab_parallel_options
        vocab_start = vp.start if vp is not None else 0

        pending = params.pending_valids
        params.pending_valids = None

        # The filtered backward can skip recomputing logit tiles that provably hold nothing above the
        # threshold if the forward records each tile's largest logit; worth it only when every
        # gradient that will be asked for is filtered (and the bias, whose gradient sums every
        # entry, asks for none).
        want_tile_max = (
            params.filter_eps is not None
            and (e_info.requires_grad or c_info.requires_grad)
            and (params.filter_e_grad or not e_info.requires_grad)
            and (params.filter_c_grad or not c_info.requires_grad)
            and not (bias_info is not None and bias_info.requires_grad)
        )
        # a vocabulary order only matters to the block-list backward, which is what tile_max is for
        order_mode = _VOCAB_ORDERING if want_tile_max else "off"
        if params.reduction not in ("mean", "sum", "none"):
            raise ValueError(f"Unknown reduction {params.reduction}")
        # (lse, -correct logit) of the valid rows sit side by side in one buffer, sized for every row
        # until the length of the row list is known: the tail kernel (and, under vocab parallelism,
        # the one all-gather) reads them as a [2, B] block.
        stats_flat = torch.empty((2 * e.size(0),), dtype=torch.float32, device=e.device)
        # a pending row list is waited for inside the launcher, after everything that does not need it
        if pending is not None and pending.count_dev is not None:
            # nothing is read back: the whole list buffer goes in, its length stays on the device
            params.valids, params.n_rows_dev = pending.rows, pending.count_dev
            pending = None
        n_dev = params.n_rows_dev
        # the backward reads the same gathered rows of e: keep the forward's staged copy for it
        # (only when e itself is what the backward will be given, i.e. no autocast cast happened)
        want_packed_e = e_info.requires_grad or c_info.requires_grad or (bias_info is not None and bias_info.requires_grad)
        ret = cce_lse_forward_kernel(
            e=e,
            c=c,
            bias=bias,
            valids=pending if pending is not None else params.valids,
            softcap=params.softcap,
            return_tile_max=want_tile_max,
            stats_flat=stats_flat,
            return_logit_avg=order_mode == "mean",
            return_col_max=order_mode != "off",
            n_rows_dev=n_dev,
            return_packed_e=want_packed_e,
        )
        if pending is not None:
            params.valids = pending.resolve()
        ret = list(ret) if isinstance(ret, tuple) else [ret]
        lse = ret.pop(0)
        logit_avg = ret.pop(0) if order_mode == "mean" else None
        tile_max = ret.pop(0) if want_tile_max else None
        col_max = ret.pop(0) if order_mode != "off" else None
        packed_e = ret.pop(0) if want_packed_e else None
        order_key = logit_avg if order_mode == "mean" else col_max
        assert isinstance(lse, torch.Tensor)
        n_rows = lse.numel()
        stats = stats_flat[: 2 * n_rows].view(1, 2, n_rows)
        if lse.data_ptr() != stats_flat.data_ptr():  # a launcher that allocated its own result
            stats[0, 0].copy_(lse)
        # labels this rank does not own give 0, so the same call serves the vocab-parallel case
        indexed_neg_dot_forward_kernel(
            e=e,
            c=c,
            inds=params.targets,
            bias=bias,
            shift=params.shift,
            valids=params.valids,
            softcap=params.softcap,
            out_dtype=torch.float32,
            vocab_start=vocab_start,
            out=stats[0, 1],
            n_rows_dev=n_dev,
        )
        if vp is not None:
            stats = vp_gather_stats(stats[0], vp.group)  # [world, 2, B]

        # one launch: merge over the ranks, nll = lse - correct logit, mean / sum / scatter
        loss, lse_out, lse_rows = loss_tail_kernel(
            stats,
            params.valids,
            params.shift,
            params.batch_shape,
            params.reduction,
            return_lse=params.return_lse,
            want_lse_rows=vp is not None,
            n_rows_dev=n_dev,
        )
        if vp is not None:
            assert lse_rows is not None
            lse = lse_rows  # the global log-sum-exp; without vocab parallelism it is stats[0, 0] itself
        else:
            lse = stats[0, 0]

        ctx.save_for_backward(e, c, bias, lse, params.targets, params.valids, tile_max, col_max, order_key, n_dev, packed_e)
        ctx.params = params
        ctx.e_info, ctx.c_info, ctx.bias_info = e_info, c_info, bias_info
        return loss, lse_out

    @staticmethod
    @torch.amp.custom_bwd(device_type="cuda")
    def backward(
        ctx, grad_out: torch.Tensor, grad_lse_out: torch.Tensor | None
    ) -> tuple[torch.Tensor | None, torch.Tensor | None, torch.Tensor | None, None]:
        e, c, bias, lse, targets, valids, tile_max, col_max, order_key, n_dev, packed_e = ctx.saved_tensors
        # integer keys (column maxima) and float keys (mean logits) both sort with the hottest entry first
        vocab_ordering = sort_logit_avg(order_key) if order_key is not None else None
        params = cast(CCEParams, ctx.params)

        if params.reduction == "mean":
            # with the count on the device, lse has a slot per row and the division happens in the kernel
            grad_scale = 1.0 if n_dev is not None else 1.0 / max(lse.numel(), 1)
        elif params.reduction in ("sum", "none"):
            grad_scale = 1.0
        else:
            raise ValueError(f"Unknown reduction {params.reduction}")
        if params.reduction == "none":
            grad_out = grad_out.reshape(-1)
        if grad_lse_out is not None:
            grad_lse_out = grad_lse_out.reshape(-1)

        vp = params.vocab_parallel_options
        de, dc, dbias = cce_backward_kernel(
            do=grad_out,
            dlse=grad_lse_out,
            e=e,
            e_info=ctx.e_info,
            c=c,
            c_info=ctx.c_info,
            bias=bias,
            bias_info=ctx.bias_info,
            lse=lse,
            valids=valids,
            softcap=params.softcap,
            filter_eps=params.filter_eps,
            targets=targets,
            shift=params.shift,
            vocab_ordering=vocab_ordering,
            grad_scale=grad_scale,
            accum_e_fp32=params.accum_e_fp32,
            accum_c_fp32=params.accum_c_fp32,
            filter_e_grad=params.filter_e_grad,
            filter_c_grad=params.filter_c_grad,
            reduce_e_grad=vp.reduce_e_grad if vp is not None else False,
            pg=vp.group if vp is not None else None,
            vocab_start=vp.start if vp is not None else 0,
            tile_max=tile_max,
            col_max=col_max,
            n_rows_dev=n_dev,
            scale_by_inv_rows=n_dev is not None and params.reduction == "mean",
            packed_e=packed_e,
        )
        return de, dc, dbias, None


def linear_cross_entropy_apply(
    e: torch.Tensor,
    c: torch.Tensor,
    bias: torch.Tensor | None,
    params: CCEParams,
) -> tuple[torch.Tensor, torch.Tensor | None]:
    loss, lse = cast(
        tuple[torch.Tensor, torch.Tensor | None],
        LinearCrossEntropyFunction.apply(e, c, bias, params),
    )
    # with a shift, position j of the outputs belongs to label j: drop the first `shift` slots
    if params.shift != 0 and params.reduction == "none":
        loss = loss[..., params.shift :]
    if params.return_lse and params.shift != 0:
        assert lse is not None
        lse = lse[..., params.shift :]
    return loss, lse


def cce_linear_cross_entropy(
    e: torch.Tensor,
    c: torch.Tensor,
    targets: torch.Tensor,
    bias: torch.Tensor | None = None,
    ignore_index: int = IGNORE_INDEX,
    softcap: float | None = None,
    reduction: str = "mean",
    shift: bool | int = 0,
    return_lse: bool = False,
    filter_eps: float | str | None = "auto",
    accum_e_fp32: bool = False,
    accum_c_fp32: bool = False,
    filter_e_grad: bool = True,
    filter_c_grad: bool = True,
    vocab_parallel_options: VocabParallelOptions | None = None,
) -> tuple[torch.Tensor, torch.Tensor | None]:
    """Loss (and optionally the log-sum-exp) of ``softcap(e @ c.T + bias)`` against ``targets``
    without materialising the logits.  See :func:`cut_cross_entropy.linear_cross_entropy`."""
    assert e.size()[0:-1] == targets.size()
    assert e.size(-1) == c.size(1)
    if not (torch.cuda.is_available() and e.is_cuda):
        raise RuntimeError(
            "Cut Cross Entropy (B200 backend) requires CUDA tensors on an sm_100 GPU; there is no CPU path."
        )

    batch_shape = targets.size()
    e = e.contiguous()
    targets = targets.contiguous()
    shift = int(shift)
    pending = launch_flat_valids(targets, ignore_index, shift, count_on_device=_SYNC_FREE)

    e = e.flatten(0, -2)
    targets = targets.flatten()

    amp_dtype = torch.get_autocast_dtype("cuda") if torch.is_autocast_enabled("cuda") else e.dtype
    params = CCEParams(
        targets=targets,
        valids=None,
        softcap=softcap,
        reduction=reduction,
        filter_eps=_handle_eps(filter_eps, amp_dtype),
        shift=shift,
        batch_shape=batch_shape,
        accum_e_fp32=accum_e_fp32,
        accum_c_fp32=accum_c_fp32,
        filter_e_grad=filter_e_grad and filter_eps is not None,
        filter_c_grad=filter_c_grad and filter_eps is not None,
        vocab_parallel_options=vocab_parallel_options,
        return_lse=return_lse,
        pending_valids=pending,
    )
    return linear_cross_entropy_apply(e, c, bias, params)
