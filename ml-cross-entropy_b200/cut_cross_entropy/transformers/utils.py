"""Options of a patched model and the call that replaces ``lm_head`` + ``loss_function``.

Reference behaviour followed here: ``cut_cross_entropy/transformers/utils.py:14-78``.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from ..linear_cross_entropy import linear_cross_entropy


@dataclass
class PatchOptions:
    impl: str
    reduction: str
    filter_eps: float | str | None
    accum_e_fp32: bool
    accum_c_fp32: bool
    filter_e_grad: bool
    filter_c_grad: bool
    train_only: bool

    def to_kwargs(self) -> dict:
        return dict(
            impl=self.impl,
            reduction=self.reduction,
            filter_eps=self.filter_eps,
            accum_e_fp32=self.accum_e_fp32,
            accum_c_fp32=self.accum_c_fp32,
            filter_e_grad=self.filter_e_grad,
            filter_c_grad=self.filter_c_grad,
        )

    def use_lce(self, labels: torch.Tensor | None, training: bool) -> bool:
        """The fused loss replaces the logits only when there are labels (and, with
        ``train_only``, only in training mode); otherwise the model's own forward runs."""
        if labels is None:
            return False
        return training or not self.train_only


def apply_lce(
    e: torch.Tensor,
    c: torch.Tensor,
    labels: torch.Tensor,
    opts: PatchOptions,
    bias: torch.Tensor | None = None,
    softcap: float | None = None,
    **loss_kwargs,
) -> torch.Tensor:
    """Next-token loss of hidden states ``e`` against ``labels`` (shifted by one inside the kernel).

    With ``num_items_in_batch`` (gradient accumulation in ``Trainer``) a ``mean`` becomes the sum
    divided by that count, as ``transformers``' own loss does (reference utils.py:59-76).
    """
    num_items_in_batch = loss_kwargs.get("num_items_in_batch", None)
    kwargs = opts.to_kwargs()
    if num_items_in_batch is not None and kwargs["reduction"] == "mean":
        kwargs["reduction"] = "sum"
    else:
        num_items_in_batch = None
    loss = linear_cross_entropy(e, c, labels.to(e.device), bias=bias, softcap=softcap, shift=True, **kwargs)
    if num_items_in_batch is not None:
        if torch.is_tensor(num_items_in_batch):
            num_items_in_batch = num_items_in_batch.to(loss.device)
        loss = loss / num_items_in_batch
    return loss
