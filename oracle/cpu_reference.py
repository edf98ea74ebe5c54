"""CPU port of the reference's ``impl="torch_compile"`` path, for TIMING on host cores.
TEST/BENCH INFRASTRUCTURE ONLY — never imported by the package.

The reference's CPU-runnable implementation materialises the logits and lets autograd
differentiate them (``cut_cross_entropy/torch_compile.py:18-49`` called from ``:53-117``):
``logits = e @ c.T (+ bias) -> soft-cap -> cross_entropy(logits.float())``, in the input dtype
(bf16 matmul on CPU), after gathering the valid rows (``:78-80``).  This file restates exactly
that with eager PyTorch so ``bench.py`` can time it with all host threads.  Its numbers are a
reported baseline, not a correctness reference (use ``cce_oracle`` for that).
"""

from __future__ import annotations

import time

import torch
import torch.nn.functional as F


def torch_compile_path_step(e, c, targets, bias=None, softcap=None, ignore_index=-100, reduction="mean"):
    """One forward+backward of the materialised-logits loss; returns (loss, dE, dC)."""
    e = e.detach().requires_grad_(True)
    c = c.detach().requires_grad_(True)
    keep = (targets != ignore_index).nonzero().squeeze(1)  # torch_compile.py:74-80
    rows = e[keep]
    logits = rows @ c.T
    if bias is not None:
        logits = logits + bias
    if softcap is not None:
        logits = torch.tanh(logits / softcap) * softcap
    loss = F.cross_entropy(logits.float(), targets[keep], ignore_index=ignore_index, reduction=reduction)
    loss.backward()
    return loss.detach(), e.grad, c.grad


def time_sample(e, c, targets, bias=None, softcap=None, warmup=1, iters=2):
    """Seconds per step (best of ``iters``) for the given sample of rows."""
    for _ in range(warmup):
        torch_compile_path_step(e, c, targets, bias, softcap)
    best = float("inf")
    for _ in range(iters):
        t0 = time.perf_counter()
        torch_compile_path_step(e, c, targets, bias, softcap)
        best = min(best, time.perf_counter() - t0)
    return best
