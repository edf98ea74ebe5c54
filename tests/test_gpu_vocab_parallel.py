"""Vocab parallelism on real GPUs: one process per GPU over NCCL (skipped with fewer than 2 GPUs).

Mirrors the reference's tests/test_vocab_parallel.py:27-150: every rank holds the whole batch and
its slice of the classifier; the loss and lse must equal the single-GPU values, the local dC must
equal the matching slice of the single-GPU dC, and dE (summed over ranks in fp32) the single-GPU dE.
"""

from __future__ import annotations

import sys
from pathlib import Path

import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def _run_ranks(target, world: int, args: tuple, timeout_s: float = 180.0) -> None:
    """Start one process per rank, collect one message per rank, and never leave a rank behind:
    whatever happens, children that are still alive are terminated before returning (a child
    blocked in a rendezvous would otherwise keep the test process from exiting)."""
    import queue
    import tempfile
    import time

    _run_ranks(_worker, world, (impl, z_loss))
