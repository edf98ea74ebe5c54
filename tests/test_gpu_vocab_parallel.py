"""Vocab parallelism on real GPUs: one process per GPU over NCCL (skipped with fewer than 2 GPUs).

Mirrors the reference's tests/test_vocab_parallel.py:27-150: every rank holds the whole batch and
its slice of the classifier; the loss and lse must equal the single-GPU values, the local dC must
equal the matching slice of the single-GPU dC, and dE (summed over ranks in fp32) the single-GPU dE.
"""

from __future__ import annotations

import os
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

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    with tempfile.TemporaryDirectory() as tmp:
        init_method = f"file://{tmp}/rendezvous"
        procs = [ctx.Process(target=target, args=(r, world, init_method, *args, q), daemon=True) for r in range(world)]
        for p in procs:
            p.start()
        results, deadline = [], time.monotonic() + timeout_s
        try:
            while len(results) < world and time.monotonic() < deadline:
                try:
                    results.append(q.get(timeout=1.0))
                except queue.Empty:
                    if any(p.exitcode not in (None, 0) for p in procs):
                        break  # a rank died without reporting: do not wait for its peers
        finally:
            for p in procs:
                p.join(timeout=10 if len(results) == world else 0.1)
            for p in procs:
                if p.is_alive():
                    p.terminate()
            for p in procs:
                p.join(timeout=5)
                if p.is_alive():
                    p.kill()
    assert len(results) == world, f"only {len(results)} of {world} ranks reported: {results}"
    for rank, msg in sorted(results):
        assert msg == "ok", f"rank {rank}: {msg}"


def _worker(rank: int, world: int, init_method: str, impl: str, z_loss: bool, q):
    for p in (ROOT / "ml-cross-entropy_b200", ROOT, ROOT / "tests"):
        sys.path.insert(0, str(p))
    import torch.distributed as dist

    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    import datetime

    dist.init_process_group("nccl", init_method=init_method, rank=rank, world_size=world, device_id=dev,
                            timeout=datetime.timedelta(seconds=120))  # fmt: skip
    try:
        from conftest import planted_inputs

        from cut_cross_entropy import VocabParallelOptions, linear_cross_entropy
        from cut_cross_entropy.utils import compute_z_loss

        N, T, V, D = 1024, 256, 4099, 256
        e, c, bias, t = planted_inputs(N, V, D, torch.bfloat16, dev, seed=21, bias=True, ignored=0.2)
        e = e.view(N // T, T, D)
        t = t.view(N // T, T)

        def run(vp):
            ee = e.clone().requires_grad_(True)
            if vp is None:
                cc, bb = c.clone().requires_grad_(True), bias.clone().requires_grad_(True)
            else:
                cc = c[vp.start : vp.stop].clone().requires_grad_(True)
                bb = bias[vp.start : vp.stop].clone().requires_grad_(True)
            loss, lse = linear_cross_entropy(ee, cc, t, bias=bb, softcap=30.0, shift=1, impl=impl,
                                             vocab_parallel_options=vp, return_lse=True)  # fmt: skip
            total = loss + (1e-2 * compute_z_loss(lse, t, 1) if z_loss else 0.0)
            total.backward()
            return loss.detach(), lse.detach(), ee.grad, cc.grad, bb.grad

        ref = run(None)
        vp = VocabParallelOptions.from_vocab(V)
        got = run(vp)
        torch.testing.assert_close(got[0], ref[0], rtol=1e-5, atol=1e-5)
        torch.testing.assert_close(got[1], ref[1], rtol=0, atol=1e-4)
        for g, r in ((got[2], ref[2]), (got[3], ref[3][vp.start : vp.stop]), (got[4], ref[4][vp.start : vp.stop])):
            assert (g.float() - r.float()).abs().max().item() <= 1e-2 * r.float().abs().max().item() + 1e-6
        # every rank holds the same dE
        mx = got[2].float().clone()
        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        torch.testing.assert_close(mx, got[2].float(), rtol=0, atol=0)
        # dE was summed by the product kernels through the ranks' mapped accumulators ...
        from cut_cross_entropy.vocab_parallel import peer_reduce

        states = list(peer_reduce._STATE.values())
        assert len(states) == 1 and states[0] is not None and states[0].world == world, states
        # ... and agrees with the sum the process group computes (fp32 sums in a different order, one rounding to bf16)
        os.environ["CCE_B200_PEER_REDUCE"] = "0"
        try:
            by_group = run(vp)
        finally:
            os.environ["CCE_B200_PEER_REDUCE"] = "1"
        scale = by_group[2].float().abs().max().item()
        assert (got[2].float() - by_group[2].float()).abs().max().item() <= 2.0 ** -7 * scale
        os.environ["CCE_B200_PEER_GATHER"] = "0"  # second half by the process group's all-gather instead of peer stores
        try:
            by_gather = run(vp)
        finally:
            os.environ["CCE_B200_PEER_GATHER"] = "1"
        assert (got[2].float() - by_gather[2].float()).abs().max().item() <= 2.0 ** -7 * scale
        again = run(vp)  # the accumulators were left clear: a second step gives the same sums
        assert (again[2].float() - got[2].float()).abs().max().item() <= 2.0 ** -7 * scale
        peer_reduce.release_peer_accumulators(None)
        q.put((rank, "ok"))
    except Exception as ex:
        import traceback

        q.put((rank, f"{type(ex).__name__}: {ex}\n{traceback.format_exc()}"))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("impl", ["cce_exact", "cce"])
@pytest.mark.parametrize("z_loss", [False, True])
def test_vocab_parallel_nccl(impl, z_loss):
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least 2 GPUs")
    _run_ranks(_worker, world, (impl, z_loss))
