"""Vocab-parallel host logic on 2 CPU ranks over gloo.

The three kernel launchers are replaced, in this test only, by CPU stand-ins built on the
oracle, so what runs for real is the package's own orchestration: label ownership, the single
all-gather of the per-rank (lse, correct logit) blocks, the fp32 all-reduce of dE, the local dC.
"""

from __future__ import annotations

import sys
from pathlib import Path

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

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


def _install_cpu_stand_ins():
    from oracle import cce_oracle as O

    import cut_cross_entropy.cce as cce_mod
    import cut_cross_entropy.cce_backward as bwd_mod

    def lse_kernel(e, c, bias=None, valids=None, softcap=None, return_logit_avg=False, return_tile_max=False,
                   stats_flat=None, return_col_max=False, n_rows_dev=None, return_packed_e=False):
        assert not return_tile_max and not return_col_max and not return_logit_avg
        lse = O.lse_forward(e, c, bias, valids, softcap).float()
        return (lse, None) if return_packed_e else lse  # no staged copy of e on this stand-in

    def dot_kernel(e, c, inds, bias=None, shift=0, valids=None, softcap=None, out_dtype=None, vocab_start=0,
                   out=None, n_rows_dev=None):
        r = O.indexed_neg_dot(e, c, inds, bias, shift, valids, softcap, vocab_start=vocab_start).to(out_dtype)
        return r if out is None else out.copy_(r)

    def tail_kernel(stats, valids, shift, batch_shape, reduction, return_lse, want_lse_rows, n_rows_dev=None):
        # what cce_b200_loss_tail computes, in PyTorch
        lse = torch.logsumexp(stats[:, 0], dim=0)
        nll = lse + stats[:, 1].sum(dim=0)

        def scatter(x):
            if valids is None:
                return x.view(batch_shape)
            full = x.new_zeros((batch_shape.numel(),))
            full[valids.long() + shift] = x
            return full.view(batch_shape)

        loss = {"mean": nll.mean, "sum": nll.sum, "none": lambda: scatter(nll)}[reduction]()
        return loss, (scatter(lse) if return_lse else None), (lse if want_lse_rows else None)

    def launch(do, dlse, e, c, bias, lse, valids, softcap, filter_eps, targets, shift, grad_scale,
               filter_e, filter_c, vocab_start, de, dc, dbias, tile_max=None, vocab_ordering=None, col_max=None,
               n_rows_dev=None, scale_by_inv_rows=False, packed_e=None, de_ready=None, peers=None):
        assert peers is None  # accumulators in peer memory exist on GPUs only
        # restates one rank of cce_backward.py:182-310 with the global lse
        n = e.size(0)
        rows = torch.arange(n) if valids is None else valids.long()
        x = e[rows].double() @ c.double().T
        if bias is not None:
            x = x + bias.double()
        if softcap is not None:
            x = torch.tanh(x / softcap) * softcap
        p = torch.exp(x - lse.double()[:, None])
        t = targets[rows + shift] - vocab_start
        own = (t >= 0) & (t < c.size(0))
        g = grad_scale * (do.double().expand(n)[rows + shift] if do.numel() == 1 else do.double()[rows + shift])
        l = torch.zeros_like(g) if dlse is None else dlse.double()[rows + shift]
        ds = p * (g + l)[:, None]
        idx = own.nonzero().squeeze(1)
        ds[idx, t[idx]] -= g[idx]
        if softcap is not None:
            ds = ds * (1 - (x / softcap) ** 2)
        if de is not None:
            de.zero_()
            de[rows] = (ds @ c.double()).to(de.dtype)
        if dc is not None:
            dc.copy_((ds.T @ e[rows].double()).to(dc.dtype))
        if dbias is not None:
            dbias.copy_(ds.sum(0).to(dbias.dtype))

    cce_mod.cce_lse_forward_kernel = lse_kernel
    cce_mod.indexed_neg_dot_forward_kernel = dot_kernel
    cce_mod.loss_tail_kernel = tail_kernel
    bwd_mod._launch = launch
    # no CUDA stream on CPU
    import cut_cross_entropy._native as nat

    nat.make_operands = None


def _worker(rank: int, world: int, init_method: str, reduce_e_grad: bool, out_q):
    for p in (ROOT / "ml-cross-entropy_b200", ROOT, ROOT / "tests"):
        sys.path.insert(0, str(p))
    import datetime

    dist.init_process_group("gloo", init_method=init_method, rank=rank, world_size=world,
                            timeout=datetime.timedelta(seconds=120))
    try:
        from oracle import cce_oracle as O

        from cut_cross_entropy import VocabParallelOptions
        from cut_cross_entropy.cce import CCEParams, linear_cross_entropy_apply
        from cut_cross_entropy.utils import _build_flat_valids, compute_z_loss

        _install_cpu_stand_ins()
        g = torch.Generator().manual_seed(11)
        N, T, V, D = 48, 12, 101, 24
        e = (torch.randn(N, D, generator=g) / D**0.5).float()
        c = torch.randn(V, D, generator=g).float()
        c[: N // 2] = e[: N // 2]
        bias = torch.randn(V, generator=g).float() * 0.02
        targets = torch.randint(0, V, (N // T, T), generator=g)
        targets[torch.rand(N // T, T, generator=g) < 0.2] = -100
        shift = 1

        vp = VocabParallelOptions.from_vocab(V, None, reduce_e_grad=reduce_e_grad)
        assert (vp.start, vp.stop) == O.partition_n_into_range(V, rank, world)
        e_r = e.clone().requires_grad_(True)
        c_r = c[vp.start : vp.stop].clone().requires_grad_(True)
        b_r = bias[vp.start : vp.stop].clone().requires_grad_(True)
        params = CCEParams(
            targets=targets.flatten(), valids=_build_flat_valids(targets, -100, shift), softcap=20.0,
            reduction="mean", filter_eps=None, shift=shift, batch_shape=targets.size(), accum_e_fp32=True,
            accum_c_fp32=True, filter_e_grad=False, filter_c_grad=False, vocab_parallel_options=vp, return_lse=True,
        )  # fmt: skip
        loss, lse = linear_cross_entropy_apply(e_r, c_r, b_r, params)
        (loss + 1e-2 * compute_z_loss(lse, targets, shift)).backward()

        # the unsharded answer from the oracle
        e3 = e.view(N // T, T, D)
        ref_loss, ref_lse = O.linear_cross_entropy(e3, c, targets, bias, softcap=20.0, shift=shift, return_lse=True)
        keep = (targets[:, shift:] != -100).double()
        d_lse = 1e-2 * 2.0 * ref_lse * keep / keep.sum()
        rde, rdc, rdb = O.linear_cross_entropy_grads(e3, c, targets, bias, softcap=20.0, shift=shift, d_lse=d_lse)
        torch.testing.assert_close(loss.double(), ref_loss, rtol=1e-5, atol=1e-6)
        torch.testing.assert_close(lse.double(), ref_lse, rtol=1e-5, atol=1e-5)
        torch.testing.assert_close(c_r.grad.double(), rdc[vp.start : vp.stop], rtol=1e-4, atol=1e-6)
        torch.testing.assert_close(b_r.grad.double(), rdb[vp.start : vp.stop], rtol=1e-4, atol=1e-6)
        de = e_r.grad.double()
        if not reduce_e_grad:  # partial sums are left to the caller: add them up here
            dist.all_reduce(de)
        torch.testing.assert_close(de, rde.view(N, D), rtol=1e-4, atol=1e-6)
        out_q.put((rank, "ok"))
    except Exception as ex:  # report instead of hanging the peer
        import traceback

        out_q.put((rank, f"{type(ex).__name__}: {ex}\n{traceback.format_exc()}"))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("reduce_e_grad", [True, False])
def test_vocab_parallel_two_ranks_gloo(reduce_e_grad):
    _run_ranks(_worker, 2, (reduce_e_grad,))


def _worker_rank1_dies(rank: int, world: int, init_method: str, q):
    """Rank 1 exits before the rendezvous; rank 0 would wait for it (up to the group timeout)."""
    if rank == 1:
        raise SystemExit(3)
    import datetime

    dist.init_process_group("gloo", init_method=init_method, rank=rank, world_size=world,
                            timeout=datetime.timedelta(seconds=120))
    q.put((rank, "ok"))


def test_a_dead_rank_fails_the_test_quickly_and_leaves_no_process_behind():
    import time

    t0 = time.monotonic()
    with pytest.raises(AssertionError, match="ranks reported"):
        _run_ranks(_worker_rank1_dies, 2, ())
    assert time.monotonic() - t0 < 60
    assert not [p for p in mp.active_children() if p.is_alive()]
