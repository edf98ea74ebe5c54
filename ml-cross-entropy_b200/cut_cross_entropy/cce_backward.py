"""Gradients of the loss with respect to ``e``, ``c`` and ``bias``.

Same call as the reference launcher ``cce_backward_kernel``
(``cut_cross_entropy/cce_backward.py:346-521``); the work is done by
``cce_b200_backward``: per vocabulary chunk the logit tile is recomputed on the
tensor cores, turned into the logit gradient in registers, and fed to two more
tensor-core products (dC = G^T E, dE += G C) that skip blocks the filter cleared.
"""

from __future__ import annotations

import os

import torch

from . import _native
from .utils import TensorInfo
from .vocab_parallel.peer_reduce import finish_peer_reduce, peer_accumulators
from .vocab_parallel.utils import vp_reduce_e_grad_, vp_reduce_e_grad_cast


_REDUCE_STREAMS: dict = {}


def _reduce_stream(dev: torch.device) -> "torch.cuda.Stream":
    """One side stream per device for the cross-rank sum of dE."""
    key = (dev.type, dev.index if dev.index is not None else torch.cuda.current_device())
    if key not in _REDUCE_STREAMS:
        _REDUCE_STREAMS[key] = torch.cuda.Stream(device=dev)
    return _REDUCE_STREAMS[key]


def _exchange_sms(n_rows: int, d: int, fused: bool) -> int:
    """SMs the last dC product leaves to the kernels that exchange dE beside it.  The product is a
    persistent kernel with one CTA per SM, so with 0 the exchange starts only when the product ends.
    ``CCE_B200_EXCHANGE_SMS`` sets the number; unset, 32 SMs are left free while the fp32 partial dE
    is at most 128 MB and none above that.  Measured on 8 GPUs at the Gemma-2-2B head (dE 75 MB):
    1.327 ms per step with 0, 1.271 with 32, 1.279 with 48 free SMs.  A large dE comes with a dC
    product that is long compared with the exchange, which then loses more to the missing SMs than
    the overlap returns (not measured: an estimate from the kernel times of the 32768 x 4096 head)."""
    env = os.environ.get("CCE_B200_EXCHANGE_SMS")
    if env is not None:
        try:
            return max(0, int(env))
        except ValueError:
            pass
    # with the process group's reduce-scatter beside it the product lost more than the overlap gave
    # (1.53 against 1.41 ms per step on 8 GPUs), so only the fused exchange gets SMs by default
    return 32 if fused and n_rows * d * 4 <= (128 << 20) else 0


def _launch(do, dlse, e, c, bias, lse, valids, softcap, filter_eps, targets, shift, grad_scale,
            filter_e, filter_c, vocab_start, de, dc, dbias, tile_max=None, vocab_ordering=None, col_max=None,
            n_rows_dev=None, scale_by_inv_rows=False, packed_e=None, de_ready=None, peers=None) -> torch.Tensor:
    """Fill the (pre-allocated, possibly ``None``) outputs ``de``/``dc``/``dbias`` through the C ABI.
    With ``peers`` (:class:`PeerAccumulators`) the dE products add into the ranks' accumulators
    instead of writing ``de``.  Returns the call's workspace (its first word is the status word)."""
    dev = e.device
    a = _native.BackwardArgs()
    a.op = _native.make_operands(e, c, bias, valids, softcap, n_rows_dev)
    a.lse = lse.data_ptr()
    a.targets = targets.data_ptr()
    a.shift = shift
    a.vocab_start = vocab_start
    a.d_out = do.data_ptr()
    a.d_out_numel = do.numel()
    a.d_lse = _native._ptr(dlse)
    a.grad_scale = grad_scale
    a.grad_scale_by_inv_rows = int(scale_by_inv_rows)
    if packed_e is not None:
        a.e_packed, a.e_packed_ld = packed_e.data_ptr(), packed_e.stride(0)
    if de_ready is not None:
        a.de_ready_event = de_ready.cuda_event
        a.exchange_sms = _exchange_sms(a.op.n_rows, a.op.D, peers is not None)
    if peers is not None:
        a.de_peer_world = peers.world
        for r, ptr in enumerate(peers.ptrs):
            a.de_peer_acc[r] = ptr
    a.has_filter = int(filter_eps is not None)
    a.filter_eps = float(filter_eps) if filter_eps is not None else 0.0
    a.filter_e = int(filter_e)
    a.filter_c = int(filter_c)
    a.d_e = _native._ptr(de)
    a.d_e_f32 = int(de is not None and de.dtype == torch.float32)
    a.d_c = _native._ptr(dc)
    a.d_bias = _native._ptr(dbias)
    a.tile_max = _native._ptr(tile_max)
    if vocab_ordering is not None and col_max is not None and tile_max is not None:
        a.vocab_order = vocab_ordering.data_ptr()
        a.col_max_key = col_max.data_ptr()
    L = _native.lib()
    ws = _native.workspace(L.cce_b200_backward_workspace_bytes(a), dev)
    with torch.cuda.device(dev):
        rc = L.cce_b200_backward(a, ws.data_ptr(), ws.numel(), _native.stream_ptr(dev))
    _native.check(rc, "cce_b200_backward")
    _native.finish(ws, "cce_b200_backward")
    return ws


def cce_backward_kernel(
    do: torch.Tensor,
    dlse: torch.Tensor | None,
    e: torch.Tensor,
    e_info: TensorInfo,
    c: torch.Tensor,
    c_info: TensorInfo,
    bias: torch.Tensor | None,
    bias_info: TensorInfo | None,
    lse: torch.Tensor,
    valids: torch.Tensor | None,
    softcap: float | None,
    filter_eps: float | None,
    targets: torch.Tensor | None = None,
    shift: int = 0,
    vocab_ordering: torch.Tensor | None = None,
    grad_scale: float = 1.0,
    accum_e_fp32: bool = False,
    accum_c_fp32: bool = False,
    filter_e_grad: bool = True,
    filter_c_grad: bool = True,
    reduce_e_grad: bool = False,
    pg: "torch.distributed.ProcessGroup | None" = None,
    vocab_start: int = 0,
    tile_max: torch.Tensor | None = None,
    col_max: torch.Tensor | None = None,
    n_rows_dev: torch.Tensor | None = None,
    scale_by_inv_rows: bool = False,
    packed_e: torch.Tensor | None = None,
) -> tuple[torch.Tensor | None, torch.Tensor | None, torch.Tensor | None]:
    """Returns ``(de, dc, dbias)``, each ``None`` unless its ``*_info.requires_grad``.

    ``do`` is the upstream gradient of the loss (one element, or one per entry of
    ``targets`` and read at the label position), ``dlse`` the upstream gradient of
    the returned log-sum-exp (or ``None``).  ``targets`` holds global labels;
    ``vocab_start`` is the first label this rank's ``c`` covers.  ``vocab_ordering``
    (int32 permutation of the local vocabulary, reference ``cce_backward.py:154-155``) makes
    the backward form its tiles from consecutive entries of that order; it takes effect when
    the block-list backward runs (both products filtered, ``tile_max`` and ``col_max`` given,
    no bias gradient) and is ignored otherwise.  The ``accum_*_fp32`` switches are accepted
    and ignored: every accumulation is fp32.  With
    ``reduce_e_grad`` the fp32 partial ``de`` is summed over ``pg`` before the cast.
    ``n_rows_dev`` (one int64 on the device) is the number of valid rows when the host never read
    it (``valids`` and ``lse`` are then sized for all rows); ``scale_by_inv_rows`` divides
    ``grad_scale`` by that number on the device (``reduction="mean"``).
    ``packed_e`` is the staged copy of ``e`` from ``cce_lse_forward_kernel(return_packed_e=True)``
    for the same ``e`` and ``valids``.
    ``tile_max`` / ``col_max`` are the optional by-products of
    ``cce_lse_forward_kernel(return_tile_max=True, return_col_max=True)``.
    """
    assert targets is not None
    assert do.numel() in (e.size(0), 1)
    assert c.size(1) == e.size(1)
    assert lse.size(0) == e.size(0) or (valids is not None and lse.size(0) == valids.size(0))
    if dlse is not None and do.numel() > 1:
        assert dlse.numel() == do.numel()

    dev = e.device
    if e.stride(1) != 1 or (e.size(0) > 1 and e.stride(0) < e.size(1)):
        e = e.contiguous()
    if c.stride(1) != 1:
        c = c.contiguous()
    do = do.reshape(-1).to(dtype=torch.float32).contiguous()
    lse = lse.to(dtype=torch.float32).contiguous()
    if dlse is not None:
        dlse = dlse.reshape(-1).to(dtype=torch.float32).contiguous()
    targets = targets.contiguous()
    if targets.dtype != torch.int64:
        targets = targets.long()
    if bias is not None:
        bias = bias.contiguous()
    if valids is not None:
        valids = valids.contiguous()
    if vocab_ordering is not None:
        assert vocab_ordering.ndim == 1 and vocab_ordering.numel() == c.size(0)
        vocab_ordering = vocab_ordering.to(torch.int32).contiguous()

    want_de = e_info.requires_grad
    want_dc = c_info.requires_grad
    want_dbias = bias is not None and bias_info is not None and bias_info.requires_grad
    reduce_de = bool(reduce_e_grad and want_de)

    # The cross-rank sum of dE.  On one NVLink node the dE product adds its tiles straight into the
    # owning ranks' accumulators (vocab_parallel/peer_reduce.py) and de keeps e's type; otherwise the
    # partial dE is produced in fp32 and summed by the process group.
    n_rows_bound = valids.size(0) if valids is not None else e.size(0)
    peers, acc_rows = None, 0
    if reduce_de and dev.type == "cuda" and n_rows_bound > 0:
        acc_rows = int(_native.lib().cce_b200_de_peer_rows(n_rows_bound, torch.distributed.get_world_size(pg)))
        world = torch.distributed.get_world_size(pg)
        peers = peer_accumulators(pg, dev, acc_rows * e.size(1) * 4, world * acc_rows * e.size(1) * e.element_size())
    de_f32 = reduce_de and peers is None

    de = torch.empty(e.shape, dtype=torch.float32 if de_f32 else e.dtype, device=dev) if want_de else None
    dc = torch.empty((c.size(0), c.size(1)), dtype=c.dtype, device=dev) if want_dc else None
    dbias = torch.empty((c.size(0),), dtype=torch.float32, device=dev) if want_dbias else None

    # With a cross-rank sum of dE to do, the library is asked to finish dE before the last dC product
    # and to record an event there: the exchange then runs on a side stream beside that product.
    overlap = reduce_de and dev.type == "cuda"
    de_ready = None
    if overlap:
        de_ready = torch.cuda.Event()
        de_ready.record(torch.cuda.current_stream(dev))  # creates the handle; the library records it again
    ws = None
    if want_de or want_dc or want_dbias:
        ws = _launch(do, dlse, e, c, bias, lse, valids, softcap, filter_eps, targets, int(shift), float(grad_scale),
                     bool(filter_e_grad), bool(filter_c_grad), int(vocab_start), de, dc, dbias, tile_max,
                     vocab_ordering, col_max, n_rows_dev, bool(scale_by_inv_rows), packed_e, de_ready, peers)

    if reduce_de:
        assert de is not None
        if overlap:
            main, side = torch.cuda.current_stream(dev), _reduce_stream(dev)
            side.wait_event(de_ready)
            with torch.cuda.stream(side):
                if peers is not None:
                    # barrier, cast of the rows this rank owns, 16-bit all-gather, rows to their places
                    # (ws and de are used on the side stream without record_stream: the main stream
                    # waits for the side stream below, before anything can reuse their memory)
                    assert ws is not None
                    finish_peer_reduce(peers, pg, de, acc_rows, valids, n_rows_bound, n_rows_dev, ws)
                elif e_info.dtype in (torch.float16, torch.bfloat16):
                    # fp32 reduce-scatter, cast, 16-bit all-gather: the fp32 sum of the reference with less traffic
                    reduced = vp_reduce_e_grad_cast(de, e_info.dtype, pg)
                    de.record_stream(side)
                    de = reduced
                else:
                    vp_reduce_e_grad_(de, pg)
            if peers is None:
                de.record_stream(main)
                de.record_stream(side)
            main.wait_stream(side)  # enqueued after the last dC product, which therefore overlaps the exchange
        else:
            vp_reduce_e_grad_(de, pg)

    if dbias is not None:
        assert bias_info is not None
        dbias = dbias.to(dtype=bias_info.dtype)
    if dc is not None:
        dc = dc.to(dtype=c_info.dtype)
    if de is not None:
        de = de.to(dtype=e_info.dtype)
    return de, dc, dbias
