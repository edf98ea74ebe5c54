"""Accumulators for the cross-rank sum of ``dE`` that the product kernel performs itself.

Under vocabulary parallelism every rank computes a partial ``dE`` over its slice of the
vocabulary, and the partial sums have to be added over the ranks (reference
``cut_cross_entropy/vocab_parallel/utils.py:68-76``: an fp32 all-reduce after the kernel).  On one
NVLink/NVSwitch node this package lets the ``dE`` product do the first half of that exchange:
each rank owns every ``world``-th block of 128 rows, holds an fp32 accumulator for the blocks it
owns, maps the other ranks' accumulators into its own address space (CUDA inter-process memory
handles), and the product's epilogue adds each finished tile into the owner's accumulator with
bulk adds (``cce_b200_backward_args.de_peer_world``).  What is left afterwards
(:func:`finish_peer_reduce`) is a barrier, a cast of the owned rows and their exchange: either a
16-bit all-gather of the process group, or (``CCE_B200_PEER_GATHER=1``, the default) stores of the cast
rows straight into a gather buffer of every rank, which sits behind the accumulator in the same
mapped allocation, followed by a second barrier.

The accumulators are plain device memory and every load or store that touches a peer's memory is
an ordinary global-memory instruction.  ``CCE_B200_PEER_REDUCE=0`` switches the path off; the
backward then reduces with the process group's reduce-scatter / all-gather instead.
"""

from __future__ import annotations

import ctypes
import os
import socket
from dataclasses import dataclass, field

import torch
import torch.distributed as dist

from .. import _native


def _enabled() -> bool:
    return os.environ.get("CCE_B200_PEER_REDUCE", "1") not in ("", "0")


def _push_gather() -> bool:
    return os.environ.get("CCE_B200_PEER_GATHER", "1") not in ("", "0")


@dataclass
class PeerAccumulators:
    """The ranks' accumulators as seen from this process (``ptrs[rank]`` is this rank's own)."""

    world: int
    rank: int
    nbytes: int  # of each rank's allocation: accumulator, then gather buffer
    acc_bytes: int  # room for the accumulator; the gather buffer starts there
    ptrs: list[int]
    token: torch.Tensor  # one element; its all-reduce is the barrier between the adds and the collect
    opened: list[int] = field(default_factory=list)


# (group, device index) -> PeerAccumulators, or None when the group cannot use the path
_STATE: dict = {}


def _key(pg, dev: torch.device):
    return (pg if pg is not None else "default", dev.index if dev.index is not None else torch.cuda.current_device())


def _same_host(pg, dev: torch.device) -> bool:
    world = dist.get_world_size(pg)
    names = [None] * world
    dist.all_gather_object(names, socket.gethostname(), group=pg)
    return len(set(names)) == 1


def _agree(ok: bool, pg, dev: torch.device) -> bool:
    """True when ``ok`` holds on every rank."""
    flag = torch.tensor([1 if ok else 0], dtype=torch.int32, device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=pg)
    return bool(flag.item())


def _release(st: PeerAccumulators, pg, dev: torch.device) -> None:
    """Unmaps the peers' buffers and frees this rank's (a collective: every rank calls it)."""
    L = _native.lib()
    torch.cuda.synchronize(dev)
    dist.barrier(group=pg)  # nobody adds into anybody's buffer any more
    for p in st.opened:
        L.cce_b200_peer_buffer_close(p)
    dist.barrier(group=pg)  # every mapping of this rank's buffer is gone
    L.cce_b200_peer_buffer_destroy(st.ptrs[st.rank])


def _create(pg, dev: torch.device, acc_bytes: int, gather_bytes: int) -> PeerAccumulators | None:
    L = _native.lib()
    world, rank = dist.get_world_size(pg), dist.get_rank(pg)
    acc_bytes = -(-acc_bytes // 256) * 256
    nbytes = acc_bytes + max(gather_bytes, 256)
    own = ctypes.c_void_p()
    handle = (ctypes.c_uint8 * _native.PEER_HANDLE_BYTES)()
    with torch.cuda.device(dev):
        rc = L.cce_b200_peer_buffer_create(nbytes, ctypes.byref(own), handle)
    ok = rc == 0
    mine = torch.tensor(list(handle), dtype=torch.uint8, device=dev)
    handles = torch.empty((world, _native.PEER_HANDLE_BYTES), dtype=torch.uint8, device=dev)
    dist.all_gather_into_tensor(handles.view(-1), mine, group=pg)
    handles = handles.cpu()
    ptrs, opened = [0] * world, []
    if _agree(ok, pg, dev):
        for r in range(world):
            if r == rank:
                ptrs[r] = own.value
                continue
            buf = (ctypes.c_uint8 * _native.PEER_HANDLE_BYTES)(*handles[r].tolist())
            p = ctypes.c_void_p()
            with torch.cuda.device(dev):
                if L.cce_b200_peer_buffer_open(buf, ctypes.byref(p)) != 0:
                    ok = False
                    break
            ptrs[r] = p.value
            opened.append(p.value)
    else:
        ok = False
    if not _agree(ok, pg, dev):  # some rank could not map some buffer: nobody uses the path
        for p in opened:
            L.cce_b200_peer_buffer_close(p)
        dist.barrier(group=pg)
        if own.value:
            L.cce_b200_peer_buffer_destroy(own)
        return None
    token = torch.zeros(1, dtype=torch.float32, device=dev)
    return PeerAccumulators(world, rank, nbytes, acc_bytes, ptrs, token, opened)


def peer_accumulators(pg, dev: torch.device, acc_bytes: int, gather_bytes: int) -> PeerAccumulators | None:
    """The group's buffers with room for an accumulator of ``acc_bytes`` and a gather buffer of
    ``gather_bytes`` on each rank, or ``None`` when the path is off or unusable (switched off, not
    NCCL, more than ``MAX_PEERS`` ranks, ranks on several hosts, or the buffers cannot be mapped).
    Collective on first use and whenever the buffers have to grow; all ranks call it with the same
    arguments."""
    if not _enabled() or dev.type != "cuda" or not dist.is_available() or not dist.is_initialized():
        return None
    key = _key(pg, dev)
    if key in _STATE:
        st = _STATE[key]
        if st is None or (st.acc_bytes >= acc_bytes and st.nbytes - st.acc_bytes >= gather_bytes):
            return st
        acc_bytes = max(acc_bytes, st.acc_bytes)
        gather_bytes = max(gather_bytes, st.nbytes - st.acc_bytes)
        _release(st, pg, dev)
        del _STATE[key]
    world = dist.get_world_size(pg)
    with torch.cuda.device(dev):
        usable = 1 < world <= _native.MAX_PEERS and dist.get_backend(pg) == "nccl" and _same_host(pg, dev)
        _STATE[key] = _create(pg, dev, acc_bytes, gather_bytes) if usable else None
    return _STATE[key]


def release_peer_accumulators(pg=None) -> None:
    """Frees the accumulators of ``pg`` (a collective).  Call before destroying the process group."""
    for key in [k for k in _STATE if k[0] == (pg if pg is not None else "default")]:
        st = _STATE.pop(key)
        if st is not None:
            _release(st, pg, torch.device("cuda", key[1]))


def finish_peer_reduce(
    st: PeerAccumulators,
    pg,
    de: torch.Tensor,
    acc_rows: int,
    valids: torch.Tensor | None,
    n_rows: int,
    n_rows_dev: torch.Tensor | None,
    status_ws: torch.Tensor,
) -> None:
    """Second half of the fused reduction, on the current stream: barrier over the ranks (every
    rank's adds have landed), this rank's sums cast to ``de``'s type (the accumulator is cleared)
    and handed to every rank, rows copied to their places in ``de`` ``[n_total, D]``.  The token's
    value is never read: its all-reduce is the barrier."""
    L = _native.lib()
    dev = de.device
    D = de.size(1)
    dt = _native._DTYPE_CODE[de.dtype]
    sp = _native.stream_ptr(dev)
    dist.all_reduce(st.token, group=pg)
    rows_dt = _native.IDX_I64 if valids is not None and valids.dtype == torch.int64 else _native.IDX_I32
    if _push_gather():
        # cast rows go straight into every rank's gather buffer; a second barrier, then the local copy
        gather = (ctypes.c_void_p * st.world)(*[p + st.acc_bytes for p in st.ptrs])
        with torch.cuda.device(dev):
            rc = L.cce_b200_de_peer_collect_push(st.ptrs[st.rank], acc_rows, D, gather, st.world, st.rank, dt,
                                                 status_ws.data_ptr(), sp)  # fmt: skip
        _native.check(rc, "cce_b200_de_peer_collect_push")
        dist.all_reduce(st.token, group=pg)
        gathered_ptr = st.ptrs[st.rank] + st.acc_bytes
    else:
        piece = torch.empty((acc_rows, D), dtype=de.dtype, device=dev)
        with torch.cuda.device(dev):
            rc = L.cce_b200_de_peer_collect(st.ptrs[st.rank], acc_rows, D, piece.data_ptr(), dt, status_ws.data_ptr(), sp)
        _native.check(rc, "cce_b200_de_peer_collect")
        gathered = torch.empty((st.world * acc_rows, D), dtype=de.dtype, device=dev)
        dist.all_gather_into_tensor(gathered, piece, group=pg)
        gathered_ptr = gathered.data_ptr()
    with torch.cuda.device(dev):
        rc = L.cce_b200_de_peer_scatter(gathered_ptr, st.world, acc_rows, D, dt, _native._ptr(valids), rows_dt,
                                        n_rows, _native._ptr(n_rows_dev), de.data_ptr(), sp)  # fmt: skip
    _native.check(rc, "cce_b200_de_peer_scatter")
