"""ctypes binding of ``libcce_b200.so`` — the only way the host layer reaches the GPU kernels.

The structures below mirror ``include/cce_b200.h`` field by field.  There is no
fallback: if the library is missing, :func:`lib` raises, and every kernel wrapper
of this package fails with it.
"""

from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, Structure, c_char_p, c_float, c_int32, c_int64, c_size_t, c_void_p
from pathlib import Path

import torch

LIB_PATH = Path(__file__).resolve().parent / "libcce_b200.so"

DT_F16, DT_BF16, DT_F32 = 0, 1, 2
IDX_I32, IDX_I64 = 0, 1
MAX_PEERS = 8  # CCE_B200_MAX_PEERS
PEER_HANDLE_BYTES = 64  # CCE_B200_PEER_HANDLE_BYTES

_DTYPE_CODE = {torch.float16: DT_F16, torch.bfloat16: DT_BF16, torch.float32: DT_F32}

EXPORTS = (
    "cce_b200_lse_workspace_bytes",
    "cce_b200_lse_forward",
    "cce_b200_tile_max_elems",
    "cce_b200_lse_packed_e",
    "cce_b200_lse_forward_ex",
    "cce_b200_logit_avg_workspace_bytes",
    "cce_b200_logit_avg",
    "cce_b200_lse_forward_static",
    "cce_b200_indexed_neg_dot",
    "cce_b200_loss_tail",
    "cce_b200_valid_rows_workspace_bytes",
    "cce_b200_valid_rows",
    "cce_b200_backward_workspace_bytes",
    "cce_b200_backward",
    "cce_b200_peer_buffer_create",
    "cce_b200_peer_buffer_open",
    "cce_b200_peer_buffer_close",
    "cce_b200_peer_buffer_destroy",
    "cce_b200_de_peer_rows",
    "cce_b200_de_peer_collect",
    "cce_b200_de_peer_collect_push",
    "cce_b200_de_peer_scatter",
    "cce_b200_gemm",
    "cce_b200_read_status",
    "cce_b200_lse_forward_static_status",
    "cce_b200_selftest_wait",
    "cce_b200_launch_count",
    "cce_b200_profile_enable",
    "cce_b200_profile_wait_counters",
    "cce_b200_profile_read",
    "cce_b200_profile_clock_words",
    "cce_b200_profile_tile_counts",
    "cce_b200_strerror",
    "cce_b200_last_cuda_error",
    "cce_b200_version",
)


class Operands(Structure):
    _fields_ = [
        ("e", c_void_p),
        ("c", c_void_p),
        ("bias", c_void_p),
        ("valids", c_void_p),
        ("n_total", c_int64),
        ("n_rows", c_int64),
        ("V", c_int64),
        ("D", c_int64),
        ("lde", c_int64),
        ("ldc", c_int64),
        ("dtype", c_int32),
        ("bias_dtype", c_int32),
        ("valids_dtype", c_int32),
        ("has_softcap", c_int32),
        ("softcap", c_float),
        ("n_rows_dev", c_void_p),
    ]


class BackwardArgs(Structure):
    _fields_ = [
        ("op", Operands),
        ("lse", c_void_p),
        ("targets", c_void_p),
        ("shift", c_int64),
        ("vocab_start", c_int64),
        ("d_out", c_void_p),
        ("d_out_numel", c_int64),
        ("d_lse", c_void_p),
        ("grad_scale", c_float),
        ("grad_scale_by_inv_rows", c_int32),
        ("has_filter", c_int32),
        ("filter_eps", c_float),
        ("filter_e", c_int32),
        ("filter_c", c_int32),
        ("d_e", c_void_p),
        ("d_e_f32", c_int32),
        ("d_c", c_void_p),
        ("d_bias", c_void_p),
        ("tile_max", c_void_p),
        ("vocab_order", c_void_p),
        ("col_max_key", c_void_p),
        ("e_packed", c_void_p),
        ("e_packed_ld", c_int64),
        ("de_ready_event", c_void_p),
        ("de_peer_world", c_int32),
        ("exchange_sms", c_int32),
        ("de_peer_acc", c_void_p * MAX_PEERS),
    ]


class NativeError(RuntimeError):
    """A C-ABI call returned a negative status."""


_lib = None


def lib() -> ctypes.CDLL:
    """Load the library once; raise loudly if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    path = Path(os.environ.get("CCE_B200_LIB", LIB_PATH))
    if not path.exists():
        raise RuntimeError(
            f"{path} is missing: build it with `python -m cut_cross_entropy._build` "
            "(needs nvcc).  This backend has no fallback path."
        )
    L = ctypes.CDLL(str(path))
    L.cce_b200_lse_workspace_bytes.restype = c_size_t
    L.cce_b200_lse_workspace_bytes.argtypes = [POINTER(Operands)]
    L.cce_b200_lse_forward.restype = c_int32
    L.cce_b200_lse_forward.argtypes = [POINTER(Operands), c_void_p, c_void_p, c_void_p, c_size_t, c_void_p]
    L.cce_b200_lse_forward_ex.restype = c_int32
    L.cce_b200_lse_forward_ex.argtypes = [POINTER(Operands), c_void_p, c_void_p, c_void_p, c_void_p, c_size_t, c_void_p]
    L.cce_b200_logit_avg_workspace_bytes.restype = c_size_t
    L.cce_b200_logit_avg_workspace_bytes.argtypes = [POINTER(Operands)]
    L.cce_b200_logit_avg.restype = c_int32
    L.cce_b200_logit_avg.argtypes = [POINTER(Operands), c_void_p, c_void_p, c_size_t, c_void_p]
    L.cce_b200_lse_packed_e.restype = c_int32
    L.cce_b200_lse_packed_e.argtypes = [POINTER(Operands), POINTER(c_size_t), POINTER(c_int64)]
    L.cce_b200_tile_max_elems.restype = c_size_t
    L.cce_b200_tile_max_elems.argtypes = [POINTER(Operands)]
    L.cce_b200_lse_forward_static.restype = c_int32
    L.cce_b200_lse_forward_static.argtypes = [POINTER(Operands), c_void_p, c_void_p]
    L.cce_b200_indexed_neg_dot.restype = c_int32
    L.cce_b200_indexed_neg_dot.argtypes = [POINTER(Operands), c_void_p, c_int64, c_int64, c_void_p, c_void_p]
    L.cce_b200_loss_tail.restype = c_int32
    L.cce_b200_loss_tail.argtypes = [
        c_void_p, c_int32, c_int64, c_void_p, c_int32, c_int64, c_int64, c_int32, c_void_p, c_void_p, c_void_p,
        c_void_p, c_void_p, c_void_p,
    ]  # fmt: skip
    L.cce_b200_lse_forward_static_status.restype = c_int32
    L.cce_b200_lse_forward_static_status.argtypes = [c_void_p, POINTER(c_int32)]
    L.cce_b200_selftest_wait.restype = c_int32
    L.cce_b200_selftest_wait.argtypes = [c_int64, c_void_p, c_void_p]
    L.cce_b200_profile_clock_words.restype = c_int32
    L.cce_b200_profile_clock_words.argtypes = [c_void_p]
    L.cce_b200_profile_tile_counts.restype = c_int32
    L.cce_b200_profile_tile_counts.argtypes = [c_void_p]
    L.cce_b200_valid_rows_workspace_bytes.restype = c_size_t
    L.cce_b200_valid_rows_workspace_bytes.argtypes = [c_int64]
    L.cce_b200_valid_rows.restype = c_int32
    L.cce_b200_valid_rows.argtypes = [
        c_void_p, c_int64, c_int64, c_int64, c_int64, c_void_p, c_int32, c_void_p, c_void_p, c_size_t, c_void_p,
    ]  # fmt: skip
    L.cce_b200_backward_workspace_bytes.restype = c_size_t
    L.cce_b200_backward_workspace_bytes.argtypes = [POINTER(BackwardArgs)]
    L.cce_b200_backward.restype = c_int32
    L.cce_b200_backward.argtypes = [POINTER(BackwardArgs), c_void_p, c_size_t, c_void_p]
    L.cce_b200_peer_buffer_create.restype = c_int32
    L.cce_b200_peer_buffer_create.argtypes = [c_size_t, POINTER(c_void_p), c_void_p]
    L.cce_b200_peer_buffer_open.restype = c_int32
    L.cce_b200_peer_buffer_open.argtypes = [c_void_p, POINTER(c_void_p)]
    L.cce_b200_peer_buffer_close.restype = c_int32
    L.cce_b200_peer_buffer_close.argtypes = [c_void_p]
    L.cce_b200_peer_buffer_destroy.restype = c_int32
    L.cce_b200_peer_buffer_destroy.argtypes = [c_void_p]
    L.cce_b200_de_peer_rows.restype = c_int64
    L.cce_b200_de_peer_rows.argtypes = [c_int64, c_int32]
    L.cce_b200_de_peer_collect.restype = c_int32
    L.cce_b200_de_peer_collect.argtypes = [c_void_p, c_int64, c_int64, c_void_p, c_int32, c_void_p, c_void_p]
    L.cce_b200_de_peer_collect_push.restype = c_int32
    L.cce_b200_de_peer_collect_push.argtypes = [
        c_void_p, c_int64, c_int64, POINTER(c_void_p), c_int32, c_int32, c_int32, c_void_p, c_void_p,
    ]  # fmt: skip
    L.cce_b200_de_peer_scatter.restype = c_int32
    L.cce_b200_de_peer_scatter.argtypes = [
        c_void_p, c_int32, c_int64, c_int64, c_int32, c_void_p, c_int32, c_int64, c_void_p, c_void_p, c_void_p,
    ]  # fmt: skip
    L.cce_b200_gemm.restype = c_int32
    L.cce_b200_gemm.argtypes = [
        c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_int64, c_int64,
        c_int32, c_int32, c_int32, c_int32, c_int32, c_void_p, c_void_p, c_void_p,
    ]  # fmt: skip
    L.cce_b200_read_status.restype = c_int32
    L.cce_b200_read_status.argtypes = [c_void_p, c_void_p, POINTER(c_int32)]
    L.cce_b200_profile_enable.restype = c_int32
    L.cce_b200_profile_enable.argtypes = [c_int32]
    L.cce_b200_profile_wait_counters.restype = c_int32
    L.cce_b200_profile_wait_counters.argtypes = [c_void_p]
    L.cce_b200_profile_read.restype = c_int32
    L.cce_b200_profile_read.argtypes = [POINTER(ctypes.c_double), POINTER(c_int64)]
    L.cce_b200_launch_count.restype = c_int64
    L.cce_b200_launch_count.argtypes = []
    L.cce_b200_strerror.restype = c_char_p
    L.cce_b200_strerror.argtypes = [c_int32]
    L.cce_b200_last_cuda_error.restype = c_int32
    L.cce_b200_version.restype = c_int32
    _lib = L
    return L


def check(rc: int, what: str) -> None:
    if rc != 0:
        L = lib()
        msg = L.cce_b200_strerror(rc).decode()
        raise NativeError(f"{what}: {msg} (code {rc}, cuda {L.cce_b200_last_cuda_error()})")


def _ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def stream_ptr(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def debug_checks() -> bool:
    """``CCE_B200_DEBUG=1``: read the device status word back after every call (synchronises)."""
    return os.environ.get("CCE_B200_DEBUG", "0") not in ("", "0")


def make_operands(
    e: torch.Tensor,
    c: torch.Tensor,
    bias: torch.Tensor | None,
    valids: torch.Tensor | None,
    softcap: float | None,
    n_rows_dev: torch.Tensor | None = None,
) -> Operands:
    """Describe ``e`` [n_total, D], ``c`` [V, D], ``bias`` and the valid-row list for the C ABI.

    ``n_rows_dev`` (one int64 on the device) is the length of the list when the host never read it:
    ``valids`` is then the whole list buffer and its size the upper bound of the row count."""
    if not e.is_cuda:
        raise RuntimeError("cut_cross_entropy (B200 backend) needs CUDA tensors; it has no CPU path")
    if e.dtype not in (torch.float16, torch.bfloat16, torch.float32):
        raise NotImplementedError(f"e/c of dtype {e.dtype} are not supported by this backend (bf16, fp16, fp32 are)")
    assert e.dim() == 2 and c.dim() == 2 and e.dtype == c.dtype
    assert e.stride(1) == 1 and c.stride(1) == 1
    if valids is not None:
        assert valids.dim() == 1 and valids.is_contiguous() and valids.dtype in (torch.int32, torch.int64)
    if bias is not None:
        assert bias.dim() == 1 and bias.is_contiguous() and bias.dtype in _DTYPE_CODE
    op = Operands()
    op.e, op.c, op.bias, op.valids = e.data_ptr(), c.data_ptr(), _ptr(bias), _ptr(valids)
    op.n_total = e.size(0)
    op.n_rows = e.size(0) if valids is None else valids.numel()
    op.V, op.D = c.size(0), c.size(1)
    op.lde, op.ldc = e.stride(0) if e.size(0) > 1 else e.size(1), c.stride(0) if c.size(0) > 1 else c.size(1)
    op.dtype = _DTYPE_CODE[e.dtype]
    op.bias_dtype = _DTYPE_CODE[bias.dtype] if bias is not None else DT_F32
    op.valids_dtype = IDX_I64 if (valids is not None and valids.dtype == torch.int64) else IDX_I32
    op.has_softcap = int(softcap is not None)
    op.softcap = float(softcap) if softcap is not None else 0.0
    if n_rows_dev is not None:
        assert valids is not None and n_rows_dev.dtype == torch.int64 and n_rows_dev.is_cuda
        op.n_rows_dev = n_rows_dev.data_ptr()
    return op


def workspace(nbytes: int, device: torch.device) -> torch.Tensor:
    return torch.empty(max(int(nbytes), 256), dtype=torch.uint8, device=device)


def finish(ws: torch.Tensor, what: str) -> None:
    """Optional post-call check of the kernels' status word."""
    if debug_checks():
        word = c_int32(0)
        rc = lib().cce_b200_read_status(ws.data_ptr(), stream_ptr(ws.device), ctypes.byref(word))
        if rc != 0:
            raise NativeError(f"{what}: kernel status word {word.value:#x} ({lib().cce_b200_strerror(rc).decode()})")
