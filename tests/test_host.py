"""CPU tests: host-side logic of the package and the shape of the C-ABI library.
No kernel is launched here."""

from __future__ import annotations

import ctypes
import re
from pathlib import Path

import pytest
import torch

from oracle import cce_oracle as O

ROOT = Path(__file__).resolve().parent.parent


def test_library_loads_and_exports_every_declared_symbol():
    from cut_cross_entropy import _build, _native

    _build.build()
    declared = set()
    for header in sorted((ROOT / "include").glob("*.h")):  # the product ABI and the test/measurement hooks
        found = set(re.findall(r"\b(cce_b200_[a-z_0-9]+)\s*\(", header.read_text()))
        assert found, f"no declarations found in {header.name}"
        declared |= found
    L = _native.lib()
    for name in sorted(declared):
        assert hasattr(L, name), f"{name} declared under include/ but not exported"
    assert declared == set(_native.EXPORTS)
    assert L.cce_b200_version() >= 1
    assert L.cce_b200_strerror(0) == b"ok" and b"workspace" in L.cce_b200_strerror(-3)
    assert L.cce_b200_launch_count() >= 0


def test_ctypes_structs_match_the_header_layout():
    from cut_cross_entropy import _native

    # 4 pointers, 6 int64, 4 int32, 1 float -> 100 bytes, padded to 8-byte alignment, then 1 pointer
    assert ctypes.sizeof(_native.Operands) == 112 and _native.Operands.n_rows_dev.offset == 104
    assert _native.BackwardArgs.op.offset == 0 and _native.BackwardArgs.lse.offset == 112
    # no GPU here: argument checks must reject, not crash
    L = _native.lib()
    op = _native.Operands()
    assert L.cce_b200_lse_workspace_bytes(op) == 0
    assert L.cce_b200_lse_forward(op, None, None, None, 0, None) == -1
    assert L.cce_b200_backward(None, None, 0, None) == -1


def test_presets():
    from cut_cross_entropy.cce_utils import CCEPreset, CCEPresets, LinearCrossEntropyImpl

    user = CCEPreset(filter_eps=1e-3, accum_e_fp32=False, accum_c_fp32=False, filter_e_grad=False, filter_c_grad=True)
    assert CCEPresets.build_for_impl("cce", user) == user
    for name in ("cce_exact", "cce_kahan_full", "cce_kahan_full_c_full_e"):
        o = CCEPresets.build_for_impl(name, user)
        assert o["filter_eps"] is None and o["accum_e_fp32"] and o["accum_c_fp32"]
    o = CCEPresets.build_for_impl("cce_kahan_full_c", user)
    assert (o["filter_eps"], o["filter_c_grad"], o["filter_e_grad"]) == ("auto", False, True)
    o = CCEPresets.build_for_impl("cce_kahan_full_e", user)
    assert (o["filter_eps"], o["filter_c_grad"], o["filter_e_grad"]) == ("auto", True, False)
    o = CCEPresets.build_for_impl("cce_kahan", user)
    assert o["filter_eps"] == 1e-3 and o["accum_e_fp32"] and o["accum_c_fp32"] and not o["filter_e_grad"]
    with pytest.raises(ValueError):
        CCEPresets.build_for_impl("torch_compile", user)
    assert {m.name.lower() for m in LinearCrossEntropyImpl} - {"torch_compile"} == CCEPresets.names
    assert user["filter_eps"] == 1e-3  # the caller's dict is not modified


@pytest.mark.parametrize("shift", [0, 1, 3])
@pytest.mark.parametrize("frac", [0.0, 0.3])
def test_flat_valids_against_oracle(shift, frac):
    from cut_cross_entropy.utils import _build_flat_valids, handle_reduction_none

    g = torch.Generator().manual_seed(shift)
    t = torch.randint(0, 50, (3, 11), generator=g)
    if frac:
        t[torch.rand(3, 11, generator=g) < frac] = -100
    got = _build_flat_valids(t, -100, shift)
    want = O.flat_valids(t, -100, shift)
    if shift == 0 and frac == 0.0:
        assert got is None
    else:
        assert got.dtype == (torch.int32 if shift == 0 else torch.int64)
        assert torch.equal(got.long(), want)
        vals = torch.arange(1.0, want.numel() + 1)
        assert torch.equal(handle_reduction_none(t.shape, got, shift, vals), O.scatter_none(t.shape, want, shift, vals))


def test_eps_and_z_loss_known_answers():
    from cut_cross_entropy.utils import _handle_eps, compute_z_loss

    assert _handle_eps("auto", torch.bfloat16) == 2.0**-12
    assert _handle_eps("auto", torch.float16) == 2.0**-15
    assert _handle_eps(None, torch.float16) is None and _handle_eps(0.5, torch.float16) == 0.5
    with pytest.raises(RuntimeError):
        _handle_eps("big", torch.float16)
    lse = torch.arange(1, 11, dtype=torch.float64)
    assert compute_z_loss(lse, reduction="sum").item() == pytest.approx(385.0)
    targets = torch.full((10,), -100)
    targets[3], targets[5] = 1, 2
    assert compute_z_loss(lse, targets, reduction="mean").item() == pytest.approx((16.0 + 36.0) / 2)
    assert compute_z_loss(lse[:9], targets, shift=1, reduction="sum").item() == pytest.approx(9.0 + 25.0)
    with pytest.raises(ValueError):
        compute_z_loss(lse, reduction="max")


def test_public_api_validation_and_no_cpu_path():
    from cut_cross_entropy import VocabParallelOptions, linear_cross_entropy

    e, c, t = torch.randn(4, 8, 16).bfloat16(), torch.randn(32, 16).bfloat16(), torch.randint(0, 32, (4, 8))
    with pytest.raises(ValueError, match="Shift must be"):
        linear_cross_entropy(e, c, t, shift=8)
    with pytest.raises(ValueError, match="Bias has"):
        linear_cross_entropy(e, c, t, bias=torch.zeros(31))
    with pytest.raises(ValueError, match="Expected c.size"):
        linear_cross_entropy(e, c, t, vocab_parallel_options=VocabParallelOptions(0, 16))
    with pytest.raises(NotImplementedError):
        linear_cross_entropy(e, c, t, impl="torch_compile")
    # CPU tensors: the backend refuses instead of falling back
    with pytest.raises(RuntimeError, match="no CPU path"):
        linear_cross_entropy(e, c, t)


def test_partition():
    from cut_cross_entropy.vocab_parallel import partition_n_into_range

    for n, w in ((10, 3), (262144, 8), (5, 8)):
        for r in range(w):
            assert partition_n_into_range(n, r, w) == O.partition_n_into_range(n, r, w)


def _operands(n_total, n_rows, V, D, dtype=1, valids=False):
    """A description with dummy (never dereferenced) 256-byte aligned addresses: the planning
    functions of the C ABI are host arithmetic on shapes, strides and alignments."""
    from cut_cross_entropy import _native

    op = _native.Operands()
    op.e, op.c = 0x10000, 0x20000
    op.valids = 0x30000 if valids else None
    op.n_total, op.n_rows, op.V, op.D = n_total, n_rows, V, D
    op.lde = op.ldc = D
    op.dtype, op.bias_dtype, op.valids_dtype = dtype, 2, 0
    return op


def test_workspace_planning_is_host_arithmetic_with_the_documented_sizes():
    from cut_cross_entropy import _native

    L = _native.lib()
    # Gemma-2-2B head, dense aligned bf16 operands, no row list: only the status block and the
    # per-band partial sums -> "about 4 MiB", as the header says of the no-allocation entry point
    op = _operands(8192, 8192, 256000, 2304)
    need = L.cce_b200_lse_workspace_bytes(op)
    assert 3 << 20 < need < 5 << 20
    assert L.cce_b200_tile_max_elems(op) == (8192 // 128) * 4 * 1000
    # a row list adds the packed copy of the listed rows; fp32 operands add three-term bf16 splits
    # of both matrices (3 x 2 bytes per element)
    with_rows = L.cce_b200_lse_workspace_bytes(_operands(8192, 7783, 256000, 2304, valids=True))
    assert 0 < with_rows - need < 7783 * 2304 * 2 + (1 << 20)
    split = L.cce_b200_lse_workspace_bytes(_operands(8192, 8192, 256000, 2304, dtype=2))
    assert split - need >= (8192 + 256000) * 2304 * 6
    # an odd hidden size is padded to a multiple of 8 elements in staged copies of both operands
    odd = L.cce_b200_lse_workspace_bytes(_operands(256, 256, 512, 123))
    assert odd >= (256 + 512) * 128 * 2
    # nonsense is refused with size 0
    assert L.cce_b200_lse_workspace_bytes(_operands(8, 9, 512, 64)) == 0  # more listed rows than rows
    assert L.cce_b200_lse_workspace_bytes(_operands(8, 8, 0, 64)) == 0
    assert L.cce_b200_lse_workspace_bytes(_operands(8, 8, 512, 64, dtype=7)) == 0
    # the row-list builder: one int per block of 2048 labels, rounded up to 256 bytes
    assert L.cce_b200_valid_rows_workspace_bytes(1) == 256
    assert L.cce_b200_valid_rows_workspace_bytes(2048 * 64) == 256
    assert L.cce_b200_valid_rows_workspace_bytes(2048 * 64 + 1) == 512
    assert L.cce_b200_valid_rows_workspace_bytes(-1) == 0


def test_backward_planning_respects_the_logit_gradient_buffer_cap(monkeypatch):
    """The backward never holds more than the cap (512 MiB unless CCE_B200_GBUF_MB says otherwise)
    of recomputed logit gradients, whatever the problem size; everything else in its workspace is
    the fp32 dE scratch, staged operands and index arrays."""
    from cut_cross_entropy import _native

    L = _native.lib()

    def need(n, V, D, tile_max, mb=None, **kw):
        if mb is None:
            monkeypatch.delenv("CCE_B200_GBUF_MB", raising=False)
        else:
            monkeypatch.setenv("CCE_B200_GBUF_MB", str(mb))
        a = _native.BackwardArgs()
        a.op = _operands(n, n, V, D)
        a.lse, a.targets, a.d_out, a.d_e, a.d_c = 0x40000, 0x50000, 0x60000, 0x70000, 0x80000
        a.d_out_numel, a.grad_scale = 1, 1.0
        a.has_filter, a.filter_eps, a.filter_e, a.filter_c = 1, 2.0**-12, 1, 1
        a.tile_max = 0x90000 if tile_max else None
        for k, v in kw.items():
            setattr(a, k, v)
        return L.cce_b200_backward_workspace_bytes(a)

    de32 = 8192 * 2304 * 4
    for tile_max in (False, True):  # chunked form / block-list form
        total = need(8192, 256000, 2304, tile_max)
        assert (512 << 20) * 0.5 < total - de32 < (512 << 20) + (16 << 20), (tile_max, total)
    # a tenth of the cap: a tenth of the buffer
    small = need(8192, 256000, 2304, True, mb=52)
    assert small - de32 < (52 << 20) + (16 << 20)
    # a problem whose every tile fits the pool asks for exactly its tiles, not for the cap
    tiny = need(256, 1024, 128, True)
    assert tiny < 2 << 20
    # without a gradient for e there is no fp32 dE scratch
    assert need(8192, 256000, 2304, True) - need(8192, 256000, 2304, True, d_e=None) >= de32
    # a long batch (chunked form): the buffer grows so that 16 chunks suffice, up to 2 GB; an explicit cap is kept
    g16 = 2 * 65536 * 152064 / 16
    long_batch = need(65536, 152064, 3584, False)
    # (the chunk width is then rounded down to whole waves of CTAs, to no less than half of it)
    assert g16 / 2 - (64 << 20) < long_batch - 65536 * 3584 * 4 < g16 + (64 << 20), long_batch
    assert long_batch > need(65536, 152064, 3584, False, mb=512)
    assert need(65536, 152064, 3584, False, mb=512) - 65536 * 3584 * 4 < (512 << 20) + (64 << 20)
    assert need(400000, 152064, 3584, False) - 400000 * 3584 * 4 < (2048 << 20) + (256 << 20)
    # refused descriptions
    assert L.cce_b200_backward_workspace_bytes(None) == 0


def test_entry_points_reject_bad_arguments_before_touching_the_gpu():
    from cut_cross_entropy import _native

    L = _native.lib()
    op = _operands(128, 128, 512, 64)
    # missing outputs, workspaces and label arrays
    assert L.cce_b200_lse_forward(op, None, None, None, 0, None) == -1
    assert L.cce_b200_lse_forward(op, 0x1000, None, 0x1001, 1 << 30, None) == -2  # workspace not 256-byte aligned
    assert L.cce_b200_lse_forward(op, 0x1000, None, 0x1000, 16, None) == -3  # workspace too small
    assert L.cce_b200_indexed_neg_dot(op, None, 0, 0, 0x1000, None) == -1
    assert L.cce_b200_indexed_neg_dot(op, 0x1000, -1, 0, 0x1000, None) == -1  # negative shift
    # the fixed scratch of the no-allocation entry point is 8 MiB: a packed copy of 65536 x 4096
    # rows cannot fit, and is refused before anything is looked up on a device
    big = _operands(65536, 65536, 262144, 4096, valids=True)
    assert L.cce_b200_lse_forward_static(big, 0x1000, None) == -7
    # the row-list builder
    args = (0x1000, 64, 16, 0, -100, 0x2000, _native.IDX_I32, 0x3000, 0x4000)
    assert L.cce_b200_valid_rows(*args[:7], None, args[8], 256, None) == -1  # nowhere to put the count
    assert L.cce_b200_valid_rows(0x1000, 64, 24, 0, -100, 0x2000, 0, 0x3000, 0x4000, 256, None) == -1  # 64 % 24
    assert L.cce_b200_valid_rows(0x1000, 64, 16, -1, -100, 0x2000, 0, 0x3000, 0x4000, 256, None) == -1
    assert L.cce_b200_valid_rows(0x1000, 64, 16, 0, -100, 0x2000, 9, 0x3000, 0x4000, 256, None) == -1  # index type
    assert L.cce_b200_valid_rows(0x1000, 64, 16, 0, -100, 0x2000, 0, 0x3000, 0x4000, 0, None) == -3  # workspace
    assert L.cce_b200_valid_rows(0x1000, 1 << 31, 1, 0, -100, 0x2000, 0, 0x3000, 0x4000, 1 << 30, None) == -7  # int32 rows
    for code in range(0, -9, -1):
        assert L.cce_b200_strerror(code) != b"unknown error"
    assert L.cce_b200_strerror(-99) == b"unknown error"


def test_pending_row_list_resolution_rules():
    """What `resolve()` hands on once the length is known (the reference's conventions,
    utils.py:28-49): `None` without a shift when every row is listed, else the first `count`
    entries of the buffer; the wait happens once."""
    from cut_cross_entropy.utils import PendingValidRows

    class Done:
        waits = 0

        def synchronize(self):
            Done.waits += 1

    rows = torch.arange(10, dtype=torch.int32)
    p = PendingValidRows(rows, torch.tensor([10]), Done(), n_total=10, shift=0)
    assert p.resolve() is None and p.resolve() is None and Done.waits == 1
    p = PendingValidRows(rows, torch.tensor([7]), Done(), n_total=10, shift=0)
    assert torch.equal(p.resolve(), rows[:7]) and p.resolve().data_ptr() == rows.data_ptr()
    p = PendingValidRows(rows.long(), torch.tensor([10]), Done(), n_total=10, shift=1)
    assert p.resolve().numel() == 10  # with a shift the list is always returned
    p = PendingValidRows(rows, torch.tensor([0]), Done(), n_total=10, shift=0)
    assert p.resolve().numel() == 0


def test_reference_arm_of_the_benchmark_prints_the_contract_line():
    """Without a GPU `bench.py --impl reference` times the CPU port on a bounded sample and prints
    one JSON line with the metric, the config and the keys of the GPU arm's line.  It uses every
    host core it may run on even when the launcher exported OMP_NUM_THREADS=1, as torchrun does."""
    import json
    import os
    import subprocess
    import sys

    out = subprocess.run(
        [sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--config", "gemma2-2b-head-small",
         "--steps", "3", "--warmup", "3"],
        check=True, capture_output=True, text=True, timeout=600, cwd=ROOT, env=dict(os.environ, OMP_NUM_THREADS="1"),
    )  # fmt: skip
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["metric"] == "linear-CE fwd+bwd tokens/s"
    assert line["unit"] == "tokens/s" and line["higher_is_better"] is True and line["n_gpus"] == 1
    assert line["steps"] == 3 and line["warmup"] == 3 and line["ms_per_step"] > 0 and line["value"] > 0
    assert line["config"]["workload"] == "gemma2-2b-head-small" and line["vs_baseline"] is None
    cb = line["cpu_baseline"]
    assert cb["kind"] == "port" and cb["value"] == line["value"] and "1024 rows" in cb["sample"]
    assert cb["cores"] == len(os.sched_getaffinity(0)) and line["reference_kind"] == "cpu_port"
    assert line["e2e"] == {"value": line["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert line["gpu_launches"] == 0


def test_reference_and_this_package_import_side_by_side():
    """baseline/reference_loader.py files the unmodified reference under another name without
    disturbing this repository's package of the same name (skipped where the reference is not installed)."""
    import sys

    from baseline.reference_loader import load_reference, reference_available

    ok, why = reference_available()
    if not ok:
        pytest.skip(why)
    import cut_cross_entropy as ours

    ref = load_reference()
    import cut_cross_entropy as again

    assert again is ours and ref is not ours
    assert "baseline/_ref" in ref.__file__ and "ml-cross-entropy_b200" in ours.__file__
    assert sys.modules["cce_reference"] is ref and "cce_reference.utils" in sys.modules
    assert hasattr(ref, "linear_cross_entropy") and ref.linear_cross_entropy is not ours.linear_cross_entropy


def test_mode_switches_of_the_python_layer():
    """set_sync_free / set_vocab_ordering return the previous setting and reject unknown modes."""
    from cut_cross_entropy import cce

    prev = cce.set_sync_free(False)
    assert cce.set_sync_free(True) is False and cce.set_sync_free(prev) is True
    prev = cce.set_vocab_ordering("mean")
    assert cce.set_vocab_ordering(True) == "mean" and cce.set_vocab_ordering(False) == "max"
    assert cce.set_vocab_ordering(prev) == "off"
    with pytest.raises(ValueError):
        cce.set_vocab_ordering("alphabetical")
    k = torch.tensor([0.5, 3.0, -1.0, 2.0])
    assert cce.sort_logit_avg(k).tolist() == [1, 3, 0, 2] and cce.sort_logit_avg(k).dtype == torch.int32


def test_host_side_of_the_fused_de_reduction(monkeypatch):
    """Row ownership arithmetic, argument checks and switches of the cross-rank sum of dE that the
    dE product performs (reference: the all-reduce of vocab_parallel/utils.py:68-76); no GPU."""
    from cut_cross_entropy import _native, cce_backward
    from cut_cross_entropy.vocab_parallel import peer_reduce

    L = _native.lib()
    # whole 128-row blocks dealt round-robin: rank r owns blocks r, r + world, ...
    assert L.cce_b200_de_peer_rows(7782, 8) == 1024  # 61 blocks -> 8 per rank
    assert L.cce_b200_de_peer_rows(7782, 2) == 31 * 128
    assert L.cce_b200_de_peer_rows(128, 8) == 128 and L.cce_b200_de_peer_rows(0, 8) == 0
    assert L.cce_b200_de_peer_rows(-1, 8) == 0 and L.cce_b200_de_peer_rows(10, 0) == 0
    # the struct carries the accumulators of at most MAX_PEERS ranks, after the event handle
    a = _native.BackwardArgs()
    assert _native.BackwardArgs.de_peer_acc.offset == _native.BackwardArgs.de_peer_world.offset + 8
    assert len(a.de_peer_acc) == _native.MAX_PEERS == 8
    # argument checks reject before any CUDA call
    p = ctypes.c_void_p()
    assert L.cce_b200_peer_buffer_create(0, ctypes.byref(p), None) == -1
    assert L.cce_b200_peer_buffer_open(None, ctypes.byref(p)) == -1
    assert L.cce_b200_peer_buffer_close(None) == -1 and L.cce_b200_peer_buffer_destroy(None) == -1
    assert L.cce_b200_de_peer_collect(None, 128, 64, None, _native.DT_BF16, None, None) == -1
    assert L.cce_b200_de_peer_collect_push(None, 128, 64, None, 2, 0, _native.DT_BF16, None, None) == -1
    assert L.cce_b200_de_peer_scatter(None, 2, 128, 64, _native.DT_BF16, None, 0, 100, None, None, None) == -1
    # SMs left to the exchange: by size unless the environment says otherwise
    monkeypatch.delenv("CCE_B200_EXCHANGE_SMS", raising=False)
    assert cce_backward._exchange_sms(8192, 2304, True) == 32  # 75 MB of fp32 partial sums
    assert cce_backward._exchange_sms(8192, 2304, False) == 0  # the process group's reduction keeps every SM busy itself
    assert cce_backward._exchange_sms(32768, 4096, True) == 0  # 537 MB
    monkeypatch.setenv("CCE_B200_EXCHANGE_SMS", "48")
    assert cce_backward._exchange_sms(32768, 4096, False) == 48
    # no process group, or CPU tensors: the process group's reduction is used
    assert peer_reduce.peer_accumulators(None, torch.device("cpu"), 1 << 20, 1 << 20) is None
    monkeypatch.setenv("CCE_B200_PEER_REDUCE", "0")
    assert not peer_reduce._enabled()
