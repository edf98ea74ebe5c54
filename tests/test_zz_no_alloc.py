"""The no-allocation form of the forward log-sum-exp, called through the C ABI.

`cce_b200_lse_forward_static` serves callers that cannot give the library a workspace: programs
without a device allocator of their own, processes whose device memory is already fully reserved
by something else, loops that must avoid the device-wide synchronisation of cudaMalloc/cudaFree.
Its scratch is a fixed array inside the library, shared by all calls on a device, so the test
checks two calls in a row (the second on a different, smaller problem, so stale contents of the
array would show) against the workspace form, and that an oversized problem is refused.

Collected last on purpose (file name): a run that stops at the first failure has then already
run every other test.  It passes on its own in a fresh process and after the other tests.
"""

from __future__ import annotations

import pytest
import torch
from conftest import planted_inputs

pytestmark = pytest.mark.gpu


def _static_lse(e, c, bias, softcap):
    from cut_cross_entropy import _native

    L = _native.lib()
    op = _native.make_operands(e, c, bias, None, softcap)
    lse = torch.full((e.size(0),), float("nan"), dtype=torch.float32, device=e.device)
    rc = L.cce_b200_lse_forward_static(op, lse.data_ptr(), torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    return rc, lse


def test_static_scratch_entry_point_matches_workspace_entry_point():
    from cut_cross_entropy import _native
    from cut_cross_entropy.cce_lse_forward import cce_lse_forward_kernel

    L = _native.lib()
    cases = [(1000, 5000, 256, True, 20.0), (255, 507, 128, False, None)]
    for n, v, d, has_bias, softcap in cases:  # two calls in a row on the shared array
        e, c, bias, _ = planted_inputs(n, v, d, torch.bfloat16, "cuda", seed=n, bias=has_bias)
        bias = None if bias is None else bias.float()
        rc, got = _static_lse(e, c, bias, softcap)
        assert rc == 0, L.cce_b200_strerror(rc)
        want = cce_lse_forward_kernel(e, c, bias, softcap=softcap)
        torch.testing.assert_close(got, want, rtol=0, atol=1e-6)
        gt = e.float() @ c.float().T
        if bias is not None:
            gt = gt + bias
        if softcap is not None:
            gt = torch.tanh(gt / softcap) * softcap
        torch.testing.assert_close(got, torch.logsumexp(gt, -1), rtol=0, atol=2e-3)


def test_static_scratch_entry_point_refuses_what_does_not_fit():
    from cut_cross_entropy import _native

    L = _native.lib()
    # a valid-row list forces a packed copy of e (4096 x 2048 x 2 bytes = 16 MiB) > 8 MiB of scratch
    e = torch.zeros(4096, 2048, dtype=torch.bfloat16, device="cuda")
    c = torch.zeros(512, 2048, dtype=torch.bfloat16, device="cuda")
    valids = torch.arange(4096, device="cuda", dtype=torch.int32)
    op = _native.make_operands(e, c, None, valids, None)
    assert L.cce_b200_lse_workspace_bytes(op) > (8 << 20)
    lse = torch.empty(4096, device="cuda")
    rc = L.cce_b200_lse_forward_static(op, lse.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert rc == -7 and b"fixed buffer" in L.cce_b200_strerror(rc)
