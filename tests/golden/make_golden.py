"""Generates the golden fixtures in this folder from the reference implementation.

Usage (in a container that has the reference checkout; it is not needed to run the tests):

    TORCH_COMPILE_DISABLE=1 python tests/golden/make_golden.py /path/to/ml-cross-entropy [case ...]

(with case names, only those fixtures are rewritten).

It imports the reference's ``cut_cross_entropy`` package from that path and calls its
``linear_cross_entropy(..., impl="torch_compile")`` — the materialised-logits code in
``cut_cross_entropy/torch_compile.py:18-117`` — on CPU, in float32, and differentiates it with
autograd.  ``TORCH_COMPILE_DISABLE=1`` makes ``torch.compile`` a no-op, so the same Python
runs eagerly (no inductor build).  Inputs are drawn in bf16 (the dtype of the GPU tests) and
widened to float32 for the reference, so that the fixtures hold the exact answer for the
stored low-precision inputs.  Each fixture stores inputs, options and outputs.
"""

from __future__ import annotations

import os
import sys
from pathlib import Path

import torch

HERE = Path(__file__).resolve().parent

# name, N(rows), T(sequence length for the 2-D view), V, D, options
CASES = [
    ("plain", 128, 32, 300, 72, dict()),
    ("ignored", 128, 32, 300, 72, dict(ignored=0.2)),
    ("bias_softcap", 128, 32, 300, 72, dict(bias=True, softcap=20.0, ignored=0.2)),
    ("shift1_sum", 128, 32, 300, 72, dict(shift=1, reduction="sum", ignored=0.2)),
    ("shift2_none_zloss", 128, 32, 300, 72, dict(shift=2, reduction="none", z_loss=True, bias=True, ignored=0.2)),
    ("mean_zloss_softcap", 128, 32, 300, 72, dict(z_loss=True, softcap=30.0)),
    ("odd_shapes", 252, 63, 507, 123, dict(bias=True, ignored=0.2, shift=1)),
    ("wide_vocab", 64, 64, 1100, 64, dict(reduction="sum", bias=True)),
    # large enough for several forward bands, and (with a 1 MB logit-gradient buffer) for several
    # vocabulary chunks / several passes of the block-list backward
    ("multi_band", 700, 100, 2500, 192, dict(ignored=0.2, bias=True, softcap=25.0, z_loss=True)),
]


def make_inputs(N, T, V, D, opts, seed):
    g = torch.Generator().manual_seed(seed)
    e = (torch.randn(N, D, generator=g) / D**0.5).to(torch.bfloat16)
    c = torch.randn(V, D, generator=g).to(torch.bfloat16)
    half = min(N, V) // 2
    c[:half] = e[:half]  # half the rows get one dominant logit, as in the reference's tests
    bias = (torch.randn(V, generator=g) * 0.02).to(torch.bfloat16) if opts.get("bias") else None
    targets = torch.randint(0, V, (N,), generator=g)
    frac = opts.get("ignored", 0.0)
    if frac:
        idx = torch.randperm(N, generator=g)[: int(frac * N)]
        targets[idx] = -100
    return e.view(N // T, T, D), c, bias, targets.view(N // T, T)


def main(ref_root: str, only: tuple[str, ...] = ()) -> None:
    assert os.environ.get("TORCH_COMPILE_DISABLE") == "1", "run with TORCH_COMPILE_DISABLE=1"
    sys.path.insert(0, ref_root)
    import cut_cross_entropy as ref
    from cut_cross_entropy.utils import compute_z_loss

    assert Path(ref.__file__).resolve().is_relative_to(Path(ref_root).resolve()), ref.__file__
    torch.set_float32_matmul_precision("highest")
    for i, (name, N, T, V, D, opts) in enumerate(CASES):
        if only and name not in only:
            continue
        e16, c16, b16, targets = make_inputs(N, T, V, D, opts, seed=100 + i)
        e = e16.float().requires_grad_(True)
        c = c16.float().requires_grad_(True)
        b = b16.float().requires_grad_(True) if b16 is not None else None
        shift = opts.get("shift", 0)
        reduction = opts.get("reduction", "mean")
        loss, lse = ref.linear_cross_entropy(
            e, c, targets, bias=b, softcap=opts.get("softcap"), shift=shift, reduction=reduction,
            impl="torch_compile", return_lse=True,
        )
        total = loss.sum()
        z = None
        if opts.get("z_loss"):
            z = compute_z_loss(lse, targets, shift)
            total = total + 1e-2 * z
        total.backward()
        out = dict(
            name=name, opts=opts, e=e16, c=c16, bias=b16, targets=targets,
            loss=loss.detach(), lse=lse.detach(), z_loss=None if z is None else z.detach(),
            z_coef=1e-2, de=e.grad.detach(), dc=c.grad.detach(),
            dbias=None if b is None else b.grad.detach(),
        )
        torch.save(out, HERE / f"{name}.pt")
        print(f"{name}: loss {loss.detach().flatten()[:3].tolist()} |de| {e.grad.abs().max():.3e} |dc| {c.grad.abs().max():.3e}")


if __name__ == "__main__":
    if len(sys.argv) < 2:
        raise SystemExit("usage: make_golden.py /path/to/ml-cross-entropy [case ...]")
    main(sys.argv[1], tuple(sys.argv[2:]))
