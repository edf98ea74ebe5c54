"""Implementation names and the option presets behind them.

Mirrors ``cut_cross_entropy/cce_utils.py:8-70`` of the reference: the same enum
members and the same mapping from an ``impl`` name to the five backward options.
One name is added: ``cce_kahan`` (the reference README describes it at
``README.md:108`` but its enum lacks it): filtered like ``cce``, accumulated in fp32.

On this backend every gradient is accumulated in fp32 (TMEM accumulators and fp32
scratch), so ``accum_e_fp32`` / ``accum_c_fp32`` do not change the arithmetic; they
are carried so that callers written against the reference keep working.
"""

from __future__ import annotations

import enum
from typing import TypedDict


class LinearCrossEntropyImpl(enum.IntEnum):
    CCE = enum.auto()
    TORCH_COMPILE = enum.auto()
    CCE_KAHAN_FULL_C = enum.auto()
    CCE_KAHAN_FULL_E = enum.auto()
    CCE_EXACT = enum.auto()
    CCE_KAHAN_FULL_C_FULL_E = enum.auto()
    CCE_KAHAN_FULL = enum.auto()
    CCE_KAHAN = enum.auto()


class CCEPreset(TypedDict):
    filter_eps: float | str | None
    accum_e_fp32: bool
    accum_c_fp32: bool
    filter_e_grad: bool
    filter_c_grad: bool


# impl name -> options it forces (None for "take the caller's")
_FORCED: dict[str, dict] = {
    "cce": {},
    "cce_kahan": dict(accum_e_fp32=True, accum_c_fp32=True),
    "cce_exact": dict(filter_eps=None, accum_e_fp32=True, accum_c_fp32=True),
    "cce_kahan_full": dict(filter_eps=None, accum_e_fp32=True, accum_c_fp32=True),
    "cce_kahan_full_c_full_e": dict(filter_eps=None, accum_e_fp32=True, accum_c_fp32=True),
    "cce_kahan_full_c": dict(
        filter_eps="auto", accum_e_fp32=True, accum_c_fp32=True, filter_e_grad=True, filter_c_grad=False
    ),
    "cce_kahan_full_e": dict(
        filter_eps="auto", accum_e_fp32=True, accum_c_fp32=True, filter_e_grad=False, filter_c_grad=True
    ),
}


class CCEPresets:
    names: set[str] = set(_FORCED)

    @classmethod
    def build_for_impl(cls, impl: str, opts: CCEPreset) -> CCEPreset:
        if impl not in cls.names:
            raise ValueError(f"{impl!r} not in {cls.names}")
        out = CCEPreset(**opts)
        out.update(_FORCED[impl])  # type: ignore[typeddict-item]
        return out
