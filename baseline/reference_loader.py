"""Imports the UNMODIFIED reference (apple/ml-cross-entropy) beside this repository's package.

Both packages are called ``cut_cross_entropy``.  The reference is installed, untouched, under
``baseline/_ref`` (``python -m pip install --no-index --no-build-isolation --no-deps --target
baseline/_ref <reference checkout>``).  :func:`load_reference` imports it from there while this
repository's modules are set aside, then files the reference's modules under the prefix
``cce_reference`` in ``sys.modules`` and puts this repository's modules back, so that

    import cut_cross_entropy                       # this repository
    ref = load_reference()                         # the reference, same process
    ref.linear_cross_entropy(e, c, t, impl="cce")  # its Triton kernels

work side by side.  All of the reference's imports are module-level and absolute, so once it is
imported its functions keep referring to its own modules.  Used by ``bench.py`` (the reference arm
and the ``ref_gpu`` figures) and by ``tests/test_gpu_reference.py``; nothing under
``ml-cross-entropy_b200/`` imports this file.
"""

from __future__ import annotations

import importlib
import sys
from pathlib import Path
from types import ModuleType

REF_DIR = Path(__file__).resolve().parent / "_ref"
_PKG = "cut_cross_entropy"
_ALIAS = "cce_reference"
_loaded: ModuleType | None = None


def reference_available() -> tuple[bool, str]:
    """(True, "") when the reference is installed under ``baseline/_ref``, else (False, why)."""
    if not (REF_DIR / _PKG / "__init__.py").exists():
        return False, f"{REF_DIR}/{_PKG} is missing (reference not installed in this checkout)"
    return True, ""


def load_reference() -> ModuleType:
    """The reference's top-level package object (``linear_cross_entropy``, ``VocabParallelOptions``, ...)."""
    global _loaded
    if _loaded is not None:
        return _loaded
    ok, why = reference_available()
    if not ok:
        raise ImportError(why)

    def ours() -> dict[str, ModuleType]:
        return {k: v for k, v in sys.modules.items() if k == _PKG or k.startswith(_PKG + ".")}

    saved = ours()
    for k in saved:
        del sys.modules[k]
    sys.path.insert(0, str(REF_DIR))
    try:
        ref = importlib.import_module(_PKG)
        for sub in ("utils", "vocab_parallel", "cce", "torch_compile"):
            importlib.import_module(f"{_PKG}.{sub}")
        origin = Path(ref.__file__).resolve()
        assert REF_DIR in origin.parents, f"imported {origin}, not the copy under {REF_DIR}"
        mods = ours()
    finally:
        sys.path.remove(str(REF_DIR))
        for k in ours():
            del sys.modules[k]
        sys.modules.update(saved)
    for k, v in mods.items():
        sys.modules[_ALIAS + k[len(_PKG):]] = v
    _loaded = ref
    return ref
