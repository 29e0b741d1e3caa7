"""Imports the reference's own model files, unmodified, on top of the NumPy stand-ins in
`oracle/_shim` (TEST INFRASTRUCTURE ONLY; used to make and to check the `tests/golden/ref_*.npz`
fixtures, never by the library or by a timed benchmark region).

The reference checkout is found through the environment variable CSSM_REFERENCE_ROOT (default
`/root/reference`).  Where it is absent `available()` is False and callers skip: the committed
fixtures carry the reference's outputs to machines without the checkout.

`src/models/__init__.py` of the reference imports every backbone; the loader avoids running it by
registering an empty package object whose `__path__` is the reference's `src/models` folder and
importing the wanted files (`cssm`, `simple_cssm`, `cssm_shvit`, ...) as its submodules, so
their relative imports (`from .math import ...`) resolve to the reference's own files.
"""
from __future__ import annotations

import importlib
import os
import sys
import types

_PKG = "cssm_reference_models"
_SHIM = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_shim")


def reference_root() -> str:
    return os.environ.get("CSSM_REFERENCE_ROOT", "/root/reference")


def available() -> bool:
    return os.path.isfile(os.path.join(reference_root(), "src", "models", "cssm.py"))


def _ensure_shim():
    real = [m for m in ("jax", "flax") if m in sys.modules
            and not getattr(sys.modules[m], "__file__", "").startswith(_SHIM)]
    if real:
        raise RuntimeError(f"real {real} already imported; the stand-ins cannot take their names")
    if _SHIM not in sys.path:
        sys.path.insert(0, _SHIM)
    import jax  # noqa: F401
    import flax  # noqa: F401


def load(module: str = "cssm"):
    """Returns the reference's `src/models/<module>.py` as an imported module object."""
    if not available():
        raise FileNotFoundError(f"no reference checkout under {reference_root()}")
    _ensure_shim()
    if _PKG not in sys.modules:
        pkg = types.ModuleType(_PKG)
        pkg.__path__ = [os.path.join(reference_root(), "src", "models")]
        pkg.__package__ = _PKG
        sys.modules[_PKG] = pkg
    return importlib.import_module(f"{_PKG}.{module}")
