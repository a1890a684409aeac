"""Loads the compiled reference CPU kernels (``oracle/_ref/ossm_ref_kernels.so``).

TEST INFRASTRUCTURE ONLY (see ``oracle/build_ref.py``).  Returns ``None`` when
the shared object has not been built.
"""
from __future__ import annotations

import importlib.machinery
import importlib.util
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "_ref", "ossm_ref_kernels.so")
_MOD = None


def load_reference_kernels():
    global _MOD
    if _MOD is not None:
        return _MOD
    if not os.path.exists(_SO):
        return None
    import torch  # noqa: F401  (libtorch must be loaded before the extension)

    loader = importlib.machinery.ExtensionFileLoader("ossm_ref_kernels", _SO)
    spec = importlib.util.spec_from_loader("ossm_ref_kernels", loader)
    mod = importlib.util.module_from_spec(spec)
    loader.exec_module(mod)
    _MOD = mod
    return mod
