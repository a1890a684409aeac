"""Installs this package behind ossm's own plugin boundary.

ossm's op shims do ``from ossm import _kernels`` at import time
(``_dlinoss_scan.py:165``, ``_linoss_scan.py:14``, ``_selective_scan.py:75``).
Seeding ``sys.modules["ossm._kernels"]`` with :mod:`ossm_b200.kernels` *before*
``import ossm`` makes every shim (and the ``torch.ops.ossm.*`` library it
registers) call into ``libossm_b200.so``.  ``patch_ops=True`` additionally swaps
ossm's op functions for the leaner ones of this package (no full-state
materialisation, CUDA backward for LinOSS, bf16 selective scan, selective D-LinOSS from chunk carries).
"""
from __future__ import annotations

import importlib
import sys


def install_as_ossm_kernels(patch_ops: bool = True) -> None:
    from . import kernels

    already = "ossm" in sys.modules
    sys.modules["ossm._kernels"] = kernels
    if already:
        # shims captured their kernel module at import; make the attribute agree at least
        setattr(sys.modules["ossm"], "_kernels", kernels)
    if not patch_ops:
        return
    try:
        ossm = importlib.import_module("ossm")
    except ImportError:
        return
    setattr(ossm, "_kernels", kernels)
    from . import diag, dlinoss, linoss, sdlinoss, selective_scan

    mods = {}
    for name in ("_dlinoss_scan", "dlinoss", "_sdlinoss_scan", "sdlinoss", "_linoss_scan", "linoss", "_selective_scan",
                 "mambarec", "lru", "s5"):
        try:
            mods[name] = importlib.import_module(f"ossm.models.{name}")
        except ImportError:
            continue
    for name in ("_dlinoss_scan", "dlinoss"):
        if name in mods:
            mods[name].run_dlinoss = dlinoss.run_dlinoss
    # selective D-LinOSS: the layer imports run_sdlinoss by name (sdlinoss.py:13)
    for name in ("_sdlinoss_scan", "sdlinoss"):
        if name in mods:
            mods[name].run_sdlinoss = sdlinoss.run_sdlinoss
    if "linoss" in mods:
        mods["linoss"]._run_associative_scan = linoss.run_associative_scan
        mods["linoss"].try_run_scan = linoss.try_run_scan
    if "_linoss_scan" in mods:
        mods["_linoss_scan"].try_run_scan = linoss.try_run_scan
    # LRU / S5: the layers call ``_LRUScanFn.apply`` / ``_S5ScanFn.apply`` (lru.py:176, s5.py:294)
    if "lru" in mods:
        mods["lru"]._LRUScanFn = diag.DiagScanFn
    if "s5" in mods:
        mods["s5"]._S5ScanFn = diag.DiagScanFn
    if "_selective_scan" in mods:
        mods["_selective_scan"].try_selective_scan = selective_scan.try_selective_scan
    if "mambarec" in mods:
        # the mixer binds the function under a private alias (mambarec.py:13)
        mods["mambarec"]._try_selective_scan = selective_scan.try_selective_scan
