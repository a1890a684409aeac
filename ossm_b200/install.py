"""Installs this package behind ossm's own plugin boundary.

ossm's op shims do ``from ossm import _kernels`` at import time
(``_dlinoss_scan.py:165``, ``_linoss_scan.py:14``, ``_selective_scan.py:75``).
Seeding ``sys.modules["ossm._kernels"]`` with :mod:`ossm_b200.kernels` *before*
``import ossm`` makes every shim (and the ``torch.ops.ossm.*`` library it
registers) call into ``libossm_b200.so``.  ``patch_ops=True`` additionally swaps
ossm's op functions for the leaner ones of this package (no full-state
materialisation, CUDA backward for LinOSS, bf16 selective scan, selective D-LinOSS from chunk carries).

Scope rule of the swapped functions: inputs this library covers -- CUDA tensors in
float32 / complex64 (plus bfloat16 and ``d_state <= 256`` for the selective scan)
-- always run its kernels, and a failure there raises; nothing on a GPU falls back
silently.  Everything else (CPU tensors of a model moved to the host for export or
evaluation, float64 / complex128 gradcheck inputs, float16, larger state sizes)
is handed to ossm's own function, which takes its PyTorch path exactly as it does
without this package (``_dlinoss_scan.py:648-680``, ``_selective_scan.py:141-145``,
``mambarec.py:172-180``).
"""
from __future__ import annotations

import importlib
import sys

import torch

MAX_D_STATE = 256   # largest Mamba state size of the CUDA kernels (the reference's MAX_DSTATE, selective_scan_common.h:41)


def _covered_complex(bu, *coeffs) -> bool:
    """CUDA, complex64 forcing and float32 coefficients: what the oscillator kernels take."""
    return bool(bu.is_cuda and bu.dtype == torch.complex64
                and all(c is None or (c.is_cuda and c.dtype == torch.float32) for c in coeffs))


def _wrap_dlinoss(ours, original):
    def run_dlinoss(variant, a_diag, g_diag, step, bu):
        if _covered_complex(bu, a_diag, g_diag, step):
            return ours(variant, a_diag, g_diag, step, bu)
        return original(variant, a_diag, g_diag, step, bu)

    run_dlinoss.__doc__ = ours.__doc__
    run_dlinoss.__wrapped__ = original
    return run_dlinoss


def _wrap_sdlinoss(ours, module):
    original = module.run_sdlinoss
    normalize = getattr(module, "_normalize_param", None)
    from_views = getattr(module, "_reference_sdlinoss_states_from_views", None)

    def run_sdlinoss(variant, a_diag, g_diag, step, bu):
        if torch.is_tensor(bu) and bu.dim() == 3 and _covered_complex(bu, a_diag, g_diag, step):
            return ours(variant, a_diag, g_diag, step, bu)
        if (normalize is None or from_views is None or not torch.is_tensor(bu) or bu.dim() != 3
                or not bu.is_complex() or bu.size(0) == 0):
            return original(variant, a_diag, g_diag, step, bu)
        # ossm's run_sdlinoss has no fallback once kernels are present (_sdlinoss_scan.py:414-452);
        # evaluate its own PyTorch recurrence for inputs the kernels do not take
        length, batch, ssm = bu.shape
        real = torch.float64 if bu.dtype == torch.complex128 else torch.float32
        views = [normalize(p, n, length, batch, ssm, device=bu.device, dtype=real)
                 for p, n in ((a_diag, "A"), (g_diag, "G"), (step, "step"))]
        return from_views(variant.lower(), views[0], views[1], views[2], bu)[..., 1]

    run_sdlinoss.__wrapped__ = original
    return run_sdlinoss


def _wrap_try_run_scan(ours):
    def try_run_scan(m11, m12, m21, m22, b_seq):
        if b_seq.is_cuda and b_seq.dtype == torch.complex64:
            return ours(m11, m12, m21, m22, b_seq)
        return None     # ossm's contract for "no kernel": the caller runs its doubling scan (linoss.py:69-76)

    return try_run_scan


def _wrap_associative_scan(ours, original):
    def _run_associative_scan(a_matrix, b_seq):
        if b_seq.is_cuda and b_seq.dtype == torch.complex64:
            return ours(a_matrix, b_seq)
        return original(a_matrix, b_seq)

    return _run_associative_scan


def _wrap_diag_fn(ours, original):
    class _DiagScanDispatch:
        """Stands where ``_LRUScanFn`` / ``_S5ScanFn`` stood: the layers only call ``.apply``."""

        @staticmethod
        def apply(lambda_bar, b_seq):
            if b_seq.is_cuda and b_seq.dtype == torch.complex64:
                return ours.apply(lambda_bar, b_seq)
            return original.apply(lambda_bar, b_seq)

    _DiagScanDispatch.__wrapped__ = original
    return _DiagScanDispatch


def _wrap_try_selective_scan(ours):
    def try_selective_scan(inputs, dt, A, B, C, gate):
        covered = (inputs.is_cuda and inputs.dtype in (torch.float32, torch.bfloat16) and A.dim() == 2
                   and 0 < A.size(1) <= MAX_D_STATE and (gate is None or gate.dtype == inputs.dtype)
                   and B.dtype == inputs.dtype and C.dtype == inputs.dtype)
        if covered:
            return ours(inputs, dt, A, B, C, gate)
        return None     # ossm's contract for "no kernel": the mixer runs _selective_scan_mamba (mambarec.py:172-180)

    return try_selective_scan


def _wrap_mixer_forward(original):
    def forward(self, inputs):
        covered = (inputs.is_cuda and inputs.dtype in (torch.float32, torch.bfloat16) and self.d_conv <= 4
                   and 0 < self.d_state <= MAX_D_STATE and not torch.is_autocast_enabled())
        if covered:
            from .mixer import mamba_mixer_forward

            return mamba_mixer_forward(self, inputs.float()).to(inputs.dtype)
        return original(self, inputs)

    forward.__wrapped__ = original
    return forward


def _layer_covered(self, inputs) -> bool:
    """What the fused layer body takes: a float32 / bfloat16 / float16 CUDA batch of non-empty sequences, float32
    parameters on the same device, no autocast region (ossm's matmuls would then run in the autocast dtype)."""
    return bool(torch.is_tensor(inputs) and inputs.is_cuda and inputs.dim() == 3 and inputs.numel() > 0
                and inputs.dtype in (torch.float32, torch.bfloat16, torch.float16)
                and inputs.size(-1) == self.hidden_dim and self.B.is_cuda and self.B.dtype == torch.float32
                and not torch.is_autocast_enabled())


def _wrap_dlinoss_layer_forward(original):
    def forward(self, inputs):
        if _layer_covered(self, inputs):
            from .dlinoss_layer import dlinoss_layer

            # the class's own parameter projection (dlinoss.py:252-267), then the fused body (dlinoss.py:217-247)
            a_diag, g_diag, step = self._project_parameters(device=inputs.device, dtype=torch.float32)
            y = dlinoss_layer(self.variant, a_diag, g_diag, step, self.B, self.C, self.D, inputs.float())
            return y.to(inputs.dtype)
        return original(self, inputs)

    forward.__wrapped__ = original
    return forward


def _wrap_linoss_layer_forward(original):
    def forward(self, inputs):
        if _layer_covered(self, inputs) and inputs.dtype == torch.float32 and self.discretization in ("IM", "IMEX"):
            from .dlinoss_layer import dlinoss_layer

            # linoss.py:213-214 (parameter projection) and :216-243 (the body)
            a_diag, step = torch.relu(self.A_diag), torch.sigmoid(self.steps)
            return dlinoss_layer("linoss_im" if self.discretization == "IM" else "linoss_imex", a_diag, None, step,
                                 self.B, self.C, self.D, inputs)
        return original(self, inputs)

    forward.__wrapped__ = original
    return forward


def install_as_ossm_kernels(patch_ops: bool = True, fuse_mixer: bool = False, fuse_layer: bool = False) -> None:
    """``fuse_layer=True`` replaces ``DampedLinOSSLayer.forward`` and ``LinOSSLayer.forward`` (the classes, their
    parameters and state dicts stay ossm's) by :func:`ossm_b200.dlinoss_layer.dlinoss_layer`: the four GEMMs on the
    tcgen05 tensor cores with the permutes and the ``D*u`` term inside them, around this package's scan.
    ``fuse_mixer=True`` also replaces ``_MambaMixer.forward`` (the class, its parameters and its state dict
    stay ossm's) by :func:`ossm_b200.mixer.mamba_mixer_forward`: causal conv1d + SiLU in one kernel and
    ``softplus(dt_proj(.))`` folded into the scan (``mambarec.py:143-171``); inputs outside the library's scope
    keep ossm's own forward."""
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
    if "_dlinoss_scan" in mods:
        original = mods["_dlinoss_scan"].run_dlinoss
        original = getattr(original, "__wrapped__", original)      # installing twice must not nest wrappers
        wrapped = _wrap_dlinoss(dlinoss.run_dlinoss, original)
        for name in ("_dlinoss_scan", "dlinoss"):
            if name in mods:
                mods[name].run_dlinoss = wrapped
    # selective D-LinOSS: the layer imports run_sdlinoss by name (sdlinoss.py:13)
    if "_sdlinoss_scan" in mods:
        module = mods["_sdlinoss_scan"]
        if hasattr(module.run_sdlinoss, "__wrapped__"):
            module.run_sdlinoss = module.run_sdlinoss.__wrapped__
        wrapped = _wrap_sdlinoss(sdlinoss.run_sdlinoss, module)
        for name in ("_sdlinoss_scan", "sdlinoss"):
            if name in mods:
                mods[name].run_sdlinoss = wrapped
    if "linoss" in mods:
        original = getattr(mods["linoss"]._run_associative_scan, "__wrapped__", mods["linoss"]._run_associative_scan)
        wrapped = _wrap_associative_scan(linoss.run_associative_scan, original)
        wrapped.__wrapped__ = original
        mods["linoss"]._run_associative_scan = wrapped
        mods["linoss"].try_run_scan = _wrap_try_run_scan(linoss.try_run_scan)
    if "_linoss_scan" in mods:
        mods["_linoss_scan"].try_run_scan = _wrap_try_run_scan(linoss.try_run_scan)
    # LRU / S5: the layers call ``_LRUScanFn.apply`` / ``_S5ScanFn.apply`` (lru.py:176, s5.py:294)
    for name, attr in (("lru", "_LRUScanFn"), ("s5", "_S5ScanFn")):
        if name in mods:
            original = getattr(mods[name], attr)
            original = getattr(original, "__wrapped__", original)
            setattr(mods[name], attr, _wrap_diag_fn(diag.DiagScanFn, original))
    if fuse_layer:
        if "dlinoss" in mods:
            cls = mods["dlinoss"].DampedLinOSSLayer
            cls.forward = _wrap_dlinoss_layer_forward(getattr(cls.forward, "__wrapped__", cls.forward))
        if "linoss" in mods:
            cls = mods["linoss"].LinOSSLayer
            cls.forward = _wrap_linoss_layer_forward(getattr(cls.forward, "__wrapped__", cls.forward))
    if fuse_mixer and "mambarec" in mods:
        cls = mods["mambarec"]._MambaMixer
        original = getattr(cls.forward, "__wrapped__", cls.forward)
        cls.forward = _wrap_mixer_forward(original)
    wrapped = _wrap_try_selective_scan(selective_scan.try_selective_scan)
    if "_selective_scan" in mods:
        mods["_selective_scan"].try_selective_scan = wrapped
    if "mambarec" in mods:
        # the mixer binds the function under a private alias (mambarec.py:13)
        mods["mambarec"]._try_selective_scan = wrapped
