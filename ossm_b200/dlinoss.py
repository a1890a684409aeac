"""D-LinOSS scan op with ossm's signature: ``run_dlinoss(variant, a_diag, g_diag, step, bu)``.

Mirror of ``src/ossm/models/_dlinoss_scan.py`` (``run_dlinoss`` :630-680, the
four ``autograd.Function`` bridges :458-627 and the ``torch.library`` ops
:182-404) for B200.  Differences from the reference, all on purpose:

* one ``autograd.Function`` serves the four variants; it saves the chunk carries
  (16 B per series per 32 steps) instead of the full ``[L,B,P,2]`` trajectory and
  returns a contiguous ``x`` instead of a stride-2 view;
* CUDA tensors never fall back to PyTorch: a kernel error is raised to the
  caller (the reference swallows it and reruns in Python, :656-680);
* float64 / complex128 inputs are rejected instead of silently taking a
  different code path.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
from torch import Tensor

from . import kernels

__all__ = ["run_dlinoss", "run_dlinoss_imex1", "has_kernels", "extension_error", "DLinossScanFn"]

_SUPPORTED_VARIANTS: Tuple[str, ...] = ("imex1", "imex2", "im", "ex")

# ---- torch.library registration ---------------------------------------------
# Same schemas as the reference's ``ossm::dlinoss_*`` ops, under this package's
# own namespace (the reference registers ``ossm::*`` itself once this package is
# installed as ``ossm._kernels``; defining them here as well would collide).
_LIB: Optional[torch.library.Library] = None


def _register_ops() -> None:
    global _LIB
    if _LIB is not None:
        return
    lib = torch.library.Library("ossm_b200", "DEF")
    for variant in _SUPPORTED_VARIANTS:
        fwd = getattr(kernels, f"dlinoss_{variant}_forward")
        bwd = getattr(kernels, f"dlinoss_{variant}_backward")
        lib.define(f"dlinoss_{variant}_forward(Tensor a_diag, Tensor g_diag, Tensor step, Tensor bu) -> Tensor")
        lib.define(f"dlinoss_{variant}_backward(Tensor a_diag, Tensor g_diag, Tensor step, Tensor bu, "
                   "Tensor states, Tensor grad_output) -> (Tensor, Tensor, Tensor, Tensor)")
        lib.impl(f"dlinoss_{variant}_forward", fwd, "CUDA")
        lib.impl(f"dlinoss_{variant}_backward", bwd, "CUDA")

        def _fwd_meta(a_diag, g_diag, step, bu):
            return bu.new_empty((*bu.shape, 2))

        def _bwd_meta(a_diag, g_diag, step, bu, states, grad_output):
            return (torch.empty_like(a_diag), torch.empty_like(g_diag), torch.empty_like(step),
                    torch.empty_like(bu))

        lib.impl(f"dlinoss_{variant}_forward", _fwd_meta, "Meta")
        lib.impl(f"dlinoss_{variant}_backward", _bwd_meta, "Meta")
    _LIB = lib


_register_ops()


def has_kernels(variant: Optional[str] = None) -> bool:
    """``True`` when the compiled library is loadable (``_dlinoss_scan.py:416-435``)."""
    if variant is not None and variant.lower() not in _SUPPORTED_VARIANTS:
        raise ValueError(f"Unknown D-LinOSS variant '{variant}'.")
    try:
        from . import _lib

        _lib.load()
        return True
    except (RuntimeError, OSError):
        return False


def extension_error() -> Optional[Exception]:
    try:
        from . import _lib

        _lib.load()
        return None
    except (RuntimeError, OSError) as exc:
        return exc


class DLinossScanFn(torch.autograd.Function):
    """Autograd bridge (counterpart of ``_DlinossImex1Fn`` etc., ``_dlinoss_scan.py:458-627``)."""

    @staticmethod
    def forward(ctx, variant: str, a_diag: Tensor, g_diag: Tensor, step: Tensor, bu: Tensor) -> Tensor:
        needs_grad = any(ctx.needs_input_grad[1:])
        x, _, carries = kernels.lti_scan_forward(variant, a_diag, g_diag, step, bu, want_carries=needs_grad)
        ctx.variant = variant
        if needs_grad:
            ctx.save_for_backward(a_diag, g_diag, step, bu, carries)
        return x

    @staticmethod
    def backward(ctx, grad_output: Tensor):
        a_diag, g_diag, step, bu, carries = ctx.saved_tensors
        grad_a, grad_g, grad_step, grad_bu = kernels.lti_scan_backward(
            ctx.variant, a_diag, g_diag, step, bu, carries, grad_output.contiguous())
        return None, grad_a, grad_g, grad_step, grad_bu


def run_dlinoss(variant: str, a_diag: Tensor, g_diag: Tensor, step: Tensor, bu: Tensor) -> Tensor:
    """Evaluate the D-LinOSS recurrence; returns ``x`` with the shape of ``bu`` ``[L,B,P]``.

    ``a_diag, g_diag, step``: float32 ``[P]`` (already projected by the layer),
    ``bu``: complex64 ``[L,B,P]`` time-major, on a CUDA device.
    """
    variant = variant.lower()
    if variant not in _SUPPORTED_VARIANTS:
        raise ValueError(f"Unknown D-LinOSS variant '{variant}'.")
    if bu.numel() == 0:
        return bu
    if (a_diag.dtype == torch.float64 or g_diag.dtype == torch.float64 or step.dtype == torch.float64
            or bu.dtype == torch.complex128):
        raise RuntimeError("ossm_b200: the D-LinOSS scan runs in float32/complex64; float64 inputs are not supported")
    if not bu.is_contiguous():
        bu = bu.contiguous()
    return DLinossScanFn.apply(variant, a_diag.contiguous(), g_diag.contiguous(), step.contiguous(), bu)


def run_dlinoss_imex1(a_diag: Tensor, g_diag: Tensor, step: Tensor, bu: Tensor) -> Tensor:
    """Backward-compatible wrapper (``_dlinoss_scan.py:683-686``)."""
    return run_dlinoss("imex1", a_diag, g_diag, step, bu)
