"""Selective D-LinOSS scan with ossm's ``run_sdlinoss`` signature.

Mirror of ``src/ossm/models/_sdlinoss_scan.py:382-452`` (``run_sdlinoss`` and the four
``_Sdlinoss*Fn`` autograd functions): same argument meaning, shape rules and messages, but the
forward keeps the state only every 32 steps (16 B per series per chunk) instead of the full
``[L,B,M,2]`` trajectory, and there is no PyTorch fallback -- tensors must be float32 /
complex64 on a CUDA device.
"""
from __future__ import annotations

from typing import Tuple

import torch
from torch import Tensor

from . import kernels

__all__ = ["SdlinossScanFn", "run_sdlinoss", "has_kernels"]

_SUPPORTED_VARIANTS: Tuple[str, ...] = kernels.SDLINOSS_VARIANTS


def has_kernels(variant=None) -> bool:
    if variant is None:
        return True
    if variant.lower() not in _SUPPORTED_VARIANTS:
        raise ValueError(f"Unknown selective D-LinOSS variant '{variant}'.")
    return True


def _normalize_param(param: Tensor, name: str, length: int, batch: int, ssm: int, *, device, dtype) -> Tensor:
    # _sdlinoss_scan.py:105-141
    if param.device != device:
        raise ValueError(f"{name} must be on device {device}, got {param.device}.")
    if param.dtype != dtype:
        raise TypeError(f"{name} must have dtype {dtype}, got {param.dtype}.")
    if param.dim() == 1 and param.shape[0] == ssm:
        return param.unsqueeze(0).unsqueeze(0)
    if param.dim() == 2 and param.shape[1] == ssm:
        if param.shape[0] == length:
            return param.unsqueeze(1)
        if param.shape[0] == batch:
            return param.unsqueeze(0)
    if param.dim() == 3 and param.shape[2] == ssm:
        if param.shape[0] in (1, length) and param.shape[1] in (1, batch):
            return param
    raise ValueError(f"{name} must be shaped as (M,), (L,M), (B,M), or (L,B,M); got {tuple(param.shape)}.")


class SdlinossScanFn(torch.autograd.Function):
    """``x = scan(A, G, step, bu)`` for parameters already viewed as ``[L|1, B|1, M]``."""

    @staticmethod
    def forward(ctx, variant: str, A: Tensor, G: Tensor, step: Tensor, bu: Tensor) -> Tensor:
        needs_grad = any(ctx.needs_input_grad)
        A, G, step, bu = (t.contiguous() for t in (A, G, step, bu))
        x, _, carries = kernels.sdlinoss_scan_forward(variant, A, G, step, bu, want_carries=needs_grad)
        ctx.variant = variant
        if needs_grad:
            ctx.save_for_backward(A, G, step, bu, carries)
        return x

    @staticmethod
    def backward(ctx, grad_output: Tensor):
        A, G, step, bu, carries = ctx.saved_tensors
        grad_A, grad_G, grad_step, grad_bu = kernels.sdlinoss_scan_backward(
            ctx.variant, A, G, step, bu, grad_output.contiguous(), carries=carries)
        return None, grad_A, grad_G, grad_step, grad_bu


def run_sdlinoss(variant: str, a_diag: Tensor, g_diag: Tensor, step: Tensor, bu: Tensor) -> Tensor:
    """``x [L,B,M]`` of the selective D-LinOSS recurrence; ``a_diag, g_diag, step`` shaped ``(M,)``,
    ``(L,M)``, ``(B,M)`` or ``(L,B,M)``, ``bu`` complex64 ``[L,B,M]``."""
    variant = variant.lower()
    if variant not in _SUPPORTED_VARIANTS:
        raise ValueError(f"Unsupported variant '{variant}'. Expected one of {', '.join(_SUPPORTED_VARIANTS)}.")
    if bu.dim() != 3:
        raise ValueError("bu must be (length, batch, ssm_size) complex.")
    if not bu.is_complex():
        raise TypeError("bu must be complex valued.")
    if bu.dtype != torch.complex64:
        raise TypeError(f"ossm_b200: the selective scan runs in complex64 only, got {bu.dtype}.")
    length, batch, ssm = bu.shape
    views = [_normalize_param(p, n, length, batch, ssm, device=bu.device, dtype=torch.float32)
             for p, n in ((a_diag, "A"), (g_diag, "G"), (step, "step"))]
    if length == 0:
        return bu.new_empty((0, batch, ssm))
    return SdlinossScanFn.apply(variant, views[0], views[1], views[2], bu)
