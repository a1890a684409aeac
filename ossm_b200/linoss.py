"""LinOSS scans with ossm's signatures.

* :func:`run_associative_scan` / :class:`LinossScanFn` / :func:`try_run_scan`
  mirror ``_run_associative_scan``, ``_LinossScanFn`` and ``try_run_scan``
  (``src/ossm/models/linoss.py:57-157``, ``_linoss_scan.py:44-63``): generic
  complex 2x2 transition, materialised ``[L,B,P,2]`` states.  The backward is one
  CUDA kernel instead of the reference's Python loop over ``L``.
* :func:`run_linoss` / :func:`linoss_recurrence` are the path the LinOSS layer
  needs (``LinOSSLayer._apply_im`` / ``_apply_imex`` / ``_run_recurrence``,
  ``linoss.py:244-315``): real transition built from ``(A, step)`` inside the
  kernel, no ``b_elems`` / state tensors, backward by carry recompute.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
from torch import Tensor

from . import kernels

__all__ = ["try_run_scan", "LinossScanFn", "run_associative_scan", "run_linoss", "linoss_recurrence"]


def try_run_scan(m11: Tensor, m12: Tensor, m21: Tensor, m22: Tensor, b_seq: Tensor) -> Optional[Tensor]:
    """Same contract as ``_linoss_scan.try_run_scan`` except that errors raise
    (there is no Python fallback to return ``None`` for)."""
    if b_seq.numel() == 0:
        return b_seq
    return kernels.linoss_scan(m11, m12, m21, m22, b_seq)


class LinossScanFn(torch.autograd.Function):
    """Counterpart of ``_LinossScanFn`` (``linoss.py:57-151``)."""

    @staticmethod
    def forward(ctx, a_matrix: Tensor, b_seq: Tensor) -> Tensor:
        length = b_seq.size(0)
        if length <= 1:
            ctx.trivial = True
            ctx.save_for_backward(a_matrix, b_seq)
            return b_seq
        ctx.trivial = False
        b_seq = b_seq.contiguous()
        cd = b_seq.dtype
        m = [a_matrix[:, i, j].to(dtype=cd).contiguous() for i in (0, 1) for j in (0, 1)]
        states = kernels.linoss_scan(m[0], m[1], m[2], m[3], b_seq)
        ctx.save_for_backward(a_matrix, states)
        return states

    @staticmethod
    def backward(ctx, grad_output: Tensor) -> Tuple[Tensor, Tensor]:
        a_matrix, states = ctx.saved_tensors
        if grad_output.size(0) == 0:
            return torch.zeros_like(a_matrix), grad_output
        if ctx.trivial:
            # length-1 sequences: s_0 = b_0, no dependence on the transition
            return torch.zeros_like(a_matrix), grad_output
        grad_output = grad_output.contiguous()
        cd = grad_output.dtype
        m = [a_matrix[:, i, j].to(dtype=cd).contiguous() for i in (0, 1) for j in (0, 1)]
        grad_m, grad_b = kernels.linoss_scan_backward(m[0], m[1], m[2], m[3], states, grad_output)
        if not torch.is_complex(a_matrix):
            grad_m = grad_m.real            # linoss.py:133-138
        return grad_m.to(dtype=a_matrix.dtype), grad_b


def run_associative_scan(a_matrix: Tensor, b_seq: Tensor) -> Tensor:
    """``_run_associative_scan(a_matrix [P,2,2], b_seq [L,B,P,2])`` (``linoss.py:154-157``)."""
    return LinossScanFn.apply(a_matrix, b_seq)


class LinossLayerScanFn(torch.autograd.Function):
    """Fused LinOSS IM / IMEX recurrence on a time-major ``bu``."""

    @staticmethod
    def forward(ctx, variant: str, a_diag: Tensor, step: Tensor, bu: Tensor) -> Tensor:
        needs_grad = any(ctx.needs_input_grad[1:])
        x, _, carries = kernels.lti_scan_forward(variant, a_diag, None, step, bu, want_carries=needs_grad)
        ctx.variant = variant
        if needs_grad:
            ctx.save_for_backward(a_diag, step, bu, carries)
        return x

    @staticmethod
    def backward(ctx, grad_output: Tensor):
        a_diag, step, bu, carries = ctx.saved_tensors
        grad_a, _, grad_step, grad_bu = kernels.lti_scan_backward(ctx.variant, a_diag, None, step, bu, carries,
                                                                  grad_output.contiguous())
        return None, grad_a, grad_step, grad_bu


def run_linoss(discretization: str, a_diag: Tensor, step: Tensor, bu_seq: Tensor) -> Tensor:
    """LinOSS recurrence on ``bu_seq [L,B,P]`` complex64 (time-major); returns ``x [L,B,P]``.

    ``a_diag = relu(A_diag)`` and ``step = sigmoid(steps)`` as the layer passes them
    (``linoss.py:213-214``)."""
    if discretization not in ("IM", "IMEX"):
        raise ValueError(f"Unsupported discretization '{discretization}'.")
    if bu_seq.numel() == 0:
        return bu_seq
    if a_diag.dtype == torch.float64 or step.dtype == torch.float64 or bu_seq.dtype == torch.complex128:
        raise RuntimeError("ossm_b200: the LinOSS scan runs in float32/complex64; float64 inputs are not supported")
    variant = "linoss_im" if discretization == "IM" else "linoss_imex"
    return LinossLayerScanFn.apply(variant, a_diag.contiguous(), step.contiguous(), bu_seq.contiguous())


def linoss_recurrence(discretization: str, a_diag: Tensor, step: Tensor, bu: Tensor) -> Tensor:
    """``LinOSSLayer._apply_im`` / ``_apply_imex`` (``linoss.py:244-315``): ``bu`` is
    batch-major ``[B,L,P]`` and so is the result."""
    batch, length, ssm = bu.shape
    if length == 0:
        return bu.new_zeros(batch, 0, ssm)
    x = run_linoss(discretization, a_diag, step, bu.permute(1, 0, 2).contiguous())
    return x.permute(1, 0, 2).contiguous()
