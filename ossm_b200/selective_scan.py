"""Mamba selective scan with ossm's signature:
``try_selective_scan(inputs, dt, A, B, C, gate)`` (``src/ossm/models/_selective_scan.py:127-196``)
and the autograd bridge ``_SelectiveScanFn`` (:199-297).

Differences from the reference, on purpose: bfloat16 ``inputs/B/C/gate`` are
accepted (state arithmetic stays float32) where the reference returns ``None``
for anything but float32; an optional skip vector ``D`` is supported; the
backward recomputes the ungated output instead of saving it; errors raise
instead of returning ``None``.
"""
from __future__ import annotations

from typing import Optional

import torch
from torch import Tensor

from . import kernels

__all__ = ["try_selective_scan", "selective_scan", "SelectiveScanFn", "has_kernels"]


def has_kernels() -> bool:
    try:
        from . import _lib

        _lib.load()
        return True
    except (RuntimeError, OSError):
        return False


class SelectiveScanFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, inputs: Tensor, dt: Tensor, A: Tensor, B: Tensor, C: Tensor, gate: Optional[Tensor],
                D: Optional[Tensor]) -> Tensor:
        needs_grad = any(ctx.needs_input_grad)
        out, states = kernels.selective_scan_fwd(inputs, dt, A, B, C, gate, D, save_states=needs_grad)
        ctx.has_gate = gate is not None
        ctx.has_skip = D is not None
        if needs_grad:
            ctx.save_for_backward(inputs, dt, A, B, C, gate if gate is not None else inputs.new_empty(0),
                                  D if D is not None else inputs.new_empty(0), states)
        return out

    @staticmethod
    def backward(ctx, grad_output: Tensor):
        inputs, dt, A, B, C, gate, D, states = ctx.saved_tensors
        du, ddt, dA, dB, dC, dz, dD = kernels.selective_scan_bwd(
            grad_output, inputs, dt, A, B, C, gate if ctx.has_gate else None, states, D if ctx.has_skip else None)
        return du, ddt, dA, dB, dC, dz, dD


def selective_scan(inputs: Tensor, dt: Tensor, A: Tensor, B: Tensor, C: Tensor, gate: Optional[Tensor] = None,
                   D: Optional[Tensor] = None) -> Tensor:
    """``out[b,d,t] = (sum_n C[b,t,n] h[b,d,t,n] + D[d] u) * silu(gate)`` with
    ``h_t = exp(dt A) h_{t-1} + dt B u``.  Shapes: ``inputs, dt, gate [B,D,L]``, ``A [D,N]``,
    ``B, C [B,L,N]``, ``D [D]``."""
    if inputs.numel() == 0:
        return inputs
    return SelectiveScanFn.apply(inputs, dt, A, B, C, gate, D)


def try_selective_scan(inputs: Tensor, dt: Tensor, A: Tensor, B: Tensor, C: Tensor,
                       gate: Optional[Tensor]) -> Optional[Tensor]:
    """Drop-in for ``ossm.models._selective_scan.try_selective_scan``."""
    return selective_scan(inputs, dt, A, B, C, gate)
