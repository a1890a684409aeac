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
                D: Optional[Tensor], delta_bias: Optional[Tensor] = None, delta_softplus: bool = False) -> Tensor:
        needs_grad = any(ctx.needs_input_grad)
        out, states = kernels.selective_scan_fwd(inputs, dt, A, B, C, gate, D, save_states=needs_grad,
                                                 delta_bias=delta_bias, delta_softplus=delta_softplus)
        ctx.has_gate = gate is not None
        ctx.has_skip = D is not None
        ctx.has_bias = delta_bias is not None
        ctx.delta_softplus = bool(delta_softplus)
        if needs_grad:
            none = inputs.new_empty(0)
            ctx.save_for_backward(inputs, dt, A, B, C, gate if gate is not None else none,
                                  D if D is not None else none, delta_bias if delta_bias is not None else none,
                                  states)
        return out

    @staticmethod
    def backward(ctx, grad_output: Tensor):
        inputs, dt, A, B, C, gate, D, bias, states = ctx.saved_tensors
        res = kernels.selective_scan_bwd(
            grad_output, inputs, dt, A, B, C, gate if ctx.has_gate else None, states, D if ctx.has_skip else None,
            delta_bias=bias if ctx.has_bias else None, delta_softplus=ctx.delta_softplus)
        du, ddt, dA, dB, dC, dz, dD = res[:7]
        dbias = res[7] if len(res) > 7 else None
        return du, ddt, dA, dB, dC, dz, dD, dbias, None


def selective_scan(inputs: Tensor, dt: Tensor, A: Tensor, B: Tensor, C: Tensor, gate: Optional[Tensor] = None,
                   D: Optional[Tensor] = None, delta_bias: Optional[Tensor] = None,
                   delta_softplus: bool = False) -> Tensor:
    """``out[b,d,t] = (sum_n C[b,t,n] h[b,d,t,n] + D[d] u) * silu(gate)`` with
    ``h_t = exp(dt A) h_{t-1} + dt B u``.  Shapes: ``inputs, dt, gate [B,D,L]``, ``A [D,N]``,
    ``B, C [B,L,N]``, ``D [D]``.  ``delta_bias [D]`` / ``delta_softplus`` fold the mixer's
    ``softplus(dt_proj(.))`` (``mambarec.py:155``) into the scan: pass the projection without its bias
    as ``dt`` and the bias here, and the separate softplus pass over ``[B,D,L]`` disappears."""
    if inputs.numel() == 0:
        return inputs
    return SelectiveScanFn.apply(inputs, dt, A, B, C, gate, D, delta_bias, delta_softplus)


def try_selective_scan(inputs: Tensor, dt: Tensor, A: Tensor, B: Tensor, C: Tensor,
                       gate: Optional[Tensor]) -> Optional[Tensor]:
    """Drop-in for ``ossm.models._selective_scan.try_selective_scan``."""
    return selective_scan(inputs, dt, A, B, C, gate)
