"""Neighbours of the selective scan inside ossm's Mamba mixer, folded into kernels of this library.

``_MambaMixer.forward`` (``src/ossm/models/mambarec.py:136-184``) runs, around the scan,

* ``transpose -> F.pad -> conv1d(groups=D) -> SiLU -> transpose`` on ``x [B, L, D]``: here one kernel
  (:func:`causal_conv1d_silu`) that reads ``x`` once and writes the result both time-contiguous (the scan's
  operand) and channel-contiguous (the ``x_proj`` GEMM's operand);
* ``dt = softplus(dt_proj(dt_raw))`` as a separate pass over ``[B, D, L]``: here the scan takes the projection
  without its bias, the bias as ``delta_bias`` and ``delta_softplus=True``.

:func:`mamba_mixer_forward` is the mixer's forward written with those two; ``install_as_ossm_kernels(
fuse_mixer=True)`` puts it behind the unmodified ``_MambaMixer`` class (same parameters, same state dict).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.nn.functional as F
from torch import Tensor

from . import _lib
from .kernels import _p, _require_cuda, _stream

__all__ = ["causal_conv1d_silu", "mamba_mixer_forward", "MAX_TAPS"]

MAX_TAPS = 4


def _row_pitch(x: Tensor) -> int:
    """``x [B, L, D]`` with contiguous channels and rows ``ldx`` floats apart (a dense tensor or the first /
    second half of a ``[B, L, 2D]`` one); raises otherwise."""
    B, L, D = x.shape
    if x.stride(2) != 1 or (L > 1 and x.stride(0) != L * x.stride(1)) or x.stride(1) < D:
        raise RuntimeError("ossm_b200: causal_conv1d_silu needs x [B, L, D] with contiguous channels and evenly spaced rows")
    return int(x.stride(1))


class _ConvSiluFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x: Tensor, weight: Tensor, bias: Optional[Tensor]) -> Tuple[Tensor, Tensor]:
        B, L, D = x.shape
        taps = weight.size(-1)
        w2 = weight.reshape(D, taps).contiguous()
        b1 = bias.contiguous() if bias is not None else None
        ldx = _row_pitch(x)
        out_bdl = torch.empty((B, D, L), dtype=torch.float32, device=x.device)
        out_bld = torch.empty((B, L, D), dtype=torch.float32, device=x.device)
        with torch.cuda.device(x.device):
            rc = _lib.load().ossm_b200_conv1d_silu_forward(_p(x), ldx, _p(w2), _p(b1), _p(out_bdl), _p(out_bld), B, L, D,
                                                           taps, _stream(x.device))
        _lib.check(rc, "conv1d_silu_forward")
        ctx.save_for_backward(x, w2, b1 if b1 is not None else x.new_empty(0))
        ctx.has_bias = bias is not None
        ctx.weight_shape = tuple(weight.shape)
        return out_bdl, out_bld

    @staticmethod
    def backward(ctx, g_bdl: Optional[Tensor], g_bld: Optional[Tensor]):
        x, w2, b1 = ctx.saved_tensors
        bias = b1 if ctx.has_bias else None
        B, L, D = x.shape
        taps = w2.size(1)
        g1 = g_bdl.contiguous() if g_bdl is not None else None
        g2 = g_bld.contiguous() if g_bld is not None else None
        grad_x = torch.empty((B, L, D), dtype=torch.float32, device=x.device)
        grad_w = torch.empty_like(w2)
        grad_b = torch.empty(D, dtype=torch.float32, device=x.device) if bias is not None else None
        if g1 is None and g2 is None:
            return torch.zeros_like(grad_x), torch.zeros(ctx.weight_shape, device=x.device), (
                torch.zeros_like(grad_b) if grad_b is not None else None)
        with torch.cuda.device(x.device):
            rc = _lib.load().ossm_b200_conv1d_silu_backward(_p(x), _row_pitch(x), _p(w2), _p(bias), _p(g1), _p(g2),
                                                            _p(grad_x), _p(grad_w), _p(grad_b), B, L, D, taps,
                                                            _stream(x.device))
        _lib.check(rc, "conv1d_silu_backward")
        return grad_x, grad_w.view(ctx.weight_shape), grad_b


def causal_conv1d_silu(x: Tensor, weight: Tensor, bias: Optional[Tensor] = None) -> Tuple[Tensor, Tensor]:
    """``silu(conv1d(left-padded x^T) + bias)`` for ``x [B, L, D]`` float32 (channels contiguous, rows evenly
    spaced), ``weight [D, 1, K]`` or ``[D, K]`` (``K <= 4``), ``bias [D]``.  Returns the result as ``[B, D, L]``
    and as ``[B, L, D]``."""
    _require_cuda("x", x)
    if x.dim() != 3 or x.dtype != torch.float32:
        raise RuntimeError("ossm_b200: causal_conv1d_silu needs a float32 [B, L, D] tensor")
    D = x.size(2)
    if weight.numel() % max(D, 1) or weight.size(0) != D or weight.size(-1) > MAX_TAPS or weight.dtype != torch.float32:
        raise RuntimeError(f"ossm_b200: conv weight must be float32 [D, 1, K] with K <= {MAX_TAPS}")
    if bias is not None and (bias.shape != (D,) or bias.dtype != torch.float32):
        raise RuntimeError("ossm_b200: conv bias must be float32 [D]")
    if x.numel() == 0:
        return x.new_zeros(x.size(0), D, x.size(1)), x.new_zeros(x.shape)
    return _ConvSiluFn.apply(x, weight, bias)


def mamba_mixer_forward(mixer, inputs: Tensor) -> Tensor:
    """Forward of ossm's ``_MambaMixer`` (``mambarec.py:136-184``) on its own parameters with the conv + SiLU
    kernel and the step transform folded into the scan.  ``inputs [B, L, d_model]`` on a CUDA device."""
    from .selective_scan import selective_scan

    if inputs.ndim != 3:
        raise ValueError("Inputs to Mamba mixer must have shape (batch, length, channels)")
    batch, seqlen, _ = inputs.shape
    if seqlen == 0:
        return torch.zeros_like(inputs)
    xz = mixer.in_proj(inputs).float()
    d_inner = mixer.d_inner
    x, z = xz[..., :d_inner], xz[..., d_inner:]
    x_bdl, x_bld = causal_conv1d_silu(x, mixer.conv1d.weight.float(),
                                      mixer.conv1d.bias.float() if mixer.conv1d.bias is not None else None)
    proj = mixer.x_proj(x_bld.to(mixer.x_proj.weight.dtype)).float()
    dt_raw, B_gen, C_gen = torch.split(proj, [mixer.dt_rank, mixer.d_state, mixer.d_state], dim=-1)
    # dt_proj without its bias, produced time-contiguous [B, D, L]; bias and softplus happen inside the scan
    dt_bdl = torch.matmul(mixer.dt_proj.weight.float(), dt_raw.transpose(1, 2))
    A = -torch.exp(mixer.A_log.float())
    gated = selective_scan(x_bdl, dt_bdl, A, B_gen, C_gen, z.transpose(1, 2), None,
                           delta_bias=mixer.dt_proj.bias.float(), delta_softplus=True)
    return mixer.out_proj(gated.transpose(1, 2).to(mixer.out_proj.weight.dtype))
