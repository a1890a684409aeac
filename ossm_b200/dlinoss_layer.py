"""The D-LinOSS layer body as one op: ``y = Re(C x) + D u`` with ``x = scan(u B^T)``.

Counterpart of ``DampedLinOSSLayer.forward`` after the parameter projection
(``src/ossm/models/dlinoss.py:217-247``, ``_apply_dlinoss`` :269-278).  The reference runs four real
library GEMMs (``u B_re^T``, ``u B_im^T``, ``x.real C_re^T``, ``x.imag C_im^T``), two permute copies
between batch-major ``[B,L,*]`` and time-major ``[L,B,*]`` and the scan.  Here the projections run on
the tcgen05 tensor cores through :func:`ossm_b200.kernels.gemm_tf32x3` (three TF32 products of split
operands: float32-level accuracy), which read and write the time-major complex scan operands in place:

  forward    bu = gemm(u, [B_re|B_im])  ->  x = scan(bu)  ->  y = gemm(x, [C_re|-C_im]) + D*u   (fused)
  backward   grad_x = gemm(grad_y, [C_re|-C_im]^T)  ->  scan backward  ->
             grad_u = gemm(grad_bu, [B_re|B_im]^T) + D*grad_y                                   (fused)

No permute copy, no real / imaginary split and no separate ``D*u`` pass exist.  The two weight
gradients (``grad_B``, ``grad_C``: reductions over all ``B*L`` rows into ``[2P, H]``) run on the tensor
cores as well (:func:`ossm_b200.kernels.wgrad_tf32x3`, split over the rows, partials summed in a fixed
order) when ``2P`` and ``H`` are multiples of 32, else as strided batched library GEMMs.

Parameters have the reference's shapes: ``B [P, H, 2]``, ``C [H, P, 2]`` (real / imaginary last,
``dlinoss.py:93-98``), ``D [H]``; ``a_diag, g_diag, step [P]`` are the projected coefficients the
layer passes to ``run_dlinoss``.  CUDA float32 only; there is no other path.
"""
from __future__ import annotations

from typing import Optional

import torch
from torch import Tensor

from . import kernels

__all__ = ["dlinoss_layer", "DLinossLayerFn", "pack_input_weights", "pack_output_weights"]


def pack_input_weights(B: Tensor) -> Tensor:
    """``[P, H, 2] -> [2P, H]`` with rows ``(B_re[p], B_im[p])`` interleaved: the GEMM then writes ``bu`` as
    interleaved (re, im) pairs, i.e. complex64."""
    P, H, _ = B.shape
    return B.permute(0, 2, 1).reshape(2 * P, H).contiguous()


def pack_output_weights(C: Tensor) -> Tensor:
    """``[H, P, 2] -> [H, 2P]`` with columns ``(C_re[:,p], -C_im[:,p])`` interleaved, so that the product
    with the interleaved (re, im) pairs of ``x`` is ``Re(C x)``."""
    H, P, _ = C.shape
    # no host constant: a tensor made from a Python list would cost a blocking host-to-device copy per call
    return torch.stack((C[..., 0], -C[..., 1]), dim=-1).reshape(H, 2 * P)


def weight_gradient(X: Tensor, x_time_major: bool, Y: Tensor, y_time_major: bool, batch: int, length: int) -> Tensor:
    """``sum_(b,l) X[row(b,l)]^T Y[row(b,l)]`` -> ``[M, N]``.  On the tensor cores when both widths are multiples of
    32 (column blocks of the operand tiles), otherwise one strided batched library GEMM (cuBLAS, float32)."""
    M, N = X.size(1), Y.size(1)
    if M % 32 == 0 and N % 32 == 0:
        return kernels.wgrad_tf32x3(X, x_time_major, Y, y_time_major, batch, length)
    xb = X.view(length, batch, M).permute(1, 2, 0) if x_time_major else X.view(batch, length, M).transpose(1, 2)
    yb = Y.view(length, batch, N).permute(1, 0, 2) if y_time_major else Y.view(batch, length, N)
    return torch.bmm(xb, yb).sum(0)


class DLinossLayerFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, variant: str, a_diag: Tensor, g_diag: Tensor, step: Tensor, B: Tensor, C: Tensor, D: Tensor,
                u: Tensor) -> Tensor:
        batch, length, hidden = u.shape
        ssm = a_diag.numel()
        dev = u.device
        u2 = u.contiguous().view(batch * length, hidden)
        w_in = pack_input_weights(B)                         # [2P, H]
        w_out = pack_output_weights(C)                       # [H, 2P]
        bu = torch.empty((length, batch, ssm), dtype=torch.complex64, device=dev)
        kernels.gemm_tf32x3(u2, *kernels.split_tf32(w_in), torch.view_as_real(bu).view(length * batch, 2 * ssm),
                            row_map=kernels.ROWS_BATCH_TO_TIME, batch=batch, length=length)
        needs_grad = any(ctx.needs_input_grad)
        x, _, carries = kernels.lti_scan_forward(variant, a_diag, g_diag, step, bu, want_carries=needs_grad)
        y = torch.empty((batch, length, hidden), dtype=torch.float32, device=dev)
        kernels.gemm_tf32x3(torch.view_as_real(x).view(length * batch, 2 * ssm), *kernels.split_tf32(w_out),
                            y.view(batch * length, hidden), aux=u2, diag=D.contiguous(),
                            row_map=kernels.ROWS_TIME_TO_BATCH, batch=batch, length=length)
        ctx.variant = variant
        if needs_grad:
            ctx.save_for_backward(a_diag, g_diag, step, w_in, w_out, D, u2, bu, x, carries)
        return y

    @staticmethod
    def backward(ctx, grad_y: Tensor):
        a_diag, g_diag, step, w_in, w_out, D, u2, bu, x, carries = ctx.saved_tensors
        length, batch, ssm = bu.shape
        hidden = u2.size(1)
        dev = u2.device
        gy = grad_y.contiguous().view(batch * length, hidden)
        # grad_x (torch's convention for complex tensors: d/dre + i d/dim) = grad_y C_re - i grad_y C_im
        grad_x = torch.empty_like(bu)
        kernels.gemm_tf32x3(gy, *kernels.split_tf32(w_out.t().contiguous()),
                            torch.view_as_real(grad_x).view(length * batch, 2 * ssm),
                            row_map=kernels.ROWS_BATCH_TO_TIME, batch=batch, length=length)
        grad_a, grad_g, grad_step, grad_bu = kernels.lti_scan_backward(ctx.variant, a_diag, g_diag, step, bu, carries,
                                                                       grad_x)
        grad_u = torch.empty((batch, length, hidden), dtype=torch.float32, device=dev)
        gbu2 = torch.view_as_real(grad_bu).view(length, batch, 2 * ssm)
        kernels.gemm_tf32x3(gbu2.view(length * batch, 2 * ssm), *kernels.split_tf32(w_in.t().contiguous()),
                            grad_u.view(batch * length, hidden), aux=gy, diag=D.contiguous(),
                            row_map=kernels.ROWS_TIME_TO_BATCH, batch=batch, length=length)
        # weight gradients: sums over every (b, l) row of products of a time-major and a batch-major matrix
        x2 = torch.view_as_real(x).view(length, batch, 2 * ssm)
        grad_w_in = weight_gradient(gbu2.view(length * batch, 2 * ssm), True, u2, False, batch, length)     # [2P, H]
        grad_w_out = weight_gradient(gy, False, x2.view(length * batch, 2 * ssm), True, batch, length)      # [H, 2P]
        grad_D = kernels.colwise_dot(gy, u2) if hidden % 4 == 0 else (gy * u2).sum(0)
        grad_B = grad_w_in.view(ssm, 2, hidden).permute(0, 2, 1).contiguous()
        g3 = grad_w_out.view(hidden, ssm, 2)
        grad_C = torch.stack((g3[..., 0], -g3[..., 1]), dim=-1)
        return None, grad_a, grad_g, grad_step, grad_B, grad_C, grad_D, grad_u


def dlinoss_layer(variant: str, a_diag: Tensor, g_diag: Optional[Tensor], step: Tensor, B: Tensor, C: Tensor, D: Tensor,
                  u: Tensor) -> Tensor:
    """``y [B, L, H]`` of the D-LinOSS layer body for ``u [B, L, H]`` (float32, CUDA).  The LinOSS layer has the same
    body around an undamped recurrence (``linoss.py:199-243``): variants ``linoss_im`` / ``linoss_imex`` with
    ``g_diag=None``."""
    variant = variant.lower()
    if variant not in ("imex1", "imex2", "im", "ex", "linoss_im", "linoss_imex"):
        raise ValueError(f"Unknown D-LinOSS variant '{variant}'.")
    if variant.startswith("linoss"):
        g_diag = None
    elif g_diag is None:
        raise ValueError("the damped variants need g_diag")
    if u.dim() != 3:
        raise ValueError("inputs must have shape (batch, length, hidden_dim).")
    if not u.is_cuda or u.dtype != torch.float32:
        raise RuntimeError("ossm_b200: dlinoss_layer needs float32 CUDA tensors (there is no CPU path)")
    batch, length, hidden = u.shape
    ssm = a_diag.numel()
    if tuple(B.shape) != (ssm, hidden, 2) or tuple(C.shape) != (hidden, ssm, 2) or tuple(D.shape) != (hidden,):
        raise ValueError("B must be [P, H, 2], C [H, P, 2] and D [H]")
    if length == 0 or batch == 0:
        return u.new_zeros(batch, length, hidden)
    # TMA wants 16-byte rows: hidden a multiple of 4 floats, 2P a multiple of 4.  Odd sizes are padded with
    # zero channels / idle oscillators (zero rows of B, zero columns of C), which leave the result unchanged
    # and whose gradients are dropped by the slicing below.
    pad_h = (-hidden) % 4
    pad_p = ssm % 2
    if pad_h or pad_p:
        pad = torch.nn.functional.pad
        u = pad(u, (0, pad_h))
        B = pad(B, (0, 0, 0, pad_h, 0, pad_p))
        C = pad(C, (0, 0, 0, pad_p, 0, pad_h))
        D = pad(D, (0, pad_h))
        a_diag = pad(a_diag, (0, pad_p))
        g_diag = pad(g_diag, (0, pad_p)) if g_diag is not None else None
        step = pad(step, (0, pad_p), value=0.5)
    y = DLinossLayerFn.apply(variant, a_diag.contiguous(), g_diag.contiguous() if g_diag is not None else None,
                             step.contiguous(), B, C, D, u)
    return y[..., :hidden] if pad_h else y
