"""Complex diagonal scan of ossm's LRU and S5 layers, ``x_t = lambda x_{t-1} + b_t``.

Mirror of ``_LRUScanFn`` / ``_S5ScanFn`` (``src/ossm/models/lru.py:33-80``,
``s5.py``): same call, but the forward keeps chunk carries instead of relying on
the saved states for the backward, and the backward is one CUDA kernel instead
of a Python loop over the sequence.
"""
from __future__ import annotations

import torch
from torch import Tensor

from . import kernels

__all__ = ["DiagScanFn", "run_diag_scan"]


class DiagScanFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, lambda_bar: Tensor, b_seq: Tensor) -> Tensor:
        if b_seq.size(0) == 0:
            ctx.empty = True
            ctx.save_for_backward(lambda_bar)
            return b_seq
        ctx.empty = False
        lam_re = lambda_bar.real.contiguous().float()
        lam_im = lambda_bar.imag.contiguous().float()
        b_seq = b_seq.contiguous()
        needs_grad = any(ctx.needs_input_grad)
        x, carries = kernels.diag_scan_forward(lam_re, lam_im, b_seq, want_carries=needs_grad)
        if needs_grad:
            ctx.save_for_backward(lambda_bar, lam_re, lam_im, b_seq, carries)
        return x

    @staticmethod
    def backward(ctx, grad_output: Tensor):
        if ctx.empty:
            (lambda_bar,) = ctx.saved_tensors
            return torch.zeros_like(lambda_bar), grad_output
        lambda_bar, lam_re, lam_im, b_seq, carries = ctx.saved_tensors
        grad_lambda, grad_b = kernels.diag_scan_backward(lam_re, lam_im, b_seq, carries, grad_output.contiguous())
        return grad_lambda.to(lambda_bar.dtype), grad_b


def run_diag_scan(lambda_bar: Tensor, b_seq: Tensor) -> Tensor:
    """``lambda_bar`` complex64 ``[P]``, ``b_seq`` complex64 ``[L,B,P]`` on a CUDA device."""
    if b_seq.dtype != torch.complex64:
        raise RuntimeError("ossm_b200: the diagonal scan runs in complex64 only")
    return DiagScanFn.apply(lambda_bar, b_seq)
