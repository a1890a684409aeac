"""D-LinOSS layer with the oscillators sharded over GPUs (BASELINE config 4).

Every rank holds a contiguous shard of the ``P`` oscillators -- the matching
entries of ``(A, G, step)``, rows of ``B`` and columns of ``C`` -- and the whole
input ``u`` (replicated).  It projects ``bu_r = u B_r^T``, scans its own series
(no exchange: series never interact), forms the partial output
``Re(C_r x_r)`` and the partial outputs are summed over ranks (NCCL all-reduce
over NVLink); ``D*u`` is added after the sum.  In the backward pass the upstream
gradient is already replicated, so the only exchange is the sum of the
per-shard input gradients.  The math of one shard is the body of
``DampedLinOSSLayer.forward`` (``src/ossm/models/dlinoss.py:217-247``); the
reference has no distributed code, the oracle is the single-device result.

The projections are plain library GEMMs (torch.matmul); the scan is this
package's CUDA op.  The sum over ranks is issued per batch slice on a side
stream so that it overlaps the projection of the next slice.
"""
from __future__ import annotations

from typing import Callable, Optional

import torch
import torch.distributed as dist
from torch import Tensor

__all__ = ["sharded_dlinoss_layer", "CopyToShards", "SumOverShards"]


class CopyToShards(torch.autograd.Function):
    """Identity on a replicated tensor; its gradient is the sum over ranks."""

    @staticmethod
    def forward(ctx, x: Tensor, group) -> Tensor:
        ctx.group = group
        return x.view_as(x)

    @staticmethod
    def backward(ctx, grad: Tensor):
        grad = grad.contiguous()
        if dist.is_initialized() and dist.get_world_size(ctx.group) > 1:
            dist.all_reduce(grad, op=dist.ReduceOp.SUM, group=ctx.group)
        return grad, None


class SumOverShards(torch.autograd.Function):
    """Sum of per-rank partial results (replicated afterwards); gradient passes through."""

    @staticmethod
    def forward(ctx, partial: Tensor, group, slices: int) -> Tensor:
        out = partial.contiguous().clone()
        if not (dist.is_initialized() and dist.get_world_size(group) > 1):
            return out
        if slices <= 1 or out.size(0) < slices:
            dist.all_reduce(out, op=dist.ReduceOp.SUM, group=group)
            return out
        works = [dist.all_reduce(piece, op=dist.ReduceOp.SUM, group=group, async_op=True)
                 for piece in out.tensor_split(slices, dim=0)]
        for w in works:
            w.wait()
        return out

    @staticmethod
    def backward(ctx, grad: Tensor):
        return grad, None, None


def sharded_dlinoss_layer(variant: str, a: Tensor, g: Tensor, step: Tensor, B_re: Tensor, B_im: Tensor,
                          C_re: Tensor, C_im: Tensor, D: Tensor, u: Tensor, *, group=None,
                          scan: Optional[Callable[[str, Tensor, Tensor, Tensor, Tensor], Tensor]] = None,
                          slices: int = 1) -> Tensor:
    """``y = sum_r Re(C_r x_r) + D*u`` with ``x_r = scan(bu_r)``, ``bu_r = u B_r^T``.

    Shapes on each rank: ``a, g, step [P_r]`` (already projected), ``B_re, B_im [P_r, H]``,
    ``C_re, C_im [H, P_r]``, ``D [H]`` and ``u [B, L, H]`` replicated.  Returns ``y [B, L, H]``
    replicated.  ``scan(variant, a, g, step, bu_seq)`` defaults to :func:`ossm_b200.dlinoss.run_dlinoss`.
    """
    if scan is None:
        from .dlinoss import run_dlinoss as scan
    batch, length, hidden = u.shape
    u_in = CopyToShards.apply(u, group)
    flat = u_in.reshape(batch * length, hidden)
    bu = torch.complex(flat @ B_re.t(), flat @ B_im.t()).reshape(batch, length, -1)
    x = scan(variant, a, g, step, bu.permute(1, 0, 2).contiguous())           # [L, B, P_r]
    xf = x.permute(1, 0, 2).reshape(batch * length, -1)
    partial = (xf.real @ C_re.t() - xf.imag @ C_im.t()).reshape(batch, length, hidden)
    y = SumOverShards.apply(partial, group, slices)
    return y + u * D
