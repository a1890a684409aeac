"""D-LinOSS layer with the oscillators sharded over GPUs (one process per GPU).

Every rank holds a contiguous shard of the ``P`` oscillators -- the matching entries of
``(A, G, step)``, rows of ``B`` and columns of ``C`` -- and the whole input ``u`` (replicated).  It
projects ``bu_r = u B_r^T`` on the tensor cores, scans its own series (no exchange: series never
interact) and forms the partial output ``Re(C_r x_r)``.  The only exchange of the forward pass is
the sum of the partial outputs over the ranks.  With ``scatter_output=True`` (default) that sum is
a reduce-scatter over the hidden dimension: rank ``r`` ends with ``y[..., H_r]``, half the bytes of
an all-reduce, and the term ``D*u`` is added on the shard (``D`` is then the rank's ``H_r`` slice).
The time axis is cut into ``chunks`` pieces for the output projection: the reduce-scatter of piece
``k`` (NCCL, on its own stream) runs while the tensor-core GEMM of piece ``k+1`` computes, and the
GEMM writes each piece directly as one plane per destination rank, so nothing is repacked or cloned
before the collective.

Backward: the gradient of the shard is all-gathered (the transpose of the reduce-scatter) in the same
time pieces, the gather of piece ``k+1`` running beside the two GEMMs of piece ``k``; every rank
computes ``grad_x_r``, runs its scan backward and the local weight gradients; the gradient of the
replicated input is one all-reduce, started before the weight gradient of ``B`` so that it runs
beside it: every rank contributes ``grad_bu_r B_r`` plus, on its own hidden columns, ``grad_y D``.

The math of one shard is the body of ``DampedLinOSSLayer.forward``
(``src/ossm/models/dlinoss.py:217-247``); the reference has no distributed code, the oracle is the
single-device result.  ``scan`` / ``gemm`` can be replaced by plain PyTorch callables so that the
sharding logic runs on CPU ranks (gloo) in tests.
"""
from __future__ import annotations

from typing import Callable, Optional

import torch
import torch.distributed as dist
from torch import Tensor

__all__ = ["sharded_dlinoss_layer", "CopyToShards", "hidden_shard"]


COMM_SMS = 0    # SMs the tensor-core kernels leave to NCCL while a collective runs beside them; 0 = none (measured on
                # 2 GPUs: 16 / 32 reserved SMs slow the GEMMs by more than the collectives gain)


def _reserve(group, use_kernels: bool):
    """Context for the projection / weight-gradient launches that overlap a collective."""
    if use_kernels and COMM_SMS > 0 and _world(group) > 1:
        from . import kernels

        return kernels.reserved_sms(COMM_SMS)
    import contextlib

    return contextlib.nullcontext()


def _world(group) -> int:
    return dist.get_world_size(group) if dist.is_available() and dist.is_initialized() else 1


def _rank(group) -> int:
    return dist.get_rank(group) if dist.is_available() and dist.is_initialized() else 0


def hidden_shard(hidden: int, group=None) -> slice:
    """Columns of the output this rank owns after the reduce-scatter (``hidden`` must divide evenly)."""
    world, rank = _world(group), _rank(group)
    if hidden % world:
        raise ValueError(f"hidden_dim {hidden} must be a multiple of the number of ranks {world}")
    hs = hidden // world
    return slice(rank * hs, (rank + 1) * hs)


class CopyToShards(torch.autograd.Function):
    """Identity on a replicated tensor; its gradient is the sum over ranks."""

    @staticmethod
    def forward(ctx, x: Tensor, group) -> Tensor:
        ctx.group = group
        return x.view_as(x)

    @staticmethod
    def backward(ctx, grad: Tensor):
        grad = grad.contiguous()
        if _world(ctx.group) > 1:
            dist.all_reduce(grad, op=dist.ReduceOp.SUM, group=ctx.group)
        return grad, None


# ---- the two projections as autograd functions over a pluggable GEMM ---------------------------------
def _torch_project(a2d: Tensor, w: Tensor) -> Tensor:
    return a2d @ w.t()


class _SkipTerm(torch.autograd.Function):
    """``y + u[..., cols] * D`` on the rank's own hidden columns.  The gradient of this term on the replicated ``u``
    is not returned here: it is left in ``box`` for :class:`_ProjectIn`, whose backward adds it to the rank's
    columns of ``grad_u`` before the all-reduce it starts anyway (each rank contributes its own columns once, so
    the sum over ranks assembles the whole term without a second collective)."""

    @staticmethod
    def forward(ctx, y: Tensor, u: Tensor, D: Tensor, cols: slice, box: dict) -> Tensor:
        u_own = u[..., cols]
        ctx.save_for_backward(u_own, D)
        ctx.box = box
        return y + u_own * D

    @staticmethod
    def backward(ctx, grad: Tensor):
        u_own, D = ctx.saved_tensors
        grad = grad.contiguous()
        if grad.is_cuda and grad.size(-1) % 4 == 0:
            from . import kernels

            grad_D = kernels.colwise_dot(grad.view(-1, grad.size(-1)), u_own.contiguous().view(-1, grad.size(-1)))
        else:
            grad_D = (grad * u_own).sum(dim=(0, 1))
        ctx.box["skip"] = grad * D
        return grad, None, grad_D, None, None


class _ProjectIn(torch.autograd.Function):
    """``bu [L, B, P_r]`` complex64 (time-major) from a replicated ``u [B, L, H]`` and ``W_in [2 P_r, H]``.  The
    gradient on ``u`` is summed over the ranks here, started before the weight gradient so that the all-reduce
    runs beside it."""

    @staticmethod
    def forward(ctx, u: Tensor, w_in: Tensor, use_kernels: bool, group, box: Optional[dict], cols) -> Tensor:
        ctx.group, ctx.box, ctx.cols = group, box, cols
        batch, length, hidden = u.shape
        p2 = w_in.size(0)
        u2 = u.contiguous().view(batch * length, hidden)
        if use_kernels:
            from . import kernels

            bu = torch.empty((length, batch, p2 // 2), dtype=torch.complex64, device=u.device)
            kernels.gemm_tf32x3(u2, *kernels.split_tf32(w_in), torch.view_as_real(bu).view(length * batch, p2),
                                row_map=kernels.ROWS_BATCH_TO_TIME, batch=batch, length=length)
        else:
            flat = _torch_project(u2, w_in).view(batch, length, p2 // 2, 2).permute(1, 0, 2, 3).contiguous()
            bu = torch.view_as_complex(flat)
        ctx.use_kernels = use_kernels
        ctx.save_for_backward(u2, w_in)
        ctx.shape = (batch, length, hidden)
        return bu

    @staticmethod
    def backward(ctx, grad_bu: Tensor):
        u2, w_in = ctx.saved_tensors
        batch, length, hidden = ctx.shape
        p2 = w_in.size(0)
        g = torch.view_as_real(grad_bu.contiguous()).view(length, batch, p2)
        if ctx.use_kernels:
            from . import kernels

            grad_u = torch.empty((batch, length, hidden), dtype=torch.float32, device=u2.device)
            kernels.gemm_tf32x3(g.view(length * batch, p2), *kernels.split_tf32(w_in.t().contiguous()),
                                grad_u.view(batch * length, hidden), row_map=kernels.ROWS_TIME_TO_BATCH, batch=batch,
                                length=length)
        else:
            grad_u = (g.permute(1, 0, 2).reshape(batch * length, p2) @ w_in).view(batch, length, hidden)
        if ctx.box is not None and ctx.box.get("skip") is not None:
            grad_u[..., ctx.cols] += ctx.box.pop("skip")        # the D*u term of this rank's output columns
        work = None
        if _world(ctx.group) > 1:
            work = dist.all_reduce(grad_u, op=dist.ReduceOp.SUM, group=ctx.group, async_op=True)
        if ctx.use_kernels:
            from .dlinoss_layer import weight_gradient

            with _reserve(ctx.group, True):
                grad_w = weight_gradient(g.view(length * batch, p2), True, u2, False, batch, length)
        else:
            grad_w = torch.bmm(g.permute(1, 2, 0), u2.view(batch, length, hidden)).sum(0)
        if work is not None:
            work.wait()
        return grad_u, grad_w, None, None, None, None


class _ProjectOutReduce(torch.autograd.Function):
    """Sum over ranks of ``x_r W_out_r^T``: ``x [L, B, P_r]`` complex64 (time-major), ``W_out [H, 2 P_r]``.
    Returns ``[B, L, H / world]`` (reduce-scatter) or ``[B, L, H]`` (all-reduce)."""

    @staticmethod
    def forward(ctx, x: Tensor, w_out: Tensor, group, chunks: int, scatter: bool, use_kernels: bool) -> Tensor:
        length, batch, ssm = x.shape
        hidden = w_out.size(0)
        world = _world(group)
        xr = torch.view_as_real(x.contiguous()).view(length, batch, 2 * ssm)
        planes = world if scatter else 1
        hs = hidden // planes
        out = torch.empty((batch, length, hs), dtype=torch.float32, device=x.device)
        chunks = max(1, min(int(chunks), length))
        bounds = [(length * i) // chunks for i in range(chunks + 1)]
        if use_kernels:
            from . import kernels

            w_hi, w_lo = kernels.split_tf32(w_out)
        pending = []
        for l0, l1 in zip(bounds[:-1], bounds[1:]):
            lc = l1 - l0
            if lc == 0:
                continue
            rows = xr[l0:l1].reshape(lc * batch, 2 * ssm)
            # one plane [B, lc, hs] per destination rank, written by the GEMM itself
            part = torch.empty((planes, batch, lc, hs), dtype=torch.float32, device=x.device)
            if use_kernels:
                with _reserve(group, True):
                    kernels.gemm_tf32x3(rows, w_hi, w_lo, part.view(planes, batch * lc, hs),
                                        row_map=kernels.ROWS_TIME_TO_BATCH, batch=batch, length=lc, col_block=hs)
            else:
                full = _torch_project(rows, w_out).view(lc, batch, planes, hs)
                part.copy_(full.permute(2, 1, 0, 3))
            if world == 1:
                out[:, l0:l1].copy_(part[0])
                continue
            if scatter:
                mine = torch.empty((batch, lc, hs), dtype=torch.float32, device=x.device)
                work = dist.reduce_scatter_tensor(mine, part.view(planes * batch, lc, hs), op=dist.ReduceOp.SUM, group=group,
                                                  async_op=True)
            else:
                mine = part[0]
                work = dist.all_reduce(mine, op=dist.ReduceOp.SUM, group=group, async_op=True)
            pending.append((work, mine, part, l0, l1))      # the collective runs while the next piece is projected
        for work, mine, _part, l0, l1 in pending:
            work.wait()
            out[:, l0:l1].copy_(mine)
        ctx.group, ctx.scatter, ctx.use_kernels, ctx.chunks = group, scatter, use_kernels, chunks
        ctx.save_for_backward(xr, w_out)
        return out

    @staticmethod
    def backward(ctx, grad_out: Tensor):
        xr, w_out = ctx.saved_tensors
        length, batch, p2 = xr.shape
        hidden = w_out.size(0)
        group, world = ctx.group, _world(ctx.group)
        gathering = ctx.scatter and world > 1
        gy = grad_out.contiguous()                              # [B, L, H / world] or [B, L, H]
        grad_x = torch.empty((length, batch, p2 // 2), dtype=torch.complex64, device=xr.device)
        gxr = torch.view_as_real(grad_x).view(length, batch, p2)
        if ctx.use_kernels:
            from . import kernels
            from .dlinoss_layer import weight_gradient

            wt_hi, wt_lo = kernels.split_tf32(w_out.t().contiguous())
        # the time axis in pieces, as in the forward: the all-gather of piece k+1 (NCCL, its own stream) runs while
        # the two GEMMs of piece k (grad_x and the weight gradient) compute
        chunks = max(1, min(int(ctx.chunks), length)) if gathering else 1
        bounds = [(length * i) // chunks for i in range(chunks + 1)]
        spans = [(l0, l1) for l0, l1 in zip(bounds[:-1], bounds[1:]) if l1 > l0]
        pending = []
        if gathering:
            hs = gy.size(-1)
            for l0, l1 in spans:
                mine = gy[:, l0:l1].contiguous()
                got = torch.empty((world, batch, l1 - l0, hs), dtype=gy.dtype, device=gy.device)
                work = dist.all_gather_into_tensor(got.view(world * batch, l1 - l0, hs), mine, group=group, async_op=True)
                pending.append((work, got, mine))
        grad_w = None
        for i, (l0, l1) in enumerate(spans):
            lc = l1 - l0
            if gathering:
                work, got, _mine = pending[i]
                work.wait()
                piece = got.permute(1, 2, 0, 3).reshape(batch * lc, hidden)     # [B, lc, H] again, dense
            else:
                piece = gy.view(batch * length, hidden)
            if ctx.use_kernels:
                with _reserve(group, True):
                    kernels.gemm_tf32x3(piece, wt_hi, wt_lo, gxr[l0:l1].view(lc * batch, p2),
                                        row_map=kernels.ROWS_BATCH_TO_TIME, batch=batch, length=lc)
                    part = weight_gradient(piece, False, xr[l0:l1].reshape(lc * batch, p2), True, batch, lc)
            else:
                gxr[l0:l1].copy_((piece @ w_out).view(batch, lc, p2).permute(1, 0, 2))
                part = torch.bmm(piece.view(batch, lc, hidden).transpose(1, 2), xr[l0:l1].permute(1, 0, 2)).sum(0)
            grad_w = part if grad_w is None else grad_w + part
        return grad_x, grad_w, None, None, None, None


def sharded_dlinoss_layer(variant: str, a: Tensor, g: Tensor, step: Tensor, B: Tensor, C: Tensor, D: Tensor, u: Tensor, *,
                          group=None, scan: Optional[Callable[[str, Tensor, Tensor, Tensor, Tensor], Tensor]] = None,
                          chunks: int = 4, scatter_output: bool = True, use_kernels: Optional[bool] = None) -> Tensor:
    """``y = sum_r Re(C_r x_r) + D*u`` with ``x_r = scan(u B_r^T)``.

    On each rank: ``a, g, step [P_r]`` (already projected), ``B [P_r, H, 2]``, ``C [H, P_r, 2]`` (the layer's
    parameter layout, ``dlinoss.py:93-98``), ``u [B, L, H]`` replicated.  ``scatter_output=True``: ``D`` is the
    rank's slice ``[H / world]`` and the result is ``y[..., hidden_shard(H)]``; ``False``: ``D [H]`` replicated
    and the whole ``y`` on every rank.  ``scan(variant, a, g, step, bu_seq)`` defaults to
    :func:`ossm_b200.dlinoss.run_dlinoss`; ``use_kernels=False`` runs the projections with ``torch.matmul``
    (CPU tests of the sharding logic)."""
    from .dlinoss_layer import pack_input_weights, pack_output_weights

    if use_kernels is None:
        use_kernels = u.is_cuda
    if scan is None:
        from .dlinoss import run_dlinoss as scan
    box = {} if scatter_output else None
    cols = hidden_shard(u.size(-1), group) if scatter_output else None
    bu = _ProjectIn.apply(u, pack_input_weights(B), use_kernels, group, box, cols)    # [L, B, P_r]
    x = scan(variant, a, g, step, bu)
    y = _ProjectOutReduce.apply(x, pack_output_weights(C), group, chunks, scatter_output, use_kernels)
    if scatter_output:
        # each rank adds D*u on its own columns; the gradients of these terms on u are disjoint slices
        return _SkipTerm.apply(y, u, D, cols, box)
    # replicated output and replicated D: every rank adds the whole term, so it stays outside the summed gradient
    return y + u * D
