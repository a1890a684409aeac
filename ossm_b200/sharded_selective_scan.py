"""Mamba selective scan with the channels sharded over GPUs.

The (batch, channel) series of the scan never interact, so a rank that holds a
contiguous shard of the ``D`` channels -- its slices of ``inputs``, ``dt``,
``gate``, the rows of ``A`` and the entries of ``D`` -- scans them without any
exchange; ``B_t`` and ``C_t`` are shared by all channels and therefore
replicated.  Their gradients are sums over channels, i.e. over ranks: the only
collective is one all-reduce of ``dB`` and one of ``dC`` (float32 ``[B, L, N]``
each) in the backward pass.  Splitting the batch instead needs no collective at
all.  The reference has no distributed code; the oracle is the unsharded scan.
"""
from __future__ import annotations

from typing import Callable, Optional

from torch import Tensor

from .sharded_layer import CopyToShards

__all__ = ["sharded_selective_scan"]


def sharded_selective_scan(inputs: Tensor, dt: Tensor, A: Tensor, B: Tensor, C: Tensor, gate: Optional[Tensor] = None,
                           D: Optional[Tensor] = None, *, delta_bias: Optional[Tensor] = None,
                           delta_softplus: bool = False, scan: Optional[Callable] = None, group=None) -> Tensor:
    """``inputs, dt, gate [B, D_local, L]``, ``A [D_local, N]``, ``D, delta_bias [D_local]`` are this rank's channel
    shard; ``B, C [B, L, N]`` are replicated.  Returns this rank's ``[B, D_local, L]`` outputs.  ``scan`` replaces
    the CUDA op (same signature as :func:`ossm_b200.selective_scan.selective_scan`) in CPU tests of the sharding."""
    if scan is None:
        from .selective_scan import selective_scan as scan
    B_all = CopyToShards.apply(B, group)    # identity; the gradient is summed over the ranks
    C_all = CopyToShards.apply(C, group)
    if delta_bias is None and not delta_softplus:
        return scan(inputs, dt, A, B_all, C_all, gate, D)
    return scan(inputs, dt, A, B_all, C_all, gate, D, delta_bias=delta_bias, delta_softplus=delta_softplus)
