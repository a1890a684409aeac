"""D-LinOSS scan for callers whose tensors live in (pinned) host memory.

``scan_from_host`` runs forward + backward of the scan on host buffers and
returns host buffers.  PCIe is the bottleneck of such a call (the scan itself
runs at HBM speed), so the work is cut into slices and pipelined: while slice
``i`` is scanned, slice ``i+1`` is on its way up and the results of slice ``i-1``
are on their way down, which keeps both PCIe directions busy.  The slices are
pieces of the TIME axis: a time slice of a time-major ``[L, B, P]`` tensor is one
dense block (plain ``cudaMemcpyAsync``), and the kernels hand the recurrence state
from one slice to the next on the device.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
from torch import Tensor

from . import kernels

__all__ = ["scan_from_host"]


def scan_from_host(variant: str, a: Tensor, g: Optional[Tensor], step: Tensor, bu_host: Tensor,
                   grad_x_host: Optional[Tensor], x_host: Tensor, grad_bu_host: Optional[Tensor] = None, *,
                   slices: int = 16, device: Optional[torch.device] = None, copies_only: bool = False
                   ) -> Optional[Tuple[Tensor, Optional[Tensor], Tensor]]:
    """Forward (and, when ``grad_x_host`` is given, backward) of the oscillator scan on
    pinned host tensors ``[L, B, P]`` complex64; results are written to ``x_host`` /
    ``grad_bu_host``.  ``a, g, step`` are device tensors ``[P]``.  Returns the coefficient
    gradients ``(grad_a, grad_g, grad_step)`` on the device (``None`` without backward).
    The call returns when all results are in host memory.  ``copies_only=True`` moves the same bytes
    through the same pipeline without launching the kernels (the results are then meaningless): the
    ceiling the host and PCIe side puts on this call, for measurements.

    The sequence is cut into ``slices`` pieces along TIME: in the time-major layout a time slice is one
    contiguous block, so every transfer is a plain ``cudaMemcpyAsync`` of a dense range.  The recurrence
    state is handed from slice to slice on the device (``lti_scan_forward_slice`` / ``_backward_slice``);
    ``bu`` stays resident between its forward and backward use.  Upload order: ``bu`` first to last slice,
    then ``grad_x`` last to first; download order: ``x`` first to last, then ``grad_bu`` last to first -- both
    PCIe directions are busy from the second slice on.
    """
    dev = device or a.device
    L, B, P = bu_host.shape
    for t in (bu_host, grad_x_host, x_host, grad_bu_host):
        if t is not None and (t.dtype != torch.complex64 or not t.is_contiguous() or not t.is_pinned()
                              or tuple(t.shape) != (L, B, P)):
            raise RuntimeError("ossm_b200: host tensors must be pinned, contiguous complex64 [L, B, P]")
    backward = grad_x_host is not None
    if backward and grad_bu_host is None:
        raise RuntimeError("ossm_b200: grad_bu_host is required for the backward pass")
    if L == 0 or B == 0 or P == 0:
        if not backward:
            return None
        return tuple(torch.zeros_like(t) if t is not None else None for t in (a, g, step))
    chunk = kernels.lti_chunk()
    nchunks = (L + chunk - 1) // chunk
    slices = max(1, min(slices, nchunks))
    # slice boundaries on multiples of the carry interval
    bounds = sorted({min(L, ((nchunks * i) // slices) * chunk) for i in range(slices)} | {L})
    spans = list(zip(bounds[:-1], bounds[1:]))
    lmax = max(l1 - l0 for l0, l1 in spans)
    with torch.cuda.device(dev):
        main = torch.cuda.current_stream()
        up, down = torch.cuda.Stream(), torch.cuda.Stream()
        bu_dev = torch.empty((L, B, P), dtype=torch.complex64, device=dev) if backward else None
        # rotating buffers: slice i+1 arrives / slice i-1 leaves while slice i is scanned
        def ring(n):
            return [torch.empty((lmax, B, P), dtype=torch.complex64, device=dev) for _ in range(n)]

        xbuf = ring(2)
        bubuf = ring(2) if not backward else None
        gxbuf, gbubuf = (ring(2), ring(2)) if backward else (None, None)
        free_x = [torch.cuda.Event(), torch.cuda.Event()]       # download of the buffer finished
        free_in = [torch.cuda.Event(), torch.cuda.Event()]      # kernel reading the upload buffer finished
        for e in free_x + free_in:
            e.record(main)
        states = [None]          # state entering slice i
        carries = []
        # ---- forward, first slice to last ------------------------------------------------------------
        for i, (l0, l1) in enumerate(spans):
            n = l1 - l0
            src = bu_dev[l0:l1] if backward else bubuf[i % 2][:n]
            if not backward:
                up.wait_event(free_in[i % 2])
            with torch.cuda.stream(up):
                src.copy_(bu_host[l0:l1], non_blocking=True)
                arrived = torch.cuda.Event()
                arrived.record(up)
            main.wait_event(arrived)
            main.wait_event(free_x[i % 2])
            xv = xbuf[i % 2][:n]
            if not copies_only:
                _, car, st_out = kernels.lti_scan_forward_slice(variant, a, g, step, src, state_in=states[-1],
                                                                want_state_out=backward or i + 1 < len(spans), x_out=xv)
                carries.append(car if backward else None)
                states.append(st_out)
            done = torch.cuda.Event()
            done.record(main)
            if not backward:
                free_in[i % 2] = done
            with torch.cuda.stream(down):
                down.wait_event(done)
                x_host[l0:l1].copy_(xv, non_blocking=True)
                free_x[i % 2] = torch.cuda.Event()
                free_x[i % 2].record(down)
        grads = None
        if backward:
            # ---- backward, last slice to first -------------------------------------------------------
            adjoint = None
            free_g = [torch.cuda.Event(), torch.cuda.Event()]
            free_gb = [torch.cuda.Event(), torch.cuda.Event()]
            for e in free_g + free_gb:
                e.record(main)
            for j, i in enumerate(reversed(range(len(spans)))):
                l0, l1 = spans[i]
                n = l1 - l0
                gv = gxbuf[j % 2][:n]
                with torch.cuda.stream(up):
                    up.wait_event(free_g[j % 2])
                    gv.copy_(grad_x_host[l0:l1], non_blocking=True)
                    arrived = torch.cuda.Event()
                    arrived.record(up)
                main.wait_event(arrived)
                main.wait_event(free_gb[j % 2])
                gb = gbubuf[j % 2][:n]
                if not copies_only:
                    ga, gg, gs, _, adjoint = kernels.lti_scan_backward_slice(
                        variant, a, g, step, bu_dev[l0:l1], carries[i], gv, state_in=states[i], adjoint_in=adjoint,
                        want_adjoint_out=i > 0, grad_bu_out=gb)
                    part = (ga, gg, gs)
                    grads = part if grads is None else tuple(
                        (p + q) if p is not None else None for p, q in zip(grads, part))
                done = torch.cuda.Event()
                done.record(main)
                free_g[j % 2] = done
                with torch.cuda.stream(down):
                    down.wait_event(done)
                    grad_bu_host[l0:l1].copy_(gb, non_blocking=True)
                    free_gb[j % 2] = torch.cuda.Event()
                    free_gb[j % 2].record(down)
        main.wait_stream(down)
        main.wait_stream(up)
        main.synchronize()
    return grads if backward else None
