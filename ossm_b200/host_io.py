"""D-LinOSS scan for callers whose tensors live in (pinned) host memory.

``scan_from_host`` runs forward + backward of the scan on host buffers and
returns host buffers.  PCIe is the bottleneck of such a call (the scan itself
runs at HBM speed), so the work is cut into batch slices -- independent series --
and pipelined: while slice ``i`` is scanned, slice ``i+1`` is on its way up and
the results of slice ``i-1`` are on their way down, which keeps both PCIe
directions busy.  A batch slice of a time-major ``[L, B, P]`` tensor is a pitched
2-D region; it is moved with ``cudaMemcpy2DAsync`` (one call per slice and
tensor) into a dense device buffer, which is what the kernels take.
"""
from __future__ import annotations

import ctypes
from typing import Optional, Tuple

import torch
from torch import Tensor

from . import kernels

__all__ = ["scan_from_host"]

_H2D, _D2H = 1, 2
_cudart = None


def _rt():
    global _cudart
    if _cudart is None:
        import glob
        import os

        cands = []
        for base in (os.path.join(os.path.dirname(torch.__file__), "lib"), "/usr/local/cuda/lib64"):
            cands += sorted(glob.glob(os.path.join(base, "libcudart.so*")))
        for root, _dirs, files in os.walk(os.path.join(os.path.dirname(os.path.dirname(torch.__file__)), "nvidia")):
            cands += [os.path.join(root, f) for f in files if f.startswith("libcudart.so")]
        last = None
        for path in cands + ["libcudart.so.12", "libcudart.so"]:
            try:
                _cudart = ctypes.CDLL(path)
                break
            except OSError as exc:
                last = exc
        if _cudart is None:
            raise RuntimeError(f"ossm_b200: cannot load the CUDA runtime for pitched copies: {last}")
        _cudart.cudaMemcpy2DAsync.restype = ctypes.c_int
        _cudart.cudaMemcpy2DAsync.argtypes = [ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p, ctypes.c_size_t,
                                              ctypes.c_size_t, ctypes.c_size_t, ctypes.c_int, ctypes.c_void_p]
    return _cudart


def _copy2d(dst_ptr: int, dst_pitch: int, src_ptr: int, src_pitch: int, width: int, height: int, kind: int,
            stream: torch.cuda.Stream) -> None:
    rc = _rt().cudaMemcpy2DAsync(ctypes.c_void_p(dst_ptr), dst_pitch, ctypes.c_void_p(src_ptr), src_pitch, width,
                                 height, kind, ctypes.c_void_p(stream.cuda_stream))
    if rc != 0:
        raise RuntimeError(f"ossm_b200: cudaMemcpy2DAsync failed with error {rc}")


def scan_from_host(variant: str, a: Tensor, g: Optional[Tensor], step: Tensor, bu_host: Tensor,
                   grad_x_host: Optional[Tensor], x_host: Tensor, grad_bu_host: Optional[Tensor] = None, *,
                   slices: int = 8, device: Optional[torch.device] = None, copies_only: bool = False
                   ) -> Optional[Tuple[Tensor, Optional[Tensor], Tensor]]:
    """Forward (and, when ``grad_x_host`` is given, backward) of the oscillator scan on
    pinned host tensors ``[L, B, P]`` complex64; results are written to ``x_host`` /
    ``grad_bu_host``.  ``a, g, step`` are device tensors ``[P]``.  Returns the coefficient
    gradients ``(grad_a, grad_g, grad_step)`` on the device (``None`` without backward).
    The call returns when all results are in host memory.  ``copies_only=True`` moves the same bytes
    through the same pipeline without launching the kernels (the results are then meaningless): the
    ceiling the host and PCIe side puts on this call, for measurements.
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
    slices = max(1, min(slices, B))
    bounds = [(B * i) // slices for i in range(slices + 1)]
    bmax = max(b1 - b0 for b0, b1 in zip(bounds, bounds[1:]))
    with torch.cuda.device(dev):
        main = torch.cuda.current_stream()
        up, down = torch.cuda.Stream(), torch.cuda.Stream()
        # two sets of device buffers so that slice i+1 can arrive while slice i is in use
        bufs = [{k: torch.empty((L, bmax, P), dtype=torch.complex64, device=dev)
                 for k in (("bu", "gx", "x", "gbu") if backward else ("bu", "x"))} for _ in range(2)]
        free = [torch.cuda.Event(), torch.cuda.Event()]      # buffer set no longer read or written
        for e in free:
            e.record(main)
        grads = None
        elem = 8
        pitch_h = B * P * elem
        for i, (b0, b1) in enumerate(zip(bounds, bounds[1:])):
            nb = b1 - b0
            if nb == 0:
                continue
            set_ = bufs[i % 2]
            width = nb * P * elem
            views = {k: v.view(-1)[: L * nb * P].view(L, nb, P) for k, v in set_.items()}
            up.wait_event(free[i % 2])
            off = b0 * P * elem
            _copy2d(views["bu"].data_ptr(), width, bu_host.data_ptr() + off, pitch_h, width, L, _H2D, up)
            arrived_bu = torch.cuda.Event()
            arrived_bu.record(up)
            if backward:
                _copy2d(views["gx"].data_ptr(), width, grad_x_host.data_ptr() + off, pitch_h, width, L, _H2D, up)
                arrived_gx = torch.cuda.Event()
                arrived_gx.record(up)
            main.wait_event(arrived_bu)
            if not copies_only:
                x, _, carries = kernels.lti_scan_forward(variant, a, g, step, views["bu"], want_carries=backward)
                views["x"].copy_(x)     # device-to-device into the staging buffer (keeps `x` out of the copy stream)
            done_fwd = torch.cuda.Event()
            done_fwd.record(main)
            down.wait_event(done_fwd)
            _copy2d(x_host.data_ptr() + off, pitch_h, views["x"].data_ptr(), width, width, L, _D2H, down)
            if backward:
                main.wait_event(arrived_gx)
                if not copies_only:
                    ga, gg, gs, gbu = kernels.lti_scan_backward(variant, a, g, step, views["bu"], carries, views["gx"])
                    views["gbu"].copy_(gbu)
                    part = (ga, gg, gs)
                    grads = part if grads is None else tuple(
                        (p + q) if p is not None else None for p, q in zip(grads, part))
                done_bwd = torch.cuda.Event()
                done_bwd.record(main)
                down.wait_event(done_bwd)
                _copy2d(grad_bu_host.data_ptr() + off, pitch_h, views["gbu"].data_ptr(), width, width, L, _D2H, down)
            free[i % 2] = torch.cuda.Event()
            free[i % 2].record(down)
        main.wait_stream(down)
        main.synchronize()
    return grads if backward else None
