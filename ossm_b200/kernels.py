"""Stand-in for ``ossm._kernels`` on B200: same function names, argument order
and error behaviour as the reference's pybind11 module
(``src/ossm/csrc/bindings.cpp:159-223``), implemented by calls into the C ABI of
``libossm_b200.so``.  Tensors must live on a CUDA device; there is no CPU path.

Besides the reference-compatible functions (``dlinoss_*_forward/backward``,
``linoss_scan``, ``selective_scan_cuda`` ...) it exposes the leaner entry points
the autograd wrappers of this package use (``lti_scan_forward`` /
``lti_scan_backward``: no full-state materialisation, states recomputed from
chunk carries in the backward).
"""
from __future__ import annotations

import ctypes
from typing import Optional, Tuple

import torch
from torch import Tensor

from . import _lib

VARIANT_IDS = {
    "imex1": 0, "imex2": 1, "im": 2, "ex": 3, "linoss_im": 4, "linoss_imex": 5, "diag": 6,
}


def _p(t: Optional[Tensor]):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _stream(device) -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def _require_cuda(name: str, t: Tensor) -> None:
    if not t.is_cuda:
        raise RuntimeError(
            f"ossm_b200: {name} must be a CUDA tensor (this library has no CPU path)")


def lti_chunk() -> int:
    return int(_lib.load().ossm_b200_lti_chunk())


def _check_lti_inputs(a: Tensor, g: Optional[Tensor], step: Optional[Tensor], bu: Tensor) -> Tuple[int, int, int]:
    # same checks and messages as dlinoss_imex1.cpp:321-341
    coeffs = [t for t in (a, step, g) if t is not None]
    if any(c.dim() != 1 for c in coeffs):
        raise RuntimeError("Coefficient diagonals must be 1-D tensors")
    if bu.dim() != 3:
        raise RuntimeError("bu must have shape (length, batch, ssm_size)")
    length, batch, ssm = bu.shape
    if any(c.size(0) != ssm for c in coeffs):
        raise RuntimeError("Coefficient diagonals must match state size")
    _require_cuda("bu", bu)
    if bu.dtype != torch.complex64 or any(c.dtype != torch.float32 for c in coeffs):
        raise RuntimeError("ossm_b200: the scan runs in float32 / complex64 only")
    if any(c.device != bu.device for c in coeffs):
        raise RuntimeError("ossm_b200: coefficient tensors must be on the device of bu")
    if length > 0:
        if not all(c.is_contiguous() for c in coeffs):
            raise RuntimeError("Coefficient diagonals must be contiguous")
        if not bu.is_contiguous():
            raise RuntimeError("bu must be contiguous")
    return int(length), int(batch), int(ssm)


def lti_scan_forward(variant: str, a: Tensor, g: Optional[Tensor], step: Tensor, bu: Tensor, *,
                     want_x: bool = True, want_states: bool = False,
                     want_carries: bool = True) -> Tuple[Optional[Tensor], Optional[Tensor], Optional[Tensor]]:
    """Runs the oscillator scan.  Returns ``(x [L,B,P], states [L,B,P,2], carries)``
    (entries not asked for are ``None``)."""
    vid = VARIANT_IDS[variant]
    L, B, P = _check_lti_inputs(a, g, step, bu)
    lib = _lib.load()
    dev = bu.device
    x = torch.empty((L, B, P), dtype=torch.complex64, device=dev) if want_x else None
    states = torch.empty((L, B, P, 2), dtype=torch.complex64, device=dev) if want_states else None
    carries = None
    if want_carries:
        rows = max((L + lti_chunk() - 1) // lti_chunk() - 1, 0)
        carries = torch.empty((rows, B, P, 2), dtype=torch.complex64, device=dev)
    if L == 0 or B == 0 or P == 0:
        return x, states, carries
    ws_bytes = int(lib.ossm_b200_lti_forward_workspace_bytes(L, B, P))
    workspace = torch.empty(ws_bytes, dtype=torch.uint8, device=dev) if ws_bytes else None
    with torch.cuda.device(dev):
        rc = lib.ossm_b200_lti_scan_forward_ws(vid, _p(a), _p(g), _p(step), _p(bu), _p(x), _p(states),
                                               _p(carries) if carries is not None and carries.numel() else None,
                                               _p(workspace), ws_bytes, L, B, P, _stream(dev))
    _lib.check(rc, "lti_scan_forward")
    return x, states, carries


def _lti_backward(fn_name: str, variant: str, a: Tensor, g: Optional[Tensor], step: Tensor, bu: Tensor,
                  carry_src: Optional[Tensor], grad_x: Tensor):
    vid = VARIANT_IDS[variant]
    L, B, P = _check_lti_inputs(a, g, step, bu)
    if grad_x.shape != bu.shape:
        raise RuntimeError("grad_output must match bu shape")
    dev = bu.device
    grad_a = torch.empty_like(a)
    grad_g = torch.empty_like(g) if g is not None else None
    grad_step = torch.empty_like(step) if step is not None else None
    grad_bu = torch.empty_like(bu)
    if L == 0 or B == 0 or P == 0:
        grad_a.zero_()
        if grad_step is not None:
            grad_step.zero_()
        if grad_g is not None:
            grad_g.zero_()
        return grad_a, grad_g, grad_step, grad_bu
    if grad_x.dtype != torch.complex64 or grad_x.device != dev:
        raise RuntimeError("ossm_b200: grad_output must be complex64 on the device of bu")
    if not grad_x.is_contiguous():
        raise RuntimeError("states and grad_output must be contiguous")
    lib = _lib.load()
    ws_bytes = int(lib.ossm_b200_lti_backward_workspace_bytes(L, B, P))
    workspace = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
    fn = getattr(lib, fn_name)
    with torch.cuda.device(dev):
        rc = fn(vid, _p(a), _p(g), _p(step), _p(bu),
                _p(carry_src) if carry_src is not None and carry_src.numel() else None,
                _p(grad_x), _p(grad_bu), _p(grad_a), _p(grad_g), _p(grad_step), _p(workspace), ws_bytes,
                L, B, P, _stream(dev))
    _lib.check(rc, fn_name)
    return grad_a, grad_g, grad_step, grad_bu


def lti_scan_backward(variant: str, a: Tensor, g: Optional[Tensor], step: Tensor, bu: Tensor,
                      carries: Optional[Tensor], grad_x: Tensor):
    """Gradients ``(grad_a, grad_g, grad_step, grad_bu)`` from the carries saved by
    :func:`lti_scan_forward` (``grad_g`` is ``None`` for the LinOSS variants)."""
    if carries is not None:
        if carries.dtype != torch.complex64 or not carries.is_contiguous():
            raise RuntimeError("ossm_b200: carries must be a contiguous complex64 tensor")
        L = bu.shape[0] if bu.dim() == 3 else 0
        rows = max((L + lti_chunk() - 1) // lti_chunk() - 1, 0)
        if tuple(carries.shape) != (rows, *bu.shape[1:], 2):
            raise RuntimeError("ossm_b200: carries do not match bu (wrong sequence length or chunk)")
    return _lti_backward("ossm_b200_lti_scan_backward", variant, a, g, step, bu, carries, grad_x)


def lti_scan_forward_slice(variant: str, a: Tensor, g: Optional[Tensor], step: Tensor, bu: Tensor, *,
                           state_in: Optional[Tensor] = None, want_state_out: bool = True,
                           x_out: Optional[Tensor] = None) -> Tuple[Tensor, Tensor, Optional[Tensor]]:
    """The scan over one time slice of a longer sequence: ``state_in [B, P, 2]`` complex64 is the state entering
    the slice (``None`` = zero).  Returns ``(x, carries, state_out)``; ``x_out`` receives ``x`` when given."""
    vid = VARIANT_IDS[variant]
    L, B, P = _check_lti_inputs(a, g, step, bu)
    dev = bu.device
    x = x_out if x_out is not None else torch.empty((L, B, P), dtype=torch.complex64, device=dev)
    if tuple(x.shape) != (L, B, P) or x.dtype != torch.complex64 or not x.is_contiguous() or x.device != dev:
        raise RuntimeError("ossm_b200: x_out must be a contiguous complex64 [L, B, P] tensor on the device of bu")
    rows = max((L + lti_chunk() - 1) // lti_chunk() - 1, 0)
    carries = torch.empty((rows, B, P, 2), dtype=torch.complex64, device=dev)
    state_out = torch.empty((B, P, 2), dtype=torch.complex64, device=dev) if want_state_out else None
    if state_in is not None and (tuple(state_in.shape) != (B, P, 2) or state_in.dtype != torch.complex64
                                 or not state_in.is_contiguous()):
        raise RuntimeError("ossm_b200: state_in must be a contiguous complex64 [B, P, 2] tensor")
    with torch.cuda.device(dev):
        rc = _lib.load().ossm_b200_lti_scan_forward_slice(
            vid, _p(a), _p(g), _p(step), _p(bu), _p(x), _p(carries) if carries.numel() else None, _p(state_in),
            _p(state_out), L, B, P, _stream(dev))
    _lib.check(rc, "lti_scan_forward_slice")
    return x, carries, state_out


def lti_scan_backward_slice(variant: str, a: Tensor, g: Optional[Tensor], step: Tensor, bu: Tensor, carries: Tensor,
                            grad_x: Tensor, *, state_in: Optional[Tensor] = None, adjoint_in: Optional[Tensor] = None,
                            want_adjoint_out: bool = True, grad_bu_out: Optional[Tensor] = None):
    """Backward of one time slice (slices run last to first): returns ``(grad_a, grad_g, grad_step, grad_bu,
    adjoint_out)`` where the coefficient gradients are this slice's share."""
    vid = VARIANT_IDS[variant]
    L, B, P = _check_lti_inputs(a, g, step, bu)
    dev = bu.device
    if grad_x.shape != bu.shape or grad_x.dtype != torch.complex64 or not grad_x.is_contiguous():
        raise RuntimeError("grad_output must match bu shape")
    grad_bu = grad_bu_out if grad_bu_out is not None else torch.empty_like(bu)
    grad_a = torch.empty_like(a)
    grad_g = torch.empty_like(g) if g is not None else None
    grad_step = torch.empty_like(step)
    adjoint_out = torch.empty((B, P, 2), dtype=torch.complex64, device=dev) if want_adjoint_out else None
    lib = _lib.load()
    ws_bytes = int(lib.ossm_b200_lti_backward_workspace_bytes(L, B, P))
    workspace = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev):
        rc = lib.ossm_b200_lti_scan_backward_slice(
            vid, _p(a), _p(g), _p(step), _p(bu), _p(carries) if carries is not None and carries.numel() else None,
            _p(state_in), _p(grad_x), _p(adjoint_in), _p(adjoint_out), _p(grad_bu), _p(grad_a), _p(grad_g),
            _p(grad_step), _p(workspace), ws_bytes, L, B, P, _stream(dev))
    _lib.check(rc, "lti_scan_backward_slice")
    return grad_a, grad_g, grad_step, grad_bu, adjoint_out


# ---- reference-compatible D-LinOSS entry points ----------------------------
def _make_dlinoss(variant: str):
    def forward(a_diag: Tensor, g_diag: Tensor, step: Tensor, bu: Tensor) -> Tensor:
        _, states, _ = lti_scan_forward(variant, a_diag, g_diag, step, bu, want_x=False, want_states=True,
                                        want_carries=False)
        return states

    def backward(a_diag: Tensor, g_diag: Tensor, step: Tensor, bu: Tensor, states: Tensor, grad_output: Tensor):
        if states.dim() != 4 or states.size(3) != 2:
            raise RuntimeError("states must have shape (length, batch, ssm_size, 2)")
        if bu.dim() == 3 and tuple(states.shape[:3]) != tuple(bu.shape):
            raise RuntimeError("states must have shape (length, batch, ssm_size, 2)")
        if bu.dim() == 3 and bu.size(0) > 0 and (not states.is_contiguous() or states.dtype != torch.complex64):
            raise RuntimeError("states and grad_output must be contiguous")
        ga, gg, gs, gbu = _lti_backward("ossm_b200_lti_scan_backward_states", variant, a_diag, g_diag, step, bu,
                                        states, grad_output)
        return ga, gg, gs, gbu

    forward.__name__ = f"dlinoss_{variant}_forward"
    backward.__name__ = f"dlinoss_{variant}_backward"
    forward.__doc__ = (f"``ossm._kernels.dlinoss_{variant}_forward`` (bindings.cpp:161-168): returns the full "
                       "state trajectory ``[L,B,P,2]`` complex64.")
    backward.__doc__ = (f"``ossm._kernels.dlinoss_{variant}_backward``: ``(grad_a, grad_g, grad_step, grad_bu)``.")
    return forward, backward


dlinoss_imex1_forward, dlinoss_imex1_backward = _make_dlinoss("imex1")
dlinoss_imex2_forward, dlinoss_imex2_backward = _make_dlinoss("imex2")
dlinoss_im_forward, dlinoss_im_backward = _make_dlinoss("im")
dlinoss_ex_forward, dlinoss_ex_backward = _make_dlinoss("ex")


def set_tuning(key: str, value: int) -> None:
    _lib.check(_lib.load().ossm_b200_lti_set_tuning(key.encode(), int(value)), "lti_set_tuning")


# ---- generic LinOSS scan (reference-compatible) ------------------------------
def linoss_scan(m11: Tensor, m12: Tensor, m21: Tensor, m22: Tensor, b_seq: Tensor) -> Tensor:
    """``ossm._kernels.linoss_scan`` (linoss_scan.cpp:115-146): complex per-channel
    2x2 transition, ``b_seq`` ``[L,B,P,2]`` complex64 -> states of the same shape."""
    out = torch.empty_like(b_seq)
    if b_seq.size(0) == 0:
        return out
    if b_seq.dim() != 4 or b_seq.size(-1) != 2:
        raise RuntimeError(f"b_seq must have shape (length, batch, ssm_size, 2), got {tuple(b_seq.shape)}")
    _require_cuda("b_seq", b_seq)
    coeffs = (m11, m12, m21, m22)
    if not all(c.is_contiguous() for c in coeffs):
        raise RuntimeError("Coefficient tensors must be contiguous")
    if not b_seq.is_contiguous():
        raise RuntimeError("b_seq must be contiguous")
    L, B, P, _ = b_seq.shape
    if b_seq.dtype != torch.complex64 or any(c.dtype != torch.complex64 or c.numel() != P or c.device != b_seq.device
                                             for c in coeffs):
        raise RuntimeError("ossm_b200: linoss_scan needs complex64 coefficients of length P on the device of b_seq")
    if B == 0 or P == 0:
        return out
    dev = b_seq.device
    with torch.cuda.device(dev):
        rc = _lib.load().ossm_b200_linoss_scan_forward(_p(m11), _p(m12), _p(m21), _p(m22), _p(b_seq), _p(out),
                                                       L, B, P, _stream(dev))
    _lib.check(rc, "linoss_scan_forward")
    return out


def linoss_scan_backward(m11: Tensor, m12: Tensor, m21: Tensor, m22: Tensor, states: Tensor,
                         grad_output: Tensor) -> Tuple[Tensor, Tensor]:
    """Adjoint of :func:`linoss_scan` (what ``_LinossScanFn.backward`` computes in a
    Python loop, linoss.py:83-151): returns ``(grad_m [P,2,2] complex64, grad_b [L,B,P,2])``."""
    L, B, P, _ = grad_output.shape
    dev = grad_output.device
    _require_cuda("grad_output", grad_output)
    grad_m = torch.zeros((P, 2, 2), dtype=torch.complex64, device=dev)
    grad_b = torch.empty_like(grad_output)
    if L == 0 or B == 0 or P == 0:
        return grad_m, grad_b
    if not (states.is_contiguous() and grad_output.is_contiguous()):
        raise RuntimeError("states and grad_output must be contiguous")
    if states.shape != grad_output.shape or states.dtype != torch.complex64 or grad_output.dtype != torch.complex64:
        raise RuntimeError("ossm_b200: states and grad_output must be complex64 tensors of the same shape")
    lib = _lib.load()
    ws_bytes = int(lib.ossm_b200_linoss_scan_backward_workspace_bytes(L, B, P))
    workspace = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev):
        rc = lib.ossm_b200_linoss_scan_backward(_p(m11), _p(m12), _p(m21), _p(m22), _p(states), _p(grad_output),
                                                _p(grad_b), _p(grad_m), _p(workspace), ws_bytes, L, B, P,
                                                _stream(dev))
    _lib.check(rc, "linoss_scan_backward")
    return grad_m, grad_b


# ---- Mamba selective scan ----------------------------------------------------
_IO_DTYPES = {torch.float32: 0, torch.bfloat16: 1}


def set_selective_scan_tuning(key: str, value: int) -> None:
    """``"serial"``: 1 (default) = serial-in-time kernels for the state sizes they cover (16; 32 / 64 / 128 / 256 with
    the states of a channel split over lanes), 0 = the time-parallel kernels for every size.  Forward and backward of
    one scan must agree.  ``"split_bwd_wide_from"``: state size from which the split backward uses 8-warp CTAs.
    ``"split_flush_parts"``: threads that share one item of the split backward's ``dB_t / dC_t`` sums (0 = the
    measured default for the state size)."""
    _lib.check(_lib.load().ossm_b200_selective_scan_set_tuning(key.encode(), int(value)), "selective_scan_set_tuning")


def selective_scan_chunk(d_state: int) -> int:
    return int(_lib.load().ossm_b200_selective_scan_chunk(int(d_state)))


def _time_major_bc(t: Tensor) -> Tensor:
    """``[B, L, N]`` (ossm's argument) -> contiguous ``[B, N, L]``; free when the caller
    already holds the operand time-contiguous and passes a transposed view."""
    tt = t.transpose(1, 2)
    return tt if tt.is_contiguous() else tt.contiguous()


def _bc_operands(lib, B: Tensor, C: Tensor, n: int):
    """``(B, C, pitch)`` as handed to the library.  ``pitch == 0``: time-contiguous ``[B, N, L]`` (free when the
    caller passed transposed views of such tensors, else a transposing copy).  ``pitch > 0``: ossm's ``[B, L, N]``
    tensors as they are -- dense, or column slices of one projection as in the mixer, ``pitch`` elements between
    the rows of consecutive steps -- where the kernels of this state size read them in that order (no copy)."""
    tb, tc = B.transpose(1, 2), C.transpose(1, 2)
    if tb.is_contiguous() and tc.is_contiguous():
        return tb, tc, 0
    if lib.ossm_b200_selective_scan_step_major_bc(n) == 1:
        length = B.size(1)
        pitch = B.stride(1)
        if (B.stride(2) == 1 and C.stride(2) == 1 and C.stride(1) == pitch and pitch >= n
                and B.stride(0) == length * pitch and C.stride(0) == length * pitch):
            return B, C, pitch
        return B.contiguous(), C.contiguous(), n
    return tb.contiguous(), tc.contiguous(), 0


def _check_selective(inputs: Tensor, dt: Tensor, A: Tensor, B: Tensor, C: Tensor, gate: Optional[Tensor]):
    # mirrors _check_inputs of selective_scan_cpu.cpp / selective_scan_cuda.cu:196-250
    if inputs.dim() != 3:
        raise RuntimeError("inputs must have shape (batch, channels, length)")
    if dt.shape != inputs.shape:
        raise RuntimeError("dt must match the shape of inputs")
    if A.dim() != 2 or A.size(0) != inputs.size(1):
        raise RuntimeError("A must have shape (channels, state)")
    bsz, _, length = inputs.shape
    n = A.size(1)
    if tuple(B.shape) != (bsz, length, n) or tuple(C.shape) != (bsz, length, n):
        raise RuntimeError("B and C must have shape (batch, length, state)")
    if gate is not None and gate.shape != inputs.shape:
        raise RuntimeError("gate must match the shape of inputs")
    _require_cuda("inputs", inputs)
    if inputs.dtype not in _IO_DTYPES:
        raise RuntimeError("ossm_b200: selective scan supports float32 or bfloat16 inputs")
    for name, t in (("B", B), ("C", C), ("gate", gate)):
        if t is not None and t.dtype != inputs.dtype:
            raise RuntimeError(f"ossm_b200: {name} must have the dtype of inputs ({inputs.dtype})")
    for t in (dt, A, B, C, gate):
        if t is not None and t.device != inputs.device:
            raise RuntimeError("ossm_b200: all selective-scan operands must be on one device")


def _delta_bias(delta_bias: Optional[Tensor], ch: int, dev) -> Optional[Tensor]:
    if delta_bias is None:
        return None
    if delta_bias.dim() != 1 or delta_bias.size(0) != ch or delta_bias.device != dev:
        raise RuntimeError("delta_bias must have shape (channels,) on the device of inputs")
    return delta_bias.float().contiguous()


def selective_scan_fwd(inputs: Tensor, dt: Tensor, A: Tensor, B: Tensor, C: Tensor, gate: Optional[Tensor] = None,
                       D: Optional[Tensor] = None, save_states: bool = True, delta_bias: Optional[Tensor] = None,
                       delta_softplus: bool = False) -> Tuple[Tensor, Optional[Tensor]]:
    """Fused selective scan; returns ``(out [B,D,L], chunk_states or None)``.
    ``inputs/gate/B/C`` float32 or bfloat16, ``dt``/``A``/``D`` float32 (cast if not).  With
    ``delta_bias [D]`` / ``delta_softplus`` the kernel uses ``softplus(dt + delta_bias[d])`` as the step."""
    _check_selective(inputs, dt, A, B, C, gate)
    bsz, ch, length = inputs.shape
    n = A.size(1)
    dev = inputs.device
    out = torch.empty_like(inputs, memory_format=torch.contiguous_format)
    lib = _lib.load()
    states = None
    if save_states:
        chunk = selective_scan_chunk(n) if n > 0 else 1
        states = torch.empty((bsz, ch, (length + chunk - 1) // chunk, n), dtype=torch.float32, device=dev)
    if inputs.numel() == 0:
        return out, states
    if n == 0:
        raise RuntimeError("A must have a positive state dimension")
    u = inputs.contiguous()
    dtc = dt.float().contiguous()
    Ac = A.float().contiguous()
    Bt, Ct, pitch = _bc_operands(lib, B, C, n)
    zc = gate.contiguous() if gate is not None else None
    Dc = D.float().contiguous() if D is not None else None
    bias = _delta_bias(delta_bias, ch, dev)
    head = (_p(u), _p(dtc), _p(Ac), _p(Bt), _p(Ct), _p(zc), _p(Dc), _p(bias), int(bool(delta_softplus)), _p(out),
            _p(states), bsz, ch, length, n)
    tail = (_IO_DTYPES[inputs.dtype], _stream(dev))
    with torch.cuda.device(dev):
        if pitch:
            rc = lib.ossm_b200_selective_scan_forward_step_major_bc(*head, pitch, *tail)
        else:
            rc = lib.ossm_b200_selective_scan_forward(*head, *tail)
    _lib.check(rc, "selective_scan_forward")
    return out, states


def selective_scan_bwd(grad_output: Tensor, inputs: Tensor, dt: Tensor, A: Tensor, B: Tensor, C: Tensor,
                       gate: Optional[Tensor], chunk_states: Tensor, D: Optional[Tensor] = None,
                       delta_bias: Optional[Tensor] = None, delta_softplus: bool = False):
    """Gradients ``(du, ddt, dA, dB, dC, dgate, dD)`` (``dgate``/``dD`` ``None`` when absent).  With
    ``delta_bias`` / ``delta_softplus`` (as given to the forward) ``ddt`` is the gradient of the raw
    step and the gradient of ``delta_bias`` (``None`` without a bias) is appended as an eighth entry."""
    _check_selective(inputs, dt, A, B, C, gate)
    if grad_output.shape != inputs.shape:
        raise RuntimeError("grad_output must match the shape of inputs")
    bsz, ch, length = inputs.shape
    n = A.size(1)
    dev = inputs.device
    du = torch.empty_like(inputs, memory_format=torch.contiguous_format)
    ddt = torch.empty(inputs.shape, dtype=torch.float32, device=dev)
    dA = torch.empty((ch, n), dtype=torch.float32, device=dev)
    dBt = torch.empty((bsz, n, length), dtype=torch.float32, device=dev)
    dCt = torch.empty((bsz, n, length), dtype=torch.float32, device=dev)
    dz = torch.empty_like(du) if gate is not None else None
    dD = torch.empty(ch, dtype=torch.float32, device=dev) if D is not None else None
    bias = _delta_bias(delta_bias, ch, dev)
    dbias = torch.empty(ch, dtype=torch.float32, device=dev) if bias is not None else None
    if inputs.numel() == 0 or n == 0:
        for t in (dA, dBt, dCt, dD, dbias):
            if t is not None:
                t.zero_()
    else:
        lib = _lib.load()
        ws_bytes = int(lib.ossm_b200_selective_scan_backward_workspace_bytes(bsz, ch, length, n))
        workspace = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
        u = inputs.contiguous()
        dtc = dt.float().contiguous()
        Ac = A.float().contiguous()
        Bt, Ct, pitch = _bc_operands(lib, B, C, n)
        zc = gate.contiguous() if gate is not None else None
        Dc = D.float().contiguous() if D is not None else None
        go = grad_output.to(inputs.dtype).contiguous()
        chunk = selective_scan_chunk(n)
        if (chunk_states.dtype != torch.float32 or not chunk_states.is_contiguous()
                or tuple(chunk_states.shape) != (bsz, ch, (length + chunk - 1) // chunk, n)):
            raise RuntimeError("ossm_b200: chunk_states do not belong to these inputs")
        with torch.cuda.device(dev):
            head = (_p(u), _p(dtc), _p(Ac), _p(Bt), _p(Ct), _p(zc), _p(Dc), _p(bias), int(bool(delta_softplus)),
                    _p(go), _p(chunk_states), _p(du), _p(ddt), _p(dA), _p(dBt), _p(dCt), _p(dz), _p(dD), _p(dbias),
                    _p(workspace), ws_bytes, bsz, ch, length, n)
            tail = (_IO_DTYPES[inputs.dtype], _stream(dev))
            if pitch:
                rc = lib.ossm_b200_selective_scan_backward_step_major_bc(*head, pitch, *tail)
            else:
                rc = lib.ossm_b200_selective_scan_backward(*head, *tail)
        _lib.check(rc, "selective_scan_backward")
    dB = dBt.transpose(1, 2).to(B.dtype)
    dC = dCt.transpose(1, 2).to(C.dtype)
    res = (du, ddt.to(dt.dtype), dA.to(A.dtype), dB, dC, dz, (dD.to(D.dtype) if dD is not None else None))
    if delta_bias is not None or delta_softplus:
        res = res + ((dbias.to(delta_bias.dtype) if dbias is not None else None),)
    return res


# reference-compatible names (bindings.cpp:180-222)
def selective_scan_cuda(inputs: Tensor, dt: Tensor, A: Tensor, B: Tensor, C: Tensor, gate: Optional[Tensor] = None,
                        chunk_length: int = 16):
    """Returns ``(outputs, chunk_states, raw_outputs)``.  ``chunk_length`` is accepted and
    ignored, as in the reference wrapper (selective_scan_cuda.cu:259); ``raw_outputs`` is an
    empty tensor because the backward recomputes the ungated output instead of reading it."""
    out, states = selective_scan_fwd(inputs, dt, A, B, C, gate)
    return out, states, inputs.new_empty(0)


def selective_scan_cuda_backward(grad_output: Tensor, inputs: Tensor, dt: Tensor, A: Tensor, B: Tensor, C: Tensor,
                                 gate: Optional[Tensor], chunk_states: Tensor, raw_outputs: Tensor,
                                 chunk_length: int):
    du, ddt, dA, dB, dC, dz, _ = selective_scan_bwd(grad_output, inputs, dt, A, B, C, gate, chunk_states)
    if dz is None:
        dz = torch.zeros_like(inputs)           # the reference returns zeros for an absent gate
    return du, ddt, dA, dB, dC, dz


def selective_scan(inputs: Tensor, dt: Tensor, A: Tensor, B: Tensor, C: Tensor, gate: Optional[Tensor] = None):
    """Name of the reference's CPU entry point; here it needs CUDA tensors like everything else."""
    return selective_scan_fwd(inputs, dt, A, B, C, gate, save_states=False)[0]


def selective_scan_backward(grad_output: Tensor, inputs: Tensor, dt: Tensor, A: Tensor, B: Tensor, C: Tensor,
                            gate: Optional[Tensor] = None):
    _, states = selective_scan_fwd(inputs, dt, A, B, C, gate)
    return selective_scan_cuda_backward(grad_output, inputs, dt, A, B, C, gate, states, inputs.new_empty(0), 0)


# ---- complex diagonal scan of the LRU / S5 layers ------------------------------
def diag_scan_forward(lambda_real: Tensor, lambda_imag: Tensor, b_seq: Tensor, want_carries: bool = True):
    """``x_t = lambda * x_{t-1} + b_t`` with ``b_seq`` complex64 ``[L,B,P]``; returns ``(x, carries)``."""
    x, _, carries = lti_scan_forward("diag", lambda_real, lambda_imag, None, b_seq, want_carries=want_carries)
    return x, carries


def diag_scan_backward(lambda_real: Tensor, lambda_imag: Tensor, b_seq: Tensor, carries: Optional[Tensor],
                       grad_x: Tensor):
    """Returns ``(grad_lambda complex64 [P], grad_b complex64 [L,B,P])`` as ``_LRUScanFn.backward``
    computes them in a Python loop (lru.py:53-80)."""
    gre, gim, _, gb = lti_scan_backward("diag", lambda_real, lambda_imag, None, b_seq, carries, grad_x)
    return torch.complex(gre, gim), gb


def _diag_compat(name: str):
    def scan(lambda_real: Tensor, lambda_imag: Tensor, b_seq: Tensor) -> Tensor:
        # same checks as lru_scan.cpp:75-88; b_seq is the real view [L, B, P, 2]
        if lambda_real.dim() != 1:
            raise RuntimeError("lambda_real must be 1-D")
        if lambda_imag.dim() != 1:
            raise RuntimeError("lambda_imag must be 1-D")
        if b_seq.dim() != 4 or b_seq.size(-1) != 2:
            raise RuntimeError("b_seq must have shape (length, batch, state, 2)")
        if lambda_real.size(0) != b_seq.size(2):
            raise RuntimeError("lambda_real must match state dimension")
        if lambda_imag.size(0) != b_seq.size(2):
            raise RuntimeError("lambda_imag must match state dimension")
        _require_cuda("b_seq", b_seq)
        if b_seq.dtype != torch.float32:
            raise RuntimeError(f"ossm_b200: {name} runs in float32 only")
        if b_seq.numel() == 0:
            return torch.empty_like(b_seq)
        x, _ = diag_scan_forward(lambda_real.contiguous(), lambda_imag.contiguous(),
                                 torch.view_as_complex(b_seq.contiguous()), want_carries=False)
        return torch.view_as_real(x)

    scan.__name__ = name
    scan.__doc__ = f"``ossm._kernels.{name}(lambda_real, lambda_imag, b_seq)`` (bindings.cpp:177-179)."
    return scan


lru_scan = _diag_compat("lru_scan")
s5_scan = _diag_compat("s5_scan")


# ---- selective D-LinOSS (per-step coefficients) -------------------------------
SDLINOSS_VARIANTS = ("imex1", "imex2", "im", "ex")


def _sd_field(t: Tensor, name: str, L: int, B: int, M: int):
    """(tensor, element strides over (L, B, M)) of a parameter given with 1, 2 or 3 dimensions; an
    axis of extent 1 is a broadcast axis (stride 0).  Axis assignment and messages follow
    ``make_strided3`` (dlinoss_common.h:86-185): a 2-D parameter's first axis is time when its
    extent is the length (or 1), else batch."""
    if t.dim() < 1 or t.dim() > 3:
        raise RuntimeError(f"Selective D-LinOSS expects parameters with 1, 2, or 3 dimensions; got {t.dim()}")
    sizes, strides = [1, 1, 1], [0, 0, 0]

    def put(axis: int, dim: int, expected: int, what: str):
        size = int(t.shape[dim])
        if size != expected and size != 1:
            raise RuntimeError(f"Expected size {expected} or 1 along {what} axis but got {size}")
        sizes[axis] = size
        strides[axis] = 0 if size == 1 else int(t.stride(dim))

    if t.dim() == 1:
        put(2, 0, M, "M")
    elif t.dim() == 2:
        size0 = int(t.shape[0])
        if size0 == L or size0 == 1:
            put(0, 0, L, "length")
        elif size0 == B:
            put(1, 0, B, "batch")
        else:
            raise RuntimeError(f"First dimension must match length or batch (or be 1), got {size0}")
        put(2, 1, M, "last")
    else:
        put(0, 0, L, "length")
        put(1, 1, B, "batch")
        put(2, 2, M, "state")
    return t, strides


def _sd_prepare(A: Tensor, G: Tensor, step: Tensor, bu: Tensor):
    if bu.dim() != 3:
        raise RuntimeError("bu must have shape (length, batch, ssm_size)")
    _require_cuda("bu", bu)
    if any(t.device != bu.device for t in (A, G, step)):
        raise RuntimeError("All tensors must live on the same device")
    if bu.dtype != torch.complex64 or any(t.dtype != torch.float32 for t in (A, G, step)):
        raise RuntimeError("ossm_b200: the selective scan runs in float32 / complex64 only")
    L, B, M = (int(v) for v in bu.shape)
    fields = []
    for name, t in (("A", A), ("G", G), ("step", step)):
        t = t if t.is_contiguous() else t.contiguous()
        fields.append(_sd_field(t, name, L, B, M))
    return L, B, M, fields


def _sd_carry_rows(L: int) -> int:
    step = int(_lib.load().ossm_b200_sdlinoss_carry_interval())
    return max((L + step - 1) // step - 1, 0)


def _i64x3(strides):
    return (ctypes.c_int64 * 3)(*strides)


def sdlinoss_scan_forward(variant: str, A: Tensor, G: Tensor, step: Tensor, bu: Tensor, *, want_x: bool = True,
                          want_states: bool = False, want_carries: bool = True):
    """Selective D-LinOSS scan; returns ``(x [L,B,M], states [L,B,M,2], carries)`` (entries not asked
    for are ``None``).  ``A, G, step`` may be ``(M,)``, ``(L,M)``, ``(B,M)`` or ``(L|1,B|1,M)``."""
    vid = VARIANT_IDS[variant]
    L, B, M, fields = _sd_prepare(A, G, step, bu)
    dev = bu.device
    x = torch.empty((L, B, M), dtype=torch.complex64, device=dev) if want_x else None
    states = torch.empty((L, B, M, 2), dtype=torch.complex64, device=dev) if want_states else None
    carries = None
    if want_carries:
        carries = torch.empty((_sd_carry_rows(L), B, M, 2), dtype=torch.complex64, device=dev)
    if L == 0 or B == 0 or M == 0:
        return x, states, carries
    if not bu.is_contiguous():
        raise RuntimeError("bu must be contiguous")
    (a, sa), (g, sg), (s, ss) = fields
    with torch.cuda.device(dev):
        rc = _lib.load().ossm_b200_sdlinoss_forward(
            vid, _p(a), _i64x3(sa), _p(g), _i64x3(sg), _p(s), _i64x3(ss), _p(bu), _p(x), _p(states),
            _p(carries) if carries is not None and carries.numel() else None, L, B, M, _stream(dev))
    _lib.check(rc, "sdlinoss_forward")
    return x, states, carries


def sdlinoss_scan_backward(variant: str, A: Tensor, G: Tensor, step: Tensor, bu: Tensor, grad_x: Tensor, *,
                           carries: Optional[Tensor] = None, states: Optional[Tensor] = None):
    """``(grad_A, grad_G, grad_step, grad_bu)``, the parameter gradients in the shapes of the
    parameters (broadcast axes summed).  Needs ``carries`` (from :func:`sdlinoss_scan_forward`) or
    the full ``states``."""
    vid = VARIANT_IDS[variant]
    L, B, M, fields = _sd_prepare(A, G, step, bu)
    if grad_x.shape != bu.shape:
        raise RuntimeError("grad_output must match bu shape")
    dev = bu.device
    grads = []
    for (t, strides), orig in zip(fields, (A, G, step)):
        dense = strides == [B * M, M, 1] or L * B * M == 0
        grads.append(torch.empty_like(t) if dense and t.numel() == L * B * M else torch.zeros_like(t))
    grad_bu = torch.empty_like(bu)
    if L == 0 or B == 0 or M == 0:
        return (*[gr.zero_().view(o.shape) for gr, o in zip(grads, (A, G, step))], grad_bu)
    if grad_x.dtype != torch.complex64 or grad_x.device != dev:
        raise RuntimeError("ossm_b200: grad_output must be complex64 on the device of bu")
    if not (bu.is_contiguous() and grad_x.is_contiguous()):
        raise RuntimeError("states and grad_output must be contiguous on CUDA")
    for name, t, shape in (("carries", carries, (_sd_carry_rows(L), B, M, 2)),
                           ("states", states, (L, B, M, 2))):
        if t is not None and (t.dtype != torch.complex64 or not t.is_contiguous() or tuple(t.shape) != shape):
            raise RuntimeError(f"ossm_b200: {name} must be a contiguous complex64 tensor of shape {shape}")
    (a, sa), (g, sg), (s, ss) = fields
    with torch.cuda.device(dev):
        rc = _lib.load().ossm_b200_sdlinoss_backward(
            vid, _p(a), _i64x3(sa), _p(g), _i64x3(sg), _p(s), _i64x3(ss), _p(bu),
            _p(carries) if carries is not None and carries.numel() else None,
            _p(states) if states is not None and states.numel() else None,
            _p(grad_x), _p(grads[0]), _p(grads[1]), _p(grads[2]), _p(grad_bu), L, B, M, _stream(dev))
    _lib.check(rc, "sdlinoss_backward")
    return grads[0], grads[1], grads[2], grad_bu


def _make_sdlinoss(variant: str):
    def forward(A: Tensor, G: Tensor, step: Tensor, bu: Tensor) -> Tensor:
        _, states, _ = sdlinoss_scan_forward(variant, A, G, step, bu, want_x=False, want_states=True,
                                             want_carries=False)
        return states

    def backward(A: Tensor, G: Tensor, step: Tensor, bu: Tensor, states: Tensor, grad_output: Tensor):
        if states.dim() != 4 or states.size(3) != 2:
            raise RuntimeError("states must have shape (length, batch, ssm_size, 2)")
        if bu.dim() != 3:
            raise RuntimeError("bu must have shape (length, batch, ssm_size)")
        return sdlinoss_scan_backward(variant, A, G, step, bu, grad_output, states=states)

    forward.__name__ = f"sdlinoss_{variant}_forward"
    backward.__name__ = f"sdlinoss_{variant}_backward"
    forward.__doc__ = (f"``ossm._kernels.sdlinoss_{variant}_forward(A, G, step, bu)`` (sdlinoss_{variant}.cpp): "
                       "the state trajectory ``[L,B,M,2]`` complex64.")
    backward.__doc__ = (f"``ossm._kernels.sdlinoss_{variant}_backward``: ``(grad_A, grad_G, grad_step, grad_bu)``.")
    return forward, backward


sdlinoss_imex1_forward, sdlinoss_imex1_backward = _make_sdlinoss("imex1")
sdlinoss_imex2_forward, sdlinoss_imex2_backward = _make_sdlinoss("imex2")
sdlinoss_im_forward, sdlinoss_im_backward = _make_sdlinoss("im")
sdlinoss_ex_forward, sdlinoss_ex_backward = _make_sdlinoss("ex")


def set_sdlinoss_tuning(key: str, value: int) -> None:
    _lib.check(_lib.load().ossm_b200_sdlinoss_set_tuning(key.encode(), int(value)), "sdlinoss_set_tuning")


# ---- projections of the D-LinOSS layer on the tensor cores ----------------------
ROWS_IDENTITY, ROWS_BATCH_TO_TIME, ROWS_TIME_TO_BATCH = 0, 1, 2


def split_tf32(w: Tensor) -> Tuple[Tensor, Tensor]:
    """``(hi, lo)`` halves of a float32 matrix: ``hi`` keeps the 10 mantissa bits a TF32 tensor-core operand
    has, ``lo = w - hi`` the rest; ``hi*hi + hi*lo + lo*hi`` reproduces float32 products."""
    _require_cuda("w", w)
    if w.dtype != torch.float32:
        raise RuntimeError("ossm_b200: split_tf32 needs a float32 tensor")
    w = w.contiguous()
    hi, lo = torch.empty_like(w), torch.empty_like(w)
    if w.numel():
        with torch.cuda.device(w.device):
            rc = _lib.load().ossm_b200_split_tf32(_p(w), _p(hi), _p(lo), w.numel(), _stream(w.device))
        _lib.check(rc, "split_tf32")
    return hi, lo


def gemm_tf32x3(A: Tensor, w_hi: Tensor, w_lo: Tensor, out: Tensor, *, aux: Optional[Tensor] = None,
                diag: Optional[Tensor] = None, row_map: int = ROWS_IDENTITY, batch: int = 0, length: int = 0,
                col_block: int = 0) -> Tensor:
    """``out[dest(m), n] = sum_k A[m,k] W[n,k] (+ diag[n] * aux[dest(m), n])`` on the tcgen05 tensor cores with
    float32-level accuracy (three TF32 products of split operands).  ``A [M,K]``, ``w_hi / w_lo [N,K]`` (from
    :func:`split_tf32`) and ``out / aux [M,N]`` are dense float32 CUDA matrices; ``row_map`` permutes the output
    rows between batch-major (``b*length + l``) and time-major (``l*batch + b``) order.  With ``col_block`` the
    output is ``[N // col_block, M, col_block]``: one plane per block of output columns (what a reduce-scatter
    over the columns takes)."""
    for name, t in (("A", A), ("w_hi", w_hi), ("w_lo", w_lo), ("out", out), ("aux", aux), ("diag", diag)):
        if t is None:
            continue
        _require_cuda(name, t)
        if t.dtype != torch.float32 or not t.is_contiguous() or t.device != A.device:
            raise RuntimeError(f"ossm_b200: {name} must be a contiguous float32 tensor on the device of A")
    if A.dim() != 2 or w_hi.dim() != 2 or w_hi.shape != w_lo.shape or A.size(1) != w_hi.size(1):
        raise RuntimeError("ossm_b200: gemm_tf32x3 needs A [M,K] and W [N,K]")
    M, K = A.shape
    N = w_hi.size(0)
    if out.numel() != M * N or (aux is not None and aux.numel() != M * N) or (diag is not None and diag.numel() != N):
        raise RuntimeError("ossm_b200: gemm_tf32x3 output / aux / diag extents do not match")
    if (aux is None) != (diag is None):
        raise RuntimeError("ossm_b200: aux and diag come together")
    if M == 0 or N == 0:
        return out
    ldo, plane = N, 0
    if col_block and col_block < N:
        if N % col_block:
            raise RuntimeError("ossm_b200: col_block must divide N")
        ldo, plane = col_block, M * col_block
    with torch.cuda.device(A.device):
        rc = _lib.load().ossm_b200_gemm_tf32x3(_p(A), _p(w_hi), _p(w_lo), _p(out), _p(aux), _p(diag), M, N, K, ldo,
                                               int(col_block or 0), plane, int(row_map), int(batch), int(length),
                                               _stream(A.device))
    _lib.check(rc, "gemm_tf32x3")
    return out


def wgrad_tf32x3(X: Tensor, x_time_major: bool, Y: Tensor, y_time_major: bool, batch: int, length: int) -> Tensor:
    """``out [M, N] = sum_(b,l) X[row(b,l), :]^T Y[row(b,l), :]`` on the tensor cores (three TF32 products of split
    operands).  ``X [batch*length, M]``, ``Y [batch*length, N]`` dense float32; each has its rows in batch-major
    (``b*length + l``) or time-major (``l*batch + b``) order.  ``M`` and ``N`` must be multiples of 32."""
    for name, t in (("X", X), ("Y", Y)):
        _require_cuda(name, t)
        if t.dtype != torch.float32 or not t.is_contiguous() or t.dim() != 2 or t.size(0) != batch * length:
            raise RuntimeError(f"ossm_b200: {name} must be a contiguous float32 [batch*length, C] CUDA matrix")
    M, N = X.size(1), Y.size(1)
    lib = _lib.load()
    ws_bytes = int(lib.ossm_b200_wgrad_tf32x3_workspace_bytes(M, N, batch, length))
    partial = torch.empty(ws_bytes // 4, dtype=torch.float32, device=X.device)
    splits = ctypes.c_int(0)
    with torch.cuda.device(X.device):
        rc = lib.ossm_b200_wgrad_tf32x3(_p(X), int(bool(x_time_major)), _p(Y), int(bool(y_time_major)), _p(partial),
                                        ws_bytes, ctypes.byref(splits), M, N, int(batch), int(length),
                                        _stream(X.device))
    _lib.check(rc, "wgrad_tf32x3")
    return partial[: splits.value * M * N].view(splits.value, M, N).sum(0)


class reserved_sms:
    """``with reserved_sms(16): ...``: the projection / weight-gradient kernels launched inside leave that many SMs free,
    so that a collective launched meanwhile (NCCL on its own stream) finds room to run beside them."""

    def __init__(self, count: int):
        self.count = int(count)

    def __enter__(self):
        if self.count > 0:
            _lib.check(_lib.load().ossm_b200_layer_set_tuning(b"reserve_sms", self.count), "layer_set_tuning")
        return self

    def __exit__(self, *exc):
        if self.count > 0:
            _lib.check(_lib.load().ossm_b200_layer_set_tuning(b"reserve_sms", 0), "layer_set_tuning")
        return False


def colwise_dot(X: Tensor, Y: Tensor) -> Tensor:
    """``out[n] = sum_m X[m, n] * Y[m, n]`` for dense float32 ``[rows, cols]`` CUDA matrices (``cols`` a multiple of 4):
    the layer's ``grad_D`` in one pass over both operands."""
    for name, t in (("X", X), ("Y", Y)):
        _require_cuda(name, t)
        if t.dtype != torch.float32 or not t.is_contiguous() or t.dim() != 2 or t.shape != X.shape:
            raise RuntimeError(f"ossm_b200: {name} must be a contiguous float32 [rows, cols] CUDA matrix")
    rows, cols = X.shape
    lib = _lib.load()
    partial = torch.empty((int(lib.ossm_b200_colwise_dot_partials(rows)), cols), dtype=torch.float32, device=X.device)
    with torch.cuda.device(X.device):
        rc = lib.ossm_b200_colwise_dot(_p(X), _p(Y), _p(partial), rows, cols, _stream(X.device))
    _lib.check(rc, "colwise_dot")
    return partial.sum(0)


# ---- names ossm calls unconditionally but that are outside this library ------
def _out_of_scope(name: str):
    def stub(*_args, **_kwargs):
        # ossm's shims catch RuntimeError and take their own PyTorch path
        # (_lru_scan.py:33, _s5_scan.py, _rnn_scan.py:38).
        raise RuntimeError(f"ossm_b200 does not provide {name}; use ossm's PyTorch implementation")

    stub.__name__ = name
    return stub


linear_rnn_scan = _out_of_scope("linear_rnn_scan")
