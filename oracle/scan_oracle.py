"""CPU oracle for the recurrent-scan hot path (numpy).

TEST INFRASTRUCTURE ONLY -- never imported by the product package
(``ossm_b200``); only ``tests/``, ``__graft_entry__.smoke()`` and the
``cpu_baseline`` / ``--impl reference`` legs of ``bench.py`` may use it.

Every function is a plain restatement of the reference algorithm named in its
docstring (paths are relative to the ossm checkout).  All arithmetic runs in
the dtype of the inputs; the parity tests feed float64/complex128 copies of
the float32 inputs so that the oracle is the "exact" answer the CUDA kernels
are compared with.

Pinning: ``tests/test_oracle_golden.py`` checks this file against the golden
vectors the reference's own tests hold (``tests/dlinoss_reference_cases.json``,
the inline LinOSS snapshot of ``tests/test_linoss_parity.py``) and against
outputs of the reference's Python and compiled CPU implementations recorded in
``tests/golden/`` by ``tests/golden/make_golden.py``.
"""
from __future__ import annotations

import numpy as np

DLINOSS_VARIANTS = ("imex1", "imex2", "im", "ex")
LINOSS_VARIANTS = ("linoss_im", "linoss_imex")
ALL_VARIANTS = DLINOSS_VARIANTS + LINOSS_VARIANTS


# --------------------------------------------------------------------------
# coefficients
# --------------------------------------------------------------------------
def lti_coefficients(variant, a, g, step):
    """Per-channel real transition ``M`` (4 arrays) and forcing scales ``F`` (2 arrays).

    D-LinOSS variants follow ``src/ossm/models/_dlinoss_scan.py:54-91`` (the
    pure-PyTorch recurrence that defines all four variants; the compiled
    kernels use the same formulas, e.g. ``src/ossm/csrc/dlinoss_imex1.cpp:33-49``).
    LinOSS IM / IMEX follow ``src/ossm/models/linoss.py:244-258`` (matrices) and
    ``linoss.py:295-300`` (forcing); ``g`` is ignored for them.
    """
    a = np.asarray(a)
    step = np.asarray(step)
    one = np.ones_like(a)
    if variant == "imex1":
        g = np.asarray(g)
        denom = one + step * g
        m11 = 1.0 / denom
        m12 = -(step * step * a) / denom
        m21 = m11
        m22 = one + m12
        f1 = (step * step) / denom
        f2 = f1
    elif variant == "imex2":
        g = np.asarray(g)
        m11 = one - step * g
        m12 = -step * a
        m21 = step * (one - step * g)
        m22 = one - step ** 2 * a
        f1 = step
        f2 = step * step
    elif variant == "im":
        g = np.asarray(g)
        denom = one + step * g + step ** 2 * a
        m11 = 1.0 / denom
        m12 = -(step * a) / denom
        m21 = step / denom
        m22 = (one + step * g) / denom
        f1 = step / denom
        f2 = f1 * step
    elif variant == "ex":
        g = np.asarray(g)
        m11 = one - step * g
        m12 = -step * a
        m21 = step
        m22 = one
        f1 = step
        f2 = np.zeros_like(step)
    elif variant == "linoss_im":
        schur = 1.0 / (1.0 + step ** 2 * a)
        m11 = 1.0 - step ** 2 * a * schur
        m12 = -step * a * schur
        m21 = step * schur
        m22 = schur
        f1 = m11 * step
        f2 = m21 * step
    elif variant == "linoss_imex":
        m11 = one
        m12 = -step * a
        m21 = step
        m22 = 1.0 - step ** 2 * a
        f1 = step
        f2 = step * step
    else:
        raise ValueError(f"unknown variant {variant!r}")
    return (m11, m12, m21, m22), (f1, f2)


def lti_coefficient_grads(variant, a, g, step, dM, dF):
    """Chain rule from ``(dM11, dM12, dM21, dM22), (dF1, dF2)`` to ``(da, dg, dstep)``.

    Derived by hand from the formulas in :func:`lti_coefficients`; equals what
    autograd produces through ``_reference_dlinoss_states``
    (``_dlinoss_scan.py:26-101``) and what the compiled kernels apply after
    their time loops (``dlinoss_imex1.cpp:222-232``, ``dlinoss_im_cuda.cu:160-187``,
    ``dlinoss_imex2_cuda.cu:146-196``, ``dlinoss_ex_cuda.cu:135-160``).
    """
    d11, d12, d21, d22 = dM
    df1, df2 = dF
    s = step
    zero = np.zeros_like(a)
    if variant == "imex1":
        inv = 1.0 / (1.0 + s * g)
        s2i = s * s * inv
        d_s2i = df1 + df2 - a * (d12 + d22)
        da = -s2i * (d12 + d22)
        d_inv = d11 + d21 + s * s * d_s2i
        ds = 2.0 * s * inv * d_s2i - g * inv * inv * d_inv
        dg = -s * inv * inv * d_inv
    elif variant == "imex2":
        da = -s * d12 - s * s * d22
        dg = -s * d11 - s * s * d21
        ds = (-g * d11 - a * d12 + (1.0 - 2.0 * s * g) * d21
              - 2.0 * s * a * d22 + df1 + 2.0 * s * df2)
    elif variant == "im":
        inv = 1.0 / (1.0 + s * g + s * s * a)
        d_inv = d11 - a * s * d12 + s * d21 + (1.0 + s * g) * d22 + s * df1 + s * s * df2
        da = -s * inv * d12
        dg = s * inv * d22
        ds = -a * inv * d12 + inv * d21 + g * inv * d22 + inv * df1 + 2.0 * s * inv * df2
        d_den = -inv * inv * d_inv
        da = da + s * s * d_den
        dg = dg + s * d_den
        ds = ds + (g + 2.0 * s * a) * d_den
    elif variant == "ex":
        da = -s * d12
        dg = -s * d11
        ds = -g * d11 - a * d12 + d21 + df1
    elif variant == "linoss_im":
        schur = 1.0 / (1.0 + s * s * a)
        m11 = 1.0 - s * s * a * schur
        m21 = s * schur
        t11 = d11 + s * df1
        t21 = d21 + s * df2
        ds = m11 * df1 + m21 * df2
        d_sch = -s * s * a * t11 - s * a * d12 + s * t21 + d22
        da = -s * s * schur * t11 - s * schur * d12
        ds = ds - 2.0 * s * a * schur * t11 - a * schur * d12 + schur * t21
        da = da - schur * schur * s * s * d_sch
        ds = ds - schur * schur * 2.0 * s * a * d_sch
        dg = zero
    elif variant == "linoss_imex":
        da = -s * d12 - s * s * d22
        ds = -a * d12 + d21 - 2.0 * s * a * d22 + df1 + 2.0 * s * df2
        dg = zero
    else:
        raise ValueError(f"unknown variant {variant!r}")
    return da, dg, ds


# --------------------------------------------------------------------------
# LTI 2x2 scan on a complex 2-state (D-LinOSS, LinOSS IM/IMEX)
# --------------------------------------------------------------------------
def lti_scan_states(M, F, bu):
    """Sequential recurrence ``s_t = M s_{t-1} + F * bu_t`` with ``s_{-1} = 0``.

    ``bu`` is ``[L, B, P]`` complex, ``M``/``F`` are per-channel ``[P]`` real.
    Returns ``[L, B, P, 2]`` (component 0 = auxiliary state, 1 = position
    ``x``).  Restates ``_reference_dlinoss_states`` -> ``_run_associative_scan``
    (``_dlinoss_scan.py:93-101``) as the plain time loop that
    ``tests/test_linoss_parity.py:11-20`` uses as its naive oracle.
    """
    m11, m12, m21, m22 = M
    f1, f2 = F
    L, B, P = bu.shape
    out = np.zeros((L, B, P, 2), dtype=bu.dtype)
    s0 = np.zeros((B, P), dtype=bu.dtype)
    s1 = np.zeros((B, P), dtype=bu.dtype)
    for t in range(L):
        n0 = m11 * s0 + m12 * s1 + f1 * bu[t]
        n1 = m21 * s0 + m22 * s1 + f2 * bu[t]
        s0, s1 = n0, n1
        out[t, :, :, 0] = s0
        out[t, :, :, 1] = s1
    return out


def lti_scan_backward(M, F, bu, states, grad_states):
    """Adjoint of :func:`lti_scan_states`.

    ``grad_states`` is ``[L, B, P, 2]`` complex (the D-LinOSS ops only ever
    feed component 1; component 0 is zero there).  Returns
    ``(dM (4 arrays [P]), dF (2 arrays [P]), dbu [L,B,P])``.

    Follows the reverse loop of ``src/ossm/models/linoss.py:114-142``
    (``G_t = g_t + lambda``; ``dM_ij += Re sum_b G_i conj(p_j)``;
    ``lambda = M^T G_t``) extended by the forcing scales as the compiled
    D-LinOSS kernels do (``dlinoss_im_cuda.cu:131-158``).
    """
    m11, m12, m21, m22 = M
    f1, f2 = F
    L, B, P = bu.shape
    rdt = bu.real.dtype
    d11 = np.zeros(P, rdt); d12 = np.zeros(P, rdt)
    d21 = np.zeros(P, rdt); d22 = np.zeros(P, rdt)
    df1 = np.zeros(P, rdt); df2 = np.zeros(P, rdt)
    dbu = np.zeros_like(bu)
    l0 = np.zeros((B, P), dtype=bu.dtype)
    l1 = np.zeros((B, P), dtype=bu.dtype)
    zero = np.zeros((B, P), dtype=bu.dtype)

    def dot(x, y):
        return (x.real * y.real + x.imag * y.imag).sum(axis=0)

    for t in range(L - 1, -1, -1):
        g0 = l0 + grad_states[t, :, :, 0]
        g1 = l1 + grad_states[t, :, :, 1]
        p0 = states[t - 1, :, :, 0] if t > 0 else zero
        p1 = states[t - 1, :, :, 1] if t > 0 else zero
        d11 += dot(g0, p0); d12 += dot(g0, p1)
        d21 += dot(g1, p0); d22 += dot(g1, p1)
        df1 += dot(g0, bu[t]); df2 += dot(g1, bu[t])
        dbu[t] = f1 * g0 + f2 * g1
        l0 = m11 * g0 + m21 * g1
        l1 = m12 * g0 + m22 * g1
    return (d11, d12, d21, d22), (df1, df2), dbu


def lti_forward(variant, a, g, step, bu):
    """``run_dlinoss(variant, a, g, step, bu)`` (``_dlinoss_scan.py:630-680``) /
    ``LinOSSLayer._apply_im|_apply_imex`` on a time-major ``bu`` (``linoss.py:244-315``):
    returns the full state trajectory ``[L,B,P,2]``; the op's output is ``[..., 1]``."""
    M, F = lti_coefficients(variant, a, g, step)
    return lti_scan_states(M, F, bu)


def lti_backward(variant, a, g, step, bu, grad_x, grad_aux=None, states=None):
    """Gradients of the op wrt ``(a, g, step, bu)`` for upstream ``grad_x`` on
    the position state (and optionally ``grad_aux`` on the auxiliary state).
    Mirrors ``dlinoss_<variant>_backward`` (``dlinoss_imex1.cpp:354-390``)."""
    M, F = lti_coefficients(variant, a, g, step)
    if states is None:
        states = lti_scan_states(M, F, bu)
    gs = np.zeros(states.shape, dtype=states.dtype)
    gs[..., 1] = grad_x
    if grad_aux is not None:
        gs[..., 0] = grad_aux
    dM, dF, dbu = lti_scan_backward(M, F, bu, states, gs)
    g_arr = np.zeros_like(np.asarray(a)) if g is None else g
    da, dg, ds = lti_coefficient_grads(variant, a, g_arr, step, dM, dF)
    return da, dg, ds, dbu


# --------------------------------------------------------------------------
# generic complex 2x2 scan (ossm._kernels.linoss_scan + _LinossScanFn.backward)
# --------------------------------------------------------------------------
def linoss_scan(m11, m12, m21, m22, b_seq):
    """``linoss_scan(m11,m12,m21,m22,b_seq)``: complex (or real) per-channel 2x2
    times complex 2-vector plus ``b_t``; ``b_seq`` is ``[L,B,P,2]``.
    Restates ``src/ossm/csrc/linoss_scan.cpp:11-73``."""
    L = b_seq.shape[0]
    out = np.zeros_like(b_seq)
    s0 = np.zeros(b_seq.shape[1:3], dtype=b_seq.dtype)
    s1 = np.zeros_like(s0)
    for t in range(L):
        n0 = m11 * s0 + m12 * s1 + b_seq[t, :, :, 0]
        n1 = m21 * s0 + m22 * s1 + b_seq[t, :, :, 1]
        s0, s1 = n0, n1
        out[t, :, :, 0] = s0
        out[t, :, :, 1] = s1
    return out


def linoss_scan_backward(a_matrix, states, grad_output):
    """``_LinossScanFn.backward`` (``src/ossm/models/linoss.py:83-151``).

    ``a_matrix`` is ``[P,2,2]`` real or complex.  Returns ``(grad_a [P,2,2],
    grad_b [L,B,P,2])``; for a real ``a_matrix`` the matrix gradient keeps only
    the real part (``linoss.py:133-138``).
    """
    L, B, P, _ = grad_output.shape
    cplx = np.iscomplexobj(a_matrix)
    m = a_matrix
    gm = np.zeros((P, 2, 2), dtype=a_matrix.dtype)
    gb = np.zeros_like(grad_output)
    nxt = np.zeros((B, P, 2), dtype=grad_output.dtype)
    for t in range(L - 1, -1, -1):
        G = grad_output[t] + nxt
        gb[t] = G
        prev = states[t - 1] if t > 0 else np.zeros((B, P, 2), dtype=states.dtype)
        for i in range(2):
            for j in range(2):
                v = (G[..., i] * np.conj(prev[..., j])).sum(axis=0)
                gm[:, i, j] += v if cplx else v.real
        n0 = G[..., 0] * np.conj(m[:, 0, 0]) + G[..., 1] * np.conj(m[:, 1, 0])
        n1 = G[..., 0] * np.conj(m[:, 0, 1]) + G[..., 1] * np.conj(m[:, 1, 1])
        nxt = np.stack((n0, n1), axis=-1)
    return gm, gb


# --------------------------------------------------------------------------
# Mamba selective scan
# --------------------------------------------------------------------------
def _sigmoid(x):
    return 1.0 / (1.0 + np.exp(-x))


def delta_transform(dt_raw, delta_bias=None, delta_softplus=False):
    """The step size the scan uses: ``dt_raw + delta_bias[d]`` passed through softplus when asked
    (identity above 20), the ``delta_bias`` / ``delta_softplus`` switches of the vendored Mamba kernel
    (``src/ossm/csrc/mamba/selective_scan_fwd_kernel.cuh:123-161``; ossm's wrapper leaves them off and
    applies ``F.softplus(dt_proj(.))`` in the mixer, ``mambarec.py:155``)."""
    x = dt_raw if delta_bias is None else dt_raw + delta_bias[None, :, None]
    if delta_softplus:
        x = np.where(x <= 20.0, np.log1p(np.exp(np.minimum(x, 20.0))), x)
    return x


def delta_transform_backward(ddt, dt_raw, delta_bias=None, delta_softplus=False):
    """``(d dt_raw, d delta_bias or None)`` from the gradient with respect to the transformed step."""
    x = dt_raw if delta_bias is None else dt_raw + delta_bias[None, :, None]
    g = ddt * np.where(x <= 20.0, _sigmoid(x), 1.0) if delta_softplus else ddt
    return g, (None if delta_bias is None else g.sum(axis=(0, 2)))


def selective_scan(u, dt, A, Bm, Cm, gate=None, D=None, return_states=False, delta_bias=None,
                   delta_softplus=False):
    """Fused selective scan: ``h = exp(dt*A) h + dt*B*u ; y = <C,h> (+ D*u) ; out = y*silu(gate)``.

    Shapes: ``u, dt, gate [B,D,L]``; ``A [D,N]``; ``Bm, Cm [B,L,N]``; ``D [D]``.
    Restates ``src/ossm/csrc/selective_scan_cpu.cpp:78-166`` (ossm itself
    passes no ``D``; the skip term follows the Mamba convention and is added
    before the gate).  With ``delta_bias`` / ``delta_softplus`` the given ``dt`` is the raw
    step, see :func:`delta_transform`.
    """
    if delta_bias is not None or delta_softplus:
        dt = delta_transform(dt, delta_bias, delta_softplus)
    Bsz, Dn, L = u.shape
    N = A.shape[1]
    h = np.zeros((Bsz, Dn, N), dtype=u.dtype)
    y = np.zeros_like(u)
    hs = np.zeros((L, Bsz, Dn, N), dtype=u.dtype) if return_states else None
    for t in range(L):
        abar = np.exp(dt[:, :, t, None] * A[None])
        h = abar * h + (dt[:, :, t, None] * Bm[:, None, t, :]) * u[:, :, t, None]
        y[:, :, t] = (h * Cm[:, None, t, :]).sum(-1)
        if return_states:
            hs[t] = h
    if D is not None:
        y = y + D[None, :, None] * u
    out = y if gate is None else y * (gate * _sigmoid(gate))
    if return_states:
        return out, y, hs
    return out


def selective_scan_backward(grad_out, u, dt, A, Bm, Cm, gate=None, D=None, delta_bias=None, delta_softplus=False):
    """Gradients ``(du, ddt, dA, dB, dC, dgate, dD)`` of :func:`selective_scan`.

    Restates ``src/ossm/csrc/selective_scan_cpu.cpp:168-360`` (recompute all
    states, then the reverse loop of lines 287-351).  ``dgate``/``dD`` are
    ``None`` when the corresponding input is ``None``.  With ``delta_bias`` / ``delta_softplus``
    ``ddt`` is the gradient of the raw step and the gradient of ``delta_bias`` (or ``None``) is
    appended as an eighth entry.
    """
    if delta_bias is not None or delta_softplus:
        res = selective_scan_backward(grad_out, u, delta_transform(dt, delta_bias, delta_softplus), A, Bm, Cm, gate, D)
        g_raw, g_bias = delta_transform_backward(res[1], dt, delta_bias, delta_softplus)
        return (res[0], g_raw) + tuple(res[2:]) + (g_bias,)
    Bsz, Dn, L = u.shape
    _, y, hs = selective_scan(u, dt, A, Bm, Cm, gate=None, D=D, return_states=True)
    if gate is not None:
        sg = _sigmoid(gate)
        gy = grad_out * gate * sg
        dgate = grad_out * y * (sg * (1.0 + gate * (1.0 - sg)))
    else:
        gy = grad_out
        dgate = None
    du = np.zeros_like(u)
    ddt = np.zeros_like(dt)
    dA = np.zeros_like(A)
    dB = np.zeros_like(Bm)
    dC = np.zeros_like(Cm)
    lam = np.zeros((Bsz, Dn, A.shape[1]), dtype=u.dtype)
    for t in range(L - 1, -1, -1):
        abar = np.exp(dt[:, :, t, None] * A[None])
        hprev = hs[t - 1] if t > 0 else np.zeros_like(lam)
        G = lam + gy[:, :, t, None] * Cm[:, None, t, :]
        lam = G * abar
        dC[:, t, :] = (gy[:, :, t, None] * hs[t]).sum(1)
        dB[:, t, :] = (G * (dt[:, :, t, None] * u[:, :, t, None])).sum(1)
        du[:, :, t] = (G * dt[:, :, t, None] * Bm[:, None, t, :]).sum(-1)
        dA += (G * (dt[:, :, t, None] * abar * hprev)).sum(0)
        ddt[:, :, t] = (G * (A[None] * abar * hprev + Bm[:, None, t, :] * u[:, :, t, None])).sum(-1)
    dD = None
    if D is not None:
        du = du + gy * D[None, :, None]
        dD = (gy * u).sum(axis=(0, 2))
    return du, ddt, dA, dB, dC, dgate, dD


# --------------------------------------------------------------------------
# error metric used by the parity tests
# --------------------------------------------------------------------------
def max_rel_err(got, want):
    """``max|got - want| / max|want|`` (max-norm relative error)."""
    got = np.asarray(got)
    want = np.asarray(want)
    denom = float(np.max(np.abs(want))) if want.size else 0.0
    if denom == 0.0:
        return float(np.max(np.abs(got))) if got.size else 0.0
    return float(np.max(np.abs(got.astype(want.dtype) - want)) / denom)


# --------------------------------------------------------------------------
# complex diagonal scan (LRU / S5)
# --------------------------------------------------------------------------
def diag_scan(lam, b_seq):
    """``x_t = lam * x_{t-1} + b_t`` (``src/ossm/csrc/lru_scan.cpp:11-66``, identical in
    ``s5_scan.cpp``); ``lam`` complex ``[P]``, ``b_seq`` complex ``[L,B,P]``."""
    out = np.zeros_like(b_seq)
    x = np.zeros(b_seq.shape[1:], dtype=b_seq.dtype)
    for t in range(b_seq.shape[0]):
        x = lam * x + b_seq[t]
        out[t] = x
    return out


def diag_scan_backward(lam, states, grad_output):
    """``_LRUScanFn.backward`` (``src/ossm/models/lru.py:53-80``): returns
    ``(grad_lambda [P], grad_b [L,B,P])``."""
    L = grad_output.shape[0]
    gl = np.zeros_like(lam)
    gb = np.zeros_like(grad_output)
    nxt = np.zeros(grad_output.shape[1:], dtype=grad_output.dtype)
    for t in range(L - 1, -1, -1):
        G = grad_output[t] + nxt
        gb[t] = G
        prev = states[t - 1] if t > 0 else np.zeros_like(nxt)
        gl += (G * np.conj(prev)).sum(axis=0)
        nxt = G * np.conj(lam)
    return gl, gb


# --------------------------------------------------------------------------
# selective D-LinOSS: per-step, per-series coefficients
# --------------------------------------------------------------------------
SDLINOSS_VARIANTS = ("imex1", "imex2", "im", "ex")


def sdlinoss_param_view(param, L, B, M):
    """Broadcast view ``[L|1, B|1, M]`` of a parameter given as ``(M,)``, ``(L,M)``, ``(B,M)``
    or ``(L|1,B|1,M)`` -- the rule of ``_normalize_param``
    (``src/ossm/models/_sdlinoss_scan.py:105-141``): a 2-D parameter whose first extent equals
    the length is time-varying, else per-batch."""
    p = np.asarray(param)
    if p.ndim == 1 and p.shape[0] == M:
        return p.reshape(1, 1, M)
    if p.ndim == 2 and p.shape[1] == M:
        if p.shape[0] == L:
            return p.reshape(L, 1, M)
        if p.shape[0] == B:
            return p.reshape(1, B, M)
    if p.ndim == 3 and p.shape[2] == M and p.shape[0] in (1, L) and p.shape[1] in (1, B):
        return p
    raise ValueError(f"parameter must be shaped (M,), (L,M), (B,M) or (L,B,M); got {p.shape}")


def _sdlinoss_step_terms(variant, a, g, step_raw):
    """dt, dt^2, alpha, S_raw, 1/S, clamp mask and the partials of S_raw for one time step
    (``src/ossm/csrc/sdlinoss_imex1.cpp:60-71`` and the same lines of the three siblings)."""
    real = a.dtype.type
    dt = np.minimum(np.maximum(step_raw, real(1e-6)), real(1.0))
    dt2 = dt * dt
    one = np.ones_like(dt)
    zero = np.zeros_like(dt)
    if variant == "imex1":
        alpha, s_raw, ds_ddt, ds_dg, ds_da = one, 1 + dt * g, g + zero, dt, zero
    elif variant == "imex2":
        alpha, s_raw, ds_ddt, ds_dg, ds_da = 1 - dt * g, 1 + dt2 * a, 2 * dt * a, zero, dt2
    elif variant == "im":
        alpha, s_raw, ds_ddt, ds_dg, ds_da = one, 1 + dt * g + dt2 * a, g + 2 * dt * a, dt, dt2
    elif variant == "ex":
        alpha, s_raw, ds_ddt, ds_dg, ds_da = 1 - dt * g, one, zero, zero, zero
    else:
        raise ValueError(variant)
    if variant == "ex":
        inv_s, mask = one, zero
    else:
        inv_s = 1 / np.maximum(s_raw, real(1e-6))
        mask = (s_raw > real(1e-6)).astype(a.dtype)
    return dt, dt2, alpha, inv_s, mask, ds_ddt, ds_dg, ds_da


def sdlinoss_scan(variant, A, G, step, bu):
    """States ``[L,B,M,2]`` (``[...,0]`` = w, ``[...,1]`` = x) of
    ``w' = (alpha w + dt^2 (-a x + bu)) / S,  x' = x + w'`` with per-step ``a, g, dt``
    (``sdlinoss_imex1.cpp:33-97``, ``sdlinoss_imex2.cpp:33-100``, ``sdlinoss_im.cpp:33-98``,
    ``sdlinoss_ex.cpp:25-80``)."""
    L, B, M = bu.shape
    real = bu.real.dtype
    Av, Gv, Sv = (sdlinoss_param_view(np.asarray(p, dtype=real), L, B, M) for p in (A, G, step))
    out = np.zeros((L, B, M, 2), dtype=bu.dtype)
    w = np.zeros((B, M), dtype=bu.dtype)
    x = np.zeros((B, M), dtype=bu.dtype)
    for t in range(L):
        a, g, s = (np.broadcast_to(v[t if v.shape[0] > 1 else 0], (B, M)) for v in (Av, Gv, Sv))
        dt, dt2, alpha, inv_s, _m, _1, _2, _3 = _sdlinoss_step_terms(variant, a, g, s)
        comb = -a * x + bu[t]
        w = (alpha * w + dt2 * comb) * inv_s
        x = x + w
        out[t, :, :, 0] = w
        out[t, :, :, 1] = x
    return out


def sdlinoss_scan_backward(variant, A, G, step, bu, states, grad_out):
    """``(grad_A, grad_G, grad_step, grad_bu)`` of ``sum(Re(conj(grad_out) * x))``, the
    parameter gradients in the shapes the parameters were given in (broadcast axes summed;
    ``sdlinoss_imex1.cpp:99-243`` and siblings, reduction as ``reduce_broadcast_grad``)."""
    L, B, M = bu.shape
    real = bu.real.dtype
    shapes = [np.asarray(p).shape for p in (A, G, step)]
    Av, Gv, Sv = (sdlinoss_param_view(np.asarray(p, dtype=real), L, B, M) for p in (A, G, step))
    gA = np.zeros((L, B, M), dtype=real)
    gG = np.zeros((L, B, M), dtype=real)
    gS = np.zeros((L, B, M), dtype=real)
    gbu = np.zeros_like(bu)
    gw_next = np.zeros((B, M), dtype=bu.dtype)
    gx_next = np.zeros((B, M), dtype=bu.dtype)

    def dot(p, q):
        return p.real * q.real + p.imag * q.imag

    for t in range(L - 1, -1, -1):
        a, g, s = (np.broadcast_to(v[t if v.shape[0] > 1 else 0], (B, M)) for v in (Av, Gv, Sv))
        dt, dt2, alpha, inv_s, mask, ds_ddt, ds_dg, ds_da = _sdlinoss_step_terms(variant, a, g, s)
        step_mask = ((s > real.type(1e-6)) & (s < real.type(1.0))).astype(real)
        w_prev = states[t - 1, :, :, 0] if t > 0 else np.zeros((B, M), dtype=bu.dtype)
        x_prev = states[t - 1, :, :, 1] if t > 0 else np.zeros((B, M), dtype=bu.dtype)
        gx = grad_out[t] + gx_next
        gw = gw_next + gx
        comb = -a * x_prev + bu[t]
        tmpw = alpha * w_prev + dt2 * comb
        gt = gw * inv_s
        gs_raw = -dot(gw, tmpw) * inv_s * inv_s * mask
        g_step = gs_raw * ds_ddt + dot(gt, 2 * dt * comb)
        g_a = gs_raw * ds_da - dt2 * dot(gt, x_prev)
        g_g = gs_raw * ds_dg
        if variant in ("imex2", "ex"):
            g_step = g_step - g * dot(gt, w_prev)
            g_g = g_g - dt * dot(gt, w_prev)
        gA[t], gG[t], gS[t] = g_a, g_g, g_step * step_mask
        gbu[t] = gt * dt2
        gx_next = gx - (dt2 * a) * gt
        gw_next = gt * alpha

    def reduce(full, view_shape, orig_shape):
        r = full
        if view_shape[0] == 1 and L > 1:
            r = r.sum(axis=0, keepdims=True)
        if view_shape[1] == 1 and B > 1:
            r = r.sum(axis=1, keepdims=True)
        return r.reshape(orig_shape)

    return (reduce(gA, Av.shape, shapes[0]), reduce(gG, Gv.shape, shapes[1]), reduce(gS, Sv.shape, shapes[2]), gbu)
