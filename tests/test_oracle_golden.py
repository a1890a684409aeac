"""Pins the numpy oracle (``oracle/scan_oracle.py``) against the reference's own
golden vectors and against recorded outputs of the reference's Python and
compiled CPU implementations (``tests/golden/*.npz``)."""
import os

import numpy as np
import pytest

from oracle import scan_oracle as so

GOLD = os.path.join(os.path.dirname(__file__), "golden")


def _load(name):
    return np.load(os.path.join(GOLD, name))


REF_CASES = _load("dlinoss_reference_cases.npz")
DGEN = _load("dlinoss_generated.npz")
LGEN = _load("linoss_generated.npz")
SGEN = _load("selective_scan_generated.npz")


def _layer_forward_backward(variant, c, dtype):
    """D-LinOSS layer math around the scan (``dlinoss.py:217-247``) with the
    loss of the reference's golden test (``test_dlinoss_parity.py:123-130``)."""
    cd = np.complex128 if dtype == np.float64 else np.complex64
    a, g, step = (c[k].astype(dtype) for k in ("A_diag", "G_diag", "step"))
    Bp, Cp, D, u = (c[k].astype(dtype) for k in ("B", "C", "D", "inputs"))
    bsz, L, H = u.shape
    P = a.shape[0]
    flat = u.reshape(bsz * L, H)
    bu = (flat @ Bp[..., 0].T + 1j * (flat @ Bp[..., 1].T)).astype(cd).reshape(bsz, L, P)
    bu_seq = np.ascontiguousarray(bu.transpose(1, 0, 2))
    states = so.lti_forward(variant, a, g, step, bu_seq)
    main = states[..., 1].transpose(1, 0, 2)
    aux = states[..., 0].transpose(1, 0, 2)
    xf = main.reshape(bsz * L, P)
    y = (xf.real @ Cp[..., 0].T - xf.imag @ Cp[..., 1].T).reshape(bsz, L, H) + u * D
    dy = 2.0 * y
    dyf = dy.reshape(bsz * L, H)
    gx = (dyf @ Cp[..., 0] - 1j * (dyf @ Cp[..., 1])).reshape(bsz, L, P) + 2.0 * main
    gaux = 2.0 * aux
    da, dg, ds, dbu = so.lti_backward(
        variant, a, g, step, bu_seq,
        np.ascontiguousarray(gx.transpose(1, 0, 2)).astype(cd),
        grad_aux=np.ascontiguousarray(gaux.transpose(1, 0, 2)).astype(cd), states=states)
    dbu_f = dbu.transpose(1, 0, 2).reshape(bsz * L, P)
    dB = np.stack((dbu_f.real.T @ flat, dbu_f.imag.T @ flat), axis=-1)
    dC = np.stack((dyf.T @ xf.real, -(dyf.T @ xf.imag)), axis=-1)
    dD = (dy * u).sum(axis=(0, 1))
    return y, main, aux, dict(A_diag=da, G_diag=dg, step=ds, B=dB, C=dC, D=dD)


@pytest.mark.parametrize("variant", so.DLINOSS_VARIANTS)
@pytest.mark.parametrize("dt_key,tol", [("float64", 1e-9), ("float32", 5e-6)])
def test_reference_golden_json(variant, dt_key, tol):
    # tolerances are the reference's own (test_dlinoss_parity.py:27-28)
    dtype = np.float64 if dt_key == "float64" else np.float32
    c = {k.split("/", 2)[2]: REF_CASES[k] for k in REF_CASES.files if k.startswith(f"{variant}/{dt_key}/")}
    y, main, aux, grads = _layer_forward_backward(variant, c, dtype)
    np.testing.assert_allclose(y, c["outputs"], rtol=tol, atol=tol)
    np.testing.assert_allclose(np.stack((main.real, main.imag), -1), c["states_main"], rtol=tol, atol=tol)
    np.testing.assert_allclose(np.stack((aux.real, aux.imag), -1), c["states_aux"], rtol=tol, atol=tol)
    for k, v in grads.items():
        np.testing.assert_allclose(v, c["grad_" + k], rtol=tol, atol=tol, err_msg=k)


def test_linoss_im_snapshot():
    s = _load("linoss_im_snapshot.npz")
    # LinOSSLayer.forward (linoss.py:199-242): a = relu(A), step = sigmoid(steps)
    a = np.maximum(s["A_diag"].astype(np.float64), 0.0)
    step = 1.0 / (1.0 + np.exp(-s["steps"].astype(np.float64)))
    u = s["inputs"].astype(np.float64)
    bsz, L, H = u.shape
    Bp = s["B"].astype(np.float64)
    Cp = s["C"].astype(np.float64).reshape(H, -1, 2)
    flat = u.reshape(bsz * L, H)
    bu = (flat @ Bp[..., 0].T + 1j * (flat @ Bp[..., 1].T)).reshape(bsz, L, -1)
    x = so.lti_forward("linoss_im", a, None, step, np.ascontiguousarray(bu.transpose(1, 0, 2)))[..., 1]
    xf = x.transpose(1, 0, 2).reshape(bsz * L, -1)
    y = (xf.real @ Cp[..., 0].T - xf.imag @ Cp[..., 1].T).reshape(bsz, L, H) + u * s["D"]
    np.testing.assert_allclose(y, s["outputs"], rtol=5e-6, atol=5e-6)


@pytest.mark.parametrize("shape", ["small", "ragged", "wide"])
@pytest.mark.parametrize("variant", so.DLINOSS_VARIANTS)
def test_dlinoss_generated(shape, variant):
    p = f"{shape}/{variant}/"
    a, g, step = (DGEN[p + k].astype(np.float64) for k in ("a", "g", "step"))
    bu = DGEN[p + "bu"].astype(np.complex128)
    gx = DGEN[p + "grad_x"].astype(np.complex128)
    states = so.lti_forward(variant, a, g, step, bu)
    da, dg, ds, dbu = so.lti_backward(variant, a, g, step, bu, gx, states=states)
    # float64 run of the reference's pure-PyTorch recurrence + autograd
    np.testing.assert_allclose(states, DGEN[p + "py_f64_states"], rtol=1e-10, atol=1e-10)
    # torch's convention for complex leaves: grad = dL/dRe + i dL/dIm, as ours
    for got, key in ((da, "da"), (dg, "dg"), (ds, "dstep"), (dbu, "dbu")):
        want = DGEN[p + "py_f64_" + key]
        assert so.max_rel_err(got, want) < 1e-10, key
    # float32 runs of the reference (pure PyTorch and compiled CPU kernel)
    for tag, tol in (("py_f32", 2e-5), ("cpp", 5e-4)):
        assert so.max_rel_err(DGEN[p + tag + "_states"], states) < tol
        for got, key in ((da, "da"), (dg, "dg"), (ds, "dstep"), (dbu, "dbu")):
            assert so.max_rel_err(DGEN[p + tag + "_" + key], got) < tol, (tag, key)


@pytest.mark.parametrize("variant", ["imex1", "im"])
def test_dlinoss_raw_parameters(variant):
    p = f"raw/{variant}/"
    a, g, step = (DGEN[p + k].astype(np.float64) for k in ("a", "g", "step"))
    states = so.lti_forward(variant, a, g, step, DGEN[p + "bu"].astype(np.complex128))
    np.testing.assert_allclose(states, DGEN[p + "py_f64_states"], rtol=1e-10, atol=1e-10)


@pytest.mark.parametrize("disc", ["IM", "IMEX"])
def test_linoss_layer_generated(disc):
    p = f"layer/{disc}/"
    variant = "linoss_im" if disc == "IM" else "linoss_imex"
    a, step = LGEN[p + "a"], LGEN[p + "step"]
    bu = np.ascontiguousarray(LGEN[p + "bu"].transpose(1, 0, 2))
    gx = np.ascontiguousarray(LGEN[p + "grad_x"].transpose(1, 0, 2))
    states = so.lti_forward(variant, a, None, step, bu)
    np.testing.assert_allclose(states[..., 1].transpose(1, 0, 2), LGEN[p + "x"], rtol=1e-10, atol=1e-10)
    da, _, ds, dbu = so.lti_backward(variant, a, None, step, bu, gx, states=states)
    assert so.max_rel_err(da, LGEN[p + "da"]) < 1e-10
    assert so.max_rel_err(ds, LGEN[p + "dstep"]) < 1e-10
    assert so.max_rel_err(dbu.transpose(1, 0, 2), LGEN[p + "dbu"]) < 1e-10


@pytest.mark.parametrize("tag", ["c1", "c2"])
def test_linoss_generic_scan_generated(tag):
    p = f"scan/{tag}/"
    am = LGEN[p + "a_matrix"].astype(np.complex128)
    b = LGEN[p + "b_seq"].astype(np.complex128)
    go = LGEN[p + "grad_out"].astype(np.complex128)
    st = so.linoss_scan(am[:, 0, 0], am[:, 0, 1], am[:, 1, 0], am[:, 1, 1], b)
    assert so.max_rel_err(LGEN[p + "states"], st) < 5e-6
    ga, gb = so.linoss_scan_backward(am, st, go)
    assert so.max_rel_err(LGEN[p + "grad_a"], ga) < 5e-5
    assert so.max_rel_err(LGEN[p + "grad_b"], gb) < 5e-5
    ar = LGEN[p + "real_a_matrix"].astype(np.float64)
    st = so.linoss_scan(ar[:, 0, 0], ar[:, 0, 1], ar[:, 1, 0], ar[:, 1, 1], b)
    assert so.max_rel_err(LGEN[p + "real_states"], st) < 5e-6
    ga, gb = so.linoss_scan_backward(ar, st, go)
    assert ga.dtype == np.float64
    assert so.max_rel_err(LGEN[p + "real_grad_a"], ga) < 5e-5
    assert so.max_rel_err(LGEN[p + "real_grad_b"], gb) < 5e-5


@pytest.mark.parametrize("tag", ["n4", "n16", "n64"])
def test_selective_scan_generated(tag):
    p = f"{tag}/"
    u, dt, A, Bm, Cm, gate, go = (SGEN[p + k].astype(np.float64)
                                  for k in ("u", "dt", "A", "B", "C", "gate", "grad_out"))
    out = so.selective_scan(u, dt, A, Bm, Cm, gate)
    grads = so.selective_scan_backward(go, u, dt, A, Bm, Cm, gate)
    # reference tolerances: rtol 1e-4 / atol 5e-5 (test_scan_parity.py:81,135)
    for src in ("py", "cpp"):
        np.testing.assert_allclose(SGEN[p + src + "_out"], out, rtol=1e-4, atol=5e-5)
        for name, got in zip(("du", "ddt", "dA", "dB", "dC", "dgate"), grads):
            want = SGEN[p + src + "_" + name]
            assert so.max_rel_err(want, got) < 1e-4, (src, name)
    np.testing.assert_allclose(SGEN[p + "cpp_out_nogate"], so.selective_scan(u, dt, A, Bm, Cm, None),
                               rtol=1e-4, atol=5e-5)


@pytest.mark.parametrize("tag", ["n128", "n256"])
def test_selective_scan_large_state(tag):
    """State sizes above 64 (the shipped Mamba4Rec configuration uses 256): the oracle against the
    reference's Python loop (its float32 math under autograd) and compiled CPU kernel."""
    G = _load("selective_scan_large_state.npz")
    p = f"{tag}/"
    u, dt, A, Bm, Cm, gate, go = (G[p + k].astype(np.float64) for k in ("u", "dt", "A", "B", "C", "gate", "grad_out"))
    out = so.selective_scan(u, dt, A, Bm, Cm, gate)
    grads = so.selective_scan_backward(go, u, dt, A, Bm, Cm, gate)
    for src in ("py", "cpp"):
        np.testing.assert_allclose(G[p + src + "_out"], out, rtol=1e-4, atol=5e-5)
        for name, got in zip(("du", "ddt", "dA", "dB", "dC", "dgate"), grads):
            assert so.max_rel_err(G[p + src + "_" + name], got) < 1e-4, (src, name)


@pytest.mark.parametrize("tag", ["d1", "d2"])
def test_diag_scan_generated(tag):
    """Complex diagonal scan of the LRU / S5 layers against the reference's two autograd
    functions (Python-loop backward) and its compiled forward kernel."""
    G = _load("diag_generated.npz")
    p = f"{tag}/"
    lam = G[p + "lambda"].astype(np.complex128)
    b = G[p + "b_seq"].astype(np.complex128)
    go = G[p + "grad_out"].astype(np.complex128)
    st = so.diag_scan(lam, b)
    gl, gb = so.diag_scan_backward(lam, st, go)
    for name in ("lru", "s5"):
        assert so.max_rel_err(G[p + name + "_states"], st) < 5e-6
        assert so.max_rel_err(G[p + name + "_grad_lambda"], gl) < 5e-5
        assert so.max_rel_err(G[p + name + "_grad_b"], gb) < 5e-5
    assert so.max_rel_err(G[p + "cpp_states"], st) < 5e-6


@pytest.mark.parametrize("kind", ["LBM", "LM", "BM", "M", "clamp"])
@pytest.mark.parametrize("variant", ["imex1", "imex2", "im", "ex"])
def test_sdlinoss_generated(variant, kind):
    """Selective D-LinOSS (per-step coefficients, every broadcast form of the parameters, step
    and stability clamps hit) against the reference's compiled CPU kernels (float32) and its
    pure-PyTorch recurrence differentiated by autograd (float64)."""
    G = _load("sdlinoss_generated.npz")
    p = f"{variant}/{kind}/"
    a, g, s, bu, go = (G[p + k] for k in ("A", "G", "step", "bu", "grad_out"))
    # float64 restatement against the float64 recurrence: tight
    a64, g64, s64 = (v.astype(np.float64) for v in (a, g, s))
    st64 = so.sdlinoss_scan(variant, a64, g64, s64, bu.astype(np.complex128))
    assert so.max_rel_err(st64, G[p + "py64_states"]) < 1e-12
    gr64 = so.sdlinoss_scan_backward(variant, a64, g64, s64, bu.astype(np.complex128), st64, go.astype(np.complex128))
    for name, got in zip(("grad_A", "grad_G", "grad_step", "grad_bu"), gr64):
        want = G[p + "py64_" + name]
        assert got.shape == want.shape, name
        assert so.max_rel_err(got, want) < 1e-10, name
    # float32 restatement against the compiled float32 kernels
    st = so.sdlinoss_scan(variant, a, g, s, bu)
    assert st.dtype == np.complex64
    assert so.max_rel_err(st, G[p + "cpp_states"]) < 1e-5
    gr = so.sdlinoss_scan_backward(variant, a, g, s, bu, st, go)
    for name, got in zip(("grad_A", "grad_G", "grad_step", "grad_bu"), gr):
        want = G[p + "cpp_" + name]
        assert got.shape == want.shape, name
        assert so.max_rel_err(got, want) < 5e-5, name


@pytest.mark.parametrize("tag", ["s16", "s8"])
def test_selective_scan_step_transform(tag):
    """Selective scan with ``dt = softplus(raw + bias[d])`` folded in, against the reference's Python
    loop behind ``F.softplus`` (float64 leaves; the loop itself accumulates in float32, hence the
    tolerances; values on both sides of the softplus cut-off)."""
    G = _load("selective_scan_delta.npz")
    p = f"{tag}/"
    u, raw, bias, A, Bm, Cm, gate, go = (G[p + k].astype(np.float64) for k in
                                         ("u", "dt_raw", "delta_bias", "A", "B", "C", "gate", "grad_out"))
    out = so.selective_scan(u, raw, A, Bm, Cm, gate=gate, delta_bias=bias, delta_softplus=True)
    assert so.max_rel_err(out, G[p + "py64_out"]) < 5e-6
    grads = so.selective_scan_backward(go, u, raw, A, Bm, Cm, gate=gate, delta_bias=bias, delta_softplus=True)
    assert len(grads) == 8 and grads[6] is None
    for name, got in zip(("du", "ddt_raw", "dA", "dB", "dC", "dgate"), grads[:6]):
        assert so.max_rel_err(got, G[p + "py64_" + name]) < 5e-5, name
    assert so.max_rel_err(grads[7], G[p + "py64_ddelta_bias"]) < 5e-5
    # bias without softplus, and softplus without bias, are the same composition
    plain = so.selective_scan(u, so.delta_transform(raw, bias, False), A, Bm, Cm, gate=gate)
    assert np.array_equal(plain, so.selective_scan(u, raw, A, Bm, Cm, gate=gate, delta_bias=bias))
