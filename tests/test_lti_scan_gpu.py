"""GPU parity of the D-LinOSS / LinOSS oscillator scan (through the C ABI)
against the numpy oracle, the committed golden fixtures and size-independent
properties.

Tolerances (max-norm relative error, ``max|got-want| / max|want|``, against a
float64 evaluation of the same float32 inputs):
  * ``x``, full states, ``grad_bu``            <= 1e-5
  * coefficient gradients (A, G, step)         <= 5e-5   (their chain rule cancels
    leading digits; the reference's own float32 paths sit at 1e-6 .. 5e-6 on the
    small fixtures and grow the same way)
"""
import os

import numpy as np
import pytest
import torch

from oracle import scan_oracle as so
from _parity_report import record

pytestmark = pytest.mark.gpu

GOLD = os.path.join(os.path.dirname(__file__), "golden")
TOL_STATE = 1e-5
TOL_COEF = 5e-5
DLINOSS = ("imex1", "imex2", "im", "ex")
ALL = DLINOSS + ("linoss_im", "linoss_imex")


@pytest.fixture(scope="module")
def K():
    from ossm_b200 import kernels

    return kernels


@pytest.fixture(autouse=True)
def _status_clean():
    yield
    from ossm_b200 import _lib

    torch.cuda.synchronize()
    assert _lib.device_status() == 0


def dev(t):
    return torch.as_tensor(t).to("cuda")


def stable_params(P, gen):
    """Parameters projected into the stable band (dlinoss.py:252-267)."""
    g = torch.relu(torch.empty(P).uniform_(-0.25, 0.6, generator=gen))
    a = torch.empty(P).uniform_(0.0, 1.5, generator=gen)
    st = torch.sigmoid(torch.randn(P, generator=gen) * 0.5)
    s = st * g
    base = torch.sqrt(1 + s)
    lo = (2 + s - 2 * base) / (st * st)
    hi = (2 + s + 2 * base) / (st * st)
    a = lo + torch.relu(a - lo) - torch.relu(a - hi)
    return a, g, st


def make_case(L, B, P, seed, raw=False):
    gen = torch.Generator().manual_seed(seed)
    if raw:  # BASELINE config distributions
        a = torch.relu(torch.randn(P, generator=gen))
        g = torch.relu(torch.randn(P, generator=gen))
        st = torch.sigmoid(torch.randn(P, generator=gen))
    else:
        a, g, st = stable_params(P, gen)
    bu = torch.complex(torch.randn(L, B, P, generator=gen), torch.randn(L, B, P, generator=gen)) * 0.5
    gx = torch.complex(torch.randn(L, B, P, generator=gen), torch.randn(L, B, P, generator=gen))
    return a, g, st, bu, gx


def oracle(variant, a, g, st, bu, gx):
    a64, g64, s64 = a.double().numpy(), g.double().numpy(), st.double().numpy()
    bu64 = bu.to(torch.complex128).numpy()
    states = so.lti_forward(variant, a64, g64, s64, bu64)
    da, dg, ds, dbu = so.lti_backward(variant, a64, g64, s64, bu64, gx.to(torch.complex128).numpy(), states=states)
    return states, da, dg, ds, dbu


def run_gpu(K, variant, a, g, st, bu, gx, want_states=True):
    gv = None if variant.startswith("linoss") else dev(g)
    x, states, carries = K.lti_scan_forward(variant, dev(a), gv, dev(st), dev(bu), want_states=want_states)
    ga, gg, gs, gbu = K.lti_scan_backward(variant, dev(a), gv, dev(st), dev(bu), carries, dev(gx))
    return x, states, (ga, gg, gs, gbu)


def check_against_oracle(K, variant, case, tol_state=TOL_STATE, tol_coef=TOL_COEF):
    a, g, st, bu, gx = case
    x, states, (ga, gg, gs, gbu) = run_gpu(K, variant, a, g, st, bu, gx)
    ref, da, dg, ds, dbu = oracle(variant, a, g, st, bu, gx)
    tag = f"lti {variant} " + "x".join(map(str, bu.shape))
    assert record(tag, "x", so.max_rel_err(x.cpu().numpy(), ref[..., 1]), tol_state) <= tol_state
    assert record(tag, "states", so.max_rel_err(states.cpu().numpy(), ref), tol_state) <= tol_state
    assert record(tag, "grad_bu", so.max_rel_err(gbu.cpu().numpy(), dbu), tol_state) <= tol_state
    assert record(tag, "grad_A", so.max_rel_err(ga.cpu().numpy(), da), tol_coef) <= tol_coef
    assert record(tag, "grad_step", so.max_rel_err(gs.cpu().numpy(), ds), tol_coef) <= tol_coef
    if gg is not None:
        assert record(tag, "grad_G", so.max_rel_err(gg.cpu().numpy(), dg), tol_coef) <= tol_coef


# ---------------------------------------------------------------------------
# oracle parity over shapes that exercise every code path
# ---------------------------------------------------------------------------
SHAPES = [
    (1, 1, 1),        # single step, single series
    (1, 2, 8),
    (2, 3, 5),        # odd B*P -> plain-load kernel
    (31, 2, 16), (32, 2, 16), (33, 2, 16),   # around one chunk
    (64, 1, 2), (65, 3, 6),
    (100, 2, 35),     # P not a multiple of the tile
    (257, 4, 64),
    (96, 2, 200),     # several CTAs with a ragged last tile
]


@pytest.mark.parametrize("variant", ALL)
@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: "x".join(map(str, s)))
def test_matches_oracle(K, variant, shape):
    L, B, P = shape
    check_against_oracle(K, variant, make_case(L, B, P, seed=L * 1000 + B * 10 + P))


@pytest.mark.parametrize("variant", ALL)
def test_plain_load_path_matches_oracle(K, variant):
    K.set_tuning("force_plain", 1)
    try:
        check_against_oracle(K, variant, make_case(100, 2, 32, seed=5))
    finally:
        K.set_tuning("force_plain", 0)


@pytest.mark.parametrize("warps,ring", [(1, 2), (2, 3), (4, 2), (1, 5)])
def test_launch_shapes_agree_bitwise(K, warps, ring):
    case = make_case(130, 3, 72, seed=11)
    a, g, st, bu, gx = case
    x0, s0, g0 = run_gpu(K, "imex2", a, g, st, bu, gx)
    for key, val in (("fwd_warps", warps), ("bwd_warps", warps), ("fwd_ring", ring), ("bwd_ring", min(ring, 3))):
        K.set_tuning(key, val)
    try:
        x1, s1, g1 = run_gpu(K, "imex2", a, g, st, bu, gx)
    finally:
        for key, val in (("fwd_warps", 4), ("bwd_warps", 4), ("fwd_ring", 2), ("bwd_ring", 2)):
            K.set_tuning(key, val)
    assert torch.equal(torch.view_as_real(x0), torch.view_as_real(x1))
    assert torch.equal(torch.view_as_real(s0), torch.view_as_real(s1))
    for u, v in zip(g0, g1):
        assert torch.equal(torch.view_as_real(u) if u.is_complex() else u,
                           torch.view_as_real(v) if v.is_complex() else v)


def test_run_to_run_deterministic(K):
    a, g, st, bu, gx = make_case(300, 8, 96, seed=3)
    r0 = run_gpu(K, "im", a, g, st, bu, gx)[2]
    r1 = run_gpu(K, "im", a, g, st, bu, gx)[2]
    for u, v in zip(r0, r1):
        assert torch.equal(torch.view_as_real(u) if u.is_complex() else u,
                           torch.view_as_real(v) if v.is_complex() else v)


# ---------------------------------------------------------------------------
# golden fixtures
# ---------------------------------------------------------------------------
@pytest.mark.parametrize("shape", ["small", "ragged", "wide"])
@pytest.mark.parametrize("variant", DLINOSS)
def test_generated_fixtures(K, shape, variant):
    """Against outputs of the reference itself (float64 PyTorch recurrence +
    autograd, and its compiled float32 CPU kernels)."""
    D = np.load(os.path.join(GOLD, "dlinoss_generated.npz"))
    p = f"{shape}/{variant}/"
    a, g, st = (torch.from_numpy(D[p + k]) for k in ("a", "g", "step"))
    bu, gx = torch.from_numpy(D[p + "bu"]), torch.from_numpy(D[p + "grad_x"])
    x, states, (ga, gg, gs, gbu) = run_gpu(K, variant, a, g, st, bu, gx)
    assert so.max_rel_err(states.cpu().numpy(), D[p + "py_f64_states"]) <= TOL_STATE
    assert so.max_rel_err(gbu.cpu().numpy(), D[p + "py_f64_dbu"]) <= TOL_STATE
    for got, key in ((ga, "da"), (gg, "dg"), (gs, "dstep")):
        assert so.max_rel_err(got.cpu().numpy(), D[p + "py_f64_" + key]) <= TOL_COEF, key
        # the reference's compiled float32 kernel, same inputs
        assert so.max_rel_err(got.cpu().numpy(), D[p + "cpp_" + key]) <= 2e-4, key
    assert so.max_rel_err(states.cpu().numpy(), D[p + "cpp_states"]) <= 2e-5


@pytest.mark.parametrize("variant", DLINOSS)
def test_reference_golden_json_states(K, variant):
    """The reference's own golden vectors (tests/dlinoss_reference_cases.json):
    both state components and the layer output."""
    D = np.load(os.path.join(GOLD, "dlinoss_reference_cases.npz"))
    c = {k.split("/", 2)[2]: D[k] for k in D.files if k.startswith(f"{variant}/float32/")}
    a, g, st = (torch.from_numpy(c[k]).float() for k in ("A_diag", "G_diag", "step"))
    u = torch.from_numpy(c["inputs"]).float()
    Bp, Cp, Dv = (torch.from_numpy(c[k]).float() for k in ("B", "C", "D"))
    bsz, L, H = u.shape
    flat = u.reshape(bsz * L, H)
    bu = torch.complex(flat @ Bp[..., 0].T, flat @ Bp[..., 1].T).reshape(bsz, L, -1).permute(1, 0, 2).contiguous()
    states = getattr(K, f"dlinoss_{variant}_forward")(dev(a), dev(g), dev(st), dev(bu)).cpu()
    main = states[..., 1].permute(1, 0, 2)
    aux = states[..., 0].permute(1, 0, 2)
    np.testing.assert_allclose(torch.view_as_real(main.contiguous()).numpy(), c["states_main"], rtol=5e-6, atol=5e-6)
    np.testing.assert_allclose(torch.view_as_real(aux.contiguous()).numpy(), c["states_aux"], rtol=5e-6, atol=5e-6)
    xf = main.reshape(bsz * L, -1)
    y = (xf.real @ Cp[..., 0].T - xf.imag @ Cp[..., 1].T).reshape(bsz, L, H) + u * Dv
    np.testing.assert_allclose(y.numpy(), c["outputs"], rtol=5e-6, atol=5e-6)


@pytest.mark.parametrize("disc", ["IM", "IMEX"])
def test_linoss_layer_fixture(K, disc):
    D = np.load(os.path.join(GOLD, "linoss_generated.npz"))
    p = f"layer/{disc}/"
    variant = "linoss_im" if disc == "IM" else "linoss_imex"
    a = torch.from_numpy(D[p + "a"]).float()
    st = torch.from_numpy(D[p + "step"]).float()
    bu = torch.from_numpy(D[p + "bu"]).to(torch.complex64).permute(1, 0, 2).contiguous()
    gx = torch.from_numpy(D[p + "grad_x"]).to(torch.complex64).permute(1, 0, 2).contiguous()
    x, _, (ga, gg, gs, gbu) = run_gpu(K, variant, a, a, st, bu, gx, want_states=False)
    assert gg is None
    assert so.max_rel_err(x.cpu().permute(1, 0, 2).numpy(), D[p + "x"]) <= TOL_STATE
    assert so.max_rel_err(gbu.cpu().permute(1, 0, 2).numpy(), D[p + "dbu"]) <= TOL_STATE
    assert so.max_rel_err(ga.cpu().numpy(), D[p + "da"]) <= TOL_COEF
    assert so.max_rel_err(gs.cpu().numpy(), D[p + "dstep"]) <= TOL_COEF


# ---------------------------------------------------------------------------
# reference-compatible entry points and the autograd op
# ---------------------------------------------------------------------------
@pytest.mark.parametrize("variant", DLINOSS)
def test_compat_backward_equals_carry_backward(K, variant):
    a, g, st, bu, gx = make_case(150, 3, 40, seed=21)
    fwd = getattr(K, f"dlinoss_{variant}_forward")
    bwd = getattr(K, f"dlinoss_{variant}_backward")
    states = fwd(dev(a), dev(g), dev(st), dev(bu))
    assert states.shape == (150, 3, 40, 2) and states.dtype == torch.complex64
    ga, gg, gs, gbu = bwd(dev(a), dev(g), dev(st), dev(bu), states, dev(gx))
    x, _, ref = run_gpu(K, variant, a, g, st, bu, gx, want_states=False)
    assert torch.equal(torch.view_as_real(states[..., 1].contiguous()), torch.view_as_real(x))
    for u, v in zip((ga, gg, gs), ref[:3]):
        assert torch.equal(u, v)
    assert torch.equal(torch.view_as_real(gbu), torch.view_as_real(ref[3]))


def test_zero_length_and_single_step(K):
    a, g, st = (dev(torch.rand(4)) for _ in range(3))
    states = K.dlinoss_imex1_forward(a, g, st, torch.zeros(0, 2, 4, dtype=torch.complex64, device="cuda"))
    assert states.shape == (0, 2, 4, 2)
    grads = K.dlinoss_imex1_backward(a, g, st, torch.zeros(0, 2, 4, dtype=torch.complex64, device="cuda"), states,
                                     torch.zeros(0, 2, 4, dtype=torch.complex64, device="cuda"))
    assert all(float(t.abs().sum()) == 0.0 for t in grads[:3])   # dlinoss_imex1.cpp:366-374


@pytest.mark.parametrize("variant", DLINOSS)
def test_autograd_op(K, variant):
    from ossm_b200.dlinoss import run_dlinoss

    a, g, st, bu, gx = make_case(70, 2, 24, seed=31)
    leaves = [dev(t).requires_grad_(True) for t in (a, g, st, bu)]
    x = run_dlinoss(variant, *leaves)
    assert x.is_contiguous() and x.shape == bu.shape
    # loss = Re<x, gx>: its gradient wrt x is gx (torch convention for complex leaves)
    (x.real * dev(gx).real + x.imag * dev(gx).imag).sum().backward()
    ref, da, dg, ds, dbu = oracle(variant, a, g, st, bu, gx)
    assert so.max_rel_err(x.detach().cpu().numpy(), ref[..., 1]) <= TOL_STATE
    assert so.max_rel_err(leaves[0].grad.cpu().numpy(), da) <= TOL_COEF
    assert so.max_rel_err(leaves[1].grad.cpu().numpy(), dg) <= TOL_COEF
    assert so.max_rel_err(leaves[2].grad.cpu().numpy(), ds) <= TOL_COEF
    assert so.max_rel_err(leaves[3].grad.cpu().numpy(), dbu) <= TOL_STATE
    # no-grad path saves nothing and still matches
    with torch.no_grad():
        x2 = run_dlinoss(variant, *[t.detach() for t in leaves])
    assert torch.equal(torch.view_as_real(x2), torch.view_as_real(x.detach()))


def test_noncontiguous_grad_output(K):
    """Upstream gradients arrive as strided views (the reference wrappers call
    ``.contiguous()``, _dlinoss_scan.py:492)."""
    from ossm_b200.dlinoss import run_dlinoss

    a, g, st, bu, gx = make_case(40, 2, 16, seed=41)
    leaves = [dev(t).requires_grad_(True) for t in (a, g, st, bu)]
    x = run_dlinoss("imex1", *leaves)
    y = x.permute(1, 0, 2)                      # consumer works batch-major
    w = dev(gx).permute(1, 0, 2)
    (y.real * w.real + y.imag * w.imag).sum().backward()
    _, da, _, _, dbu = oracle("imex1", a, g, st, bu, gx)
    assert so.max_rel_err(leaves[3].grad.cpu().numpy(), dbu) <= TOL_STATE
    assert so.max_rel_err(leaves[0].grad.cpu().numpy(), da) <= TOL_COEF


# ---------------------------------------------------------------------------
# BASELINE-sized sequences
# ---------------------------------------------------------------------------
@pytest.mark.parametrize("variant,L", [("imex1", 4096), ("im", 4096), ("linoss_im", 16384), ("linoss_imex", 4096)])
def test_long_sequence_raw_parameters(K, variant, L):
    """BASELINE distributions (A, G = relu(N(0,1)), dt = sigmoid(N(0,1))): about a
    quarter of the channels are undamped double integrators whose |x| grows like
    L^2, the hard case for float32.  Batch reduced so the oracle runs in seconds."""
    check_against_oracle(K, variant, make_case(L, 2, 256, seed=77, raw=True))


def test_full_size_adjoint_and_linearity(K):
    """BASELINE config 1 (B=64, L=4096, P=256): properties that need no oracle.
    <x(bu), gx> == <bu, grad_bu(gx)> (the backward is the exact adjoint of the
    forward) and the scan is linear in bu; coefficient gradients of the full batch
    equal the sum over two half batches."""
    L, B, P = 4096, 64, 256
    gen = torch.Generator(device="cuda").manual_seed(0)
    a, g, st = stable_params(P, torch.Generator().manual_seed(1))
    a, g, st = dev(a), dev(g), dev(st)
    bu = torch.view_as_complex(torch.randn(L, B, P, 2, generator=gen, device="cuda") * 0.5)
    gx = torch.view_as_complex(torch.randn(L, B, P, 2, generator=gen, device="cuda"))
    x, _, carries = K.lti_scan_forward("imex1", a, g, st, bu)
    ga, gg, gs, gbu = K.lti_scan_backward("imex1", a, g, st, bu, carries, gx)

    def rdot(u, v):
        return float((u.real.double() * v.real.double() + u.imag.double() * v.imag.double()).sum())

    lhs, rhs = rdot(x, gx), rdot(bu, gbu)
    scale = float(x.abs().double().pow(2).sum().sqrt() * gx.abs().double().pow(2).sum().sqrt())
    assert abs(lhs - rhs) <= 1e-6 * scale
    bu2 = torch.view_as_complex(torch.randn(L, B, P, 2, generator=gen, device="cuda") * 0.5)
    x2, _, _ = K.lti_scan_forward("imex1", a, g, st, bu2, want_carries=False)
    x12, _, _ = K.lti_scan_forward("imex1", a, g, st, bu + bu2, want_carries=False)
    assert float((x12 - (x + x2)).abs().max() / x12.abs().max()) <= 1e-5
    del x2, x12, bu2
    half = B // 2
    acc = [torch.zeros(P, device="cuda", dtype=torch.float64) for _ in range(3)]
    for sl in (slice(0, half), slice(half, B)):
        b_h, g_h = bu[:, sl].contiguous(), gx[:, sl].contiguous()
        _, _, c_h = K.lti_scan_forward("imex1", a, g, st, b_h)
        part = K.lti_scan_backward("imex1", a, g, st, b_h, c_h, g_h)
        for t, q in zip(acc, part[:3]):
            t += q.double()
    for full, parts in zip((ga, gg, gs), acc):
        assert float((full.double() - parts).abs().max() / parts.abs().max()) <= 1e-5


# ---------------------------------------------------------------------------
# time slices (state handed over by the caller)
# ---------------------------------------------------------------------------
@pytest.mark.parametrize("variant", ["imex1", "im", "linoss_imex"])
@pytest.mark.parametrize("cuts", [(37,), (32, 64), (1, 50, 99)], ids=lambda c: "-".join(map(str, c)))
@pytest.mark.parametrize("P", [35, 36], ids=["plain_loads", "tma"])
def test_time_slices_match_oracle(K, variant, cuts, P):
    """A sequence scanned slice by slice (forward first to last, backward last to first, state and adjoint
    handed over) gives the oracle's answer; cuts inside and on chunk boundaries, odd (plain-load kernels) and
    even (TMA-staged kernels) series counts."""
    L, B = 100, 3
    a, g, st, bu, gx = make_case(L, B, P, seed=sum(cuts))
    ref, da, dg, ds, dbu = oracle(variant, a, g, st, bu, gx)
    gv = None if variant.startswith("linoss") else dev(g)
    ad, sd, bud, gxd = dev(a), dev(st), dev(bu), dev(gx)
    bounds = [0, *cuts, L]
    spans = list(zip(bounds[:-1], bounds[1:]))
    states, carries, xs = [None], [], []
    for l0, l1 in spans:
        x, car, out = K.lti_scan_forward_slice(variant, ad, gv, sd, bud[l0:l1].contiguous(), state_in=states[-1])
        xs.append(x)
        carries.append(car)
        states.append(out)
    x = torch.cat(xs, 0)
    assert so.max_rel_err(x.cpu().numpy(), ref[..., 1]) <= TOL_STATE
    assert so.max_rel_err(states[-1].cpu().numpy(), ref[-1]) <= TOL_STATE
    adjoint, gbus, acc = None, [None] * len(spans), None
    for i in reversed(range(len(spans))):
        l0, l1 = spans[i]
        ga, gg, gs, gbu, adjoint = K.lti_scan_backward_slice(variant, ad, gv, sd, bud[l0:l1].contiguous(), carries[i],
                                                             gxd[l0:l1].contiguous(), state_in=states[i],
                                                             adjoint_in=adjoint)
        gbus[i] = gbu
        part = [ga, gg, gs]
        acc = part if acc is None else [p + q if p is not None else None for p, q in zip(acc, part)]
    assert so.max_rel_err(torch.cat(gbus, 0).cpu().numpy(), dbu) <= TOL_STATE
    assert so.max_rel_err(acc[0].cpu().numpy(), da) <= TOL_COEF
    assert so.max_rel_err(acc[2].cpu().numpy(), ds) <= TOL_COEF
    if acc[1] is not None:
        assert so.max_rel_err(acc[1].cpu().numpy(), dg) <= TOL_COEF


# ---------------------------------------------------------------------------
# time segments (long sequences of few series)
# ---------------------------------------------------------------------------
@pytest.mark.parametrize("variant", ["imex1", "im", "linoss_imex"])
@pytest.mark.parametrize("L,segments", [(700, 3), (1024, 8), (333, 5)])
def test_time_segments_match_oracle(K, variant, L, segments):
    """The sequence split into segments (summary pass, stitching by matrix power,
    segmented scan) gives the oracle's answer, forward and backward."""
    K.set_tuning("segments", segments)
    try:
        check_against_oracle(K, variant, make_case(L, 2, 64, seed=L + segments))
    finally:
        K.set_tuning("segments", 0)


def test_time_segments_raw_parameters_long(K):
    """Undamped double-integrator channels over 16k steps in 8 segments."""
    K.set_tuning("segments", 8)
    try:
        check_against_oracle(K, "imex1", make_case(16384, 1, 128, seed=8, raw=True))
    finally:
        K.set_tuning("segments", 0)


@pytest.mark.parametrize("variant", ["imex1", "im", "linoss_imex"])
@pytest.mark.parametrize("shape", [(1024, 8, 256), (1300, 16, 131), (4097, 4, 512)], ids=lambda s: "x".join(map(str, s)))
def test_two_level_kernels_match_oracle(K, variant, shape):
    """1536 .. 8192 series and a long sequence: CTAs of 16 series whose threads split a staged tile of 256
    steps in time (scan from zero, prefix over the sub-chunks, second sweep over the same tile).  Ragged
    lengths (partial tile, partial sub-chunk) and a series count that is not a multiple of 16 included."""
    from ossm_b200 import _lib

    L, B, P = shape
    lib = _lib.load()
    assert lib.ossm_b200_lti_forward_workspace_bytes(L, B, P) == 0                   # not the segmented path
    assert lib.ossm_b200_lti_backward_workspace_bytes(L, B, P) >= 6 * 8 * B * P * 4
    # 3e-5 on x: one of these seeded cases holds a nearly undamped low-frequency channel on which a plain
    # sequential float32 evaluation of the same inputs is already 1.9e-5 away from float64
    check_against_oracle(K, variant, make_case(L, B, P, seed=L + P), tol_state=3e-5)


def test_two_level_agrees_with_wide_kernels(K):
    """Same problem through the two-level kernels and (knob off) the one-lane-per-series kernels."""
    a, g, st, bu, gx = make_case(2048, 8, 256, seed=14)
    x1, s1, g1 = run_gpu(K, "imex1", a, g, st, bu, gx)
    K.set_tuning("twolevel", 0)
    K.set_tuning("segments", 1)
    try:
        x0, s0, g0 = run_gpu(K, "imex1", a, g, st, bu, gx)
    finally:
        K.set_tuning("segments", 0)
        K.set_tuning("twolevel", 1)
    assert float((x1 - x0).abs().max() / x0.abs().max()) <= 1e-5
    assert float((s1 - s0).abs().max() / s0.abs().max()) <= 1e-5
    for u, v in zip(g1, g0):
        assert float((u - v).abs().max() / v.abs().max()) <= 5e-5


def test_two_level_raw_parameters_long(K):
    """The 256-oscillator shard shape of the sharded layer (B = 8, P = 256) at a length the oracle still
    finishes in seconds, with the benchmark's raw parameter distributions (undamped channels)."""
    case = make_case(16384, 8, 256, seed=18, raw=True)
    a, g, st, bu, gx = case
    ref, da, dg, ds, dbu = oracle("imex1", a, g, st, bu, gx)
    errs = {}
    for name, knob in (("two-level", 1), ("one lane per series", 0)):
        K.set_tuning("twolevel", knob)
        K.set_tuning("segments", 0 if knob else 1)
        try:
            x, _, (ga, gg, gs, gbu) = run_gpu(K, "imex1", a, g, st, bu, gx, want_states=False)
        finally:
            K.set_tuning("twolevel", 1)
            K.set_tuning("segments", 0)
        tag = f"lti imex1 raw 16384x8x256 ({name})"
        errs[name] = {
            "x": record(tag, "x", so.max_rel_err(x.cpu().numpy(), ref[..., 1]), 1e-5),
            "grad_bu": record(tag, "grad_bu", so.max_rel_err(gbu.cpu().numpy(), dbu), 1e-5),
            "grad_A": record(tag, "grad_A", so.max_rel_err(ga.cpu().numpy(), da), 5e-5),
            "grad_G": record(tag, "grad_G", so.max_rel_err(gg.cpu().numpy(), dg), 5e-5),
            "grad_step": record(tag, "grad_step", so.max_rel_err(gs.cpu().numpy(), ds), 1e-3),
        }
    for name, e in errs.items():
        assert e["x"] <= 1e-5 and e["grad_bu"] <= 1e-5 and e["grad_A"] <= 5e-5 and e["grad_G"] <= 5e-5, (name, e)
        # the step-size gradient of the undamped channels is limited by the float32 state itself (any float32
        # evaluation order lands within a few 1e-4 of float64 over 16384 steps); the two kernels must be alike
        assert e["grad_step"] <= 1e-3, (name, e)


def test_automatic_segments_agree_with_unsplit(K):
    """A shape the heuristic splits (few series, long sequence) against the same
    problem forced to one segment."""
    a, g, st, bu, gx = make_case(8192, 2, 128, seed=12)
    x1, _, g1 = run_gpu(K, "imex1", a, g, st, bu, gx, want_states=False)      # automatic (split)
    K.set_tuning("segments", 1)
    try:
        x0, _, g0 = run_gpu(K, "imex1", a, g, st, bu, gx, want_states=False)
    finally:
        K.set_tuning("segments", 0)
    # the two differ by the float32 rounding of the unsplit pass (the stitched entry
    # states come from a double-precision matrix power)
    assert float((x1 - x0).abs().max() / x0.abs().max()) <= 1e-5
    for u, v in zip(g1, g0):
        assert float((u - v).abs().max() / v.abs().max()) <= 5e-5
