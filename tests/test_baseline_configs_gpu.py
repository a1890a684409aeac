"""Parity at the shapes, value distributions and dtypes of the benchmark configurations.

Each case runs the CUDA path through the C ABI on seeded inputs drawn as the configuration says and
compares every output tensor with the float64 oracle (max-norm relative error
``max|got-want| / max|want|``).  Batch / channel counts are cut down so that the numpy oracle finishes in
seconds; the sequence lengths, parameter distributions and dtypes are the configurations' own.

  config 2  LinOSS-IM and LinOSS-IMEX, L = 16384, A = relu(N), dt = sigmoid(N)
  config 3  Mamba selective scan, L = 8192, N = 16, A = -(1..16), delta = softplus(N(0,1) - 4),
            D = ones, SiLU gate; bfloat16 I/O (<= 2e-2) and float32 I/O
  config 4  D-LinOSS imex1, L = 131072 with few series (the 256-oscillator shard of a P = 2048 layer at
            B = 8 has 2048 series; here B = 1, P = 128), which takes the time-split kernels
"""
import numpy as np
import pytest
import torch

from oracle import scan_oracle as so
from _parity_report import record

pytestmark = pytest.mark.gpu


def dev(t, dtype=None):
    t = torch.as_tensor(t).to("cuda")
    return t.to(dtype) if dtype is not None else t


@pytest.fixture(autouse=True)
def _status_clean():
    yield
    from ossm_b200 import _lib

    torch.cuda.synchronize()
    assert _lib.device_status() == 0


def raw_case(L, B, P, seed):
    """A, G = relu(N(0,1)), dt = sigmoid(N(0,1)): about a quarter of the channels are undamped."""
    gen = torch.Generator().manual_seed(seed)
    a = torch.relu(torch.randn(P, generator=gen))
    g = torch.relu(torch.randn(P, generator=gen))
    st = torch.sigmoid(torch.randn(P, generator=gen))
    bu = torch.complex(torch.randn(L, B, P, generator=gen), torch.randn(L, B, P, generator=gen)) * 0.5
    gx = torch.complex(torch.randn(L, B, P, generator=gen), torch.randn(L, B, P, generator=gen))
    return a, g, st, bu, gx


def reference_fp32_errors(variant, case, tag, ref, da, dg, ds, dbu):
    """Errors of the reference's own compiled float32 CPU kernels on the same inputs, recorded beside
    ours (no assertion: they are context for the bounds, and the library is only there when the
    checker side has been built)."""
    from oracle.ref_loader import load_reference_kernels

    kern = load_reference_kernels()
    if kern is None or not hasattr(kern, f"dlinoss_{variant}_forward"):
        return
    a, g, st, bu, gx = case
    states = getattr(kern, f"dlinoss_{variant}_forward")(a, g, st, bu)
    ga, gg, gs, gbu = getattr(kern, f"dlinoss_{variant}_backward")(a, g, st, bu, states, gx)
    tag = tag + " [reference float32 CPU kernel]"
    record(tag, "x", so.max_rel_err(states[..., 1].numpy(), ref[..., 1]), float("nan"))
    record(tag, "grad_bu", so.max_rel_err(gbu.numpy(), dbu), float("nan"))
    record(tag, "grad_A", so.max_rel_err(ga.numpy(), da), float("nan"))
    record(tag, "grad_step", so.max_rel_err(gs.numpy(), ds), float("nan"))
    record(tag, "grad_G", so.max_rel_err(gg.numpy(), dg), float("nan"))


def lti_errors(K, variant, case, tag, tol_state, tol_coef, tol_step=None):
    tol_step = tol_coef if tol_step is None else tol_step
    a, g, st, bu, gx = case
    gv = None if variant.startswith("linoss") else dev(g)
    x, _, carries = K.lti_scan_forward(variant, dev(a), gv, dev(st), dev(bu))
    ga, gg, gs, gbu = K.lti_scan_backward(variant, dev(a), gv, dev(st), dev(bu), carries, dev(gx))
    a64, g64, s64 = a.double().numpy(), g.double().numpy(), st.double().numpy()
    bu64 = bu.to(torch.complex128).numpy()
    ref = so.lti_forward(variant, a64, g64, s64, bu64)
    da, dg, ds, dbu = so.lti_backward(variant, a64, g64, s64, bu64, gx.to(torch.complex128).numpy(), states=ref)
    assert record(tag, "x", so.max_rel_err(x.cpu().numpy(), ref[..., 1]), tol_state) <= tol_state
    assert record(tag, "grad_bu", so.max_rel_err(gbu.cpu().numpy(), dbu), tol_state) <= tol_state
    assert record(tag, "grad_A", so.max_rel_err(ga.cpu().numpy(), da), tol_coef) <= tol_coef
    assert record(tag, "grad_step", so.max_rel_err(gs.cpu().numpy(), ds), tol_step) <= tol_step
    if gg is not None:
        assert record(tag, "grad_G", so.max_rel_err(gg.cpu().numpy(), dg), tol_coef) <= tol_coef
    reference_fp32_errors(variant, case, tag, ref, da, dg, ds, dbu)


@pytest.mark.parametrize("variant", ["imex1", "imex2", "im"])
def test_config1_length(variant):
    from ossm_b200 import kernels as K

    # imex2 with raw parameters is unstable (|eig| > 1 when dt*G > 2 is possible); its parameters are
    # drawn small enough to stay bounded, the others use the configuration's distributions as they are
    case = raw_case(4096, 2, 256, seed=1)
    if variant == "imex2":
        a, g, st, bu, gx = case
        case = (a * 0.5, g * 0.3, st, bu, gx)
    lti_errors(K, variant, case, f"config1 {variant} L=4096 B=2 P=256", 1e-5, 1e-5, tol_step=3e-5)


@pytest.mark.parametrize("variant", ["linoss_im", "linoss_imex"])
def test_config2_length(variant):
    from ossm_b200 import kernels as K

    # grad_step on the undamped channels (A > 0, no damping: |eigenvalue| = 1) over 16384 steps is limited by the
    # float32 state itself: a plain sequential float32 evaluation with float64 sums sits at 3e-5 .. 1e-4 on these
    # inputs, whatever the kernel does; every other tensor stays within 1e-5
    lti_errors(K, variant, raw_case(16384, 2, 128, seed=2), f"config2 {variant} L=16384 B=2 P=128", 1e-5, 1e-5,
               tol_step=2.5e-4)


def test_config4_shard_length_automatic_segments():
    from ossm_b200 import _lib, kernels as K

    L, B, P = 131072, 1, 128
    # the heuristic must split this shape (that is the code path of the 256-oscillator shard)
    assert _lib.load().ossm_b200_lti_forward_workspace_bytes(L, B, P) > 0
    lti_errors(K, "imex1", raw_case(L, B, P, seed=4), "config4 imex1 L=131072 B=1 P=128 (time-split)", 1e-5, 5e-5,
               tol_step=5e-4)


def test_config4_shard_full_size_properties():
    """The whole 256-oscillator shard (B = 8, P = 256, L = 131072; 2048 series, two-level kernels) with
    stable parameters: the backward is the adjoint of the forward (<x(bu), g> = <bu, grad_bu(g)>), and the
    two-level kernels agree with the time-segmented kernels on x, grad_bu and the coefficient gradients."""
    from ossm_b200 import kernels as K
    from test_lti_scan_gpu import stable_params

    L, B, P = 131072, 8, 256
    gen = torch.Generator(device="cuda").manual_seed(0)
    a, g, st = (dev(t) for t in stable_params(P, torch.Generator().manual_seed(1)))
    bu = torch.view_as_complex(torch.randn(L, B, P, 2, generator=gen, device="cuda") * 0.5)
    gx = torch.view_as_complex(torch.randn(L, B, P, 2, generator=gen, device="cuda"))
    x, _, carries = K.lti_scan_forward("imex1", a, g, st, bu)
    grads = K.lti_scan_backward("imex1", a, g, st, bu, carries, gx)

    def rdot(u, v):
        return float((u.real.double() * v.real.double() + u.imag.double() * v.imag.double()).sum())

    scale = float(x.abs().double().pow(2).sum().sqrt() * gx.abs().double().pow(2).sum().sqrt())
    assert abs(rdot(x, gx) - rdot(bu, grads[3])) <= 1e-6 * scale
    K.set_tuning("twolevel", 0)
    try:
        x0, _, carries0 = K.lti_scan_forward("imex1", a, g, st, bu)
        grads0 = K.lti_scan_backward("imex1", a, g, st, bu, carries0, gx)
    finally:
        K.set_tuning("twolevel", 1)
    tag = "config4 shard L=131072 B=8 P=256: two-level against time-segmented kernels"
    assert record(tag, "x", float((x - x0).abs().max() / x0.abs().max()), 1e-5) <= 1e-5
    assert torch.equal(torch.view_as_real(carries), torch.view_as_real(carries0)) or float(
        (carries - carries0).abs().max() / carries0.abs().max()) <= 1e-5
    for name, u, v in zip(("grad_A", "grad_G", "grad_step", "grad_bu"), grads, grads0):
        tol = 1e-5 if name == "grad_bu" else 5e-5
        assert record(tag, name, float((u - v).abs().max() / v.abs().max()), tol) <= tol


def mamba_case(Bz, Dn, L, N, seed):
    gen = torch.Generator().manual_seed(seed)
    u = torch.randn(Bz, Dn, L, generator=gen)
    z = torch.randn(Bz, Dn, L, generator=gen)
    delta = torch.nn.functional.softplus(torch.randn(Bz, Dn, L, generator=gen) - 4)
    A = -torch.arange(1, N + 1, dtype=torch.float32).repeat(Dn, 1)
    Bm = torch.randn(Bz, L, N, generator=gen)
    Cm = torch.randn(Bz, L, N, generator=gen)
    go = torch.randn(Bz, Dn, L, generator=gen)
    return u, delta, A, Bm, Cm, z, go, torch.ones(Dn)


@pytest.mark.parametrize("io,tol", [(torch.bfloat16, 2e-2), (torch.float32, 1e-4)], ids=["bf16", "f32"])
@pytest.mark.parametrize("serial", [1, 0], ids=["serial", "time_parallel"])
def test_config3_forward_and_all_gradients(io, tol, serial):
    """B = 1, D = 64: one CTA tile of channels, so dB / dC are complete sums over the channels."""
    from ossm_b200 import kernels as K

    u, delta, A, Bm, Cm, z, go, Dv = mamba_case(1, 64, 8192, 16, seed=3)
    rnd = (lambda t: t.to(io).double().numpy())
    K.set_selective_scan_tuning("serial", serial)
    try:
        args = [dev(u, io), dev(delta), dev(A), dev(Bm, io), dev(Cm, io), dev(z, io)]
        out, states = K.selective_scan_fwd(*args, dev(Dv))
        grads = K.selective_scan_bwd(dev(go, io), *args, states, dev(Dv))
    finally:
        K.set_selective_scan_tuning("serial", 1)
    oargs = [rnd(u), delta.double().numpy(), A.double().numpy(), rnd(Bm), rnd(Cm)]
    ref_out = so.selective_scan(*oargs, gate=rnd(z), D=Dv.double().numpy())
    ref_grads = so.selective_scan_backward(rnd(go), *oargs, gate=rnd(z), D=Dv.double().numpy())
    tag = f"config3 {'bf16' if io == torch.bfloat16 else 'f32'} {'serial' if serial else 'time-parallel'} L=8192 D=64"
    assert record(tag, "out", so.max_rel_err(out.float().cpu().numpy(), ref_out), tol) <= tol
    for name, got, want in zip(("du", "ddelta", "dA", "dB", "dC", "dz", "dD"), grads, ref_grads):
        assert record(tag, name, so.max_rel_err(got.float().cpu().numpy(), want), tol) <= tol, name


@pytest.mark.parametrize("variant", ["imex1", "imex2", "im", "ex"])
def test_torch_library_ops_on_cuda(variant):
    """``torch.ops.ossm_b200.dlinoss_<v>_forward / _backward`` (the schemas of the reference's
    ``ossm::dlinoss_*`` ops, _dlinoss_scan.py:183-206) dispatch to the CUDA implementation."""
    import ossm_b200.dlinoss  # noqa: F401  (registers the ops)
    from ossm_b200 import kernels as K

    gen = torch.Generator().manual_seed(9)
    P, L, B = 24, 70, 3
    a = torch.rand(P, generator=gen) * 0.8
    g = torch.rand(P, generator=gen) * 0.3
    st = torch.sigmoid(torch.randn(P, generator=gen)) * 0.5
    bu = torch.complex(torch.randn(L, B, P, generator=gen), torch.randn(L, B, P, generator=gen))
    gx = torch.complex(torch.randn(L, B, P, generator=gen), torch.randn(L, B, P, generator=gen))
    fwd = getattr(torch.ops.ossm_b200, f"dlinoss_{variant}_forward")
    bwd = getattr(torch.ops.ossm_b200, f"dlinoss_{variant}_backward")
    states = fwd(dev(a), dev(g), dev(st), dev(bu))
    assert states.shape == (L, B, P, 2) and states.is_cuda
    ga, gg, gs, gbu = bwd(dev(a), dev(g), dev(st), dev(bu), states, dev(gx))
    a64, g64, s64 = a.double().numpy(), g.double().numpy(), st.double().numpy()
    ref = so.lti_forward(variant, a64, g64, s64, bu.to(torch.complex128).numpy())
    da, dg, ds, dbu = so.lti_backward(variant, a64, g64, s64, bu.to(torch.complex128).numpy(),
                                      gx.to(torch.complex128).numpy(), states=ref)
    assert so.max_rel_err(states.cpu().numpy(), ref) <= 1e-5
    assert so.max_rel_err(gbu.cpu().numpy(), dbu) <= 1e-5
    for got, want in ((ga, da), (gg, dg), (gs, ds)):
        assert so.max_rel_err(got.cpu().numpy(), want) <= 5e-5
    # same numbers as the direct call
    assert torch.equal(torch.view_as_real(states), torch.view_as_real(getattr(K, f"dlinoss_{variant}_forward")(
        dev(a), dev(g), dev(st), dev(bu))))


def test_bounded_wait_gives_up_and_reports():
    """A wait on a barrier that nothing completes runs out after its limit, the kernel returns, and the
    status word says so (and is cleared by the read)."""
    import ctypes

    from ossm_b200 import _lib

    lib = _lib.load()
    assert _lib.device_status() == 0
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    rc = lib.ossm_b200_selftest_wait_timeout(2_000_000, ctypes.c_void_p(flag.data_ptr()),
                                             ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0, lib.ossm_b200_last_error()
    torch.cuda.synchronize()
    assert int(flag.item()) == 1
    assert _lib.device_status(clear=True) == 1
    assert _lib.device_status() == 0
