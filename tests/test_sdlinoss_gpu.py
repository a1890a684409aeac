"""GPU parity of the selective D-LinOSS scan (per-step coefficients) through the C ABI:
the reference-compatible ``sdlinoss_<v>_forward/backward`` entry points and the
``run_sdlinoss`` autograd op, against fixtures recorded from the reference and against the
float64 oracle on seeded inputs (TMA-staged and plain-load kernels, every broadcast form)."""
import math
import os

import numpy as np
import pytest
import torch

from oracle import scan_oracle as so

pytestmark = pytest.mark.gpu
G = np.load(os.path.join(os.path.dirname(__file__), "golden", "sdlinoss_generated.npz"))
VARIANTS = ("imex1", "imex2", "im", "ex")
X_TOL, GRAD_TOL = 1e-5, 5e-5     # relative to the largest magnitude of the tensor compared


def dev(t):
    return torch.as_tensor(t).to("cuda")


def fields(variant, L, B, M, gen, over_one=0.05):
    """(A, G, raw step) [L,B,M] from a pole radius / angle field, the map of the layer
    (``src/ossm/models/sdlinoss.py:186-204``); a fraction of the raw steps lies above 1.
    Long sequences of the variants with an explicit part (imex2, ex) use a field that varies
    slowly in time around a per-series pole -- a product of independent random transitions of
    those schemes grows without bound although each factor is stable."""
    if L > 64 and variant in ("imex2", "ex"):
        r = (torch.rand(1, B, M, generator=gen) * 0.6 + 0.3) + 0.03 * torch.randn(L, B, M, generator=gen)
        r = r.clamp(0.25, 0.95)
        th = (torch.rand(1, B, M, generator=gen) * 2 - 1) * 2.5 + 0.05 * torch.randn(L, B, M, generator=gen)
        raw = (torch.sigmoid(torch.randn(1, B, M, generator=gen)) * 0.9 + 0.05) * (
            1 + 0.03 * torch.randn(L, B, M, generator=gen))
    else:
        r = torch.rand(L, B, M, generator=gen) * 0.7 + 0.25
        th = (torch.rand(L, B, M, generator=gen) * 2 - 1) * 3.0
        raw = torch.sigmoid(torch.randn(L, B, M, generator=gen)) * 0.9 + 0.05
    raw = torch.where(torch.rand(L, B, M, generator=gen) < over_one, raw + 1.0, raw)
    dtc = torch.clamp(raw, min=1e-6, max=1.0)
    r2, c = r * r, torch.cos(th)
    if variant == "imex1":
        A, Gm = (r2 - 2 * r * c + 1) / (dtc * dtc * r2), (1 - r2) / (dtc * r2)
    elif variant == "imex2":
        A, Gm = (r2 - 2 * r * c + 1) / (dtc * dtc), (1 - r2) / dtc
    elif variant == "im":
        A, Gm = (r2 - 2 * r * c + 1) / (dtc * dtc * r2), (-2 * r2 + 2 * r * c) / (dtc * r2)
    else:   # explicit scheme: transition [[al, -dt^2 a], [al, 1 - dt^2 a]] with al = 1 - dt g has det r^2, trace 2 r cos
        A, Gm = (r2 - 2 * r * c + 1) / (dtc * dtc), (1 - r2) / dtc
    return A.float(), Gm.float(), raw.float()


def cplx(L, B, M, gen):
    return torch.complex(torch.randn(L, B, M, generator=gen), torch.randn(L, B, M, generator=gen))


PICK = {"M": lambda t: t[0, 0].contiguous(), "LM": lambda t: t[:, 0].contiguous(),
        "BM": lambda t: t[0].contiguous(), "LBM": lambda t: t.contiguous()}


@pytest.mark.parametrize("kind", ["LBM", "LM", "BM", "M", "clamp"])
@pytest.mark.parametrize("variant", VARIANTS)
def test_fixture(variant, kind):
    """Fixtures recorded from the reference's CPU kernels (float32) and its PyTorch recurrence
    (float64, autograd): the reference-compatible entry points and the autograd op."""
    from ossm_b200 import kernels
    from ossm_b200.sdlinoss import run_sdlinoss

    p = f"{variant}/{kind}/"
    a, g, s, bu, go = (dev(G[p + k]) for k in ("A", "G", "step", "bu", "grad_out"))
    states = getattr(kernels, f"sdlinoss_{variant}_forward")(a, g, s, bu)
    assert states.shape == (*bu.shape, 2) and states.dtype == torch.complex64
    assert so.max_rel_err(states.cpu().numpy(), G[p + "py64_states"]) <= X_TOL
    assert so.max_rel_err(states.cpu().numpy(), G[p + "cpp_states"]) <= X_TOL
    grads = getattr(kernels, f"sdlinoss_{variant}_backward")(a, g, s, bu, states, go)
    for name, got in zip(("grad_A", "grad_G", "grad_step", "grad_bu"), grads):
        want = G[p + "py64_" + name]
        assert tuple(got.shape) == want.shape, name
        assert so.max_rel_err(got.cpu().numpy(), want) <= GRAD_TOL, name
        assert so.max_rel_err(got.cpu().numpy(), G[p + "cpp_" + name]) <= 2 * GRAD_TOL, name
    # the autograd op (keeps carries, not states)
    leaves = [t.clone().requires_grad_(True) for t in (a, g, s, bu)]
    x = run_sdlinoss(variant, *leaves)
    assert torch.equal(x, states[..., 1])
    (x.real * go.real + x.imag * go.imag).sum().backward()
    for name, leaf in zip(("grad_A", "grad_G", "grad_step", "grad_bu"), leaves):
        assert so.max_rel_err(leaf.grad.cpu().numpy(), G[p + "py64_" + name]) <= GRAD_TOL, name


# N = B*M a multiple of 4 -> TMA-staged kernels; otherwise the plain-load kernels
SHAPES = [(1, 1, 4), (32, 2, 64), (33, 1, 128), (100, 3, 44), (257, 2, 200), (64, 3, 5), (97, 1, 3)]


@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: "x".join(map(str, s)))
@pytest.mark.parametrize("variant", VARIANTS)
def test_dense_matches_oracle(variant, shape):
    from ossm_b200 import kernels

    L, B, M = shape
    gen = torch.Generator().manual_seed(1000 + L)
    A, Gm, raw = fields(variant, L, B, M, gen)
    bu, go = cplx(L, B, M, gen), cplx(L, B, M, gen)
    x, states, carries = kernels.sdlinoss_scan_forward(variant, dev(A), dev(Gm), dev(raw), dev(bu), want_states=True)
    ref = so.sdlinoss_scan(variant, A.double().numpy(), Gm.double().numpy(), raw.double().numpy(),
                           bu.to(torch.complex128).numpy())
    assert so.max_rel_err(states.cpu().numpy(), ref) <= X_TOL
    assert torch.equal(x, states[..., 1])
    rg = so.sdlinoss_scan_backward(variant, A.double().numpy(), Gm.double().numpy(), raw.double().numpy(),
                                   bu.to(torch.complex128).numpy(), ref, go.to(torch.complex128).numpy())
    from_carries = kernels.sdlinoss_scan_backward(variant, dev(A), dev(Gm), dev(raw), dev(bu), dev(go), carries=carries)
    from_states = kernels.sdlinoss_scan_backward(variant, dev(A), dev(Gm), dev(raw), dev(bu), dev(go), states=states)
    for name, want, c, s in zip(("grad_A", "grad_G", "grad_step", "grad_bu"), rg, from_carries, from_states):
        assert so.max_rel_err(c.cpu().numpy(), want) <= GRAD_TOL, name
        assert torch.equal(c, s), name     # same kernel, same carry values
    # raw steps above 1 are clamped: their gradient is exactly zero
    assert torch.all(from_carries[2][dev(raw) >= 1.0] == 0)


@pytest.mark.parametrize("kind", ["M", "LM", "BM"])
@pytest.mark.parametrize("variant", VARIANTS)
def test_broadcast_forms_match_oracle(variant, kind):
    """Broadcast parameters over several chunks and several warps: gradients are summed over the
    broadcast axes (registers over time, atomics over the batch)."""
    from ossm_b200 import kernels

    L, B, M = 70, 3, 40
    gen = torch.Generator().manual_seed(77)
    A, Gm, raw = (PICK[kind](t) for t in fields(variant, L, B, M, gen, over_one=0.0))
    bu, go = cplx(L, B, M, gen), cplx(L, B, M, gen)
    x, _, carries = kernels.sdlinoss_scan_forward(variant, dev(A), dev(Gm), dev(raw), dev(bu))
    ref = so.sdlinoss_scan(variant, A.double().numpy(), Gm.double().numpy(), raw.double().numpy(),
                           bu.to(torch.complex128).numpy())
    assert so.max_rel_err(x.cpu().numpy(), ref[..., 1]) <= X_TOL
    rg = so.sdlinoss_scan_backward(variant, A.double().numpy(), Gm.double().numpy(), raw.double().numpy(),
                                   bu.to(torch.complex128).numpy(), ref, go.to(torch.complex128).numpy())
    got = kernels.sdlinoss_scan_backward(variant, dev(A), dev(Gm), dev(raw), dev(bu), dev(go), carries=carries)
    for name, want, g in zip(("grad_A", "grad_G", "grad_step", "grad_bu"), rg, got):
        assert tuple(g.shape) == want.shape, name
        assert so.max_rel_err(g.cpu().numpy(), want) <= GRAD_TOL, name


def test_mixed_forms_and_full_equivalence():
    """(M,), (L,M), (B,M) parameters in one call give what their materialised [L,B,M] fields give
    (tests/test_sdlinoss.py:80-110 of the reference)."""
    from ossm_b200.sdlinoss import run_sdlinoss

    L, B, M = 45, 4, 12
    gen = torch.Generator().manual_seed(5)
    A, Gm, raw = fields("imex1", L, B, M, gen, over_one=0.0)
    # a in [0, 1], g >= 0, dt <= 1 keeps a*dt^2 < 2*(2 + dt*g): stable for any mix of the three
    a, g, s = dev(torch.rand(M, generator=gen)), dev(Gm[:, 0].contiguous()), dev(raw[0].contiguous())
    bu = dev(cplx(L, B, M, gen))
    y = run_sdlinoss("imex1", a, g, s, bu)
    y_full = run_sdlinoss("imex1", a.expand(L, B, M).contiguous(), g.unsqueeze(1).expand(L, B, M).contiguous(),
                          s.unsqueeze(0).expand(L, B, M).contiguous(), bu)
    assert so.max_rel_err(y.cpu().numpy(), y_full.cpu().numpy()) <= 1e-6


def test_tma_and_plain_kernels_agree():
    from ossm_b200 import kernels

    L, B, M = 300, 4, 160
    gen = torch.Generator().manual_seed(9)
    A, Gm, raw = (dev(t) for t in fields("im", L, B, M, gen))
    bu, go = dev(cplx(L, B, M, gen)), dev(cplx(L, B, M, gen))
    x1, _, c1 = kernels.sdlinoss_scan_forward("im", A, Gm, raw, bu)
    g1 = kernels.sdlinoss_scan_backward("im", A, Gm, raw, bu, go, carries=c1)
    kernels.set_sdlinoss_tuning("force_plain", 1)
    try:
        x2, _, c2 = kernels.sdlinoss_scan_forward("im", A, Gm, raw, bu)
        g2 = kernels.sdlinoss_scan_backward("im", A, Gm, raw, bu, go, carries=c2)
    finally:
        kernels.set_sdlinoss_tuning("force_plain", 0)
    assert torch.equal(x1, x2) and torch.equal(c1, c2)      # same arithmetic, different staging
    for p, q in zip(g1, g2):
        assert torch.equal(p, q)


def test_zero_input_and_linearity_at_layer_size():
    """Size-independent properties on a layer-sized problem (L=2048, B=16, M=256): zero forcing
    gives an exactly zero trajectory (tests/test_sdlinoss.py:243-254), and the scan is linear in
    bu for fixed coefficients."""
    from ossm_b200 import kernels

    L, B, M = 2048, 16, 256
    gen = torch.Generator().manual_seed(3)
    A, Gm, raw = (dev(t) for t in fields("imex1", L, B, M, gen))
    z = torch.zeros(L, B, M, dtype=torch.complex64, device="cuda")
    x0, _, _ = kernels.sdlinoss_scan_forward("imex1", A, Gm, raw, z, want_carries=False)
    assert torch.count_nonzero(x0).item() == 0
    u, v = dev(cplx(L, B, M, gen)), dev(cplx(L, B, M, gen))
    xu, _, _ = kernels.sdlinoss_scan_forward("imex1", A, Gm, raw, u, want_carries=False)
    xv, _, _ = kernels.sdlinoss_scan_forward("imex1", A, Gm, raw, v, want_carries=False)
    xs, _, _ = kernels.sdlinoss_scan_forward("imex1", A, Gm, raw, u + 2 * v, want_carries=False)
    scale = xs.abs().max().item()
    assert (xs - (xu + 2 * xv)).abs().max().item() <= 2e-5 * scale
    assert kernels._lib.device_status() == 0


def test_autograd_matches_pytorch_recurrence():
    """End to end against a float64 PyTorch rollout of the recurrence differentiated by autograd."""
    from ossm_b200.sdlinoss import run_sdlinoss

    L, B, M = 40, 2, 8
    gen = torch.Generator().manual_seed(11)
    A, Gm, raw = fields("imex2", L, B, M, gen, over_one=0.0)
    bu = cplx(L, B, M, gen)
    leaves = [dev(t).requires_grad_(True) for t in (A, Gm, raw, bu)]
    y = run_sdlinoss("imex2", *leaves)
    y.abs().pow(2).sum().backward()
    ref = [t.double().requires_grad_(True) if not t.is_complex() else t.to(torch.complex128).requires_grad_(True)
           for t in (A, Gm, raw, bu)]
    a, g, s, u = ref
    w = torch.zeros(B, M, dtype=torch.complex128)
    x = torch.zeros(B, M, dtype=torch.complex128)
    xs = []
    for t in range(L):
        dt = torch.clamp(s[t], 1e-6, 1.0)
        S = torch.clamp(1 + dt * dt * a[t], min=1e-6)
        w = ((1 - dt * g[t]) * w + dt * dt * (-a[t] * x + u[t])) / S
        x = x + w
        xs.append(x)
    torch.stack(xs).abs().pow(2).sum().backward()
    for got, want in zip(leaves, ref):
        assert so.max_rel_err(got.grad.cpu().numpy(), want.grad.numpy()) <= GRAD_TOL


def test_empty_and_errors():
    from ossm_b200 import kernels
    from ossm_b200.sdlinoss import run_sdlinoss

    a = torch.ones(4, device="cuda")
    assert run_sdlinoss("imex1", a, a, a, torch.zeros(0, 2, 4, dtype=torch.complex64, device="cuda")).shape == (0, 2, 4)
    bu = torch.zeros(3, 2, 4, dtype=torch.complex64, device="cuda")
    with pytest.raises(ValueError, match="Unsupported variant"):
        run_sdlinoss("rk4", a, a, a, bu)
    with pytest.raises(ValueError, match="must be shaped"):
        run_sdlinoss("imex1", torch.ones(5, device="cuda"), a, a, bu)
    with pytest.raises(TypeError, match="complex"):
        run_sdlinoss("imex1", a, a, a, bu.real)
    with pytest.raises(TypeError, match="dtype"):
        run_sdlinoss("imex1", a.double(), a, a, bu)
    with pytest.raises(RuntimeError, match="CUDA"):
        kernels.sdlinoss_imex1_forward(a.cpu(), a.cpu(), a.cpu(), bu.cpu())
    with pytest.raises(RuntimeError, match="Expected size"):
        kernels.sdlinoss_imex1_forward(torch.ones(3, 2, 5, device="cuda"), a, a, bu)
    with pytest.raises(RuntimeError, match="states must have shape"):
        kernels.sdlinoss_ex_backward(a, a, a, bu, torch.zeros(3, 2, 4, dtype=torch.complex64, device="cuda"), bu)
    assert math.isfinite(float(kernels.sdlinoss_ex_forward(a, a, a, bu).abs().sum()))
