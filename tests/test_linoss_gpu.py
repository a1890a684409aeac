"""GPU parity of the LinOSS entry points: the generic complex 2x2 scan
(``linoss_scan`` + ``LinossScanFn``) and the layer recurrence (``run_linoss``),
against the oracle, the reference's inline snapshot and fixtures recorded from
the reference's own ``_LinossScanFn`` (Python-loop backward)."""
import os

import numpy as np
import pytest
import torch

from oracle import scan_oracle as so

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")
LGEN = np.load(os.path.join(GOLD, "linoss_generated.npz"))


def dev(t):
    return torch.as_tensor(t).to("cuda")


@pytest.mark.parametrize("tag", ["c1", "c2"])
def test_generic_scan_fixture_complex(tag):
    from ossm_b200.linoss import LinossScanFn

    p = f"scan/{tag}/"
    am = dev(LGEN[p + "a_matrix"]).requires_grad_(True)
    b = dev(LGEN[p + "b_seq"]).requires_grad_(True)
    go = dev(LGEN[p + "grad_out"])
    st = LinossScanFn.apply(am, b)
    (st.real * go.real + st.imag * go.imag).sum().backward()
    # tolerances of the reference's own test (test_linoss_parity.py:44-53): 1e-6 / 5e-5
    assert so.max_rel_err(st.detach().cpu().numpy(), LGEN[p + "states"]) <= 5e-6
    assert so.max_rel_err(am.grad.cpu().numpy(), LGEN[p + "grad_a"]) <= 5e-5
    assert so.max_rel_err(b.grad.cpu().numpy(), LGEN[p + "grad_b"]) <= 5e-5


@pytest.mark.parametrize("tag", ["c1", "c2"])
def test_generic_scan_fixture_real_matrix(tag):
    from ossm_b200.linoss import run_associative_scan

    p = f"scan/{tag}/"
    ar = dev(LGEN[p + "real_a_matrix"]).requires_grad_(True)
    b = dev(LGEN[p + "b_seq"]).requires_grad_(True)
    go = dev(LGEN[p + "grad_out"])
    st = run_associative_scan(ar, b)
    (st.real * go.real + st.imag * go.imag).sum().backward()
    assert ar.grad.dtype == torch.float32          # real matrix keeps a real gradient (linoss.py:133-138)
    assert so.max_rel_err(st.detach().cpu().numpy(), LGEN[p + "real_states"]) <= 5e-6
    assert so.max_rel_err(ar.grad.cpu().numpy(), LGEN[p + "real_grad_a"]) <= 5e-5
    assert so.max_rel_err(b.grad.cpu().numpy(), LGEN[p + "real_grad_b"]) <= 5e-5


@pytest.mark.parametrize("shape", [(2, 1, 1), (7, 3, 5), (64, 2, 33), (200, 4, 130), (33, 1, 64), (129, 2, 64),
                                   (500, 3, 70), (1000, 8, 256)],
                         ids=lambda s: "x".join(map(str, s)))
def test_generic_scan_matches_oracle(shape):
    """Tiles of 32 steps x 64 series through a four-deep ring: lengths around one tile, past the ring depth and
    with a ragged tail; series counts below, at and across the 64-series box."""
    from ossm_b200 import kernels

    L, B, P = shape
    gen = torch.Generator().manual_seed(L + B + P)
    am = (torch.complex(torch.randn(P, 2, 2, generator=gen), torch.randn(P, 2, 2, generator=gen)) * 0.2)
    b = torch.complex(torch.randn(L, B, P, 2, generator=gen), torch.randn(L, B, P, 2, generator=gen))
    go = torch.complex(torch.randn(L, B, P, 2, generator=gen), torch.randn(L, B, P, 2, generator=gen))
    m = [dev(am[:, i, j].contiguous()) for i in (0, 1) for j in (0, 1)]
    st = kernels.linoss_scan(*m, dev(b))
    gm, gb = kernels.linoss_scan_backward(*m, st, dev(go))
    am64 = am.to(torch.complex128).numpy()
    ref = so.linoss_scan(am64[:, 0, 0], am64[:, 0, 1], am64[:, 1, 0], am64[:, 1, 1], b.to(torch.complex128).numpy())
    rgm, rgb = so.linoss_scan_backward(am64, ref, go.to(torch.complex128).numpy())
    assert so.max_rel_err(st.cpu().numpy(), ref) <= 1e-5
    assert so.max_rel_err(gb.cpu().numpy(), rgb) <= 1e-5
    assert so.max_rel_err(gm.cpu().numpy(), rgm) <= 5e-5


def test_short_sequences_pass_through():
    from ossm_b200.linoss import run_associative_scan, try_run_scan

    am = dev(torch.randn(3, 2, 2, dtype=torch.complex64)).requires_grad_(True)
    b1 = dev(torch.randn(1, 2, 3, 2, dtype=torch.complex64)).requires_grad_(True)
    out = run_associative_scan(am, b1)              # linoss.py:62-65
    assert torch.equal(torch.view_as_real(out.detach()), torch.view_as_real(b1.detach()))
    out.real.sum().backward()
    assert float(am.grad.abs().sum()) == 0.0
    empty = torch.zeros(0, 2, 3, 2, dtype=torch.complex64, device="cuda")
    m = [am.detach()[:, i, j].contiguous() for i in (0, 1) for j in (0, 1)]
    assert try_run_scan(*m, empty) is empty         # _linoss_scan.py:52-53


def test_linoss_im_snapshot_through_layer_math():
    """The reference's inline golden (test_linoss_parity.py:74-204): LinOSSLayer('IM')."""
    from ossm_b200.linoss import linoss_recurrence

    s = np.load(os.path.join(GOLD, "linoss_im_snapshot.npz"))
    a = torch.relu(dev(s["A_diag"]))
    step = torch.sigmoid(dev(s["steps"]))
    u = dev(s["inputs"])
    bsz, L, H = u.shape
    Bp, Cp, D = dev(s["B"]), dev(s["C"]).view(H, -1, 2), dev(s["D"])
    flat = u.reshape(bsz * L, H)
    bu = torch.complex(flat @ Bp[..., 0].T, flat @ Bp[..., 1].T).reshape(bsz, L, -1)
    x = linoss_recurrence("IM", a, step, bu).reshape(bsz * L, -1)
    y = (x.real @ Cp[..., 0].T - x.imag @ Cp[..., 1].T).reshape(bsz, L, H) + u * D
    np.testing.assert_allclose(y.cpu().numpy(), s["outputs"], rtol=5e-6, atol=5e-6)


@pytest.mark.parametrize("disc", ["IM", "IMEX"])
def test_run_linoss_autograd(disc):
    from ossm_b200.linoss import linoss_recurrence

    p = f"layer/{disc}/"
    a = dev(LGEN[p + "a"]).float().requires_grad_(True)
    st = dev(LGEN[p + "step"]).float().requires_grad_(True)
    bu = dev(LGEN[p + "bu"]).to(torch.complex64).requires_grad_(True)
    gx = dev(LGEN[p + "grad_x"]).to(torch.complex64)
    x = linoss_recurrence(disc, a, st, bu)
    (x.real * gx.real + x.imag * gx.imag).sum().backward()
    assert so.max_rel_err(x.detach().cpu().numpy(), LGEN[p + "x"]) <= 1e-5
    assert so.max_rel_err(a.grad.cpu().numpy(), LGEN[p + "da"]) <= 5e-5
    assert so.max_rel_err(st.grad.cpu().numpy(), LGEN[p + "dstep"]) <= 5e-5
    assert so.max_rel_err(bu.grad.cpu().numpy(), LGEN[p + "dbu"]) <= 1e-5
