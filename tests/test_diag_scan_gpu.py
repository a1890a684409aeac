"""GPU parity of the complex diagonal scan (``lru_scan`` / ``s5_scan`` entry points
and the autograd op) against the oracle and fixtures recorded from the reference."""
import os

import numpy as np
import pytest
import torch

from oracle import scan_oracle as so

pytestmark = pytest.mark.gpu
G = np.load(os.path.join(os.path.dirname(__file__), "golden", "diag_generated.npz"))


def dev(t):
    return torch.as_tensor(t).to("cuda")


@pytest.mark.parametrize("tag", ["d1", "d2"])
def test_fixture(tag):
    from ossm_b200 import kernels
    from ossm_b200.diag import run_diag_scan

    p = f"{tag}/"
    lam = dev(G[p + "lambda"]).requires_grad_(True)
    b = dev(G[p + "b_seq"]).requires_grad_(True)
    go = dev(G[p + "grad_out"])
    x = run_diag_scan(lam, b)
    (x.real * go.real + x.imag * go.imag).sum().backward()
    assert so.max_rel_err(x.detach().cpu().numpy(), G[p + "lru_states"]) <= 5e-6
    assert so.max_rel_err(lam.grad.cpu().numpy(), G[p + "lru_grad_lambda"]) <= 5e-5
    assert so.max_rel_err(b.grad.cpu().numpy(), G[p + "s5_grad_b"]) <= 5e-5
    # reference-compatible entry points: real view in, real view out
    for fn in (kernels.lru_scan, kernels.s5_scan):
        raw = fn(lam.detach().real.contiguous(), lam.detach().imag.contiguous(),
                 torch.view_as_real(b.detach()).contiguous())
        assert raw.shape == (*b.shape, 2) and raw.dtype == torch.float32
        assert so.max_rel_err(torch.view_as_complex(raw.contiguous()).cpu().numpy(), G[p + "cpp_states"]) <= 5e-6


@pytest.mark.parametrize("shape", [(1, 1, 1), (33, 2, 7), (300, 3, 130), (2048, 2, 64)],
                         ids=lambda s: "x".join(map(str, s)))
def test_matches_oracle(shape):
    from ossm_b200 import kernels

    L, B, P = shape
    gen = torch.Generator().manual_seed(L)
    lam = torch.polar(torch.rand(P, generator=gen) * 0.55 + 0.44, torch.rand(P, generator=gen) * 6.28)
    b = torch.complex(torch.randn(L, B, P, generator=gen), torch.randn(L, B, P, generator=gen))
    go = torch.complex(torch.randn(L, B, P, generator=gen), torch.randn(L, B, P, generator=gen))
    lr, li = dev(lam.real.contiguous()), dev(lam.imag.contiguous())
    x, carries = kernels.diag_scan_forward(lr, li, dev(b))
    gl, gb = kernels.diag_scan_backward(lr, li, dev(b), carries, dev(go))
    lam64 = lam.to(torch.complex128).numpy()
    ref = so.diag_scan(lam64, b.to(torch.complex128).numpy())
    rgl, rgb = so.diag_scan_backward(lam64, ref, go.to(torch.complex128).numpy())
    assert so.max_rel_err(x.cpu().numpy(), ref) <= 1e-5
    assert so.max_rel_err(gb.cpu().numpy(), rgb) <= 1e-5
    assert so.max_rel_err(gl.cpu().numpy(), rgl) <= 5e-5


def test_empty_and_errors():
    from ossm_b200 import kernels

    lam = torch.zeros(4, device="cuda")
    empty = torch.zeros(0, 2, 4, 2, device="cuda")
    assert kernels.lru_scan(lam, lam, empty).shape == (0, 2, 4, 2)
    with pytest.raises(RuntimeError, match="state dimension"):
        kernels.lru_scan(lam, lam, torch.zeros(3, 2, 5, 2, device="cuda"))
    with pytest.raises(RuntimeError, match="shape"):
        kernels.s5_scan(lam, lam, torch.zeros(3, 2, 4, device="cuda"))
