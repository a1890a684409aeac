"""``scan_from_host``: pinned host buffers in, pinned host buffers out, time slices
pipelined over PCIe with the recurrence state handed from slice to slice on the device --
same numbers as the device-resident op."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("slices", [1, 3, 16])
@pytest.mark.parametrize("variant", ["imex1", "linoss_im"])
def test_scan_from_host_matches_device_op(variant, slices):
    from ossm_b200 import kernels
    from ossm_b200.host_io import scan_from_host

    gen = torch.Generator().manual_seed(slices)
    L, B, P = 150, 7, 40
    a = (torch.rand(P, generator=gen) * 0.8).cuda()
    g = None if variant.startswith("linoss") else (torch.rand(P, generator=gen) * 0.3).cuda()
    st = torch.sigmoid(torch.randn(P, generator=gen)).cuda()
    bu = (torch.complex(torch.randn(L, B, P, generator=gen), torch.randn(L, B, P, generator=gen)) * 0.5).pin_memory()
    gx = torch.complex(torch.randn(L, B, P, generator=gen), torch.randn(L, B, P, generator=gen)).pin_memory()
    x_h = torch.empty_like(bu).pin_memory()
    gbu_h = torch.empty_like(bu).pin_memory()
    grads = scan_from_host(variant, a, g, st, bu, gx, x_h, gbu_h, slices=slices)
    x, _, carries = kernels.lti_scan_forward(variant, a, g, st, bu.cuda())
    ga, gg, gs, gbu = kernels.lti_scan_backward(variant, a, g, st, bu.cuda(), carries, gx.cuda())
    # slices start on multiples of the carry interval: every step is the same arithmetic, x and grad_bu are identical
    assert torch.equal(torch.view_as_real(x_h), torch.view_as_real(x.cpu()))
    assert torch.equal(torch.view_as_real(gbu_h), torch.view_as_real(gbu.cpu()))
    # coefficient gradients are summed slice by slice: equal up to float32 summation order
    for got, want in zip(grads, (ga, gg, gs)):
        if want is None:
            assert got is None
        else:
            assert float((got - want).abs().max()) <= 1e-5 * float(want.abs().max())
    # forward only
    x2 = torch.empty_like(bu).pin_memory()
    assert scan_from_host(variant, a, g, st, bu, None, x2, slices=slices) is None
    assert torch.equal(torch.view_as_real(x2), torch.view_as_real(x_h))


def test_scan_from_host_rejects_pageable_memory():
    from ossm_b200.host_io import scan_from_host

    a = torch.rand(4).cuda()
    bu = torch.zeros(5, 2, 4, dtype=torch.complex64)
    with pytest.raises(RuntimeError, match="pinned"):
        scan_from_host("imex1", a, a, a, bu, None, torch.empty_like(bu))
