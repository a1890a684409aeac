"""The allocation-free backward entry point (``ossm_b200_lti_scan_backward_static``).

It exists for callers that are not allowed to create device memory when they call
the library (a process that pins its memory plan at start-up, or a thin
foreign-language binding with no allocator of its own): the scratch the backward
needs sits in a fixed array inside the library.  The test drives it through the
C ABI with pre-made buffers only and checks it against the regular entry point,
twice in a row, because the array keeps whatever the previous call left there.
The file name sorts last so that a run that stops at the first failure has
already covered everything else.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr())


def _case(L, B, P, seed):
    gen = torch.Generator().manual_seed(seed)
    a = torch.rand(P, generator=gen) * 0.8
    g = torch.rand(P, generator=gen) * 0.3
    st = torch.sigmoid(torch.randn(P, generator=gen))
    bu = torch.complex(torch.randn(L, B, P, generator=gen), torch.randn(L, B, P, generator=gen)) * 0.5
    gx = torch.complex(torch.randn(L, B, P, generator=gen), torch.randn(L, B, P, generator=gen))
    return [t.cuda() for t in (a, g, st, bu, gx)]


def _run_static(lib, variant, a, g, st, bu, carries, gx):
    L, B, P = bu.shape
    grad_bu = torch.empty_like(bu)
    ga, gg, gs = (torch.empty_like(a) for _ in range(3))
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    rc = lib.ossm_b200_lti_scan_backward_static(
        variant, _ptr(a), _ptr(g), _ptr(st), _ptr(bu), _ptr(carries) if carries.numel() else None, _ptr(gx),
        _ptr(grad_bu), _ptr(ga), _ptr(gg), _ptr(gs), L, B, P, stream)
    assert rc == 0, lib.ossm_b200_last_error()
    return ga, gg, gs, grad_bu


def test_static_scratch_backward_matches_workspace_backward():
    from ossm_b200 import _lib, kernels

    lib = _lib.load()
    assert lib.ossm_b200_lti_scan_backward_static_max_series() == 65536
    # two calls in a row, different shapes and variants: the second one finds the
    # scratch as the first one left it
    for (L, B, P, name, vid) in ((200, 6, 96, "imex1", 0), (97, 3, 40, "im", 2)):
        a, g, st, bu, gx = _case(L, B, P, seed=L)
        _, _, carries = kernels.lti_scan_forward(name, a, g, st, bu)
        want = kernels.lti_scan_backward(name, a, g, st, bu, carries, gx)
        got = _run_static(lib, vid, a, g, st, bu, carries, gx)
        torch.cuda.synchronize()
        for w, q in zip(want, got):
            w = torch.view_as_real(w) if w.is_complex() else w
            q = torch.view_as_real(q) if q.is_complex() else q
            # same kernels, same order of operations: the results are identical,
            # which is well inside the 1e-5 / 5e-5 bounds of the parity tests
            assert torch.equal(w, q)
    assert _lib.device_status() == 0


def test_static_scratch_with_time_segments():
    """Few series and a long sequence: the backward splits the time axis and keeps the segment
    summaries in the same built-in array.  Same split, same kernels as the workspace entry, so the
    results are identical; a second call straight after finds the array used and still agrees."""
    from ossm_b200 import _lib, kernels

    lib = _lib.load()
    for (L, B, P, name, vid) in ((2048, 2, 64, "imex1", 0), (4096, 1, 96, "im", 2)):
        assert lib.ossm_b200_lti_backward_workspace_bytes(L, B, P) > 6 * B * P * 4     # the heuristic splits it
        a, g, st, bu, gx = _case(L, B, P, seed=L + P)
        _, _, carries = kernels.lti_scan_forward(name, a, g, st, bu)
        want = kernels.lti_scan_backward(name, a, g, st, bu, carries, gx)
        for _ in range(2):
            got = _run_static(lib, vid, a, g, st, bu, carries, gx)
            torch.cuda.synchronize()
            for w, q in zip(want, got):
                w = torch.view_as_real(w) if w.is_complex() else w
                q = torch.view_as_real(q) if q.is_complex() else q
                assert torch.equal(w, q)
    assert _lib.device_status() == 0


def test_static_scratch_rejects_oversized_problems():
    from ossm_b200 import _lib

    lib = _lib.load()
    dummy = ctypes.c_void_p(256)
    rc = lib.ossm_b200_lti_scan_backward_static(0, dummy, dummy, dummy, dummy, dummy, dummy, dummy, dummy, dummy,
                                                dummy, 64, 1024, 128, None)      # 131072 series > 65536
    assert rc == -4
    assert b"exceed the built-in scratch" in lib.ossm_b200_last_error()
