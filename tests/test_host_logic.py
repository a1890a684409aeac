"""Host-side behaviour of the Python mirror of the reference interface that
needs no GPU: argument checks raise ``RuntimeError``/``ValueError`` like the
reference's TORCH_CHECKs (``dlinoss_imex1.cpp:321-341``), empty inputs return
early, CPU tensors are refused loudly (no CPU path)."""
import pytest
import torch

from ossm_b200 import kernels
from ossm_b200.dlinoss import run_dlinoss


def _params(P):
    return torch.rand(P), torch.rand(P), torch.rand(P)


def test_cpu_tensors_are_refused():
    a, g, s = _params(4)
    bu = torch.zeros(5, 2, 4, dtype=torch.complex64)
    with pytest.raises(RuntimeError, match="CUDA"):
        kernels.dlinoss_imex1_forward(a, g, s, bu)
    with pytest.raises(RuntimeError, match="CUDA"):
        run_dlinoss("imex1", a, g, s, bu)


def test_shape_checks_match_reference_messages():
    a, g, s = _params(4)
    with pytest.raises(RuntimeError, match="bu must have shape"):
        kernels.dlinoss_im_forward(a, g, s, torch.zeros(5, 4, dtype=torch.complex64))
    with pytest.raises(RuntimeError, match="must match state size"):
        kernels.dlinoss_im_forward(a, g, s, torch.zeros(5, 2, 3, dtype=torch.complex64))
    with pytest.raises(RuntimeError, match="1-D"):
        kernels.dlinoss_im_forward(a.view(2, 2), g, s, torch.zeros(5, 2, 4, dtype=torch.complex64))


def test_unknown_variant_and_empty_input():
    a, g, s = _params(4)
    with pytest.raises(ValueError, match="Unknown D-LinOSS variant"):
        run_dlinoss("imex3", a, g, s, torch.zeros(5, 2, 4, dtype=torch.complex64))
    empty = torch.zeros(0, 2, 4, dtype=torch.complex64)
    assert run_dlinoss("ex", a, g, s, empty) is empty          # _dlinoss_scan.py:641-642


def test_float64_is_rejected_not_silently_rerouted():
    a, g, s = _params(4)
    bu = torch.zeros(5, 2, 4, dtype=torch.complex128)
    with pytest.raises(RuntimeError, match="float32"):
        run_dlinoss("imex1", a.double(), g.double(), s.double(), bu)


def test_torch_library_ops_registered():
    for v in ("imex1", "imex2", "im", "ex"):
        assert hasattr(torch.ops.ossm_b200, f"dlinoss_{v}_forward")
        assert hasattr(torch.ops.ossm_b200, f"dlinoss_{v}_backward")
    # meta kernels give shapes without touching a device
    a = torch.empty(4, device="meta")
    bu = torch.empty(5, 2, 4, dtype=torch.complex64, device="meta")
    st = torch.ops.ossm_b200.dlinoss_imex1_forward(a, a, a, bu)
    assert tuple(st.shape) == (5, 2, 4, 2)
