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


def test_sdlinoss_parameter_forms_and_errors():
    """Selective D-LinOSS host logic: axis assignment of (M,), (L,M), (B,M), (L,B,M) parameters as element strides
    (0 = broadcast), the reference's messages for bad shapes, and no CPU path."""
    from ossm_b200.sdlinoss import run_sdlinoss

    L, B, M = 6, 3, 5
    full = torch.rand(L, B, M)
    assert kernels._sd_field(full, "A", L, B, M)[1] == [B * M, M, 1]
    assert kernels._sd_field(full[0, 0].contiguous(), "A", L, B, M)[1] == [0, 0, 1]
    assert kernels._sd_field(full[:, 0].contiguous(), "A", L, B, M)[1] == [M, 0, 1]        # first axis = length
    assert kernels._sd_field(full[0].contiguous(), "A", L, B, M)[1] == [0, M, 1]           # first axis = batch
    assert kernels._sd_field(full[:1].contiguous(), "A", L, B, M)[1] == [0, M, 1]
    with pytest.raises(RuntimeError, match="Expected size"):
        kernels._sd_field(torch.rand(L, B, M + 1), "A", L, B, M)
    with pytest.raises(RuntimeError, match="First dimension must match length or batch"):
        kernels._sd_field(torch.rand(4, M), "A", L, B, M)
    with pytest.raises(RuntimeError, match="1, 2, or 3 dimensions"):
        kernels._sd_field(torch.rand(1, L, B, M), "A", L, B, M)
    bu = torch.zeros(L, B, M, dtype=torch.complex64)
    a = torch.rand(M)
    with pytest.raises(ValueError, match="Unsupported variant"):
        run_sdlinoss("rk4", a, a, a, bu)
    with pytest.raises(ValueError, match="must be shaped"):
        run_sdlinoss("imex1", torch.rand(M + 1), a, a, bu)
    with pytest.raises(TypeError, match="complex"):
        run_sdlinoss("imex1", a, a, a, bu.real)
    with pytest.raises(RuntimeError, match="CUDA"):
        run_sdlinoss("imex1", a, a, a, bu)                                               # valid shapes, CPU tensors
    assert run_sdlinoss("ex", a, a, a, torch.zeros(0, B, M, dtype=torch.complex64)).shape == (0, B, M)


def test_selective_scan_host_checks():
    """Selective-scan wrappers: shape checks before any device work, tuning keys, state interval by state size."""
    u = torch.zeros(2, 3, 8)
    A = torch.zeros(3, 16)
    Bm = torch.zeros(2, 8, 16)
    with pytest.raises(RuntimeError, match="dt must match"):
        kernels.selective_scan_fwd(u, torch.zeros(2, 3, 7), A, Bm, Bm)
    with pytest.raises(RuntimeError, match="A must have shape"):
        kernels.selective_scan_fwd(u, u, torch.zeros(4, 16), Bm, Bm)
    assert kernels.selective_scan_chunk(16) == 8          # serial kernels: a saved state every 8 steps
    assert kernels.selective_scan_chunk(32) == 32         # states split over lanes: a saved state every 32 steps
    assert kernels.selective_scan_chunk(256) == 32
    assert kernels.selective_scan_chunk(24) == 64         # no serial kernel for this size: time-parallel kernels
    kernels.set_selective_scan_tuning("serial", 0)
    try:
        assert kernels.selective_scan_chunk(16) == 128
        assert kernels.selective_scan_chunk(32) == 64
    finally:
        kernels.set_selective_scan_tuning("serial", 1)
    with pytest.raises(RuntimeError, match="unknown key"):
        kernels.set_selective_scan_tuning("no_such_key", 1)


def test_selective_scan_bc_operand_choice():
    """Which form of ossm's ``B, C [B, L, N]`` arguments reaches the library: time-contiguous views as they are,
    step-major tensors (dense or pitched column slices of one projection, ``mambarec.py:153-154``) as they are where
    the kernels of the state size read that order, a transposing copy otherwise."""

    class Lib:
        def __init__(self, sizes):
            self.sizes = sizes

        def ossm_b200_selective_scan_step_major_bc(self, n):
            return 1 if n in self.sizes else 0

    lib = Lib({16, 32, 64, 128, 256})
    Bz, L, N = 2, 10, 32
    dense = torch.randn(Bz, L, N)
    b, c, pitch = kernels._bc_operands(lib, dense, dense.clone(), N)
    assert pitch == N and b.data_ptr() == dense.data_ptr() and tuple(b.shape) == (Bz, L, N)
    proj = torch.randn(Bz, L, 4 + 2 * N)
    b, c, pitch = kernels._bc_operands(lib, proj[..., 4:4 + N], proj[..., 4 + N:], N)
    assert pitch == 4 + 2 * N and b.data_ptr() == proj[..., 4:].data_ptr() and c.data_ptr() == proj[..., 4 + N:].data_ptr()
    held = torch.randn(Bz, N, L)                                   # time-contiguous, passed as a transposed view
    b, c, pitch = kernels._bc_operands(lib, held.transpose(1, 2), held.transpose(1, 2), N)
    assert pitch == 0 and b.data_ptr() == held.data_ptr() and tuple(b.shape) == (Bz, N, L)
    # different pitches of B and C: dense copies in step-major order
    b, c, pitch = kernels._bc_operands(lib, proj[..., 4:4 + N], dense, N)
    assert pitch == N and b.is_contiguous() and c.is_contiguous() and torch.equal(b, proj[..., 4:4 + N])
    # a state size whose kernels want [B, N, L]: transposing copy
    b, c, pitch = kernels._bc_operands(Lib(set()), dense, dense, N)
    assert pitch == 0 and tuple(b.shape) == (Bz, N, L) and b.is_contiguous() and torch.equal(b, dense.transpose(1, 2))
