"""The tensor-core projection GEMM (tcgen05, three TF32 products of split operands) through the C ABI
against a float64 matrix product: float32-level accuracy (max-norm relative error <= 5e-6, three orders
below plain TF32), ragged extents, every output-row permutation and the fused ``+ diag * aux`` term."""
import pytest
import torch

from _parity_report import record

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _status_clean():
    yield
    from ossm_b200 import _lib

    torch.cuda.synchronize()
    assert _lib.device_status() == 0


def rel(got, want):
    return float((got.double() - want).abs().max() / want.abs().max())


SHAPES = [(128, 64, 32), (300, 96, 64), (1000, 512, 256), (129, 40, 36), (64, 256, 512), (4096, 130, 100)]


@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: "x".join(map(str, s)))
def test_plain_product(shape):
    from ossm_b200 import kernels as K

    M, N, Kd = shape
    gen = torch.Generator().manual_seed(M + N + Kd)
    A = torch.randn(M, Kd, generator=gen).cuda()
    W = (torch.randn(N, Kd, generator=gen) / Kd ** 0.5).cuda()
    hi, lo = K.split_tf32(W)
    assert torch.equal(hi + lo, W) and int((hi.view(torch.int32) & 0x1fff).abs().max()) == 0
    out = torch.full((M, N), float("nan"), device="cuda")
    K.gemm_tf32x3(A, hi, lo, out)
    want = A.double() @ W.double().t()
    assert record(f"gemm_tf32x3 {M}x{N}x{Kd}", "out", rel(out, want), 5e-6) <= 5e-6


@pytest.mark.parametrize("row_map", [1, 2])
def test_row_permutation_and_diagonal_term(row_map):
    from ossm_b200 import kernels as K

    Bz, L, N, Kd = 3, 200, 72, 48
    gen = torch.Generator().manual_seed(row_map)
    A = torch.randn(Bz * L, Kd, generator=gen).cuda()
    W = (torch.randn(N, Kd, generator=gen) / Kd ** 0.5).cuda()
    aux = torch.randn(Bz * L, N, generator=gen).cuda()
    diag = torch.randn(N, generator=gen).cuda()
    hi, lo = K.split_tf32(W)
    out = torch.empty(Bz * L, N, device="cuda")
    K.gemm_tf32x3(A, hi, lo, out, aux=aux, diag=diag, row_map=row_map, batch=Bz, length=L)
    prod = A.double() @ W.double().t()
    if row_map == 1:      # rows of A are (b, l); rows of out are (l, b)
        prod = prod.view(Bz, L, N).permute(1, 0, 2).reshape(Bz * L, N)
    else:                 # rows of A are (l, b); rows of out are (b, l)
        prod = prod.view(L, Bz, N).permute(1, 0, 2).reshape(Bz * L, N)
    want = prod + diag.double() * aux.double()
    assert rel(out, want) <= 5e-6


def test_column_planes():
    """Output written as one plane per block of columns ([N / block, M, block]), with a row permutation."""
    from ossm_b200 import kernels as K

    Bz, L, N, Kd, blk = 2, 96, 128, 40, 32
    gen = torch.Generator().manual_seed(7)
    A = torch.randn(L * Bz, Kd, generator=gen).cuda()
    W = (torch.randn(N, Kd, generator=gen) / Kd ** 0.5).cuda()
    hi, lo = K.split_tf32(W)
    out = torch.empty(N // blk, Bz * L, blk, device="cuda")
    K.gemm_tf32x3(A, hi, lo, out, row_map=2, batch=Bz, length=L, col_block=blk)
    prod = (A.double() @ W.double().t()).view(L, Bz, N).permute(1, 0, 2).reshape(Bz * L, N)
    want = prod.view(Bz * L, N // blk, blk).permute(1, 0, 2)
    assert rel(out, want) <= 5e-6


@pytest.mark.parametrize("orders", [(True, False), (False, True), (False, False), (True, True)])
@pytest.mark.parametrize("shape", [(2, 100, 64, 32), (3, 257, 128, 256), (8, 1024, 512, 256), (1, 31, 32, 96)],
                         ids=lambda s: "x".join(map(str, s)))
def test_weight_gradient_product(shape, orders):
    """sum over (b, l) of X[row]^T Y[row] with the two row orders mixed; ragged lengths (partial last slice per
    batch entry) and more splits than slices included."""
    from ossm_b200 import kernels as K

    Bz, L, M, N = shape
    xt, yt = orders
    gen = torch.Generator().manual_seed(sum(shape))
    X = torch.randn(Bz, L, M, generator=gen)
    Y = torch.randn(Bz, L, N, generator=gen)
    want = torch.einsum("blm,bln->mn", X.double(), Y.double())
    Xd = (X.permute(1, 0, 2) if xt else X).contiguous().view(Bz * L, M).cuda()
    Yd = (Y.permute(1, 0, 2) if yt else Y).contiguous().view(Bz * L, N).cuda()
    out = K.wgrad_tf32x3(Xd, xt, Yd, yt, Bz, L)
    assert out.shape == (M, N)
    assert record(f"wgrad_tf32x3 {Bz}x{L}x{M}x{N}", "out", rel(out.cpu(), want), 5e-6) <= 5e-6


@pytest.mark.parametrize("shape", [(1, 4), (37, 8), (1000, 256), (70000, 512), (5000, 1028), (300, 2052)],
                         ids=lambda s: "x".join(map(str, s)))
def test_colwise_dot(shape):
    """``grad_D``: column sums of an elementwise product, one pass, partials added in a fixed order."""
    from ossm_b200 import kernels as K

    rows, cols = shape
    gen = torch.Generator().manual_seed(rows + cols)
    x = torch.randn(rows, cols, generator=gen).cuda()
    y = torch.randn(rows, cols, generator=gen).cuda()
    got = K.colwise_dot(x, y)
    want = (x.double() * y.double()).sum(0)
    assert got.shape == (cols,)
    assert rel(got, want) <= 2e-6
    assert torch.equal(got, K.colwise_dot(x, y))        # deterministic
    with pytest.raises(RuntimeError):
        K.colwise_dot(x[:, :3].contiguous(), y[:, :3].contiguous())


def test_rejects_bad_arguments():
    from ossm_b200 import kernels as K

    A = torch.randn(8, 6, device="cuda")          # K not a multiple of 4
    W = torch.randn(4, 6, device="cuda")
    with pytest.raises(RuntimeError):
        K.gemm_tf32x3(A, W, W, torch.empty(8, 4, device="cuda"))
    with pytest.raises(RuntimeError):
        K.gemm_tf32x3(A.cpu(), W, W, torch.empty(8, 4, device="cuda"))
