"""Drop-in boundary: ``install_as_ossm_kernels()`` puts this package behind an unmodified ossm checkout.
Needs the checkout (``$OSSM_REFERENCE``, a directory ``reference`` beside this repository, or the copy
staged by ``oracle/build_ref.py`` under ``oracle/_ref/pkg``) and is skipped without it; runs in a child
process so that the parent's module table stays clean.  No GPU: the checks are that ossm's op functions
are now this package's dispatchers, that inputs outside the library's scope (CPU tensors, float64) still
take ossm's own PyTorch path with unchanged results, and that covered inputs are routed to the CUDA ops."""
import os
import subprocess
import sys
import textwrap
import types

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def reference_src():
    for cand in (os.environ.get("OSSM_REFERENCE") and os.path.join(os.environ["OSSM_REFERENCE"], "src"),
                 os.path.join(os.path.dirname(ROOT), "reference", "src"),
                 os.path.join(ROOT, "oracle", "_ref", "pkg")):
        if cand and os.path.isdir(os.path.join(cand, "ossm")):
            return cand
    return None


CHILD = textwrap.dedent('''
    import sys
    import torch
    torch.manual_seed(0)
    import ossm                                         # first without the library: ossm's own results
    from ossm.models import dlinoss, lru, mambarec, sdlinoss, linoss
    def build():
        torch.manual_seed(1)
        return [(dlinoss.DampedLinOSSLayer(ssm_size=8, hidden_dim=4), torch.randn(2, 5, 4)),
                (sdlinoss.SelectiveDLinOSSLayer(ssm_size=8, hidden_dim=4), torch.randn(2, 5, 4)),
                (mambarec._MambaMixer(8, d_state=16, d_conv=4, expand=2), torch.randn(2, 6, 8)),
                (lru.LRULayer(ssm_size=8, hidden_dim=4), torch.randn(2, 5, 4)),
                (linoss.LinOSSLayer(ssm_size=8, hidden_dim=4, discretization="IM"), torch.randn(2, 5, 4))]
    cases = build()
    before = [m(x).detach() for m, x in cases]
    from ossm_b200.install import install_as_ossm_kernels
    import ossm_b200.kernels as K
    install_as_ossm_kernels(fuse_layer=True, fuse_mixer=True)
    install_as_ossm_kernels(fuse_layer=True, fuse_mixer=True)     # twice: wrappers must not nest
    for cls in (dlinoss.DampedLinOSSLayer, linoss.LinOSSLayer, mambarec._MambaMixer):
        assert cls.forward.__wrapped__.__module__.startswith("ossm.models"), cls
        assert not hasattr(cls.forward.__wrapped__, "__wrapped__"), cls
    from ossm.models import _dlinoss_scan, _sdlinoss_scan, _selective_scan, s5
    assert sys.modules["ossm._kernels"] is K
    assert dlinoss.run_dlinoss is _dlinoss_scan.run_dlinoss
    assert dlinoss.run_dlinoss.__wrapped__.__module__ == "ossm.models._dlinoss_scan"
    assert not hasattr(dlinoss.run_dlinoss.__wrapped__, "__wrapped__")
    assert sdlinoss.run_sdlinoss is _sdlinoss_scan.run_sdlinoss
    assert _selective_scan.try_selective_scan is mambarec._try_selective_scan
    assert lru._LRUScanFn.__wrapped__.__module__ == "ossm.models.lru"
    assert s5._S5ScanFn.__wrapped__.__module__ == "ossm.models.s5"
    # every name the reference probes or calls is present
    for name in ("dlinoss_imex1_forward", "dlinoss_ex_backward", "sdlinoss_im_forward", "sdlinoss_imex2_backward",
                 "linoss_scan", "lru_scan", "s5_scan", "linear_rnn_scan", "selective_scan", "selective_scan_backward",
                 "selective_scan_cuda", "selective_scan_cuda_backward"):
        assert hasattr(K, name), name
    # a model on the host keeps working and gives ossm's own numbers: CPU tensors are outside the
    # library's scope and go to ossm's PyTorch path, forward and backward
    for (m, x), want in zip(cases, before):
        got = m(x)
        assert torch.allclose(got, want, rtol=1e-5, atol=1e-6), type(m).__name__
        got.square().sum().backward()
        assert all(p.grad is not None and torch.isfinite(p.grad).all() for p in m.parameters() if p.requires_grad)
    # float64 (ossm's gradcheck dtype) likewise
    layer = dlinoss.DampedLinOSSLayer(ssm_size=8, hidden_dim=4).double()
    assert layer(torch.randn(2, 5, 4, dtype=torch.float64)).dtype == torch.float64
    assert _selective_scan.try_selective_scan(torch.randn(1, 2, 3), torch.rand(1, 2, 3), -torch.rand(2, 4),
                                              torch.randn(1, 3, 4), torch.randn(1, 3, 4), None) is None
    # the library itself still has no CPU path
    try:
        K.dlinoss_imex1_forward(torch.rand(4), torch.rand(4), torch.rand(4), torch.zeros(3, 2, 4, dtype=torch.complex64))
    except RuntimeError as exc:
        assert "CUDA" in str(exc), exc
    else:
        raise AssertionError("kernels accepted a CPU tensor")
    print("install ok")
''')


def test_scope_predicates_route_covered_inputs_to_the_library():
    """The dispatchers decide on device and dtype only; stand-in objects make the CUDA side testable here."""
    from ossm_b200 import install

    def fake(cuda, dtype, dim=3, shape=(4, 2, 8)):
        return types.SimpleNamespace(is_cuda=cuda, dtype=dtype, dim=lambda: dim, size=lambda i: shape[i], shape=shape)

    assert install._covered_complex(fake(True, torch.complex64), fake(True, torch.float32), None)
    assert not install._covered_complex(fake(False, torch.complex64), fake(False, torch.float32))
    assert not install._covered_complex(fake(True, torch.complex128), fake(True, torch.float64))
    calls = []
    sel = install._wrap_try_selective_scan(lambda *a: calls.append(a) or "ours")
    A16, A256, A512 = (fake(True, torch.float32, 2, (8, n)) for n in (16, 256, 512))
    u32, ubf, u16 = (fake(True, dt) for dt in (torch.float32, torch.bfloat16, torch.float16))
    assert sel(u32, None, A16, u32, u32, None) == "ours"
    assert sel(ubf, None, A256, ubf, ubf, ubf) == "ours"
    assert sel(u32, None, A512, u32, u32, None) is None          # beyond the kernels' state size: ossm's own path
    assert sel(u16, None, A16, u16, u16, None) is None
    assert sel(fake(False, torch.float32), None, A16, u32, u32, None) is None
    assert len(calls) == 2
    run = install._wrap_dlinoss(lambda *a: "ours", lambda *a: "ossm")
    assert run("imex1", fake(True, torch.float32), fake(True, torch.float32), fake(True, torch.float32),
               fake(True, torch.complex64)) == "ours"
    assert run("imex1", fake(False, torch.float32), fake(False, torch.float32), fake(False, torch.float32),
               fake(False, torch.complex64)) == "ossm"


@pytest.mark.timeout(300)
def test_install_behind_unmodified_ossm():
    src = reference_src()
    if src is None:
        pytest.skip("no ossm checkout")
    env = dict(os.environ)
    env["PYTHONPATH"] = os.pathsep.join([ROOT, src, env.get("PYTHONPATH", "")])
    res = subprocess.run([sys.executable, "-c", CHILD], capture_output=True, text=True, env=env, timeout=280)
    assert res.returncode == 0 and "install ok" in res.stdout, res.stdout + res.stderr
