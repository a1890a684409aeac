"""Drop-in boundary: ``install_as_ossm_kernels()`` puts this package behind an unmodified ossm checkout.
Needs the checkout (``$OSSM_REFERENCE`` or a directory ``reference`` beside this repository) and is
skipped without it; runs in a child process so that the parent's module table stays clean.  No GPU:
the check is that ossm's own layers now reach this library (which refuses CPU tensors loudly) instead
of their silent PyTorch fallback."""
import os
import subprocess
import sys
import textwrap

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REFERENCE = os.environ.get("OSSM_REFERENCE") or os.path.join(os.path.dirname(ROOT), "reference")

CHILD = textwrap.dedent('''
    import sys
    import torch
    from ossm_b200.install import install_as_ossm_kernels
    import ossm_b200.kernels as K
    install_as_ossm_kernels()
    import ossm
    from ossm.models import _dlinoss_scan, _sdlinoss_scan, _selective_scan, dlinoss, lru, s5, sdlinoss
    import ossm_b200.dlinoss, ossm_b200.sdlinoss, ossm_b200.selective_scan, ossm_b200.diag
    assert sys.modules["ossm._kernels"] is K
    assert _dlinoss_scan.has_kernels() and _sdlinoss_scan.has_kernels()
    assert dlinoss.run_dlinoss is ossm_b200.dlinoss.run_dlinoss
    assert sdlinoss.run_sdlinoss is ossm_b200.sdlinoss.run_sdlinoss
    assert _selective_scan.try_selective_scan is ossm_b200.selective_scan.try_selective_scan
    assert lru._LRUScanFn is ossm_b200.diag.DiagScanFn and s5._S5ScanFn is ossm_b200.diag.DiagScanFn
    # every name the reference probes or calls is present
    for name in ("dlinoss_imex1_forward", "dlinoss_ex_backward", "sdlinoss_im_forward", "sdlinoss_imex2_backward",
                 "linoss_scan", "lru_scan", "s5_scan", "linear_rnn_scan", "selective_scan", "selective_scan_backward",
                 "selective_scan_cuda", "selective_scan_cuda_backward"):
        assert hasattr(K, name), name
    # the reference layer now reaches this library: CPU tensors are refused instead of silently falling back
    layer = dlinoss.DampedLinOSSLayer(ssm_size=8, hidden_dim=4)
    try:
        layer(torch.randn(2, 5, 4))
    except RuntimeError as exc:
        assert "CUDA" in str(exc), exc
    else:
        raise AssertionError("the layer did not go through ossm_b200")
    from ossm.models import mambarec
    for make, x in ((lambda: sdlinoss.SelectiveDLinOSSLayer(ssm_size=8, hidden_dim=4), torch.randn(2, 5, 4)),
                    (lambda: mambarec._MambaMixer(8, d_state=16, d_conv=4, expand=2), torch.randn(2, 6, 8)),
                    (lambda: lru.LRULayer(ssm_size=8, hidden_dim=4), torch.randn(2, 5, 4))):
        try:
            make()(x)
        except RuntimeError as exc:
            assert "CUDA" in str(exc), exc
        else:
            raise AssertionError("a layer did not go through ossm_b200")
    print("install ok")
''')


@pytest.mark.timeout(300)
def test_install_behind_unmodified_ossm():
    if not os.path.isdir(os.path.join(REFERENCE, "src", "ossm")):
        pytest.skip("no ossm checkout")
    env = dict(os.environ)
    env["PYTHONPATH"] = os.pathsep.join([ROOT, os.path.join(REFERENCE, "src"), env.get("PYTHONPATH", "")])
    res = subprocess.run([sys.executable, "-c", CHILD], capture_output=True, text=True, env=env, timeout=280)
    assert res.returncode == 0 and "install ok" in res.stdout, res.stdout + res.stderr
