"""The reference's own layers on the GPU with this library behind them.

A child process calls ``install_as_ossm_kernels()`` and then builds *unmodified* ossm modules
(``DampedLinOSSLayer`` in its four variants, ``LinOSSLayer`` IM / IMEX, ``_MambaMixer`` with 16 and
256 states, ``SelectiveDLinOSSLayer``, ``LRULayer``), runs forward + backward on CUDA in float32 and
compares the output, the input gradient and every parameter gradient with the same module evaluated
on the CPU in float64 -- which, being outside the library's scope, takes ossm's pure-PyTorch path
(``_dlinoss_scan.py:26-101``, ``linoss.py:17-54``, ``mambarec.py:23-61``).  Run for both install modes:
``patch_ops=True`` (this package's lean ops behind ``run_dlinoss`` etc.) and ``patch_ops=False`` (only
``ossm._kernels`` replaced: ossm's own autograd functions and its ``torch.ops.ossm.*`` registration
call the reference-compatible entry points with full ``[L,B,P,2]`` states).

Counterparts in the reference's suite: ``tests/test_dlinoss.py:100-109, 141-155``,
``tests/test_dlinoss_kernels.py:36-70`` (kernel against fallback, all gradients, atol 1e-4 / rtol 5e-4),
``tests/test_linoss.py:77-86``, ``tests/test_mambarec.py:66-106``.

The ossm package is taken from ``$OSSM_REFERENCE/src``, a checkout beside this repository, or the copy
staged by ``oracle/build_ref.py`` under ``oracle/_ref/pkg``; without any of them the tests are skipped.
"""
import os
import subprocess
import sys
import textwrap

import pytest

from test_install_cpu import ROOT, reference_src

pytestmark = pytest.mark.gpu

CHILD = textwrap.dedent('''
    import copy, json, sys
    import torch
    patch_ops = sys.argv[1] in ("1", "2")
    fuse_layer = sys.argv[1] == "2"
    which = sys.argv[2]
    from ossm_b200.install import install_as_ossm_kernels
    install_as_ossm_kernels(patch_ops=patch_ops, fuse_layer=fuse_layer)
    import ossm
    from ossm.models import dlinoss, linoss, lru, mambarec, sdlinoss, _dlinoss_scan
    import ossm_b200.kernels as K
    assert sys.modules["ossm._kernels"] is K and _dlinoss_scan.has_kernels()
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False

    calls = {}
    def counted(name):
        fn = getattr(K, name)
        def wrapper(*a, **k):
            calls[name] = calls.get(name, 0) + 1
            return fn(*a, **k)
        return wrapper
    for name in ("lti_scan_forward", "lti_scan_backward", "linoss_scan", "linoss_scan_backward", "selective_scan_fwd",
                 "selective_scan_bwd", "sdlinoss_scan_forward", "sdlinoss_scan_backward", "diag_scan_forward",
                 "diag_scan_backward", "gemm_tf32x3"):
        setattr(K, name, counted(name))

    def make(kind):
        torch.manual_seed(0)
        if kind.startswith("dlinoss_"):
            return dlinoss.DampedLinOSSLayer(ssm_size=48, hidden_dim=24, variant=kind.split("_")[1]), (3, 70, 24)
        if kind.startswith("linoss_"):
            return linoss.LinOSSLayer(ssm_size=40, hidden_dim=24, discretization=kind.split("_")[1]), (3, 70, 24)
        if kind.startswith("mamba_"):
            return mambarec._MambaMixer(32, d_state=int(kind.split("_")[1]), d_conv=4, expand=2), (2, 50, 32)
        if kind == "sdlinoss":
            return sdlinoss.SelectiveDLinOSSLayer(ssm_size=32, hidden_dim=16), (2, 60, 16)
        if kind == "lru":
            return lru.LRULayer(ssm_size=40, hidden_dim=24), (3, 70, 24)
        raise ValueError(kind)

    def run(module, x):
        x = x.clone().requires_grad_(True)
        y = module(x)
        gen = torch.Generator().manual_seed(5)
        w = torch.randn(y.shape, generator=gen).to(device=y.device, dtype=y.dtype)
        (y * w).sum().backward()
        grads = {n: p.grad.detach().double().cpu() for n, p in module.named_parameters() if p.grad is not None}
        grads["input"] = x.grad.detach().double().cpu()
        return y.detach().double().cpu(), grads

    def rel(a, b):
        return float((a - b).abs().max() / b.abs().max().clamp_min(1e-30))

    report = {}
    for kind in which.split(","):
        module, shape = make(kind)
        gen = torch.Generator().manual_seed(3)
        x = torch.randn(*shape, generator=gen)
        ref_mod = copy.deepcopy(module).double()
        # CPU float64: ossm's own PyTorch path.  With only the kernel module replaced, ossm's run_sdlinoss has
        # no fallback of its own (_sdlinoss_scan.py:414-452), so its switch is used for this reference run.
        import os
        os.environ["OSSM_SDLINOSS_DISABLE_KERNEL"] = "1"
        y_ref, g_ref = run(ref_mod, x.double())
        del os.environ["OSSM_SDLINOSS_DISABLE_KERNEL"]
        calls.clear()
        y, g = run(module.cuda(), x.cuda())                        # CUDA float32: this library
        assert calls, f"{kind}: no kernel of the library was called"
        if fuse_layer and kind.split("_")[0] in ("dlinoss", "linoss"):
            assert calls.get("gemm_tf32x3", 0) >= 4, (kind, calls)      # the projections ran on the tensor cores
        errs = {"output": rel(y, y_ref)}
        assert set(g) == set(g_ref), (sorted(g), sorted(g_ref))
        for n in g_ref:
            errs[n] = rel(g[n], g_ref[n])
        report[kind] = {"errors": errs, "calls": dict(calls)}
        bad = {n: e for n, e in errs.items() if not e <= 2e-4}
        assert not bad, (kind, bad)
    from ossm_b200 import _lib
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    print("REPORT " + json.dumps(report))
''')

KINDS = ["dlinoss_imex1,dlinoss_imex2,dlinoss_im,dlinoss_ex", "linoss_IM,linoss_IMEX", "mamba_16,mamba_256",
         "sdlinoss,lru"]


@pytest.mark.timeout(600)
@pytest.mark.parametrize("kinds", KINDS[:2])
def test_fused_layer_body_behind_unmodified_classes(kinds):
    """``install_as_ossm_kernels(fuse_layer=True)``: ossm's ``DampedLinOSSLayer`` / ``LinOSSLayer`` objects, their
    parameters untouched, with the layer body (projections on the tensor cores around the scan) of this package."""
    src = reference_src()
    if src is None:
        pytest.skip("no ossm package (checkout or oracle/_ref/pkg)")
    env = dict(os.environ)
    env["PYTHONPATH"] = os.pathsep.join([ROOT, src, env.get("PYTHONPATH", "")])
    res = subprocess.run([sys.executable, "-c", CHILD, "2", kinds], capture_output=True, text=True, env=env, timeout=580)
    assert res.returncode == 0 and "REPORT " in res.stdout, res.stdout[-3000:] + res.stderr[-3000:]


@pytest.mark.timeout(600)
@pytest.mark.parametrize("patch_ops", [True, False], ids=["lean_ops", "kernels_module_only"])
@pytest.mark.parametrize("kinds", KINDS)
def test_unmodified_ossm_layers_on_cuda(kinds, patch_ops):
    src = reference_src()
    if src is None:
        pytest.skip("no ossm package (checkout or oracle/_ref/pkg)")
    env = dict(os.environ)
    env["PYTHONPATH"] = os.pathsep.join([ROOT, src, env.get("PYTHONPATH", "")])
    res = subprocess.run([sys.executable, "-c", CHILD, "1" if patch_ops else "0", kinds], capture_output=True,
                         text=True, env=env, timeout=580)
    assert res.returncode == 0 and "REPORT " in res.stdout, res.stdout[-3000:] + res.stderr[-3000:]
    path = os.environ.get("OSSM_B200_PARITY_REPORT")
    if path:
        import json

        rep = json.loads(res.stdout.split("REPORT ", 1)[1])
        with open(path, "a") as fh:
            for kind, body in rep.items():
                for tensor, err in body["errors"].items():
                    fh.write(json.dumps({"case": f"ossm layer {kind} ({'lean ops' if patch_ops else 'kernels module only'})",
                                         "tensor": tensor, "err": err, "bound": 2e-4}) + "\n")
