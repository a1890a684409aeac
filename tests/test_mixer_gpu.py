"""The Mamba mixer's neighbours of the scan: the fused causal conv1d + bias + SiLU kernel against PyTorch's
own ``F.pad -> conv1d -> silu`` (``mambarec.py:143-151``) in float64, forward and backward through both
output layouts, and the whole mixer forward (conv kernel + step transform folded into the scan) against the
unmodified ``_MambaMixer`` evaluated on the CPU."""
import os
import subprocess
import sys
import textwrap

import pytest
import torch
import torch.nn.functional as F

from _parity_report import record
from test_install_cpu import ROOT, reference_src

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _status_clean():
    yield
    from ossm_b200 import _lib

    torch.cuda.synchronize()
    assert _lib.device_status() == 0


def rel(got, want):
    return float((got.double().cpu() - want).abs().max() / want.abs().max().clamp_min(1e-30))


@pytest.mark.parametrize("shape", [(2, 70, 40, 4), (1, 1, 3, 4), (3, 130, 96, 3), (2, 64, 32, 2), (1, 200, 33, 1),
                                   (2, 512, 64, 4), (1, 1000, 200, 3), (3, 260, 36, 2), (2, 1156, 128, 4)],
                         ids=lambda s: "x".join(map(str, s)))
@pytest.mark.parametrize("strided", [False, True], ids=["dense", "half_of_xz"])
def test_conv_silu_matches_pytorch(shape, strided):
    from ossm_b200.mixer import causal_conv1d_silu

    Bz, L, D, Kw = shape
    gen = torch.Generator().manual_seed(sum(shape))
    xz = torch.randn(Bz, L, 2 * D, generator=gen)
    w = torch.randn(D, 1, Kw, generator=gen) * 0.5
    bias = torch.randn(D, generator=gen) * 0.3
    g1 = torch.randn(Bz, D, L, generator=gen)
    g2 = torch.randn(Bz, L, D, generator=gen)
    # float64 reference: the mixer's own chain
    x64 = (xz[..., :D] if strided else xz[..., :D].contiguous()).double().requires_grad_(True)
    w64, b64 = w.double().requires_grad_(True), bias.double().requires_grad_(True)
    ref = F.silu(F.conv1d(F.pad(x64.transpose(1, 2), (Kw - 1, 0)), w64, b64, groups=D))
    (ref * g1.double()).sum().backward(retain_graph=True)
    (ref.transpose(1, 2) * g2.double()).sum().backward()
    xd = xz.cuda()
    x = (xd[..., :D] if strided else xd[..., :D].contiguous()).requires_grad_(True)
    wd, bd = w.cuda().requires_grad_(True), bias.cuda().requires_grad_(True)
    o1, o2 = causal_conv1d_silu(x, wd, bd)
    assert o1.shape == (Bz, D, L) and o2.shape == (Bz, L, D)
    ((o1 * g1.cuda()).sum() + (o2 * g2.cuda()).sum()).backward()
    tag = f"conv1d+SiLU {'x'.join(map(str, shape))}"
    assert record(tag, "out", rel(o1.detach(), ref.detach()), 1e-5) <= 1e-5
    assert rel(o2.detach(), ref.detach().transpose(1, 2)) <= 1e-5
    assert record(tag, "grad_x", rel(x.grad, x64.grad), 1e-5) <= 1e-5
    assert record(tag, "grad_weight", rel(wd.grad, w64.grad), 1e-5) <= 1e-5
    assert record(tag, "grad_bias", rel(bd.grad, b64.grad), 1e-5) <= 1e-5


@pytest.mark.parametrize("length", [50, 576], ids=["vector_kernels", "staged_kernels"])
@pytest.mark.parametrize("which", [0, 1], ids=["time_contiguous_only", "channel_contiguous_only"])
def test_conv_single_output_gradient(length, which):
    """Only one of the two outputs is used downstream: the other gradient is absent, not zero-filled (the staged
    backward then leaves that operand's tile out of its stages)."""
    from ossm_b200.mixer import causal_conv1d_silu

    gen = torch.Generator().manual_seed(1 + which)
    x = torch.randn(2, length, 16, generator=gen).cuda().requires_grad_(True)
    w = (torch.randn(16, 1, 4, generator=gen) * 0.5).cuda().requires_grad_(True)
    out = causal_conv1d_silu(x, w, None)[which]
    out.square().sum().backward()
    x64, w64 = x.detach().double().cpu().requires_grad_(True), w.detach().double().cpu().requires_grad_(True)
    F.silu(F.conv1d(F.pad(x64.transpose(1, 2), (3, 0)), w64, None, groups=16)).square().sum().backward()
    assert rel(x.grad, x64.grad) <= 1e-5 and rel(w.grad, w64.grad) <= 1e-5


CHILD = textwrap.dedent('''
    import copy, json, sys
    import torch
    from ossm_b200.install import install_as_ossm_kernels
    install_as_ossm_kernels(fuse_mixer=True)
    from ossm.models import mambarec
    torch.manual_seed(0)
    report = {}
    for d_state in (16, 64):
        mixer = mambarec._MambaMixer(32, d_state=d_state, d_conv=4, expand=2)
        x = torch.randn(2, 90 if d_state == 16 else 320, 32)
        ref_mod = copy.deepcopy(mixer).double()
        xr = x.double().requires_grad_(True)
        y_ref = ref_mod(xr)                                  # CPU: ossm's own forward
        w = torch.randn(y_ref.shape, generator=torch.Generator().manual_seed(2))
        (y_ref * w.double()).sum().backward()
        m = mixer.cuda()
        xc = x.cuda().requires_grad_(True)
        y = m(xc)                                            # CUDA: conv kernel + folded step transform
        (y * w.cuda()).sum().backward()
        rel = lambda a, b: float((a.double().cpu() - b).abs().max() / b.abs().max().clamp_min(1e-30))
        errs = {"output": rel(y.detach(), y_ref.detach()), "input": rel(xc.grad, xr.grad)}
        for (n, p), (_, q) in zip(m.named_parameters(), ref_mod.named_parameters()):
            errs[n] = rel(p.grad, q.grad)
        bad = {k: v for k, v in errs.items() if not v <= 2e-4}
        assert not bad, bad
        report[d_state] = errs
    print("REPORT " + json.dumps(report))
''')


@pytest.mark.timeout(600)
def test_fused_mixer_behind_unmodified_class():
    src = reference_src()
    if src is None:
        pytest.skip("no ossm package (checkout or oracle/_ref/pkg)")
    env = dict(os.environ)
    env["PYTHONPATH"] = os.pathsep.join([ROOT, src, env.get("PYTHONPATH", "")])
    res = subprocess.run([sys.executable, "-c", CHILD], capture_output=True, text=True, env=env, timeout=580)
    assert res.returncode == 0 and "REPORT " in res.stdout, res.stdout[-3000:] + res.stderr[-3000:]
