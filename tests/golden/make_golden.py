"""Generates the committed golden fixtures in this directory.

Run in a container that holds the ossm checkout (it is *not* needed at test
time):

    python oracle/build_ref.py                       # compiled reference CPU kernels
    python tests/golden/make_golden.py [--reference /path/to/ossm]

Sources of the vectors:

* ``dlinoss_reference_cases.npz``  -- the reference's own golden file
  ``tests/dlinoss_reference_cases.json`` (upstream-JAX derived; consumed by
  ``tests/test_dlinoss_parity.py:73-138``), re-encoded as arrays.
* ``linoss_im_snapshot.npz``       -- the inline LinOSS-IM snapshot of
  ``tests/test_linoss_parity.py:74-204``.
* ``dlinoss_generated.npz``, ``linoss_generated.npz``, ``diag_generated.npz``,
  ``sdlinoss_generated.npz``, ``selective_scan_generated.npz``, ``selective_scan_large_state.npz``,
  ``selective_scan_delta.npz`` -- outputs of the reference itself run here
  on seeded inputs: its pure-PyTorch recurrences (float64 and float32, grads by
  autograd) and its compiled CPU kernels (float32).
"""
from __future__ import annotations

import argparse
import importlib.util
import json
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))


def _np(t):
    return t.detach().cpu().numpy()


def stable_params(P, gen):
    """Parameters inside the stable band (same projection the layer applies,
    ``src/ossm/models/dlinoss.py:252-267``)."""
    g = torch.empty(P).uniform_(-0.25, 0.6, generator=gen)
    a = torch.empty(P).uniform_(0.0, 1.5, generator=gen)
    step = torch.randn(P, generator=gen) * 0.5
    step_p = torch.sigmoid(step)
    g_p = torch.relu(g)
    denom = torch.clamp(step_p * step_p, min=1e-6)
    s = step_p * g_p
    base = torch.sqrt(torch.clamp(1.0 + s, min=1e-6))
    a_low = (2.0 + s - 2.0 * base) / denom
    a_high = (2.0 + s + 2.0 * base) / denom
    a_p = a_low + torch.relu(a - a_low) - torch.relu(a - a_high)
    return a_p, g_p, step_p


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("OSSM_REFERENCE") or os.path.join(os.path.dirname(ROOT), "reference"),
                    help="ossm checkout (default: $OSSM_REFERENCE, else a directory 'reference' beside this repository)")
    ap.add_argument("--only", default=None, choices=["large_state"],
                    help="regenerate one fixture file only (the others are left as they are)")
    args = ap.parse_args()
    ref = args.reference

    sys.path.insert(0, ROOT)
    from oracle.ref_loader import load_reference_kernels

    kernels = load_reference_kernels()
    if kernels is None:
        raise SystemExit("build oracle/_ref first: python oracle/build_ref.py")
    # The reference shims import ``ossm._kernels``; seed it with its own compiled
    # CPU extension before the package is imported.
    sys.modules["ossm._kernels"] = kernels
    sys.path.insert(0, os.path.join(ref, "src"))
    import ossm  # noqa: F401
    from ossm.models import _dlinoss_scan as dscan
    from ossm.models import linoss as linoss_mod
    from ossm.models.mambarec import _selective_scan_mamba

    ossm._kernels = kernels

    # ---- E3. selective scan with large state sizes (the shipped Mamba4Rec configuration uses
    # d_state = ssm_size = 256, configs/model/mambarec.yaml:3, mambarec.py:305) ----------------
    import torch.nn.functional as F
    out = {}
    gen = torch.Generator().manual_seed(256)
    for tag, (Bz, Dn, L, N) in (("n128", (1, 5, 70, 128)), ("n256", (2, 6, 45, 256))):
        u = torch.randn(Bz, Dn, L, generator=gen)
        dt = torch.rand(Bz, Dn, L, generator=gen) * 0.05
        A = -torch.exp(torch.randn(Dn, N, generator=gen))
        Bm = torch.randn(Bz, L, N, generator=gen)
        Cm = torch.randn(Bz, L, N, generator=gen)
        gate = torch.randn(Bz, Dn, L, generator=gen)
        go = torch.randn(Bz, Dn, L, generator=gen)
        pre = f"{tag}/"
        for k, v in (("u", u), ("dt", dt), ("A", A), ("B", Bm), ("C", Cm), ("gate", gate), ("grad_out", go)):
            out[pre + k] = _np(v)
        leaves = [t.double().clone().requires_grad_(True) for t in (u, dt, A, Bm, Cm, gate)]
        y = _selective_scan_mamba(inputs=leaves[0], dt=leaves[1], A=leaves[2], B_t=leaves[3], C_t=leaves[4])
        o = y.double() * F.silu(leaves[5])
        (o * go.double()).sum().backward()
        out[pre + "py_out"] = _np(o)
        for name, leaf in zip(("du", "ddt", "dA", "dB", "dC", "dgate"), leaves):
            out[pre + "py_" + name] = _np(leaf.grad)
        o2 = kernels.selective_scan(u, dt, A, Bm, Cm, gate)
        grads = kernels.selective_scan_backward(go, u, dt, A, Bm, Cm, gate)
        out[pre + "cpp_out"] = _np(o2)
        for name, gr in zip(("du", "ddt", "dA", "dB", "dC", "dgate"), grads):
            out[pre + "cpp_" + name] = _np(gr)
    np.savez_compressed(os.path.join(HERE, "selective_scan_large_state.npz"), **out)
    if args.only == "large_state":
        return

    # ---- A. the reference's own golden JSON -----------------------------
    payload = json.load(open(os.path.join(ref, "tests", "dlinoss_reference_cases.json")))
    cases = payload.get("cases", payload)
    out = {}
    for variant, by_dtype in cases.items():
        for dt_key, case in by_dtype.items():
            pre = f"{variant}/{dt_key}/"
            for key in ("A_diag", "G_diag", "step", "B", "C", "D", "inputs", "outputs"):
                out[pre + key] = np.asarray(case[key], dtype=np.float64)
            out[pre + "states_main"] = np.asarray(case["states"]["main"], dtype=np.float64)
            out[pre + "states_aux"] = np.asarray(case["states"]["aux"], dtype=np.float64)
            for key, val in case["grads"].items():
                out[pre + "grad_" + key] = np.asarray(val, dtype=np.float64)
    np.savez_compressed(os.path.join(HERE, "dlinoss_reference_cases.npz"), **out)

    # ---- B. inline LinOSS snapshot --------------------------------------
    spec = importlib.util.spec_from_file_location(
        "ref_test_linoss_parity", os.path.join(ref, "tests", "test_linoss_parity.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    snap = {k: _np(v) for k, v in mod.REFERENCE_LINOSS.items()}
    np.savez_compressed(os.path.join(HERE, "linoss_im_snapshot.npz"), **snap)

    # ---- C. D-LinOSS generated ------------------------------------------
    out = {}
    gen = torch.Generator().manual_seed(1234)
    shapes = {"small": (12, 3, 8), "ragged": (37, 3, 5), "wide": (40, 2, 35)}
    for sname, (L, B, P) in shapes.items():
        for variant in ("imex1", "imex2", "im", "ex"):
            a, g, step = stable_params(P, gen)
            bu = torch.complex(torch.randn(L, B, P, generator=gen), torch.randn(L, B, P, generator=gen)) * 0.5
            gx = torch.complex(torch.randn(L, B, P, generator=gen), torch.randn(L, B, P, generator=gen))
            pre = f"{sname}/{variant}/"
            out[pre + "a"], out[pre + "g"], out[pre + "step"] = _np(a), _np(g), _np(step)
            out[pre + "bu"], out[pre + "grad_x"] = _np(bu), _np(gx)
            for tag, rd, cd in (("f64", torch.float64, torch.complex128), ("f32", torch.float32, torch.complex64)):
                aa = a.to(rd).requires_grad_(True)
                gg = g.to(rd).requires_grad_(True)
                ss = step.to(rd).requires_grad_(True)
                bb = bu.to(cd).requires_grad_(True)
                states = dscan._reference_dlinoss_states(variant, aa, gg, ss, bb)
                x = states[..., 1]
                loss = (x.real * gx.real.to(rd)).sum() + (x.imag * gx.imag.to(rd)).sum()
                loss.backward()
                out[pre + f"py_{tag}_states"] = _np(states)
                out[pre + f"py_{tag}_da"] = _np(aa.grad)
                out[pre + f"py_{tag}_dg"] = _np(gg.grad)
                out[pre + f"py_{tag}_dstep"] = _np(ss.grad)
                out[pre + f"py_{tag}_dbu"] = _np(bb.grad)
            fwd = getattr(kernels, f"dlinoss_{variant}_forward")
            bwd = getattr(kernels, f"dlinoss_{variant}_backward")
            st = fwd(a, g, step, bu)
            da, dg, ds, dbu = bwd(a, g, step, bu, st, gx)
            out[pre + "cpp_states"] = _np(st)
            out[pre + "cpp_da"], out[pre + "cpp_dg"] = _np(da), _np(dg)
            out[pre + "cpp_dstep"], out[pre + "cpp_dbu"] = _np(ds), _np(dbu)
    # raw BASELINE-style parameters (relu'd normals: many exact zeros) for the
    # two variants that stay finite under them
    L, B, P = 64, 2, 16
    a = torch.relu(torch.randn(P, generator=gen))
    g = torch.relu(torch.randn(P, generator=gen))
    step = torch.sigmoid(torch.randn(P, generator=gen))
    bu = torch.complex(torch.randn(L, B, P, generator=gen), torch.randn(L, B, P, generator=gen)) * 0.5
    for variant in ("imex1", "im"):
        pre = f"raw/{variant}/"
        out[pre + "a"], out[pre + "g"], out[pre + "step"], out[pre + "bu"] = _np(a), _np(g), _np(step), _np(bu)
        states = dscan._reference_dlinoss_states(variant, a.double(), g.double(), step.double(), bu.to(torch.complex128))
        out[pre + "py_f64_states"] = _np(states)
    np.savez_compressed(os.path.join(HERE, "dlinoss_generated.npz"), **out)

    # ---- D. LinOSS generated ---------------------------------------------
    out = {}
    gen = torch.Generator().manual_seed(4321)
    B, L, H, P = 3, 19, 6, 7
    for disc in ("IM", "IMEX"):
        layer = linoss_mod.LinOSSLayer(P, H, disc).double()
        a_diag = torch.rand(P, generator=gen).double().requires_grad_(True)
        step = torch.sigmoid(torch.randn(P, generator=gen)).double().requires_grad_(True)
        bu = (torch.complex(torch.randn(B, L, P, generator=gen), torch.randn(B, L, P, generator=gen)) * 0.5).to(torch.complex128).requires_grad_(True)
        gx = torch.complex(torch.randn(B, L, P, generator=gen), torch.randn(B, L, P, generator=gen)).to(torch.complex128)
        x = layer._apply_im(a_diag, step, bu) if disc == "IM" else layer._apply_imex(a_diag, step, bu)
        loss = (x.real * gx.real).sum() + (x.imag * gx.imag).sum()
        loss.backward()
        pre = f"layer/{disc}/"
        out[pre + "a"], out[pre + "step"], out[pre + "bu"], out[pre + "grad_x"] = _np(a_diag), _np(step), _np(bu), _np(gx)
        out[pre + "x"] = _np(x)
        out[pre + "da"], out[pre + "dstep"], out[pre + "dbu"] = _np(a_diag.grad), _np(step.grad), _np(bu.grad)
    for tag, shape in (("c1", (9, 2, 5)), ("c2", (33, 3, 36))):
        L, B, P = shape
        a_matrix = (torch.complex(torch.randn(P, 2, 2, generator=gen), torch.randn(P, 2, 2, generator=gen)) * 0.45).to(torch.complex64)
        b_seq = torch.complex(torch.randn(L, B, P, 2, generator=gen), torch.randn(L, B, P, 2, generator=gen)).to(torch.complex64)
        go = torch.complex(torch.randn(L, B, P, 2, generator=gen), torch.randn(L, B, P, 2, generator=gen)).to(torch.complex64)
        am = a_matrix.clone().requires_grad_(True)
        bs = b_seq.clone().requires_grad_(True)
        states = linoss_mod._LinossScanFn.apply(am, bs)
        loss = (states.real * go.real).sum() + (states.imag * go.imag).sum()
        loss.backward()
        pre = f"scan/{tag}/"
        out[pre + "a_matrix"], out[pre + "b_seq"], out[pre + "grad_out"] = _np(a_matrix), _np(b_seq), _np(go)
        out[pre + "states"] = _np(states)
        out[pre + "grad_a"], out[pre + "grad_b"] = _np(am.grad), _np(bs.grad)
        # real transition matrix: gradient keeps only the real part
        ar = (torch.randn(P, 2, 2, generator=gen) * 0.45).requires_grad_(True)
        bs2 = b_seq.clone().requires_grad_(True)
        st2 = linoss_mod._LinossScanFn.apply(ar, bs2)
        loss = (st2.real * go.real).sum() + (st2.imag * go.imag).sum()
        loss.backward()
        out[pre + "real_a_matrix"], out[pre + "real_states"] = _np(ar), _np(st2)
        out[pre + "real_grad_a"], out[pre + "real_grad_b"] = _np(ar.grad), _np(bs2.grad)
    np.savez_compressed(os.path.join(HERE, "linoss_generated.npz"), **out)

    # ---- E. selective scan generated --------------------------------------
    out = {}
    gen = torch.Generator().manual_seed(99)
    import torch.nn.functional as F
    for tag, (Bz, Dn, L, N) in (("n4", (2, 8, 48, 4)), ("n16", (2, 36, 100, 16)), ("n64", (1, 6, 40, 64))):
        u = torch.randn(Bz, Dn, L, generator=gen)
        dt = torch.rand(Bz, Dn, L, generator=gen) * 0.05
        A = -torch.exp(torch.randn(Dn, N, generator=gen))
        Bm = torch.randn(Bz, L, N, generator=gen)
        Cm = torch.randn(Bz, L, N, generator=gen)
        gate = torch.randn(Bz, Dn, L, generator=gen)
        go = torch.randn(Bz, Dn, L, generator=gen)
        pre = f"{tag}/"
        for k, v in (("u", u), ("dt", dt), ("A", A), ("B", Bm), ("C", Cm), ("gate", gate), ("grad_out", go)):
            out[pre + k] = _np(v)
        leaves = [t.clone().requires_grad_(True) for t in (u, dt, A, Bm, Cm, gate)]
        y = _selective_scan_mamba(inputs=leaves[0], dt=leaves[1], A=leaves[2], B_t=leaves[3], C_t=leaves[4])
        o = y * F.silu(leaves[5])
        (o * go).sum().backward()
        out[pre + "py_out"] = _np(o)
        out[pre + "py_y"] = _np(y)
        for name, leaf in zip(("du", "ddt", "dA", "dB", "dC", "dgate"), leaves):
            out[pre + "py_" + name] = _np(leaf.grad)
        o2 = kernels.selective_scan(u, dt, A, Bm, Cm, gate)
        grads = kernels.selective_scan_backward(go, u, dt, A, Bm, Cm, gate)
        out[pre + "cpp_out"] = _np(o2)
        for name, gr in zip(("du", "ddt", "dA", "dB", "dC", "dgate"), grads):
            out[pre + "cpp_" + name] = _np(gr)
        o3 = kernels.selective_scan(u, dt, A, Bm, Cm, None)
        out[pre + "cpp_out_nogate"] = _np(o3)
    np.savez_compressed(os.path.join(HERE, "selective_scan_generated.npz"), **out)
    # ---- E2. selective scan with the step transform of the mixer folded in ---------------
    # dt = softplus(raw + bias[d]) as Mamba4Rec computes it before the scan (mambarec.py:155-157);
    # float64 run of the reference's Python loop, gradients by autograd
    out = {}
    gen = torch.Generator().manual_seed(99)
    for tag, (Bz, Dn, L, N) in (("s16", (2, 5, 45, 16)), ("s8", (1, 3, 30, 8))):
        u = torch.randn(Bz, Dn, L, generator=gen)
        raw = torch.randn(Bz, Dn, L, generator=gen) * 2.0 - 1.0
        raw[0, 0, :3] = torch.tensor([25.0, 19.5, -30.0])      # both sides of the softplus cut-off and a tiny step
        bias = torch.randn(Dn, generator=gen) * 0.5
        A = -torch.exp(torch.randn(Dn, N, generator=gen)) * 0.3
        Bm = torch.randn(Bz, L, N, generator=gen)
        Cm = torch.randn(Bz, L, N, generator=gen)
        gate = torch.randn(Bz, Dn, L, generator=gen)
        go = torch.randn(Bz, Dn, L, generator=gen)
        pre = f"{tag}/"
        for k, v in (("u", u), ("dt_raw", raw), ("delta_bias", bias), ("A", A), ("B", Bm), ("C", Cm), ("gate", gate),
                     ("grad_out", go)):
            out[pre + k] = _np(v)
        leaves = [t.double().clone().requires_grad_(True) for t in (u, raw, A, Bm, Cm, gate, bias)]
        dt = F.softplus(leaves[1] + leaves[6][None, :, None])
        y = _selective_scan_mamba(inputs=leaves[0], dt=dt, A=leaves[2], B_t=leaves[3], C_t=leaves[4])
        o = y * F.silu(leaves[5])
        (o * go.double()).sum().backward()
        out[pre + "py64_out"] = _np(o)
        for name, leaf in zip(("du", "ddt_raw", "dA", "dB", "dC", "dgate", "ddelta_bias"), leaves):
            out[pre + "py64_" + name] = _np(leaf.grad)
    np.savez_compressed(os.path.join(HERE, "selective_scan_delta.npz"), **out)
    # ---- F. complex diagonal scan (LRU / S5) ------------------------------
    from ossm.models.lru import _LRUScanFn
    from ossm.models.s5 import _S5ScanFn

    out = {}
    gen = torch.Generator().manual_seed(2024)
    for tag, (L, B, P) in (("d1", (9, 2, 5)), ("d2", (70, 3, 33))):
        mag = torch.rand(P, generator=gen) * 0.5 + 0.45
        ph = torch.rand(P, generator=gen) * 6.28
        lam = torch.polar(mag, ph).to(torch.complex64)
        b = torch.complex(torch.randn(L, B, P, generator=gen), torch.randn(L, B, P, generator=gen)).to(torch.complex64)
        go = torch.complex(torch.randn(L, B, P, generator=gen), torch.randn(L, B, P, generator=gen)).to(torch.complex64)
        pre = f"{tag}/"
        out[pre + "lambda"], out[pre + "b_seq"], out[pre + "grad_out"] = _np(lam), _np(b), _np(go)
        for name, fn in (("lru", _LRUScanFn), ("s5", _S5ScanFn)):
            lm = lam.clone().requires_grad_(True)
            bb = b.clone().requires_grad_(True)
            st = fn.apply(lm, bb)
            ((st.real * go.real).sum() + (st.imag * go.imag).sum()).backward()
            out[pre + name + "_states"] = _np(st)
            out[pre + name + "_grad_lambda"], out[pre + name + "_grad_b"] = _np(lm.grad), _np(bb.grad)
        raw = kernels.lru_scan(lam.real.contiguous(), lam.imag.contiguous(), torch.view_as_real(b).contiguous())
        out[pre + "cpp_states"] = _np(torch.view_as_complex(raw.contiguous()))
    np.savez_compressed(os.path.join(HERE, "diag_generated.npz"), **out)
    # ---- G. selective D-LinOSS (per-step coefficients) --------------------
    from ossm.models import _sdlinoss_scan as sd

    def sel_params(variant, L, B, M, gen):
        """(A, G, step) from a pole radius / angle field, the layer's own map
        (``src/ossm/models/sdlinoss.py:186-204``); a few raw steps lie above 1 so that the
        step clamp and its gradient mask are exercised."""
        r = torch.rand(L, B, M, generator=gen) * 0.7 + 0.25
        th = (torch.rand(L, B, M, generator=gen) * 2 - 1) * 3.0
        raw = torch.sigmoid(torch.randn(L, B, M, generator=gen)) * 0.9 + 0.05
        dtc = raw.clone()
        raw = torch.where(torch.rand(L, B, M, generator=gen) < 0.05, raw + 1.0, raw)
        dtc = torch.clamp(torch.minimum(raw, torch.ones(())), min=1e-6)
        r2 = r * r
        cos_t = torch.cos(th)
        if variant == "imex1":
            A = (r2 - 2.0 * r * cos_t + 1.0) / (dtc * dtc * r2)
            G = (1.0 - r2) / (dtc * r2)
        elif variant == "imex2":
            A = (r2 - 2.0 * r * cos_t + 1.0) / (dtc * dtc)
            G = (1.0 - r2) / dtc
        elif variant == "im":
            A = (r2 - 2.0 * r * cos_t + 1.0) / (dtc * dtc * r2)
            G = (-2.0 * r2 + 2.0 * r * cos_t) / (dtc * r2)
        else:
            A = (r2 - 2.0 * r * cos_t + 1.0) / (dtc * dtc)
            G = (2.0 - 2.0 * r * cos_t) / dtc
        return A.float(), G.float(), raw.float()

    out = {}
    gen = torch.Generator().manual_seed(777)
    pick = {"M": lambda t: t[0, 0].contiguous(), "LM": lambda t: t[:, 0].contiguous(),
            "BM": lambda t: t[0].contiguous(), "LBM": lambda t: t.contiguous()}
    for variant in ("imex1", "imex2", "im", "ex"):
        for kind, (L, B, M) in (("LBM", (37, 3, 11)), ("LM", (24, 2, 5)), ("BM", (24, 2, 5)), ("M", (24, 2, 5)),
                                ("clamp", (6, 2, 3))):
            A, G, raw = sel_params(variant, L, B, M, gen)
            if kind == "clamp":      # one strongly negative damping entry drives S below its floor
                G[2, 1, 1] = -3.0 / torch.clamp(raw[2, 1, 1], max=1.0)
                a, g, s = A, G, raw
            else:
                a, g, s = (pick[kind](t) for t in (A, G, raw))
            bu = torch.complex(torch.randn(L, B, M, generator=gen), torch.randn(L, B, M, generator=gen))
            go = torch.complex(torch.randn(L, B, M, generator=gen), torch.randn(L, B, M, generator=gen))
            pre = f"{variant}/{kind}/"
            for k, v in (("A", a), ("G", g), ("step", s), ("bu", bu), ("grad_out", go)):
                out[pre + k] = _np(v)
            st = getattr(kernels, f"sdlinoss_{variant}_forward")(a, g, s, bu)
            gr = getattr(kernels, f"sdlinoss_{variant}_backward")(a, g, s, bu, st, go)
            out[pre + "cpp_states"] = _np(st)
            for name, t in zip(("grad_A", "grad_G", "grad_step", "grad_bu"), gr):
                out[pre + "cpp_" + name] = _np(t)
            # the pure-PyTorch recurrence in float64, gradients by autograd
            leaves = [t.double().clone().requires_grad_(True) for t in (a, g, s)]
            bl = bu.to(torch.complex128).clone().requires_grad_(True)
            st64 = sd._reference_sdlinoss_states(variant, leaves[0], leaves[1], leaves[2], bl)
            x64 = st64[..., 1]
            ((x64.real * go.real.double()).sum() + (x64.imag * go.imag.double()).sum()).backward()
            out[pre + "py64_states"] = _np(st64)
            for name, leaf in zip(("grad_A", "grad_G", "grad_step"), leaves):
                out[pre + "py64_" + name] = _np(leaf.grad)
            out[pre + "py64_grad_bu"] = _np(bl.grad)
    np.savez_compressed(os.path.join(HERE, "sdlinoss_generated.npz"), **out)

    for f in sorted(os.listdir(HERE)):
        if f.endswith(".npz"):
            print(f, os.path.getsize(os.path.join(HERE, f)))


if __name__ == "__main__":
    main()
