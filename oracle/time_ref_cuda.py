"""Times the reference's own CUDA kernels (``oracle/_ref/ossm_ref_kernels_cuda.so``, built by
``oracle/build_ref_cuda.py``: ossm's generic kernels recompiled for sm_100) on this GPU, on the same
synthetic workloads as ``bench.py``.  MEASUREMENT INFRASTRUCTURE ONLY: a same-box comparison point for
the numbers of this package; nothing here is part of the product path.

    python oracle/time_ref_cuda.py [--steps 10]

Prints one JSON line per workload (CUDA events, warm-up 3, L2 not flushed: inputs exceed L2).
"""
from __future__ import annotations

import argparse
import importlib.machinery
import importlib.util
import json
import os
import statistics

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
SO = os.path.join(HERE, "_ref", "ossm_ref_kernels_cuda.so")


def load():
    loader = importlib.machinery.ExtensionFileLoader("ossm_ref_kernels_cuda", SO)
    spec = importlib.util.spec_from_loader("ossm_ref_kernels_cuda", loader)
    mod = importlib.util.module_from_spec(spec)
    loader.exec_module(mod)
    return mod


def timed(fwd, bwd, steps):
    for _ in range(3):
        bwd(fwd())
    torch.cuda.synchronize()
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(steps)]
    for e in ev:
        e[0].record()
        saved = fwd()
        e[1].record()
        bwd(saved)
        e[2].record()
    torch.cuda.synchronize()
    return (statistics.mean(e[0].elapsed_time(e[1]) for e in ev),
            statistics.mean(e[1].elapsed_time(e[2]) for e in ev))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=10)
    args = ap.parse_args()
    k = load()
    dev = torch.device("cuda", 0)
    gen = torch.Generator(device=dev).manual_seed(0)
    rnd = lambda *s: torch.randn(*s, generator=gen, device=dev)

    def report(name, elems, f_ms, b_ms):
        print(json.dumps({"kernel": name, "impl": "reference CUDA kernels, recompiled for sm_100", "elements": elems,
                          "forward_ms": round(f_ms, 3), "backward_ms": round(b_ms, 3),
                          "gelem_per_s": round(elems / ((f_ms + b_ms) * 1e-3) / 1e9, 2)}), flush=True)

    # D-LinOSS imex1, B=64 L=4096 P=256 (the headline workload of bench.py)
    L, B, P = 4096, 64, 256
    a, g, dt = torch.relu(rnd(P)), torch.relu(rnd(P)), torch.sigmoid(rnd(P))
    bu = torch.view_as_complex(rnd(L, B, P, 2) * 0.5)
    gx = torch.view_as_complex(rnd(L, B, P, 2))
    f, b = timed(lambda: k.dlinoss_imex1_forward(a, g, dt, bu),
                 lambda st: k.dlinoss_imex1_backward(a, g, dt, bu, st, gx), args.steps)
    report("dlinoss_imex1_forward + backward (B=64 L=4096 P=256)", L * B * P, f, b)

    # selective D-LinOSS imex1, dense per-step coefficients, same shape
    r = (torch.rand(1, B, P, generator=gen, device=dev) * 0.6 + 0.3 + 0.03 * rnd(L, B, P)).clamp_(0.25, 0.95)
    th = (torch.rand(1, B, P, generator=gen, device=dev) * 2 - 1) * 2.5 + 0.05 * rnd(L, B, P)
    dtf = ((torch.sigmoid(rnd(1, B, P)) * 0.9 + 0.05) * (1 + 0.03 * rnd(L, B, P))).clamp(1e-6, 1.0)
    Af = ((r * r - 2 * r * torch.cos(th) + 1) / (dtf * dtf * r * r)).contiguous()
    Gf = ((1 - r * r) / (dtf * r * r)).contiguous()
    del r, th
    f, b = timed(lambda: k.sdlinoss_imex1_forward(Af, Gf, dtf, bu),
                 lambda st: k.sdlinoss_imex1_backward(Af, Gf, dtf, bu, st, gx), args.steps)
    report("sdlinoss_imex1_forward + backward (B=64 L=4096 M=256, dense coefficients)", L * B * P, f, b)
    del Af, Gf, dtf, bu, gx
    torch.cuda.empty_cache()

    # Mamba selective scan, B=32 D=2048 L=8192 N=16, float32 (the reference rejects bf16)
    Bz, Dn, Ls, N = 32, 2048, 8192, 16
    u, z = rnd(Bz, Dn, Ls), rnd(Bz, Dn, Ls)
    delta = torch.nn.functional.softplus(rnd(Bz, Dn, Ls) - 4)
    A = -torch.arange(1, N + 1, device=dev, dtype=torch.float32).repeat(Dn, 1)
    Bm, Cm = rnd(Bz, Ls, N), rnd(Bz, Ls, N)
    go = rnd(Bz, Dn, Ls)
    f, b = timed(lambda: k.selective_scan_cuda(u, delta, A, Bm, Cm, z, 16),
                 lambda out: k.selective_scan_cuda_backward(go, u, delta, A, Bm, Cm, z, out[1], out[2], 16),
                 max(args.steps // 3, 2))
    report("selective_scan_cuda forward + backward (B=32 D=2048 L=8192 N=16, fp32)", Bz * Dn * Ls, f, b)


if __name__ == "__main__":
    main()
