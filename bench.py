#!/usr/bin/env python
"""Benchmark of the recurrent-scan hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" is one forward + backward pass of the D-LinOSS imex1 scan over one
synthetic batch at the op boundary (``bu`` and the upstream gradient in,
``x``, ``grad_bu`` and the three coefficient gradients out).  The workload is
BASELINE.json's config 1 (B=64, L=4096, P=256 oscillators, fp32 / complex64).
With N > 1 (launched by torchrun, one rank per GPU) every rank scans its own
256-oscillator shard of a P = 256*N layer: the series are independent, so there
is no data-path collective (weak scaling).

Prints ONE JSON line (rank 0).  ``value`` is scan elements (B*L*P) per second
with inputs resident in HBM; ``e2e`` is the same metric through the public call
for host-resident data (``ossm_b200.host_io.scan_from_host``) with pinned HOST
buffers, the host->device and device->host copies inside the timed region.

The K steps are timed as a block (barrier + synchronize on both sides, maximum over
ranks) and the block is repeated ``--repeats`` times; ``ms_per_step`` is the median
block, the spread is reported beside it.

Beside the headline the same line carries
  ``config4``          the oscillator-sharded long-sequence configuration (B=8, L=131072,
                       H=512, P=2048 split over the ranks): strong scaling at the op boundary
                       (outputs left sharded) and at the layer boundary (tensor-core
                       projections + scan + NCCL reduce-scatter), with the parts timed apart;
  ``sharded_parity``   (N > 1) a small sharded layer and sharded selective scan compared with
                       the unsharded result on every rank before anything is timed;
  ``side``             (N = 1) the other scan families at their benchmark configurations.

``--impl reference`` times the reference's own compiled CPU kernels
(``oracle/_ref``, built from the ossm checkout by ``oracle/build_ref.py``) on
the host cores instead.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "dlinoss_scan_fwd_bwd_gelem_per_s"
UNIT = "Gelem/s"
FWD_BYTES = 16      # read bu 8 + write x 8                        (per scan element)
BWD_BYTES = 24      # read grad_x 8 + read bu 8 + write grad_bu 8  (per scan element)
BWD_DRAM_BYTES_PER_ELEM = 1.608e9 / (64 * 4096 * 256)   # measured DRAM traffic of one backward launch


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--repeats", type=int, default=10, help="how many times the K-step block is timed")
    ap.add_argument("--no-side", action="store_true", help="skip the side workloads of the N=1 line")
    ap.add_argument("--no-config4", action="store_true", help="skip the sharded long-sequence configuration")
    ap.add_argument("--config4-length", type=int, default=131072)
    ap.add_argument("--workload", default="dlinoss",
                    choices=["dlinoss", "linoss", "lru", "mamba", "sdlinoss", "generic", "layer", "shard", "conv", "mixer",
                             "sharded_layer"],
                    help="dlinoss = the headline (BASELINE config 1); linoss = config 2 (LinOSS IM, B=128 L=16384 "
                         "P=128); mamba = config 3 (selective scan, bf16 I/O, B=32 D=2048 L=8192 N=16); "
                         "sharded_layer = config 4 (D-LinOSS layer, B=8 H=512 P=2048 split over the ranks; "
                         "L defaults to 32768, a quarter of the config, to bound memory)")
    ap.add_argument("--side-batch", type=int, default=0,
                    help="batch of the side workloads (0 = the BASELINE config's own: 128 / 32 / 8)")
    ap.add_argument("--variant", default="imex1")
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--length", type=int, default=4096)
    ap.add_argument("--ssm", type=int, default=256, help="oscillators per GPU")
    ap.add_argument("--side-state", type=int, default=0,
                    help="state size of the selective-scan side workload (default 16, BASELINE config 3) and of the "
                         "mixer workload (default 256, ossm's Mamba4Rec configuration)")
    ap.add_argument("--side-length", type=int, default=0,
                    help="sequence length of the linoss / mamba side workloads (0 = the BASELINE config's own)")
    ap.add_argument("--e2e-steps", type=int, default=3)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--cpu-batch", type=int, default=8, help="batch slice timed on the host cores")
    return ap.parse_args()


def workload_name(args):
    return (f"D-LinOSS {args.variant} scan fwd+bwd at the op boundary, B={args.batch} L={args.length} "
            f"P={args.ssm} per GPU, complex64 (BASELINE config 1)")


def make_params(P, device, seed):
    """BASELINE config 0/1 distributions: A=relu(N), G=relu(N), dt=sigmoid(N)."""
    import torch

    gen = torch.Generator(device="cpu").manual_seed(seed)
    a = torch.relu(torch.randn(P, generator=gen))
    g = torch.relu(torch.randn(P, generator=gen))
    dt = torch.sigmoid(torch.randn(P, generator=gen))
    return a.to(device), g.to(device), dt.to(device)


# ---------------------------------------------------------------------------
# clocks
# ---------------------------------------------------------------------------
class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU while the timed region runs.

    Uses NVML (read-only queries) from a background thread every ~2 ms, because the
    timed region of this memory-bound benchmark lasts tens of milliseconds, shorter
    than one `nvidia-smi -lms` period; falls back to `nvidia-smi` when NVML is not
    importable.
    """

    REASONS = (("hw_slowdown", 0x8), ("hw_thermal_slowdown", 0x40), ("sw_thermal_slowdown", 0x20),
               ("sw_power_cap", 0x4))

    def __init__(self, index):
        self.index = index
        self.samples = []
        self.mask = 0
        self.max_mhz = None
        self._stop = False
        self._thread = None
        self._nvml = None

    def _loop(self):
        nv, h = self._nvml
        while not self._stop:
            try:
                self.samples.append(float(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)))
                self.mask |= int(nv.nvmlDeviceGetCurrentClocksEventReasons(h))
            except Exception:
                pass
            time.sleep(0.002)

    def start(self):
        import threading

        try:
            import pynvml as nv

            nv.nvmlInit()
            h = nv.nvmlDeviceGetHandleByIndex(self._physical_index())
            self.max_mhz = float(nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM))
            self._nvml = (nv, h)
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()
        except Exception:
            self._nvml = None

    def _physical_index(self):
        vis = os.environ.get("CUDA_VISIBLE_DEVICES")
        if vis:
            ids = [v.strip() for v in vis.split(",") if v.strip()]
            if self.index < len(ids) and ids[self.index].isdigit():
                return int(ids[self.index])
        return self.index

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0, "source": "nvml"}
        if self._nvml is None:
            return self._smi_once(out)
        self._stop = True
        self._thread.join(timeout=2)
        if self.samples:
            out.update(sm_mhz=statistics.median(self.samples), sm_max_mhz=self.max_mhz, samples=len(self.samples),
                       reasons=[name for name, bit in self.REASONS if self.mask & bit])
        return out

    def _smi_once(self, out):
        try:
            txt = subprocess.run(
                ["nvidia-smi", "--query-gpu=clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
                 "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
                 "clocks_event_reasons.sw_power_cap", "--format=csv,noheader,nounits", "-i", str(self.index)],
                capture_output=True, text=True, timeout=20).stdout.strip().splitlines()[0]
            parts = [p.strip() for p in txt.split(",")]
            out.update(sm_mhz=float(parts[0]), sm_max_mhz=float(parts[1]), samples=1, source="nvidia-smi (one sample)",
                       reasons=[n for (n, _), v in zip(self.REASONS, parts[2:6]) if v.lower().startswith("active")])
        except Exception:
            pass
        return out


# ---------------------------------------------------------------------------
# reference CPU arm / cpu_baseline
# ---------------------------------------------------------------------------
def time_reference_cpu(args, min_seconds, max_steps, warmup):
    """Times the reference's compiled CPU kernels (fwd + bwd) on a batch slice of
    the workload.  Returns (Gelem/s, description dict) or (None, reason)."""
    import torch
    from oracle.ref_loader import load_reference_kernels

    ref = load_reference_kernels()
    if ref is None:
        return None, "oracle/_ref/ossm_ref_kernels.so not built (run oracle/build_ref.py where the ossm checkout is)"
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    L, B, P = args.length, min(args.cpu_batch, args.batch), args.ssm
    a, g, dt = make_params(P, "cpu", 0)
    gen = torch.Generator().manual_seed(1)
    bu = torch.complex(torch.randn(L, B, P, generator=gen), torch.randn(L, B, P, generator=gen)) * 0.5
    gx = torch.complex(torch.randn(L, B, P, generator=gen), torch.randn(L, B, P, generator=gen))
    fwd = getattr(ref, f"dlinoss_{args.variant}_forward")
    bwd = getattr(ref, f"dlinoss_{args.variant}_backward")

    def step():
        states = fwd(a, g, dt, bu)
        return bwd(a, g, dt, bu, states, gx)

    for _ in range(warmup):
        step()
    times = []
    t_start = time.perf_counter()
    while len(times) < max_steps and (len(times) < 3 or time.perf_counter() - t_start < min_seconds):
        t0 = time.perf_counter()
        step()
        times.append(time.perf_counter() - t0)
    sec = statistics.mean(times)
    elems = L * B * P
    desc = {
        "kind": "reference", "cores": cores,
        "sample": (f"reference CPU kernels dlinoss_{args.variant}_forward+backward (ossm csrc, -O3 -ffast-math, "
                   f"at::parallel_for over {cores} threads) on a batch slice B={B} of the workload "
                   f"(L={L}, P={P}); {len(times)} steps of {sec * 1e3:.1f} ms"),
        "ms_per_step": sec * 1e3, "steps": len(times), "cpu_batch": B,
    }
    return elems / sec / 1e9, desc


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    warm = max(0, min(args.warmup, 20))      # each CPU step is ~0.2 s: the driver's warm-up count, capped at a few seconds
    val, desc = time_reference_cpu(args, min_seconds=20.0, max_steps=max(args.steps, 3), warmup=warm)
    if val is None:
        print(json.dumps({"impl": "reference", "unavailable": desc}))
        return
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus,
        "steps": desc["steps"], "warmup": warm, "ms_per_step": desc["ms_per_step"],
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload_name(args), "timing": "host wall clock, CPU tensors",
                   "cpu_batch": desc["cpu_batch"],
                   "sample": f"each step scans a batch slice of {desc['cpu_batch']} of the {args.batch} sequences "
                             "(the metric is a rate, elements per second)"},
        "cpu_baseline": {"value": val, "unit": UNIT, "kind": desc["kind"], "cores": desc["cores"],
                         "sample": desc["sample"]},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# ---------------------------------------------------------------------------
# helpers of our arm
# ---------------------------------------------------------------------------
def hbm_peak():
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        return float(peaks["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)", peaks
    except Exception:
        return 6650.0, "fallback 6650 GB/s", {}


def time_pair(fwd, bwd, steps, warmup):
    """Median device times (ms) over ``steps`` steps of ``saved = fwd()``, of ``bwd(saved)`` and of the whole step,
    CUDA events on the current stream, after ``warmup`` untimed steps (the median keeps one stalled step -- an
    allocator refill, another tenant of the host -- out of the figure)."""
    import torch

    for _ in range(max(warmup, 3)):
        bwd(fwd())
    torch.cuda.synchronize()
    evs = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(steps)]
    for e in evs:
        e[0].record()
        saved = fwd()
        e[1].record()
        bwd(saved)
        e[2].record()
    torch.cuda.synchronize()
    fwd_ms = statistics.median(e[0].elapsed_time(e[1]) for e in evs)
    bwd_ms = statistics.median(e[1].elapsed_time(e[2]) for e in evs)
    return fwd_ms, bwd_ms, statistics.median(e[0].elapsed_time(e[2]) for e in evs)


def side_workload(name, args, dev):
    """Builds one side workload: returns (fwd, bwd, elems, fwd_bytes, bwd_bytes, description, metric)."""
    import torch

    from ossm_b200 import kernels

    gen = torch.Generator(device=dev).manual_seed(0)

    def cplx(L, B, P, scale=1.0):
        return torch.view_as_complex(torch.randn(L, B, P, 2, generator=gen, device=dev) * scale)

    if name == "linoss":
        L, B, P = (args.side_length or 16384), (args.side_batch or 128), 128
        a = torch.relu(torch.randn(P, generator=gen, device=dev))
        dt = torch.sigmoid(torch.randn(P, generator=gen, device=dev))
        bu, gx = cplx(L, B, P, 0.5), cplx(L, B, P)
        return (lambda: kernels.lti_scan_forward("linoss_im", a, None, dt, bu),
                lambda saved: kernels.lti_scan_backward("linoss_im", a, None, dt, bu, saved[2], gx),
                L * B * P, FWD_BYTES, BWD_BYTES,
                f"LinOSS-IM scan fwd+bwd, B={B} L={L} P={P}, complex64 (BASELINE config 2)",
                "linoss_scan_fwd_bwd_gelem_per_s")
    if name == "shard":
        # the 256-oscillator shard of the sharded long-sequence configuration: few series, long sequence
        L, B, P = (args.side_length or 131072), (args.side_batch or 8), 256
        a, g, dt = make_params(P, dev, 0)
        bu, gx = cplx(L, B, P, 0.5), cplx(L, B, P)
        return (lambda: kernels.lti_scan_forward("imex1", a, g, dt, bu),
                lambda saved: kernels.lti_scan_backward("imex1", a, g, dt, bu, saved[2], gx),
                L * B * P, FWD_BYTES, BWD_BYTES,
                f"D-LinOSS imex1 scan fwd+bwd on one 256-oscillator shard, B={B} L={L} P={P} (2048 series: the "
                "two-level kernels; BASELINE config 4 per GPU at 8 GPUs)", "dlinoss_shard_scan_fwd_bwd_gelem_per_s")
    if name == "lru":
        L, B, P = args.length, (args.side_batch or 64), args.ssm
        mag = torch.rand(P, generator=gen, device=dev) * 0.5 + 0.45
        ph = torch.rand(P, generator=gen, device=dev) * 6.28
        lam_re, lam_im = (mag * torch.cos(ph)).contiguous(), (mag * torch.sin(ph)).contiguous()
        bu, gx = cplx(L, B, P, 0.5), cplx(L, B, P)
        return (lambda: kernels.diag_scan_forward(lam_re, lam_im, bu),
                lambda saved: kernels.diag_scan_backward(lam_re, lam_im, bu, saved[1], gx),
                L * B * P, FWD_BYTES, BWD_BYTES,
                f"LRU / S5 complex diagonal scan fwd+bwd, B={B} L={L} P={P}, complex64", "diag_scan_fwd_bwd_gelem_per_s")
    if name == "generic":
        # generic complex 2x2 LinOSS scan on materialised [L,B,P,2] states (the compatibility path of _LinossScanFn)
        L, B, P = (args.side_length or 4096), (args.side_batch or 32), 256
        am = (torch.view_as_complex(torch.randn(P, 2, 2, 2, generator=gen, device=dev)) * 0.3)
        m = [am[:, i, j].contiguous() for i in (0, 1) for j in (0, 1)]
        bs = torch.view_as_complex(torch.randn(L, B, P, 2, 2, generator=gen, device=dev) * 0.5)
        go = torch.view_as_complex(torch.randn(L, B, P, 2, 2, generator=gen, device=dev))
        # forward: read b 16, write states 16; backward: read states 16 + grad 16, write grad_b 16
        return (lambda: kernels.linoss_scan(*m, bs), lambda st: kernels.linoss_scan_backward(*m, st, go),
                L * B * P, 32, 48, f"generic complex 2x2 LinOSS scan fwd+bwd on [L,B,P,2] states, B={B} L={L} P={P}",
                "linoss_generic_scan_fwd_bwd_gelem_per_s")
    if name == "sdlinoss":
        L, B, P = args.length, (args.side_batch or 64), args.ssm
        r = (torch.rand(1, B, P, generator=gen, device=dev) * 0.6 + 0.3
             + 0.03 * torch.randn(L, B, P, generator=gen, device=dev)).clamp_(0.25, 0.95)
        th = (torch.rand(1, B, P, generator=gen, device=dev) * 2 - 1) * 2.5 + 0.05 * torch.randn(
            L, B, P, generator=gen, device=dev)
        dtf = (torch.sigmoid(torch.randn(1, B, P, generator=gen, device=dev)) * 0.9 + 0.05) * (
            1 + 0.03 * torch.randn(L, B, P, generator=gen, device=dev))
        dtc = dtf.clamp(1e-6, 1.0)
        Af = (r * r - 2 * r * torch.cos(th) + 1) / (dtc * dtc * r * r)
        Gf = (1 - r * r) / (dtc * r * r)
        del r, th, dtc
        bu, gx = cplx(L, B, P, 0.5), cplx(L, B, P)
        # forward: a, g, dt 12 B + bu 8 -> x 8 ; backward: 12 + bu 8 + grad_x 8 -> grad_bu 8 + three gradients 12
        return (lambda: kernels.sdlinoss_scan_forward("imex1", Af, Gf, dtf, bu),
                lambda saved: kernels.sdlinoss_scan_backward("imex1", Af, Gf, dtf, bu, gx, carries=saved[2]),
                L * B * P, 28, 48,
                f"selective D-LinOSS imex1 scan fwd+bwd, B={B} L={L} M={P}, dense per-step coefficients, complex64",
                "sdlinoss_scan_fwd_bwd_gelem_per_s")
    if name == "conv":
        # causal conv1d + SiLU of the Mamba mixer at the selective-scan benchmark shape, on the x half of in_proj's output
        from ossm_b200.mixer import _ConvSiluFn

        Bz, Dn, L = (args.side_batch or 32), 2048, (args.side_length or 8192)
        xz = torch.randn(Bz, L, 2 * Dn, generator=gen, device=dev)
        w = torch.randn(Dn, 1, 4, generator=gen, device=dev) * 0.5
        bias = torch.randn(Dn, generator=gen, device=dev) * 0.3
        g1 = torch.randn(Bz, Dn, L, generator=gen, device=dev)
        g2 = torch.randn(Bz, L, Dn, generator=gen, device=dev)
        x = xz[..., :Dn].requires_grad_(True)
        wl, bl = w.requires_grad_(True), bias.requires_grad_(True)

        def cfwd():
            x.grad = wl.grad = bl.grad = None
            return _ConvSiluFn.apply(x, wl, bl)

        def cbwd(outs):
            torch.autograd.backward(outs, (g1, g2))

        # forward: read x 4, write both layouts 8; backward: read x 4 + two gradients 8, write grad_x 4
        return (cfwd, cbwd, Bz * Dn * L, 12, 16,
                f"causal conv1d(k=4) + bias + SiLU fwd+bwd, B={Bz} D={Dn} L={L}, float32, both output layouts",
                "conv1d_silu_fwd_bwd_gelem_per_s")
    if name == "mamba":
        Bz, Dn, L, N = (args.side_batch or 32), 2048, (args.side_length or 8192), (args.side_state or 16)
        io = torch.bfloat16
        u = torch.randn(Bz, Dn, L, generator=gen, device=dev).to(io)
        z = torch.randn(Bz, Dn, L, generator=gen, device=dev).to(io)
        delta = torch.nn.functional.softplus(torch.randn(Bz, Dn, L, generator=gen, device=dev) - 4)
        A = -torch.arange(1, N + 1, device=dev, dtype=torch.float32).repeat(Dn, 1)
        Bt = torch.randn(Bz, N, L, generator=gen, device=dev).to(io)      # given time-contiguous [B, N, L]
        Ct = torch.randn(Bz, N, L, generator=gen, device=dev).to(io)
        Dv = torch.ones(Dn, device=dev)
        go = torch.randn(Bz, Dn, L, generator=gen, device=dev).to(io)
        # u 2 + delta 4 + z 2 -> out 2 ; + dout 2 -> du 2, ddelta 4, dz 2
        return (lambda: kernels.selective_scan_fwd(u, delta, A, Bt.transpose(1, 2), Ct.transpose(1, 2), z, Dv),
                lambda saved: kernels.selective_scan_bwd(go, u, delta, A, Bt.transpose(1, 2), Ct.transpose(1, 2), z,
                                                         saved[1], Dv),
                Bz * Dn * L, 10, 18,
                f"Mamba selective scan fwd+bwd, B={Bz} D={Dn} L={L} N={N}, bf16 I/O, fp32 state " + ("(BASELINE config 3)" if N == 16 else "(time-parallel kernels)"),
                "selective_scan_fwd_bwd_gelem_per_s")
    raise ValueError(name)


def run_side(name, args, dev, steps, warmup):
    import torch

    fwd, bwd, elems, fb, bb, desc, metric = side_workload(name, args, dev)
    fwd_ms, bwd_ms, ms = time_pair(fwd, bwd, steps, warmup)
    peak, _, _ = hbm_peak()
    gbs = elems * (fb + bb) / (ms * 1e-3) / 1e9
    out = {"metric": metric, "value": elems / (ms * 1e-3) / 1e9, "unit": UNIT, "ms_per_step": ms, "steps": steps,
           "workload": desc, "kernel_ms": {"forward": fwd_ms, "backward": bwd_ms},
           "roofline": {"bound": "hbm", "achieved": gbs, "peak": peak, "unit": "GB/s", "frac": gbs / peak,
                        "algorithmic_bytes_per_elem": fb + bb,
                        "forward_frac": elems * fb / (fwd_ms * 1e-3) / 1e9 / peak,
                        "backward_frac": elems * bb / (bwd_ms * 1e-3) / 1e9 / peak}}
    del fwd, bwd
    torch.cuda.empty_cache()
    return out


def layer_workload(args, dev, batch, length, hidden, ssm):
    """The D-LinOSS layer body at the layer boundary (u in, y out; gradients of u, A, G, step, B, C, D)."""
    import torch

    from ossm_b200.dlinoss_layer import dlinoss_layer

    gen = torch.Generator(device=dev).manual_seed(0)
    a, g, dt = make_params(ssm, dev, 0)
    bound = 1.0 / hidden ** 0.5
    Bp = (torch.rand(ssm, hidden, 2, generator=gen, device=dev) * 2 - 1) * bound
    Cp = (torch.rand(hidden, ssm, 2, generator=gen, device=dev) * 2 - 1) * bound
    D = torch.randn(hidden, generator=gen, device=dev)
    u = torch.randn(batch, length, hidden, generator=gen, device=dev)
    dy = torch.randn(batch, length, hidden, generator=gen, device=dev)
    leaves = [t.requires_grad_(True) for t in (a, g, dt, Bp, Cp, D, u)]

    def fwd():
        for t in leaves:
            t.grad = None
        return dlinoss_layer(args.variant, *leaves)

    def bwd(y):
        y.backward(dy)

    return fwd, bwd


def run_layer_side(args, dev, steps, warmup):
    """Layer boundary at the headline shape, and the composition the reference layer runs (library GEMMs in float32,
    permute copies, scan op) on the same GPU beside it."""
    import torch

    from ossm_b200.dlinoss import run_dlinoss

    Bz, L, H, P = args.batch, args.length, 256, args.ssm
    fwd, bwd = layer_workload(args, dev, Bz, L, H, P)
    fwd_ms, bwd_ms, ms = time_pair(fwd, bwd, steps, warmup)
    elems = Bz * L * P
    flops = 8.0 * Bz * L * H * P            # four real GEMMs of 2*B*L*H*P each way
    peak, _, peaks = hbm_peak()
    out = {"metric": "dlinoss_layer_fwd_bwd_gelem_per_s", "value": elems / (ms * 1e-3) / 1e9, "unit": UNIT,
           "ms_per_step": ms, "steps": steps,
           "workload": f"D-LinOSS {args.variant} layer body fwd+bwd (u in, y out, 7 gradients), B={Bz} L={L} H={H} P={P}",
           "kernel_ms": {"forward": fwd_ms, "backward": bwd_ms},
           "algorithmic_bytes_per_elem": 20.0 * H / P,
           "gemm": {"useful_tflops_forward": flops / (fwd_ms * 1e-3) / 1e12,
                    "useful_flop_forward": flops, "useful_flop_backward": 2 * flops,
                    "note": "float32-accurate: every useful product is three TF32 tensor-core products; the dense "
                            "bf16 peak of this GPU is %.0f TFLOP/s, its TF32 rate half of that" % peaks.get("bf16_tflops", 0.0)}}
    del fwd, bwd
    torch.cuda.empty_cache()
    # the reference layer's composition on the same GPU
    gen = torch.Generator(device=dev).manual_seed(0)
    a, g, dt = make_params(P, dev, 0)
    bound = 1.0 / H ** 0.5
    Bp = ((torch.rand(P, H, 2, generator=gen, device=dev) * 2 - 1) * bound).requires_grad_(True)
    Cp = ((torch.rand(H, P, 2, generator=gen, device=dev) * 2 - 1) * bound).requires_grad_(True)
    D = torch.randn(H, generator=gen, device=dev).requires_grad_(True)
    u = torch.randn(Bz, L, H, generator=gen, device=dev).requires_grad_(True)
    dy = torch.randn(Bz, L, H, generator=gen, device=dev)
    a, g, dt = (t.requires_grad_(True) for t in (a, g, dt))

    def ufwd():
        for t in (a, g, dt, Bp, Cp, D, u):
            t.grad = None
        flat = u.reshape(Bz * L, H)
        bu = torch.complex(flat @ Bp[..., 0].t(), flat @ Bp[..., 1].t()).reshape(Bz, L, P)
        x = run_dlinoss(args.variant, a, g, dt, bu.permute(1, 0, 2).contiguous()).permute(1, 0, 2).reshape(Bz * L, P)
        return (x.real @ Cp[..., 0].t() - x.imag @ Cp[..., 1].t()).reshape(Bz, L, H) + u * D

    uf, ub, ums = time_pair(ufwd, lambda y: y.backward(dy), max(3, steps // 2), 3)
    out["library_gemm_composition"] = {"ms_per_step": ums, "kernel_ms": {"forward": uf, "backward": ub},
                                       "what": "torch.matmul float32 (cuBLAS) + permute copies + this package's scan op"}
    torch.cuda.empty_cache()
    return out


# ---------------------------------------------------------------------------
# sharded long-sequence configuration (BASELINE config 4) and sharded parity
# ---------------------------------------------------------------------------
def run_sharded_parity(dev, world, rank):
    """Small sharded layer and sharded selective scan against the unsharded op on every rank (same seeded
    inputs everywhere); returns the largest relative errors over all ranks."""
    import torch
    import torch.distributed as dist

    from ossm_b200.dlinoss_layer import dlinoss_layer
    from ossm_b200.selective_scan import selective_scan
    from ossm_b200.sharded_layer import hidden_shard, sharded_dlinoss_layer
    from ossm_b200.sharded_selective_scan import sharded_selective_scan
    from ossm_b200.sharding import shard_channels

    gen = torch.Generator().manual_seed(11)
    Bz, L, H, P = 2, 600, 8 * world, 32 * world
    a = torch.rand(P, generator=gen) * 0.8
    g = torch.rand(P, generator=gen) * 0.4
    st = torch.sigmoid(torch.randn(P, generator=gen))
    Bp = torch.randn(P, H, 2, generator=gen) * 0.2
    Cp = torch.randn(H, P, 2, generator=gen) * 0.2
    D = torch.randn(H, generator=gen)
    u = torch.randn(Bz, L, H, generator=gen)
    dy = torch.randn(Bz, L, H, generator=gen)
    full = [t.to(dev).requires_grad_(True) for t in (a, g, st, Bp, Cp, D, u)]
    y_ref = dlinoss_layer("imex1", *full)
    y_ref.backward(dy.to(dev))
    cols = hidden_shard(H)
    loc = [shard_channels(a.to(dev), world, rank, 0), shard_channels(g.to(dev), world, rank, 0),
           shard_channels(st.to(dev), world, rank, 0), shard_channels(Bp.to(dev), world, rank, 0),
           shard_channels(Cp.to(dev), world, rank, 1), D[cols].to(dev), u.to(dev)]
    loc = [t.requires_grad_(True) for t in loc]
    y = sharded_dlinoss_layer("imex1", *loc, chunks=3)
    y.backward(dy.to(dev)[..., cols])

    def rel(got, want):
        return float((got - want).abs().max() / want.abs().max().clamp_min(1e-30))

    def shard_of(t, dim):
        return shard_channels(t, world, rank, dim)

    errs = {"layer_y": rel(y.detach(), y_ref.detach()[..., cols]), "layer_grad_u": rel(loc[6].grad, full[6].grad),
            "layer_grad_A": rel(loc[0].grad, shard_of(full[0].grad, 0)),
            "layer_grad_step": rel(loc[2].grad, shard_of(full[2].grad, 0)),
            "layer_grad_B": rel(loc[3].grad, shard_of(full[3].grad, 0)),
            "layer_grad_C": rel(loc[4].grad, shard_of(full[4].grad, 1)),
            "layer_grad_D": rel(loc[5].grad, full[5].grad[cols])}
    # Mamba scan with the channels split over the ranks: dB / dC are all-reduced in the backward
    Dn, N, Ls = 16 * world, 16, 300
    us = torch.randn(Bz, Dn, Ls, generator=gen)
    dts = torch.rand(Bz, Dn, Ls, generator=gen) * 0.05
    A = -torch.exp(torch.randn(Dn, N, generator=gen))
    Bm = torch.randn(Bz, Ls, N, generator=gen)
    Cm = torch.randn(Bz, Ls, N, generator=gen)
    z = torch.randn(Bz, Dn, Ls, generator=gen)
    go = torch.randn(Bz, Dn, Ls, generator=gen)
    fulls = [t.to(dev).requires_grad_(True) for t in (us, dts, A, Bm, Cm, z)]
    o_ref = selective_scan(*fulls)
    o_ref.backward(go.to(dev))
    locs = [shard_of(us.to(dev), 1), shard_of(dts.to(dev), 1), shard_of(A.to(dev), 0), Bm.to(dev), Cm.to(dev),
            shard_of(z.to(dev), 1)]
    locs = [t.requires_grad_(True) for t in locs]
    o = sharded_selective_scan(*locs)
    o.backward(shard_of(go.to(dev), 1))
    errs.update({"scan_out": rel(o.detach(), shard_of(o_ref.detach(), 1)),
                 "scan_grad_u": rel(locs[0].grad, shard_of(fulls[0].grad, 1)),
                 "scan_grad_A": rel(locs[2].grad, shard_of(fulls[2].grad, 0)),
                 "scan_grad_B": rel(locs[3].grad, fulls[3].grad), "scan_grad_C": rel(locs[4].grad, fulls[4].grad)})
    keys = sorted(errs)
    t = torch.tensor([errs[k] for k in keys], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    out = {k: float(v) for k, v in zip(keys, t.tolist())}
    out["bound"] = 1e-4
    out["ok"] = all(v <= 1e-4 for k, v in out.items() if k not in ("bound",))
    out["what"] = (f"sharded D-LinOSS layer (B={Bz} L={L} H={H} P={P}, reduce-scatter output, 3 time chunks) and "
                   f"channel-sharded selective scan (D={Dn} N={N} L={Ls}) against the unsharded ops, max over "
                   f"{world} ranks of max|got-want|/max|want|")
    return out


def run_config4(args, dev, world, rank):
    """Strong scaling of the sharded long-sequence configuration.  Returns a dict (same on every rank)."""
    import torch
    import torch.distributed as dist

    from ossm_b200 import kernels
    from ossm_b200.sharded_layer import hidden_shard, sharded_dlinoss_layer
    from ossm_b200.sharding import aggregate_throughput, shard_channels

    Bz, H, P = 8, 512, 2048
    L = args.config4_length
    if P % world or H % world:
        return {"skipped": f"P={P} and H={H} must divide over {world} ranks"}
    Pr = P // world
    free, _total = torch.cuda.mem_get_info(dev)
    # op boundary: bu, x, grad_x, grad_bu (8 B each per element) + carries; layer: also u, y, grads (small)
    need = Bz * L * Pr * 8 * 5.2 + Bz * L * H * 4 * 8
    while need > 0.8 * free and L > 4096:
        L //= 2
        need = Bz * L * Pr * 8 * 5.2 + Bz * L * H * 4 * 8
    out = {"workload": f"D-LinOSS imex1, B={Bz} L={L} H={H} P={P} split {Pr} oscillators per GPU over {world} GPU(s) "
                       "(BASELINE config 4)", "scaling": "strong", "length": L,
           "length_note": None if L == args.config4_length else f"L reduced from {args.config4_length} to fit this GPU's free memory"}
    steps, warm = 5, 3

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def timed(fn, n):
        for _ in range(warm):
            fn()
        sync_all()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        sync_all()
        _, ms = aggregate_throughput(0, e0.elapsed_time(e1) / n, dev)
        return ms

    # ---- op boundary: every rank scans its oscillator shard, outputs stay sharded, no collective ------
    a, g, dt = (shard_channels(t, world, rank) for t in make_params(P, dev, 0))
    gen = torch.Generator(device=dev).manual_seed(100 + rank)
    bu = torch.view_as_complex(torch.randn(L, Bz, Pr, 2, generator=gen, device=dev).mul_(0.5))
    gx = torch.view_as_complex(torch.randn(L, Bz, Pr, 2, generator=gen, device=dev))
    state = {}

    def op_fwd():
        state["f"] = kernels.lti_scan_forward("imex1", a, g, dt, bu)

    def op_step():
        op_fwd()
        kernels.lti_scan_backward("imex1", a, g, dt, bu, state["f"][2], gx)

    fwd_ms = timed(op_fwd, steps)
    step_ms = timed(op_step, steps)
    elems = Bz * L * P
    peak, _, _ = hbm_peak()
    out["op_boundary"] = {"value": elems / (step_ms * 1e-3) / 1e9, "unit": UNIT, "ms_per_step": step_ms,
                          "forward_ms": fwd_ms, "backward_ms": step_ms - fwd_ms,
                          "hbm_frac_per_gpu": (elems / world) * (FWD_BYTES + BWD_BYTES) / (step_ms * 1e-3) / 1e9 / peak,
                          "series_per_gpu": Bz * Pr,
                          "collective": "none (outputs left sharded over the oscillators)"}
    scan_ms = step_ms
    del bu, gx
    state.clear()
    torch.cuda.empty_cache()

    # ---- layer boundary: tensor-core projections + scan + reduce-scatter of y -----------------------
    gcpu = torch.Generator().manual_seed(0)
    bound = 1.0 / H ** 0.5
    Bp = (torch.rand(P, H, 2, generator=gcpu) * 2 - 1) * bound
    Cp = (torch.rand(H, P, 2, generator=gcpu) * 2 - 1) * bound
    Dv = torch.randn(H, generator=gcpu)
    cols = hidden_shard(H) if world > 1 else slice(0, H)
    loc = [a, g, dt, shard_channels(Bp, world, rank, 0).to(dev), shard_channels(Cp, world, rank, 1).to(dev),
           Dv[cols].to(dev)]
    loc = [t.detach().clone().requires_grad_(True) for t in loc]
    gen = torch.Generator(device=dev).manual_seed(7)          # u is replicated: same seed on every rank
    u = torch.randn(Bz, L, H, generator=gen, device=dev).requires_grad_(True)
    dy = torch.randn(Bz, L, H // world if world > 1 else H, generator=gen, device=dev)

    def layer_step():
        for t in loc + [u]:
            t.grad = None
        y = sharded_dlinoss_layer("imex1", *loc, u, chunks=8, scatter_output=world > 1)
        y.backward(dy)

    layer_ms = timed(layer_step, 3)
    # the parts, each timed on its own (standalone times: inside the step they partly overlap)
    w_in = torch.randn(2 * Pr, H, device=dev) * bound
    w_out = torch.randn(H, 2 * Pr, device=dev) * bound
    hi_in, lo_in = kernels.split_tf32(w_in)
    hi_out, lo_out = kernels.split_tf32(w_out)
    hi_int, lo_int = kernels.split_tf32(w_in.t().contiguous())
    hi_outt, lo_outt = kernels.split_tf32(w_out.t().contiguous())
    ud = u.detach().view(Bz * L, H)
    buf_p = torch.empty(L * Bz, 2 * Pr, device=dev)
    buf_h = torch.empty(Bz * L, H, device=dev)

    def gemms():    # the four tensor-core projections of one forward + backward
        kernels.gemm_tf32x3(ud, hi_in, lo_in, buf_p, row_map=1, batch=Bz, length=L)
        kernels.gemm_tf32x3(buf_p, hi_out, lo_out, buf_h, row_map=2, batch=Bz, length=L)
        kernels.gemm_tf32x3(ud, hi_outt, lo_outt, buf_p, row_map=1, batch=Bz, length=L)
        kernels.gemm_tf32x3(buf_p, hi_int, lo_int, buf_h, row_map=2, batch=Bz, length=L)

    from ossm_b200.dlinoss_layer import weight_gradient

    def weight_grads():    # grad_B and grad_C: sums over all (b, l) rows, on the tensor cores as well
        weight_gradient(buf_p, True, ud, False, Bz, L)
        weight_gradient(ud, False, buf_p, True, Bz, L)

    proj_ms = timed(gemms, 3)
    wgrad_ms = timed(weight_grads, 3)
    coll_ms = 0.0
    if world > 1:
        hs = H // world
        part = torch.empty(world * Bz, L, hs, device=dev)
        mine = torch.empty(Bz, L, hs, device=dev)
        full = torch.empty(Bz, L, H, device=dev)

        def collectives():   # forward reduce-scatter of y, backward all-gather of grad_y and all-reduce of grad_u
            dist.reduce_scatter_tensor(mine, part)
            dist.all_gather_into_tensor(part, mine)
            dist.all_reduce(full)

        coll_ms = timed(collectives, 3)
    flops = 4 * 2.0 * Bz * L * H * 2 * Pr        # the four projections of this rank
    out["layer_boundary"] = {
        "value": elems / (layer_ms * 1e-3) / 1e9, "unit": UNIT, "ms_per_step": layer_ms,
        "parts_ms_standalone": {"tensor_core_projections": proj_ms, "tensor_core_weight_gradients": wgrad_ms,
                                "scan": scan_ms, "collectives": coll_ms},
        "projection_useful_tflops_per_gpu": flops / (proj_ms * 1e-3) / 1e12,
        "collective_bytes_per_gpu": 0 if world == 1 else 3 * Bz * L * H * 4,
        "pipeline": "output projection in 8 time chunks, the NCCL reduce-scatter of a chunk overlaps the GEMM of the next",
        "limit": "largest standalone part"}
    del u, dy, loc, buf_p, buf_h
    torch.cuda.empty_cache()
    return out


# ---------------------------------------------------------------------------
# our arm
# ---------------------------------------------------------------------------
def run_ours(args):
    import torch
    import torch.distributed as dist

    from ossm_b200 import _lib, kernels

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device (the scan has no CPU path; use --impl reference for the CPU arm)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    _lib.load()

    sharded_parity = run_sharded_parity(dev, world, rank) if world > 1 else None

    L, B, P = args.length, args.batch, args.ssm
    variant = args.variant
    from ossm_b200.sharding import aggregate_throughput, shard_channels

    # one layer of P * world oscillators; this rank owns a contiguous shard of P of them
    a, g, dt = (shard_channels(t, world, rank) for t in make_params(P * world, dev, seed=0))
    gen = torch.Generator(device=dev).manual_seed(100 + rank)
    bu = torch.randn(L, B, P, 2, generator=gen, device=dev)
    bu = torch.view_as_complex(bu.mul_(0.5))
    gx = torch.view_as_complex(torch.randn(L, B, P, 2, generator=gen, device=dev))
    elems = L * B * P

    def step(record=None):
        if record is not None:
            record[0].record()
        x, _, carries = kernels.lti_scan_forward(variant, a, g, dt, bu)
        if record is not None:
            record[1].record()
        grads = kernels.lti_scan_backward(variant, a, g, dt, bu, carries, gx)
        if record is not None:
            record[2].record()
        return x, grads

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step()
    sync_all()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    # the K-step block, `repeats` times; each block is bracketed by barrier + synchronize and timed on the device
    blocks = []
    total_elems = elems * world
    for _ in range(max(1, args.repeats)):
        t_begin = torch.cuda.Event(enable_timing=True)
        t_end = torch.cuda.Event(enable_timing=True)
        t_begin.record()
        for i in range(args.steps):
            step()
        t_end.record()
        sync_all()
        total_elems, block_ms = aggregate_throughput(elems, t_begin.elapsed_time(t_end), dev)   # sum of units, max of time
        blocks.append(block_ms / args.steps)
    # per-kernel durations for the roofline: the same steps again, now with an event between the kernels
    # (kept out of the K timed steps so that the extra stream operations do not stretch them)
    evs = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(min(args.steps, 50))]
    for e in evs:
        step(e)
    torch.cuda.synchronize()
    clocks = sampler.stop() if rank == 0 else None
    fwd_ms = statistics.mean(e[0].elapsed_time(e[1]) for e in evs)
    bwd_ms = statistics.mean(e[1].elapsed_time(e[2]) for e in evs)
    status = _lib.device_status()
    if status != 0:
        raise SystemExit(f"bench.py: device status {status} (a bounded wait inside a kernel gave up)")
    ms_per_step = statistics.median(blocks)
    value = total_elems / (ms_per_step * 1e-3) / 1e9

    # ---- end-to-end through the public op with host buffers ----------------
    e2e = None
    if not args.no_e2e:
        pin_to_gpu_numa_node(local_rank)
        h_bu = torch.empty((L, B, P), dtype=torch.complex64, pin_memory=True)
        h_gx = torch.empty((L, B, P), dtype=torch.complex64, pin_memory=True)
        h_bu.copy_(bu)
        h_gx.copy_(gx)
        h_x = torch.empty((L, B, P), dtype=torch.complex64, pin_memory=True)
        h_gbu = torch.empty((L, B, P), dtype=torch.complex64, pin_memory=True)
        h_pg = torch.empty((3, P), dtype=torch.float32, pin_memory=True)
        from ossm_b200.host_io import scan_from_host

        # The public call for host-resident data: time slices are copied up, scanned and
        # copied down in a pipeline so that both PCIe directions stay busy.
        def e2e_step(copies_only=False):
            grads = scan_from_host(variant, a, g, dt, h_bu, h_gx, h_x, h_gbu, slices=16, copies_only=copies_only)
            if grads is not None:
                for row, t in zip(h_pg, grads):
                    row.copy_(t, non_blocking=True)

        def time_e2e(copies_only):
            e2e_step(copies_only)
            sync_all()
            e0 = torch.cuda.Event(enable_timing=True)
            e1 = torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(args.e2e_steps):
                e2e_step(copies_only)
            e1.record()
            torch.cuda.synchronize()
            _, ms = aggregate_throughput(elems, e0.elapsed_time(e1) / args.e2e_steps, dev)
            return ms

        e2e_ms = time_e2e(False)
        copy_ms = time_e2e(True)
        e2e = {"value": total_elems / (e2e_ms * 1e-3) / 1e9, "unit": UNIT,
               "h2d_bytes_per_step": 2 * elems * 8, "d2h_bytes_per_step": 2 * elems * 8 + 3 * P * 4,
               "ms_per_step": e2e_ms,
               "copies_only": {"ms_per_step": copy_ms, "value": total_elems / (copy_ms * 1e-3) / 1e9,
                               "what": "the same pinned buffers through the same copy pipeline with no kernel launched: "
                                       "the ceiling the host and PCIe side puts on this call"},
               "api": "ossm_b200.host_io.scan_from_host (forward + backward, pinned host buffers, 16 time slices, state handed over on the device)"}
        del h_bu, h_gx, h_x, h_gbu
    del bu, gx
    torch.cuda.empty_cache()

    config4 = None
    if not args.no_config4:
        config4 = run_config4(args, dev, world, rank)

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peak, peak_src, _peaks = hbm_peak()
    bwd_gbs = elems * BWD_BYTES / (bwd_ms * 1e-3) / 1e9
    fwd_gbs = elems * FWD_BYTES / (fwd_ms * 1e-3) / 1e9
    # whole step over the K timed steps of this rank (launch gaps included)
    step_gbs = elems * (FWD_BYTES + BWD_BYTES) / (ms_per_step * 1e-3) / 1e9
    roofline = {
        "bound": "hbm", "kernel": "lti_backward_kernel (dominant; + lti_param_grad_kernel)",
        "achieved": bwd_gbs, "peak": peak, "unit": "GB/s", "frac": bwd_gbs / peak,
        "traffic": BWD_DRAM_BYTES_PER_ELEM * elems, "peak_source": peak_src,
        "peak_note": "the measured peak is a copy kernel's rate, a lower bound of what HBM3e delivers "
                     "(nominal 7.7 TB/s); fractions slightly above 1 are possible",
        "frac_of_nominal_7700": bwd_gbs / 7700.0,
        "algorithmic_bytes_per_launch": elems * BWD_BYTES, "ms_per_launch": bwd_ms,
        "forward": {"kernel": "lti_forward_kernel", "achieved": fwd_gbs, "frac": fwd_gbs / peak,
                    "algorithmic_bytes_per_launch": elems * FWD_BYTES, "ms_per_launch": fwd_ms},
        "step": {"achieved": step_gbs, "frac": step_gbs / peak,
                 "algorithmic_bytes": elems * (FWD_BYTES + BWD_BYTES)},
        # one ncu capture of one backward launch at this shape (1.608 GB for 67.1 M elements), scaled by elements
        "traffic_source": "ncu dram__bytes_read.sum + dram__bytes_write.sum of one lti_backward_kernel launch "
                          "(a constant from an earlier capture, not measured by this run)",
    }

    cpu_baseline = None
    if world == 1 and not args.no_cpu_baseline:
        val, desc = time_reference_cpu(args, min_seconds=10.0, max_steps=20, warmup=1)
        if val is not None:
            cpu_baseline = {"value": val, "unit": UNIT, "cores": desc["cores"], "kind": desc["kind"],
                            "sample": desc["sample"]}
        else:
            cpu_baseline = {"value": None, "unit": UNIT, "cores": os.cpu_count(), "kind": "reference",
                            "sample": "unavailable: " + desc}

    side = None
    if world == 1 and not args.no_side:
        side = {}
        for name, n_steps in (("linoss", 30), ("mamba", 5), ("sdlinoss", 30), ("lru", 30), ("generic", 20), ("shard", 20), ("conv", 10)):
            try:
                side[name] = run_side(name, args, dev, n_steps, 3)
            except Exception as exc:       # a side workload must not take the headline down
                side[name] = {"error": str(exc)[:300]}
        try:
            side["layer"] = run_layer_side(args, dev, 5, 3)
        except Exception as exc:
            side["layer"] = {"error": str(exc)[:300]}
        try:
            side["mixer"] = run_mixer_side(args, dev, 10, 3)
        except Exception as exc:
            side["mixer"] = {"error": str(exc)[:300]}
        if _lib.device_status() != 0:
            side["device_status"] = "non-zero"

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "ms_per_step_blocks": {"n": len(blocks), "min": min(blocks), "max": max(blocks), "median": ms_per_step,
                               "what": f"the {args.steps}-step block timed {len(blocks)} times"},
        "config": {"workload": workload_name(args), "variant": variant, "batch": B, "length": L,
                   "ssm_per_gpu": P, "sharding": f"oscillators split over {world} GPU(s), no collective",
                   "l2": "inputs (2 x %d MB) larger than L2, no flush" % (elems * 8 // 2**20)},
        "roofline": roofline, "cpu_baseline": cpu_baseline, "e2e": e2e,
        # forward, backward and the coefficient-gradient reduction per step
        "gpu_launches": 3 * args.steps * len(blocks), "clocks": clocks,
        "kernel_ms": {"forward": fwd_ms, "backward": bwd_ms},
        "config4": config4, "sharded_parity": sharded_parity, "side": side,
    }
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def pin_to_gpu_numa_node(local_rank):
    """Binds this process to the CPUs NVML reports as close to its GPU before the pinned host buffers are
    allocated and first touched, so that they land on that GPU's NUMA node (read-only NVML query)."""
    try:
        import pynvml as nv

        nv.nvmlInit()
        vis = os.environ.get("CUDA_VISIBLE_DEVICES")
        idx = local_rank
        if vis:
            ids = [v.strip() for v in vis.split(",") if v.strip()]
            if local_rank < len(ids) and ids[local_rank].isdigit():
                idx = int(ids[local_rank])
        h = nv.nvmlDeviceGetHandleByIndex(idx)
        words = (os.cpu_count() + 63) // 64
        mask = nv.nvmlDeviceGetCpuAffinity(h, words)
        cpus = [64 * w + b for w, m in enumerate(mask) for b in range(64) if (int(m) >> b) & 1]
        allowed = sorted(set(cpus) & set(os.sched_getaffinity(0)))
        if allowed:
            os.sched_setaffinity(0, allowed)
    except Exception:
        pass


def run_mixer_side(args, dev, steps, warmup):
    """Mamba mixer (ossm ``_MambaMixer``, ``mambarec.py:64-184``) forward + backward at the Mamba4Rec shape
    (``configs/model/mambarec.yaml``: d_model 64, expand 2, d_state 256, d_conv 4; batch 128 of ``training/seqrec.yaml``,
    length 200 of ``dataset/ml1m.yaml``), on a stand-in module with ossm's attribute names and initialisation ranges.
    Two arms on the same parameters: this package's fused forward (conv1d + SiLU kernel, step transform inside the
    scan), and the sequence of passes ossm's forward runs (transpose, pad, conv1d, SiLU, softplus(dt_proj)) around
    this package's selective-scan op."""
    import math

    import torch
    import torch.nn.functional as F
    from torch import nn

    from ossm_b200.mixer import mamba_mixer_forward
    from ossm_b200.selective_scan import selective_scan

    d_model, expand, d_state, d_conv = 64, 2, (args.side_state or 256), 4
    Bz, L = (args.side_batch or 128), (args.side_length or 200)

    class Mixer(nn.Module):
        def __init__(self):
            super().__init__()
            self.d_inner, self.d_state, self.d_conv = expand * d_model, d_state, d_conv
            self.dt_rank = math.ceil(d_model / 16)
            self.in_proj = nn.Linear(d_model, 2 * self.d_inner, bias=False)
            self.conv1d = nn.Conv1d(self.d_inner, self.d_inner, d_conv, groups=self.d_inner, bias=True, padding=0)
            self.x_proj = nn.Linear(self.d_inner, self.dt_rank + 2 * d_state, bias=False)
            self.dt_proj = nn.Linear(self.dt_rank, self.d_inner, bias=True)
            self.out_proj = nn.Linear(self.d_inner, d_model, bias=False)
            dt = torch.exp(torch.rand(self.d_inner) * (math.log(0.1) - math.log(0.001)) + math.log(0.001)).clamp(min=1e-4)
            with torch.no_grad():
                self.dt_proj.bias.copy_(dt + torch.log(-torch.expm1(-dt)))
            self.A_log = nn.Parameter(torch.log(torch.arange(1, d_state + 1, dtype=torch.float32).repeat(self.d_inner, 1)))

    torch.manual_seed(0)
    m = Mixer().to(dev)
    x = torch.randn(Bz, L, d_model, device=dev, requires_grad=True)
    gy = torch.randn(Bz, L, d_model, device=dev)

    def reset():
        x.grad = None
        for q in m.parameters():
            q.grad = None

    def fused():
        reset()
        return mamba_mixer_forward(m, x)

    def composed():
        reset()
        xz = m.in_proj(x)
        xi, z = xz.chunk(2, dim=-1)
        xc = m.conv1d(F.pad(xi.transpose(1, 2), (d_conv - 1, 0)))
        xc = F.silu(xc)
        proj = m.x_proj(xc.transpose(1, 2))
        dt_raw, Bg, Cg = torch.split(proj, [m.dt_rank, d_state, d_state], dim=-1)
        dt = F.softplus(m.dt_proj(dt_raw)).transpose(1, 2)
        y = selective_scan(xc, dt, -torch.exp(m.A_log.float()), Bg, Cg, z.transpose(1, 2), None)
        return m.out_proj(y.transpose(1, 2))

    f_ms, b_ms, ms = time_pair(fused, lambda y: y.backward(gy), steps, warmup)
    cf_ms, cb_ms, cms = time_pair(composed, lambda y: y.backward(gy), steps, warmup)
    with torch.no_grad():
        diff = float((fused() - composed()).abs().max())
    elems = Bz * m.d_inner * L
    out = {"metric": "mamba_mixer_fwd_bwd_gelem_per_s", "value": elems / (ms * 1e-3) / 1e9, "unit": UNIT,
           "ms_per_step": ms, "steps": steps,
           "workload": f"Mamba mixer fwd+bwd (ossm _MambaMixer), B={Bz} L={L} d_model={d_model} d_inner={m.d_inner} "
                       f"d_state={d_state} d_conv={d_conv}, float32",
           "kernel_ms": {"forward": f_ms, "backward": b_ms},
           "passes_as_in_ossm_forward": {"ms_per_step": cms, "kernel_ms": {"forward": cf_ms, "backward": cb_ms},
                                         "what": "transpose, pad, conv1d, SiLU, softplus(dt_proj) as separate library "
                                                 "passes around this package's selective-scan op",
                                         "max_abs_difference_of_outputs": diff}}
    del m
    torch.cuda.empty_cache()
    return out


def run_single(args):
    """One side workload on its own (single GPU): one JSON line with its own metric name."""
    import torch

    from ossm_b200 import _lib

    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device")
    dev = torch.device("cuda", 0)
    if args.workload == "layer":
        out = run_layer_side(args, dev, args.steps, args.warmup)
    elif args.workload == "mixer":
        out = run_mixer_side(args, dev, args.steps, args.warmup)
    else:
        out = run_side(args.workload, args, dev, args.steps, args.warmup)
    if _lib.device_status() != 0:
        raise SystemExit("bench.py: device status non-zero")
    out.update({"n_gpus": 1, "warmup": max(args.warmup, 3), "higher_is_better": True, "data": "synthetic",
                "config": {"workload": out.pop("workload")}})
    print(json.dumps(out))


def run_config4_only(args):
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    parity = run_sharded_parity(dev, world, rank) if world > 1 else None
    out = run_config4(args, dev, world, rank)
    if rank == 0:
        print(json.dumps({"metric": "dlinoss_sharded_config4", "n_gpus": world, "config4": out, "sharded_parity": parity}))
    if world > 1:
        dist.destroy_process_group()


def main():
    args = parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
    elif args.workload == "sharded_layer":
        run_config4_only(args)
    elif args.workload != "dlinoss":
        run_single(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
