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
    ap.add_argument("--workload", default="dlinoss", choices=["dlinoss", "linoss", "lru", "mamba", "sdlinoss", "sharded_layer"],
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
        "ms_per_step": sec * 1e3, "steps": len(times),
    }
    return elems / sec / 1e9, desc


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    val, desc = time_reference_cpu(args, min_seconds=20.0, max_steps=max(args.steps, 3), warmup=min(args.warmup, 2))
    if val is None:
        print(json.dumps({"impl": "reference", "unavailable": desc}))
        return
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus,
        "steps": desc["steps"], "warmup": min(args.warmup, 2), "ms_per_step": desc["ms_per_step"],
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload_name(args), "timing": "host wall clock, CPU tensors"},
        "cpu_baseline": {"value": val, "unit": UNIT, "kind": desc["kind"], "cores": desc["cores"],
                         "sample": desc["sample"]},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


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

    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
        torch.cuda.synchronize()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    t_begin = torch.cuda.Event(enable_timing=True)
    t_end = torch.cuda.Event(enable_timing=True)
    t_begin.record()
    for i in range(args.steps):
        step()
    t_end.record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
        torch.cuda.synchronize()
    total_ms = t_begin.elapsed_time(t_end)
    # per-kernel durations for the roofline: the same steps again, now with an event between the kernels
    # (kept out of the K timed steps so that the extra stream operations do not stretch them)
    evs = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(min(args.steps, 50))]
    for e in evs:
        step(e)
    torch.cuda.synchronize()
    clocks = sampler.stop() if rank == 0 else None
    fwd_ms = statistics.mean(e[0].elapsed_time(e[1]) for e in evs)
    bwd_ms = statistics.mean(e[1].elapsed_time(e[2]) for e in evs)
    total_elems, total_ms = aggregate_throughput(elems, total_ms, dev)   # sum of units, max of time over ranks
    status = _lib.device_status()
    if status != 0:
        raise SystemExit(f"bench.py: device status {status} (a bounded wait inside a kernel gave up)")
    ms_per_step = total_ms / args.steps
    value = total_elems / (ms_per_step * 1e-3) / 1e9

    # ---- end-to-end through the public op with host buffers ----------------
    e2e = None
    if not args.no_e2e:
        h_bu = torch.empty((L, B, P), dtype=torch.complex64, pin_memory=True)
        h_gx = torch.empty((L, B, P), dtype=torch.complex64, pin_memory=True)
        h_bu.copy_(bu)
        h_gx.copy_(gx)
        h_x = torch.empty((L, B, P), dtype=torch.complex64, pin_memory=True)
        h_gbu = torch.empty((L, B, P), dtype=torch.complex64, pin_memory=True)
        h_pg = torch.empty((3, P), dtype=torch.float32, pin_memory=True)
        from ossm_b200.host_io import scan_from_host

        # The public call for host-resident data: batch slices are copied up, scanned and
        # copied down in a pipeline so that both PCIe directions stay busy.
        def e2e_step():
            grads = scan_from_host(variant, a, g, dt, h_bu, h_gx, h_x, h_gbu, slices=8)
            for row, t in zip(h_pg, grads):
                row.copy_(t, non_blocking=True)

        e2e_step()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        e0 = torch.cuda.Event(enable_timing=True)
        e1 = torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.e2e_steps):
            e2e_step()
        e1.record()
        torch.cuda.synchronize()
        e2e_ms = e0.elapsed_time(e1) / args.e2e_steps
        _, e2e_ms = aggregate_throughput(elems, e2e_ms, dev)
        e2e = {"value": total_elems / (e2e_ms * 1e-3) / 1e9, "unit": UNIT,
               "h2d_bytes_per_step": 2 * elems * 8, "d2h_bytes_per_step": 2 * elems * 8 + 3 * P * 4,
               "ms_per_step": e2e_ms,
               "api": "ossm_b200.host_io.scan_from_host (forward + backward, pinned host buffers, 8 batch slices)"}

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except Exception:
        pass
    peak = float(peaks.get("hbm_gbs", 6650.0))
    peak_src = "measured (MEASURED_PEAKS.json hbm_gbs)" if "hbm_gbs" in peaks else "fallback 6650 GB/s"
    bwd_gbs = elems * BWD_BYTES / (bwd_ms * 1e-3) / 1e9
    fwd_gbs = elems * FWD_BYTES / (fwd_ms * 1e-3) / 1e9
    # whole step over the K timed steps of this rank (launch gaps included)
    step_gbs = elems * (FWD_BYTES + BWD_BYTES) / (ms_per_step * 1e-3) / 1e9
    roofline = {
        "bound": "hbm", "kernel": "lti_backward_kernel (dominant; + lti_param_grad_kernel)",
        "achieved": bwd_gbs, "peak": peak, "unit": "GB/s", "frac": bwd_gbs / peak,
        "traffic": None, "peak_source": peak_src,
        "algorithmic_bytes_per_launch": elems * BWD_BYTES, "ms_per_launch": bwd_ms,
        "forward": {"kernel": "lti_forward_kernel", "achieved": fwd_gbs, "frac": fwd_gbs / peak,
                    "algorithmic_bytes_per_launch": elems * FWD_BYTES, "ms_per_launch": fwd_ms},
        "step": {"achieved": step_gbs, "frac": step_gbs / peak,
                 "algorithmic_bytes": elems * (FWD_BYTES + BWD_BYTES)},
    }
    # dram__bytes_read.sum + dram__bytes_write.sum of one backward launch at config 1, from the ncu capture
    # summarised in profiles/lti_scan_config1_dram_traffic.md (1.608 GB for 67.1 M elements), scaled by elements.
    roofline["traffic"] = BWD_DRAM_BYTES_PER_ELEM * elems
    roofline["traffic_source"] = "ncu dram__bytes_read.sum+dram__bytes_write.sum, profiles/lti_scan_config1_dram_traffic.md"

    cpu_baseline = None
    if world == 1 and not args.no_cpu_baseline:
        val, desc = time_reference_cpu(args, min_seconds=10.0, max_steps=20, warmup=1)
        if val is not None:
            cpu_baseline = {"value": val, "unit": UNIT, "cores": desc["cores"], "kind": desc["kind"],
                            "sample": desc["sample"]}
        else:
            cpu_baseline = {"value": None, "unit": UNIT, "cores": os.cpu_count(), "kind": "reference",
                            "sample": "unavailable: " + desc}

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload_name(args), "variant": variant, "batch": B, "length": L,
                   "ssm_per_gpu": P, "sharding": f"oscillators split over {world} GPU(s), no collective",
                   "l2": "inputs (2 x %d MB) larger than L2, no flush" % (elems * 8 // 2**20)},
        "roofline": roofline, "cpu_baseline": cpu_baseline, "e2e": e2e,
        # forward, backward and the coefficient-gradient reduction per step
        "gpu_launches": 3 * args.steps, "clocks": clocks,
        "kernel_ms": {"forward": fwd_ms, "backward": bwd_ms},
    }
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def run_secondary(args):
    """Side workloads (single GPU, kernels only): BASELINE config 2 and config 3.  Same
    timing rules as the headline; one JSON line with its own metric name."""
    import torch

    from ossm_b200 import _lib, kernels

    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device")
    dev = torch.device("cuda", 0)
    gen = torch.Generator(device=dev).manual_seed(0)
    if args.workload == "linoss":
        L, B, P = (args.side_length or 16384), (args.side_batch or 128), 128
        a = torch.relu(torch.randn(P, generator=gen, device=dev))
        dt = torch.sigmoid(torch.randn(P, generator=gen, device=dev))
        bu = torch.view_as_complex(torch.randn(L, B, P, 2, generator=gen, device=dev) * 0.5)
        gx = torch.view_as_complex(torch.randn(L, B, P, 2, generator=gen, device=dev))
        elems, fb, bb = L * B * P, FWD_BYTES, BWD_BYTES
        name = f"LinOSS-IM scan fwd+bwd, B={B} L={L} P={P}, complex64 (BASELINE config 2)"
        metric = "linoss_scan_fwd_bwd_gelem_per_s"

        def fwd():
            return kernels.lti_scan_forward("linoss_im", a, None, dt, bu)

        def bwd(saved):
            return kernels.lti_scan_backward("linoss_im", a, None, dt, bu, saved[2], gx)
    elif args.workload == "lru":
        # complex diagonal scan of the LRU / S5 layers at the headline shape: x_t = lambda x_{t-1} + b_t
        L, B, P = args.length, (args.side_batch or 64), args.ssm
        mag = torch.rand(P, generator=gen, device=dev) * 0.5 + 0.45
        ph = torch.rand(P, generator=gen, device=dev) * 6.28
        lam_re, lam_im = (mag * torch.cos(ph)).contiguous(), (mag * torch.sin(ph)).contiguous()
        bu = torch.view_as_complex(torch.randn(L, B, P, 2, generator=gen, device=dev) * 0.5)
        gx = torch.view_as_complex(torch.randn(L, B, P, 2, generator=gen, device=dev))
        elems, fb, bb = L * B * P, FWD_BYTES, BWD_BYTES
        name = f"LRU / S5 complex diagonal scan fwd+bwd, B={B} L={L} P={P}, complex64"
        metric = "diag_scan_fwd_bwd_gelem_per_s"

        def fwd():
            return kernels.diag_scan_forward(lam_re, lam_im, bu)

        def bwd(saved):
            return kernels.diag_scan_backward(lam_re, lam_im, bu, saved[1], gx)
    elif args.workload == "sdlinoss":
        # selective D-LinOSS at the headline shape: per-step a, g, dt fields [L,B,M] from a slowly varying pole
        # field (the layer's map, sdlinoss.py:186-204)
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
        bu = torch.view_as_complex(torch.randn(L, B, P, 2, generator=gen, device=dev) * 0.5)
        gx = torch.view_as_complex(torch.randn(L, B, P, 2, generator=gen, device=dev))
        # forward: a, g, dt 12 B + bu 8 -> x 8 ; backward: 12 + bu 8 + grad_x 8 -> grad_bu 8 + three gradients 12
        elems, fb, bb = L * B * P, 28, 48
        name = f"selective D-LinOSS imex1 scan fwd+bwd, B={B} L={L} M={P}, dense per-step coefficients, complex64"
        metric = "sdlinoss_scan_fwd_bwd_gelem_per_s"

        def fwd():
            return kernels.sdlinoss_scan_forward("imex1", Af, Gf, dtf, bu)

        def bwd(saved):
            return kernels.sdlinoss_scan_backward("imex1", Af, Gf, dtf, bu, gx, carries=saved[2])
    else:
        Bz, Dn, L, N = (args.side_batch or 32), 2048, (args.side_length or 8192), 16
        io = torch.bfloat16
        u = torch.randn(Bz, Dn, L, generator=gen, device=dev).to(io)
        z = torch.randn(Bz, Dn, L, generator=gen, device=dev).to(io)
        delta = torch.nn.functional.softplus(torch.randn(Bz, Dn, L, generator=gen, device=dev) - 4)
        A = -torch.arange(1, N + 1, device=dev, dtype=torch.float32).repeat(Dn, 1)
        Bt = torch.randn(Bz, N, L, generator=gen, device=dev).to(io)      # given time-contiguous [B, N, L]
        Ct = torch.randn(Bz, N, L, generator=gen, device=dev).to(io)
        Dv = torch.ones(Dn, device=dev)
        go = torch.randn(Bz, Dn, L, generator=gen, device=dev).to(io)
        elems, fb, bb = Bz * Dn * L, 10, 18      # u 2 + delta 4 + z 2 -> out 2 ; + dout 2 -> du 2, ddelta 4, dz 2
        name = f"Mamba selective scan fwd+bwd, B={Bz} D={Dn} L={L} N={N}, bf16 I/O, fp32 state (BASELINE config 3)"
        metric = "selective_scan_fwd_bwd_gelem_per_s"

        def fwd():
            return kernels.selective_scan_fwd(u, delta, A, Bt.transpose(1, 2), Ct.transpose(1, 2), z, Dv)

        def bwd(saved):
            return kernels.selective_scan_bwd(go, u, delta, A, Bt.transpose(1, 2), Ct.transpose(1, 2), z, saved[1], Dv)

    for _ in range(max(args.warmup, 3)):
        bwd(fwd())
    torch.cuda.synchronize()
    evs = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(args.steps)]
    for e in evs:
        e[0].record()
        saved = fwd()
        e[1].record()
        bwd(saved)
        e[2].record()
    torch.cuda.synchronize()
    if _lib.device_status() != 0:
        raise SystemExit("bench.py: device status non-zero")
    fwd_ms = statistics.mean(e[0].elapsed_time(e[1]) for e in evs)
    bwd_ms = statistics.mean(e[1].elapsed_time(e[2]) for e in evs)
    ms = evs[0][0].elapsed_time(evs[-1][2]) / args.steps
    try:
        peak = float(json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["hbm_gbs"])
    except Exception:
        peak = 6650.0
    gbs = elems * (fb + bb) / (ms * 1e-3) / 1e9
    print(json.dumps({
        "metric": metric, "value": elems / (ms * 1e-3) / 1e9, "unit": UNIT, "n_gpus": 1, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "data": "synthetic",
        "config": {"workload": name}, "kernel_ms": {"forward": fwd_ms, "backward": bwd_ms},
        "roofline": {"bound": "hbm", "achieved": gbs, "peak": peak, "unit": "GB/s", "frac": gbs / peak,
                     "algorithmic_bytes_per_elem": fb + bb}}))


def run_sharded_layer(args):
    """BASELINE config 4: D-LinOSS layer forward + backward with the oscillators split over
    the ranks and the partial outputs summed over NVLink (ossm_b200.sharded_layer)."""
    import torch
    import torch.distributed as dist

    from ossm_b200 import _lib
    from ossm_b200.sharded_layer import sharded_dlinoss_layer
    from ossm_b200.sharding import aggregate_throughput, shard_channels

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    Bz, H, P = 8, 512, 2048
    L = 32768 if args.length == 4096 else args.length
    per_rank_gb = Bz * L * (P // world) * 8 * 8 / 2**30 + Bz * L * H * 4 * 6 / 2**30
    if per_rank_gb > 120:
        raise SystemExit(f"bench.py: sharded_layer would need ~{per_rank_gb:.0f} GB per GPU; lower --length")
    gen = torch.Generator().manual_seed(0)
    a, g, dt = make_params(P, "cpu", 0)
    bound = 1.0 / H ** 0.5
    full = dict(a=a, g=g, step=dt,
                B_re=torch.empty(P, H).uniform_(-bound, bound, generator=gen),
                B_im=torch.empty(P, H).uniform_(-bound, bound, generator=gen),
                C_re=torch.empty(H, P).uniform_(-bound, bound, generator=gen),
                C_im=torch.empty(H, P).uniform_(-bound, bound, generator=gen))
    dims = dict(a=0, g=0, step=0, B_re=0, B_im=0, C_re=1, C_im=1)
    loc = {k: shard_channels(v, world, rank, dim=dims[k]).to(dev).requires_grad_(True) for k, v in full.items()}
    Dv = torch.randn(H, generator=gen).to(dev).requires_grad_(True)
    u = torch.randn(Bz, L, H, generator=gen).to(dev).requires_grad_(True)
    dy = torch.randn(Bz, L, H, generator=gen).to(dev)

    def step():
        for t in list(loc.values()) + [Dv, u]:
            t.grad = None
        y = sharded_dlinoss_layer("imex1", loc["a"], loc["g"], loc["step"], loc["B_re"], loc["B_im"], loc["C_re"],
                                  loc["C_im"], Dv, u, slices=4)
        y.backward(dy)

    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
        torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    elems_local = Bz * L * loc["a"].numel()
    total, ms = aggregate_throughput(elems_local, e0.elapsed_time(e1), dev)
    if _lib.device_status() != 0:
        raise SystemExit("bench.py: device status non-zero")
    if rank == 0:
        ms /= args.steps
        print(json.dumps({
            "metric": "dlinoss_layer_sharded_fwd_bwd_gelem_per_s", "value": total / (ms * 1e-3) / 1e9, "unit": UNIT,
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms,
            "higher_is_better": True, "scaling": "strong", "data": "synthetic",
            "config": {"workload": f"D-LinOSS imex1 layer fwd+bwd, B={Bz} L={L} H={H} P={P} split over {world} GPU(s), "
                                   "partial outputs summed with NCCL (BASELINE config 4, reduced L)",
                       "projections": "torch.matmul fp32 (library GEMM)"}}))
    if world > 1:
        dist.destroy_process_group()


def main():
    args = parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
    elif args.workload == "sharded_layer":
        run_sharded_layer(args)
    elif args.workload != "dlinoss":
        run_secondary(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
