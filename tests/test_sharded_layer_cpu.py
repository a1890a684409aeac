"""Oscillator-sharded D-LinOSS layer on two gloo ranks (CPU) against the
single-process layer: output, input gradient and every parameter gradient, for the
reduce-scatter form (output sharded over the hidden dimension, chunked in time) and the
all-reduce form.  The scan and the projections are injected (a plain PyTorch time loop and
``torch.matmul`` stand in for the CUDA kernels, which have no CPU path), so this covers the
sharding logic and the collectives."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def torch_scan(variant, a, g, step, bu):
    """imex1 recurrence as a differentiable PyTorch loop (_dlinoss_scan.py:54-68)."""
    assert variant == "imex1"
    inv = 1.0 / (1.0 + step * g)
    s2i = step * step * inv
    w = torch.zeros_like(bu[0])
    x = torch.zeros_like(bu[0])
    out = []
    for t in range(bu.size(0)):
        w = w * inv + x * (-a * s2i) + bu[t] * s2i
        x = x + w
        out.append(x)
    return torch.stack(out, 0)


def make_problem():
    gen = torch.Generator().manual_seed(3)
    Bz, L, H, P = 2, 9, 6, 6
    p = dict(a=torch.rand(P, generator=gen), g=torch.rand(P, generator=gen) * 0.4,
             step=torch.sigmoid(torch.randn(P, generator=gen)),
             B=torch.randn(P, H, 2, generator=gen) * 0.4, C=torch.randn(H, P, 2, generator=gen) * 0.4,
             D=torch.randn(H, generator=gen))
    u = torch.randn(Bz, L, H, generator=gen)
    dy = torch.randn(Bz, L, H, generator=gen)
    return p, u, dy


SHARD_DIM = dict(a=0, g=0, step=0, B=0, C=1)


def reference_layer(p, u):
    """Single-process layer body (dlinoss.py:217-247) in plain PyTorch."""
    bsz, L, H = u.shape
    flat = u.reshape(bsz * L, H)
    bu = torch.complex(flat @ p["B"][..., 0].t(), flat @ p["B"][..., 1].t()).reshape(bsz, L, -1)
    x = torch_scan("imex1", p["a"], p["g"], p["step"], bu.permute(1, 0, 2)).permute(1, 0, 2).reshape(bsz * L, -1)
    return (x.real @ p["C"][..., 0].t() - x.imag @ p["C"][..., 1].t()).reshape(bsz, L, H) + u * p["D"]


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from ossm_b200.sharded_layer import hidden_shard, sharded_dlinoss_layer
        from ossm_b200.sharding import gather_channels, shard_channels

        params, u, dy = make_problem()
        full = {k: v.clone().requires_grad_(True) for k, v in params.items()}
        u_full = u.clone().requires_grad_(True)
        y_ref = reference_layer(full, u_full)
        y_ref.backward(dy)
        P, H = params["a"].numel(), u.size(-1)
        for scatter in (True, False):
            loc = {k: (shard_channels(v, world, rank, dim=SHARD_DIM[k]) if k in SHARD_DIM else v.clone())
                   for k, v in params.items()}
            cols = hidden_shard(H) if scatter else slice(0, H)
            loc["D"] = params["D"][cols].clone()
            loc = {k: v.requires_grad_(True) for k, v in loc.items()}
            u_loc = u.clone().requires_grad_(True)
            y = sharded_dlinoss_layer("imex1", loc["a"], loc["g"], loc["step"], loc["B"], loc["C"], loc["D"], u_loc,
                                      scan=torch_scan, chunks=2, scatter_output=scatter, use_kernels=False)
            assert y.shape == (u.size(0), u.size(1), H // world if scatter else H)
            y.backward(dy[..., cols])
            torch.testing.assert_close(y, y_ref[..., cols].detach(), rtol=1e-5, atol=1e-5)
            torch.testing.assert_close(u_loc.grad, u_full.grad, rtol=1e-5, atol=1e-5)
            torch.testing.assert_close(loc["D"].grad, full["D"].grad[cols], rtol=1e-5, atol=1e-5)
            for k, dim in SHARD_DIM.items():
                grad = loc[k].grad
                if grad.dim() == 3:         # [P_r, H, 2] / [H, P_r, 2]: gather along the oscillator axis
                    parts = [gather_channels(grad[..., c].movedim(dim, -1).contiguous(), P).movedim(-1, dim)
                             for c in (0, 1)]
                    got = torch.stack(parts, -1)
                else:
                    got = gather_channels(grad.contiguous(), P)
                torch.testing.assert_close(got, full[k].grad, rtol=1e-5, atol=1e-5, msg=f"{k} scatter={scatter}")
        out.put((rank, "ok"))
    except Exception:                                       # pragma: no cover
        import traceback

        out.put((rank, traceback.format_exc()))
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(180)
def test_sharded_layer_matches_single_process():
    world = 2
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, out)) for r in range(world)]
    for p in procs:
        p.start()
    results = [out.get(timeout=150) for _ in procs]
    for p in procs:
        p.join(timeout=30)
    assert sorted(results) == [(0, "ok"), (1, "ok")], results


def test_single_process_without_a_process_group():
    """world = 1: the same function is the plain layer (no collective is issued)."""
    from ossm_b200.sharded_layer import sharded_dlinoss_layer

    params, u, dy = make_problem()
    y = sharded_dlinoss_layer("imex1", params["a"], params["g"], params["step"], params["B"], params["C"], params["D"],
                              u, scan=torch_scan, chunks=3, use_kernels=False)
    torch.testing.assert_close(y, reference_layer(params, u), rtol=1e-5, atol=1e-5)
