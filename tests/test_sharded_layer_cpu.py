"""Oscillator-sharded D-LinOSS layer on two gloo ranks (CPU) against the
single-process layer: output, input gradient and every parameter gradient.  The
scan is injected (a plain PyTorch time loop stands in for the CUDA op, which has
no CPU path), so this covers the sharding and the two collectives."""
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
    Bz, L, H, P = 2, 9, 5, 6
    p = dict(a=torch.rand(P, generator=gen), g=torch.rand(P, generator=gen) * 0.4,
             step=torch.sigmoid(torch.randn(P, generator=gen)),
             B_re=torch.randn(P, H, generator=gen) * 0.4, B_im=torch.randn(P, H, generator=gen) * 0.4,
             C_re=torch.randn(H, P, generator=gen) * 0.4, C_im=torch.randn(H, P, generator=gen) * 0.4,
             D=torch.randn(H, generator=gen))
    u = torch.randn(Bz, L, H, generator=gen)
    dy = torch.randn(Bz, L, H, generator=gen)
    return {k: v.double() for k, v in p.items()}, u.double(), dy.double()


SHARD_DIM = dict(a=0, g=0, step=0, B_re=0, B_im=0, C_re=1, C_im=1)


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
        from ossm_b200.sharded_layer import sharded_dlinoss_layer
        from ossm_b200.sharding import gather_channels, shard_channels

        params, u, dy = make_problem()
        full = {k: v.clone().requires_grad_(True) for k, v in params.items()}
        u_full = u.clone().requires_grad_(True)
        y_ref = sharded_dlinoss_layer("imex1", full["a"], full["g"], full["step"], full["B_re"], full["B_im"],
                                      full["C_re"], full["C_im"], full["D"], u_full, scan=torch_scan,
                                      group=dist.new_group([rank]))
        y_ref.backward(dy)

        loc = {k: (shard_channels(v, world, rank, dim=SHARD_DIM[k]) if k in SHARD_DIM else v.clone())
               .requires_grad_(True) for k, v in params.items()}
        u_loc = u.clone().requires_grad_(True)
        y = sharded_dlinoss_layer("imex1", loc["a"], loc["g"], loc["step"], loc["B_re"], loc["B_im"], loc["C_re"],
                                  loc["C_im"], loc["D"], u_loc, scan=torch_scan, slices=2)
        y.backward(dy)
        torch.testing.assert_close(y, y_ref, rtol=1e-10, atol=1e-10)
        torch.testing.assert_close(u_loc.grad, u_full.grad, rtol=1e-10, atol=1e-10)
        torch.testing.assert_close(loc["D"].grad, full["D"].grad, rtol=1e-10, atol=1e-10)
        P = params["a"].numel()
        for k, dim in SHARD_DIM.items():
            got = gather_channels(loc[k].grad.movedim(dim, -1).contiguous(), P).movedim(-1, dim)
            torch.testing.assert_close(got, full[k].grad, rtol=1e-10, atol=1e-10, msg=k)
        out.put((rank, "ok"))
    except Exception as exc:                                # pragma: no cover
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
