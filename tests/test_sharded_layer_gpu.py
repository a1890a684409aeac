"""Oscillator-sharded D-LinOSS layer on two GPUs (NCCL) with the CUDA scan and the tensor-core
projections, reduce-scatter and all-reduce forms, against the same layer on one GPU.  Needs two
devices; skipped otherwise (``bench.py --gpus N`` runs the same comparison before its timed region
and reports it under ``sharded_parity``)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu

SHARD_DIM = dict(a=0, g=0, step=0, B=0, C=1)


def make_problem():
    gen = torch.Generator().manual_seed(5)
    Bz, L, H, P = 3, 130, 16, 96
    p = dict(a=torch.rand(P, generator=gen) * 0.8, g=torch.rand(P, generator=gen) * 0.4,
             step=torch.sigmoid(torch.randn(P, generator=gen)),
             B=torch.randn(P, H, 2, generator=gen) * 0.2, C=torch.randn(H, P, 2, generator=gen) * 0.2,
             D=torch.randn(H, generator=gen))
    return p, torch.randn(Bz, L, H, generator=gen), torch.randn(Bz, L, H, generator=gen)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from ossm_b200.sharded_layer import sharded_dlinoss_layer
        from ossm_b200.sharding import gather_channels, shard_channels

        params, u, dy = make_problem()
        full = {k: v.to(dev).requires_grad_(True) for k, v in params.items()}
        u_full = u.to(dev).requires_grad_(True)
        # single-GPU reference: the unsharded layer op, every oscillator on this rank, no collective
        from ossm_b200.dlinoss_layer import dlinoss_layer
        from ossm_b200.sharded_layer import hidden_shard

        H = u.size(-1)
        y_ref = dlinoss_layer("imex1", full["a"], full["g"], full["step"], full["B"], full["C"], full["D"], u_full)
        y_ref.backward(dy.to(dev))
        P = params["a"].numel()
        for scatter in (True, False):
            cols = hidden_shard(H) if scatter else slice(0, H)
            loc = {k: (shard_channels(v.to(dev), world, rank, dim=SHARD_DIM[k]) if k in SHARD_DIM else v.to(dev))
                   for k, v in params.items()}
            loc["D"] = params["D"][cols].to(dev)
            loc = {k: v.requires_grad_(True) for k, v in loc.items()}
            u_loc = u.to(dev).requires_grad_(True)
            y = sharded_dlinoss_layer("imex1", loc["a"], loc["g"], loc["step"], loc["B"], loc["C"], loc["D"], u_loc,
                                      chunks=3, scatter_output=scatter)
            y.backward(dy.to(dev)[..., cols])
            torch.testing.assert_close(y, y_ref[..., cols].detach(), rtol=2e-5, atol=2e-5)
            torch.testing.assert_close(u_loc.grad, u_full.grad, rtol=2e-5, atol=2e-5)
            for k, dim in SHARD_DIM.items():
                grad = loc[k].grad
                if grad.dim() == 3:
                    got = torch.stack([gather_channels(grad[..., c].movedim(dim, -1).contiguous(), P).movedim(-1, dim)
                                       for c in (0, 1)], -1)
                else:
                    got = gather_channels(grad.contiguous(), P)
                torch.testing.assert_close(got, full[k].grad, rtol=1e-4, atol=1e-4, msg=k)
        out.put((rank, "ok"))
    except Exception:                                       # pragma: no cover
        import traceback

        out.put((rank, traceback.format_exc()))
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(300)
def test_sharded_layer_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    world = 2
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, out)) for r in range(world)]
    for p in procs:
        p.start()
    results = [out.get(timeout=240) for _ in procs]
    for p in procs:
        p.join(timeout=30)
    assert sorted(results) == [(0, "ok"), (1, "ok")], results
