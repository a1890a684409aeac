"""Oscillator-sharded D-LinOSS layer on two GPUs (NCCL) with the CUDA scan,
against the same layer on one GPU.  Needs two devices; skipped otherwise."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu

SHARD_DIM = dict(a=0, g=0, step=0, B_re=0, B_im=0, C_re=1, C_im=1)


def make_problem():
    gen = torch.Generator().manual_seed(5)
    Bz, L, H, P = 3, 130, 16, 96
    p = dict(a=torch.rand(P, generator=gen) * 0.8, g=torch.rand(P, generator=gen) * 0.4,
             step=torch.sigmoid(torch.randn(P, generator=gen)),
             B_re=torch.randn(P, H, generator=gen) * 0.2, B_im=torch.randn(P, H, generator=gen) * 0.2,
             C_re=torch.randn(H, P, generator=gen) * 0.2, C_im=torch.randn(H, P, generator=gen) * 0.2,
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
        # single-GPU reference: same function, every oscillator on this rank, no collective
        from ossm_b200.dlinoss import run_dlinoss

        bsz, L, H = u.shape
        flat = u_full.reshape(bsz * L, H)
        bu = torch.complex(flat @ full["B_re"].t(), flat @ full["B_im"].t()).reshape(bsz, L, -1)
        x = run_dlinoss("imex1", full["a"], full["g"], full["step"], bu.permute(1, 0, 2).contiguous())
        xf = x.permute(1, 0, 2).reshape(bsz * L, -1)
        y_ref = (xf.real @ full["C_re"].t() - xf.imag @ full["C_im"].t()).reshape(bsz, L, H) + u_full * full["D"]
        y_ref.backward(dy.to(dev))

        loc = {k: (shard_channels(v.to(dev), world, rank, dim=SHARD_DIM[k]) if k in SHARD_DIM else v.to(dev))
               .requires_grad_(True) for k, v in params.items()}
        u_loc = u.to(dev).requires_grad_(True)
        y = sharded_dlinoss_layer("imex1", loc["a"], loc["g"], loc["step"], loc["B_re"], loc["B_im"], loc["C_re"],
                                  loc["C_im"], loc["D"], u_loc, slices=2)
        y.backward(dy.to(dev))
        torch.testing.assert_close(y, y_ref, rtol=2e-5, atol=2e-5)
        torch.testing.assert_close(u_loc.grad, u_full.grad, rtol=2e-5, atol=2e-5)
        P = params["a"].numel()
        for k, dim in SHARD_DIM.items():
            got = gather_channels(loc[k].grad.movedim(dim, -1).contiguous(), P).movedim(-1, dim)
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
