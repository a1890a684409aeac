"""Channel-sharded selective scan on two GPUs (NCCL) with the CUDA scan, against the unsharded scan on
one GPU.  Needs two devices; skipped otherwise."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu
CH_DIM = dict(u=1, dt=1, A=0, gate=1, D=0)


def make_problem():
    gen = torch.Generator().manual_seed(8)
    Bz, Dn, L, N = 2, 96, 200, 16
    return dict(u=torch.randn(Bz, Dn, L, generator=gen), dt=torch.rand(Bz, Dn, L, generator=gen) * 0.05,
                A=-torch.exp(torch.randn(Dn, N, generator=gen)), B=torch.randn(Bz, L, N, generator=gen),
                C=torch.randn(Bz, L, N, generator=gen), gate=torch.randn(Bz, Dn, L, generator=gen),
                D=torch.randn(Dn, generator=gen)), torch.randn(Bz, Dn, L, generator=gen)


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
        from ossm_b200.selective_scan import selective_scan
        from ossm_b200.sharded_selective_scan import sharded_selective_scan
        from ossm_b200.sharding import shard_range

        prob, go = make_problem()
        full = {k: v.to(dev).requires_grad_(True) for k, v in prob.items()}
        ref = selective_scan(full["u"], full["dt"], full["A"], full["B"], full["C"], full["gate"], full["D"])
        ref.backward(go.to(dev))

        Dn = prob["A"].size(0)
        lo, hi = shard_range(Dn, world, rank)
        loc = {k: (v.to(dev).narrow(CH_DIM[k], lo, hi - lo).contiguous() if k in CH_DIM else v.to(dev).clone())
               .requires_grad_(True) for k, v in prob.items()}
        y = sharded_selective_scan(loc["u"], loc["dt"], loc["A"], loc["B"], loc["C"], loc["gate"], loc["D"])
        y.backward(go.to(dev).narrow(1, lo, hi - lo).contiguous())
        torch.testing.assert_close(y, ref.narrow(1, lo, hi - lo), rtol=1e-5, atol=1e-5)
        for k, dim in CH_DIM.items():
            torch.testing.assert_close(loc[k].grad, full[k].grad.narrow(dim, lo, hi - lo), rtol=1e-4, atol=1e-4,
                                       msg=k)
        for k in ("B", "C"):        # summed over the ranks by the all-reduce
            torch.testing.assert_close(loc[k].grad, full[k].grad, rtol=1e-4, atol=2e-4, msg=k)
        out.put((rank, "ok"))
    except Exception:                                       # pragma: no cover
        import traceback

        out.put((rank, traceback.format_exc()))
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(300)
def test_sharded_selective_scan_two_gpus():
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
