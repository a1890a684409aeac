"""Channel-sharded selective scan on two gloo ranks (CPU) against the unsharded scan: outputs and all
gradients, including the all-reduced dB / dC.  A differentiable PyTorch loop stands in for the CUDA op
(which has no CPU path), so this covers the sharding and the collective."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def torch_scan(u, dt, A, Bm, Cm, gate=None, D=None):
    """h = exp(dt A) h + dt B u ; y = <C, h> (+ D u) ; out = y silu(gate)  (mambarec.py:23-61)."""
    Bz, Dn, L = u.shape
    h = torch.zeros(Bz, Dn, A.size(1), dtype=u.dtype)
    ys = []
    for t in range(L):
        h = torch.exp(dt[:, :, t, None] * A[None]) * h + dt[:, :, t, None] * Bm[:, None, t, :] * u[:, :, t, None]
        ys.append((h * Cm[:, None, t, :]).sum(-1))
    y = torch.stack(ys, -1)
    if D is not None:
        y = y + D[None, :, None] * u
    return y if gate is None else y * torch.nn.functional.silu(gate)


def make_problem():
    gen = torch.Generator().manual_seed(4)
    Bz, Dn, L, N = 2, 6, 11, 4
    return dict(u=torch.randn(Bz, Dn, L, generator=gen), dt=torch.rand(Bz, Dn, L, generator=gen) * 0.3,
                A=-torch.exp(torch.randn(Dn, N, generator=gen)), B=torch.randn(Bz, L, N, generator=gen),
                C=torch.randn(Bz, L, N, generator=gen), gate=torch.randn(Bz, Dn, L, generator=gen),
                D=torch.randn(Dn, generator=gen)), torch.randn(Bz, Dn, L, generator=gen)


CH_DIM = dict(u=1, dt=1, A=0, gate=1, D=0)     # channel axis of the sharded operands


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
        from ossm_b200.sharded_selective_scan import sharded_selective_scan
        from ossm_b200.sharding import shard_range

        prob, go = make_problem()
        full = {k: v.double().requires_grad_(True) for k, v in prob.items()}
        ref = torch_scan(full["u"], full["dt"], full["A"], full["B"], full["C"], full["gate"], full["D"])
        ref.backward(go.double())

        Dn = prob["A"].size(0)
        lo, hi = shard_range(Dn, world, rank)
        loc = {k: (v.double().narrow(CH_DIM[k], lo, hi - lo).clone() if k in CH_DIM else v.double().clone())
               .requires_grad_(True) for k, v in prob.items()}
        y = sharded_selective_scan(loc["u"], loc["dt"], loc["A"], loc["B"], loc["C"], loc["gate"], loc["D"],
                                   scan=torch_scan)
        y.backward(go.double().narrow(1, lo, hi - lo))
        torch.testing.assert_close(y, ref.narrow(1, lo, hi - lo), rtol=1e-12, atol=1e-12)
        for k, dim in CH_DIM.items():
            torch.testing.assert_close(loc[k].grad, full[k].grad.narrow(dim, lo, hi - lo), rtol=1e-10, atol=1e-10,
                                       msg=k)
        for k in ("B", "C"):        # summed over the ranks by the collective
            torch.testing.assert_close(loc[k].grad, full[k].grad, rtol=1e-10, atol=1e-10, msg=k)
        out.put((rank, "ok"))
    except Exception:                                       # pragma: no cover
        import traceback

        out.put((rank, traceback.format_exc()))
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(180)
def test_sharded_selective_scan_matches_single_process():
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
