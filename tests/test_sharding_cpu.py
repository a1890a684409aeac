"""Host-side logic of the multi-GPU path on two gloo ranks (CPU): shards
partition the oscillators, the gathered shards reproduce the single-device
tensor, and the benchmark aggregation is sum-of-units over max-of-time."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from ossm_b200.sharding import shard_range


def test_shard_ranges_partition():
    for total in (1, 7, 256, 2048, 2049):
        for world in (1, 2, 3, 8):
            spans = [shard_range(total, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == total
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [b - a for a, b in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard_range(8, 2, 2)


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
        from ossm_b200.sharding import aggregate_throughput, gather_channels, shard_channels

        gen = torch.Generator().manual_seed(0)             # same "global" tensors on every rank
        P = 11
        x_full = torch.complex(torch.randn(5, 3, P, generator=gen), torch.randn(5, 3, P, generator=gen))
        a_full = torch.randn(P, generator=gen)
        x_loc = shard_channels(x_full, world, rank)
        a_loc = shard_channels(a_full, world, rank)
        start, stop = shard_range(P, world, rank)
        assert x_loc.shape[-1] == stop - start and torch.equal(a_loc, a_full[start:stop])
        # stand-in for the per-shard scan: any per-channel map commutes with the sharding
        y_loc = x_loc * a_loc
        y_all = gather_channels(y_loc, P)
        assert torch.equal(torch.view_as_real(y_all), torch.view_as_real(x_full * a_full))
        r_all = gather_channels(a_loc, P)
        assert torch.equal(r_all, a_full)
        units, ms = aggregate_throughput(100 + rank, 2.0 + rank, torch.device("cpu"))
        assert units == sum(100 + r for r in range(world)) and ms == 2.0 + (world - 1)
        out.put((rank, "ok"))
    except Exception as exc:                                # pragma: no cover - reported to the parent
        out.put((rank, repr(exc)))
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(120)
def test_two_rank_gather_and_aggregate():
    world = 2
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, out)) for r in range(world)]
    for p in procs:
        p.start()
    results = [out.get(timeout=100) for _ in procs]
    for p in procs:
        p.join(timeout=30)
    assert sorted(results) == [(0, "ok"), (1, "ok")], results
