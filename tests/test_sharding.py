"""CPU suite: the scan-sharding helpers, with the N>1 path exercised by two gloo ranks."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from torchsparse_b200.sharding import (PaddedGather, balanced_assignment, gather_rows, gather_rows_padded,
                                       shard_range)


def test_shard_range_covers_everything_once():
    for n in (0, 1, 7, 32, 33):
        for world in (1, 2, 3, 8):
            seen = []
            for r in range(world):
                lo, hi = shard_range(n, world, r)
                assert 0 <= lo <= hi <= n
                seen += list(range(lo, hi))
            assert seen == list(range(n))
            sizes = [shard_range(n, world, r)[1] - shard_range(n, world, r)[0] for r in range(world)]
            assert max(sizes) - min(sizes) <= 1


def test_balanced_assignment():
    sizes = [100, 90, 80, 10, 10, 10, 5, 5]
    parts = balanced_assignment(sizes, 3)
    assert sorted(i for p in parts for i in p) == list(range(8))
    loads = [sum(sizes[i] for i in p) for p in parts]
    assert max(loads) - min(loads) <= 20
    assert balanced_assignment(sizes, 3) == parts          # deterministic


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rows = 3 + 2 * rank                                  # a different row count on every rank
        local = torch.arange(rows * 4, dtype=torch.float32).reshape(rows, 4) + 1000 * rank
        out, counts = gather_rows(local)
        lo, hi = shard_range(10, world, rank)
        q.put((rank, out.clone(), counts, (lo, hi)))
        # an empty shard on one rank must not break the gather
        local2 = torch.zeros((0 if rank == 0 else 2, 4))
        out2, counts2 = gather_rows(local2)
        q.put((rank, out2.clone(), counts2, None))
        # the variant with a known row bound: same rows, counts stay a tensor, no host read inside
        buf, cnt = gather_rows_padded(local, 8)
        q.put((rank, buf.clone(), cnt.tolist(), "padded"))
        # the same with buffers kept between calls: two calls with different row counts
        pg = PaddedGather(8, 4, torch.float32, "cpu")
        pg(local[:2])
        buf, cnt = pg(local)
        q.put((rank, buf.clone(), cnt.tolist(), "padded"))
    finally:
        dist.destroy_process_group()


def test_gather_rows_two_gloo_ranks():
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in range(4 * world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    padded = [r for r in results if r[3] == "padded"]
    results = [r for r in results if r[3] != "padded"]
    first = [r for r in results if r[3] is not None]
    second = [r for r in results if r[3] is None]
    expect = torch.cat([torch.arange(12, dtype=torch.float32).reshape(3, 4),
                        torch.arange(20, dtype=torch.float32).reshape(5, 4) + 1000])
    for rank, out, counts, rng in first:
        assert counts == [3, 5]
        assert torch.equal(out, expect)
        assert rng == ((0, 5) if rank == 0 else (5, 10))
    for rank, out, counts, _ in second:
        assert counts == [0, 2] and out.shape == (2, 4)
    assert len(padded) == 2 * world
    for rank, buf, counts, _ in padded:
        assert counts == [3, 5] and buf.shape == (2, 8, 4)
        assert torch.equal(torch.cat([buf[0, :3], buf[1, :5]]), expect)
