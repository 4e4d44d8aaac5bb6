"""CPU: the multi-rank path of the benchmark (contiguous batch shards, waves, max/sum reduction)
with world_size 2 over gloo."""
import os
import socket

import pytest

from lumi_b200 import shard


def test_shard_range_covers_everything():
    for total in (1, 7, 64, 4096):
        for world in (1, 2, 3, 8):
            spans = [shard.shard_range(total, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == total
            assert all(spans[i][1] == spans[i + 1][0] for i in range(world - 1))
            sizes = [hi - lo for lo, hi in spans]
            assert max(sizes) - min(sizes) <= 1


def test_waves():
    assert shard.waves(4096, 2048) == [(0, 2048), (2048, 4096)]
    assert shard.waves(512, 2048) == [(0, 512)]
    w = shard.waves(4096, 1500)
    assert len(w) == 3 and w[0][0] == 0 and w[-1][1] == 4096 and all(hi - lo <= 1500 for lo, hi in w)


def _worker(rank, world, port, q):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    lo, hi = shard.shard_range(101, rank, world)
    dist.barrier()
    tmax, units = shard.reduce_max_sum(dist, 10.0 + rank, float(hi - lo))
    q.put((rank, lo, hi, tmax, units))
    dist.destroy_process_group()


def test_two_ranks_gloo():
    import torch.multiprocessing as mp
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert res[0][1:3] == (0, 51) and res[1][1:3] == (51, 101)
    assert all(r[3] == 11.0 and r[4] == 101.0 for r in res)      # max over ranks, sum of units
