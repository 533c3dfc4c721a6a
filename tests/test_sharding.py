"""The multi-GPU host logic on CPU: units dealt over ranks, time reduced with MAX, coordinates
gathered in unit order. Two gloo ranks stand in for two GPUs; a deterministic function of the seed
stands in for the fold."""
import os
import socket
import sys

import numpy as np
import pytest

from mkharness import shard


def test_deal_units_partitions():
    for n, w in [(8, 1), (8, 2), (8, 4), (8, 8), (5, 2), (3, 4)]:
        seen = sorted(u for r in range(w) for u in shard.deal_units(n, r, w))
        assert seen == list(range(n))
        sizes = [len(shard.deal_units(n, r, w)) for r in range(w)]
        assert max(sizes) - min(sizes) <= 1


def fake_fold(seed):
    rng = np.random.default_rng(seed)
    return rng.standard_normal((2, 48, 3)).astype(np.float32), 10.0 + seed % 7


def test_single_process_gather():
    units = shard.deal_units(3, 0, 1)
    local, ms = shard.fold_units(fake_fold, units, 100)
    out, t = shard.gather(local, ms, 3, 0, 1)
    assert t == ms and all((out[u] == fake_fold(100 + u)[0]).all() for u in range(3))


def _worker(rank, world, port, n_units, q):
    import torch.distributed as dist

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    local, ms = shard.fold_units(fake_fold, shard.deal_units(n_units, rank, world), 100)
    out, t = shard.gather(local, ms, n_units, rank, world, dist)
    ok = all((out[u].reshape(2, 48, 3) == fake_fold(100 + u)[0]).all() for u in range(n_units))
    q.put((rank, ok, t, ms))
    dist.destroy_process_group()


@pytest.mark.parametrize("n_units", [2, 5])
def test_two_ranks_gloo(n_units):
    import torch.multiprocessing as mp

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, n_units, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert all(ok for _, ok, _, _ in res)
    assert res[0][2] == res[1][2] == max(r[3] for r in res)  # MAX over ranks of the local time
