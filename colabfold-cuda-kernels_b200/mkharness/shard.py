"""Sharding of a sampling job over the GPUs of one node.

The unit of work is one (seed, S samples) fold: one launch of the persistent sampler kernel. Units
are independent (the Philox key is the seed, the counter carries only the sample index inside the
unit), so they are dealt to ranks with no data-path collective; the only exchanges are a MAX over
ranks of the device time and a gather of the final coordinates.
"""
import numpy as np


def deal_units(n_units, rank, world):
    """Indices of the units rank `rank` folds: round-robin, so every rank gets floor or ceil of n/world."""
    return list(range(rank, n_units, world))


def unit_seed(base_seed, unit):
    return int(base_seed) + int(unit)


def fold_units(fold, units, base_seed):
    """Runs `fold(seed) -> (positions ndarray, device ms)` for each unit; returns (dict unit -> positions, total ms)."""
    out, ms = {}, 0.0
    for u in units:
        pos, t = fold(unit_seed(base_seed, u))
        out[u] = np.asarray(pos, dtype=np.float32)
        ms += float(t)
    return out, ms


def gather(local, local_ms, n_units, rank, world, dist=None, device="cpu"):
    """Every rank gets all units' positions in unit order and the max over ranks of the device time.

    `dist` is torch.distributed (initialised) or None for a single process."""
    if world == 1 or dist is None:
        return [local[u] for u in range(n_units)], local_ms
    import torch

    t = torch.tensor([local_ms], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    size = next(iter(local.values())).size if local else 0
    sizes = torch.tensor([size], dtype=torch.int64, device=device)
    dist.all_reduce(sizes, op=dist.ReduceOp.MAX)
    size = int(sizes[0])
    per_rank = (n_units + world - 1) // world
    mine = torch.zeros(per_rank, size, dtype=torch.float32, device=device)
    for i, u in enumerate(deal_units(n_units, rank, world)):
        mine[i] = torch.from_numpy(local[u].ravel()).to(device)
    parts = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(parts, mine)
    out = [None] * n_units
    for r in range(world):
        for i, u in enumerate(deal_units(n_units, r, world)):
            out[u] = parts[r][i].cpu().numpy()
    return out, float(t[0])
