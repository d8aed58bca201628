"""Multi-GPU plumbing: the path shards by independent signal / channel, one process per GPU,
with no collective on the data path.  These helpers give every rank its contiguous share and
offer the optional final gather (NCCL on GPUs, gloo in CPU tests)."""
from __future__ import annotations

from typing import List, Tuple


def shard_range(n_units: int, rank: int, world: int, group: int = 1) -> Tuple[int, int]:
    """[lo, hi) of the units rank owns: contiguous ranges [g*n/G, (g+1)*n/G).  ``group`` keeps
    units that must stay together on one GPU (the two channels of an IR pair: group=2)."""
    if n_units % group != 0:
        raise ValueError("n_units must be a multiple of group")
    g = n_units // group
    lo = (rank * g) // world * group
    hi = ((rank + 1) * g) // world * group
    return lo, hi


def all_shards(n_units: int, world: int, group: int = 1) -> List[Tuple[int, int]]:
    return [shard_range(n_units, r, world, group) for r in range(world)]


def gather_rows(local, n_units: int, group: int = 1):
    """Optional final gather, outside any timed region: every rank contributes the rows of its
    shard (a torch tensor whose first dimension is its share) and receives the full set in
    unit order.  Uses the default process group (all_gather of padded shards)."""
    import torch
    import torch.distributed as dist
    world = dist.get_world_size()
    shards = all_shards(n_units, world, group)
    most = max(hi - lo for lo, hi in shards)
    pad = torch.zeros((most,) + tuple(local.shape[1:]), dtype=local.dtype, device=local.device)
    pad[: local.shape[0]] = local
    parts = [torch.empty_like(pad) for _ in range(world)]
    dist.all_gather(parts, pad)
    return torch.cat([parts[r][: hi - lo] for r, (lo, hi) in enumerate(shards)], dim=0)


def max_over_ranks(value: float, device=None) -> float:
    """Timing rule for multi-GPU numbers: the maximum over ranks."""
    import torch
    import torch.distributed as dist
    t = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())
