"""(batch x head) sharding of the attention path over the GPUs of one node.

Every (b, h) unit is independent in all sub-steps of the path (the reference's grids are
(blocks, B*H): kernel.py:259,292,298,309; utils.py:50), so ranks own contiguous slices of the
flattened unit index and no collective is needed on the attention path. The only optional exchange
is an all-gather of the outputs, for callers that want the full (B, H, L, D) tensor on every rank.
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch
import torch.distributed as dist


def unit_range(n_units: int, rank: int, world: int) -> Tuple[int, int]:
    """Contiguous slice [lo, hi) of units owned by `rank`; the first n_units % world ranks get one more."""
    base, rem = divmod(n_units, world)
    lo = rank * base + min(rank, rem)
    return lo, lo + base + (1 if rank < rem else 0)


def unit_counts(n_units: int, world: int) -> List[int]:
    return [unit_range(n_units, r, world)[1] - unit_range(n_units, r, world)[0] for r in range(world)]


def all_gather_units(local: torch.Tensor, n_units: int, group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """Concatenate every rank's (U_r, L, D) slice along dim 0 into (n_units, L, D) on every rank.
    Uneven slices are padded to the largest one for the collective and trimmed afterwards."""
    world = dist.get_world_size(group)
    counts = unit_counts(n_units, world)
    umax = max(counts)
    pad = local
    if local.shape[0] < umax:
        pad = torch.cat([local, local.new_zeros((umax - local.shape[0],) + tuple(local.shape[1:]))])
    out = local.new_empty((world * umax,) + tuple(local.shape[1:]))
    dist.all_gather_into_tensor(out, pad.contiguous(), group=group)
    parts = [out[r * umax: r * umax + counts[r]] for r in range(world)]
    return torch.cat(parts, dim=0)


def max_over_ranks(value: float, device, group: Optional[dist.ProcessGroup] = None) -> float:
    if not (dist.is_available() and dist.is_initialized()):
        return value
    t = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())
