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


class GatheredOutput:
    """A full-size output buffer (n_units, L, D) on every rank of a (batch x head)-sharded run, which the forward
    kernel of each rank fills directly: its own slice through the ordinary store, the same slice in every peer GPU's
    buffer through plain stores over NVLink issued from the kernel's epilogue (`sla_fwd_gather`). It replaces
    `all_gather_units` after the forward: when every rank's forward has completed (`wait()`), `full` holds all units.

    The peers' buffers are mapped with CUDA IPC (every rank of the node must see every GPU, as under torchrun);
    nothing is bound to an NVLink multicast object. Construction is collective over `group`.
    """

    def __init__(self, n_units: int, L: int, D: int, dtype: torch.dtype, device, group: Optional[dist.ProcessGroup] = None):
        import ctypes as C
        from ._lib import check, lib
        self._lib = lib
        self.group = group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.n_units, self.L, self.D = n_units, L, D
        self.lo, self.hi = unit_range(n_units, self.rank, self.world)
        self.full = torch.empty((n_units, L, D), dtype=dtype, device=device)
        # export: the IPC handle of the allocation that holds `full`, and where `full` starts inside it
        hbuf, off_c = C.create_string_buffer(64), C.c_size_t(0)
        with torch.cuda.device(self.full.device):
            check(lib.sla_ipc_export(self.full.data_ptr(), hbuf, C.byref(off_c)))
        handle, offset = hbuf.raw, int(off_c.value)
        handles = [None] * self.world
        dist.all_gather_object(handles, (self.rank, handle, offset), group=group)
        self._peers = []          # (rank, mapped base address, address of that rank's `full`)
        with torch.cuda.device(self.full.device):      # mapped for THIS rank's GPU, whose kernels write there
            for r, h, off in handles:
                if r == self.rank:
                    continue
                base = C.c_void_p()
                check(lib.sla_ipc_open(h, C.byref(base)))
                self._peers.append((r, base.value, base.value + off))
        dist.barrier(group=group)

    def close(self) -> None:
        """Unmap the peers' buffers (collective in effect: no rank may still be writing them)."""
        with torch.cuda.device(self.full.device):
            for _, base, _ in self._peers:
                self._lib.sla_ipc_close(base)
        self._peers = []

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def local_view(self, shape) -> torch.Tensor:
        """This rank's slice of `full`, shaped like the operator's output (1, U, L, D)."""
        if tuple(shape) != (1, self.hi - self.lo, self.L, self.D):
            raise ValueError(f"expected this rank's units as (1, {self.hi - self.lo}, {self.L}, {self.D})")
        return self.full[self.lo:self.hi].view(1, self.hi - self.lo, self.L, self.D)

    def peer_pointers(self) -> List[int]:
        """Address, in this process, of this rank's slice inside every peer's buffer."""
        off = self.lo * self.L * self.D * self.full.element_size()
        return [addr + off for _, _, addr in self._peers]

    def wait(self) -> None:
        """Every rank's forward has completed and its stores have landed: `full` is whole on every rank."""
        torch.cuda.current_stream(self.full.device).synchronize()
        dist.barrier(group=self.group)
