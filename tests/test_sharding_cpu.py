"""Host-side logic of the (batch x head) sharding on CPU ranks (gloo, world_size 2)."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_unit_range_partitions_everything():
    from sla_b200.sharding import unit_counts, unit_range
    for n in (1, 2, 12, 16, 40, 7):
        for world in (1, 2, 4, 8):
            spans = [unit_range(n, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            for a, b in zip(spans, spans[1:]):
                assert a[1] == b[0]
            c = unit_counts(n, world)
            assert sum(c) == n and max(c) - min(c) <= 1
    assert unit_counts(12, 8) == [2, 2, 2, 2, 1, 1, 1, 1]


def _worker(rank, world, port, n_units):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from sla_b200 import synthetic
    from sla_b200.sharding import all_gather_units, max_over_ranks, unit_range
    w = synthetic.WORKLOADS["tiny"]
    lo, hi = unit_range(n_units, rank, world)
    mine = torch.stack([synthetic.make_unit(w, u, "cpu")[0].float() for u in range(lo, hi)]) if hi > lo \
        else torch.zeros(0, w.L, w.D)
    full = all_gather_units(mine, n_units)
    ref = torch.stack([synthetic.make_unit(w, u, "cpu")[0].float() for u in range(n_units)])
    assert torch.equal(full, ref), "gathered units differ from the unsharded tensor"
    assert max_over_ranks(float(rank + 1), "cpu") == float(world)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("n_units", [2, 3])
def test_all_gather_of_head_shards_gloo(n_units):
    port = 29600 + n_units
    mp.spawn(_worker, args=(2, port, n_units), nprocs=2, join=True)


def test_units_are_identical_under_any_sharding():
    from sla_b200 import synthetic
    w = synthetic.WORKLOADS["tiny"]
    a = synthetic.make_inputs(w, "cpu", units=[0, 1])[0]
    b = synthetic.make_inputs(w, "cpu", units=[1])[0]
    assert torch.equal(a[0, 1], b[0, 0])
