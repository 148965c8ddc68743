"""The forward as its own all-gather, on two GPUs of one node (skipped where fewer are visible): every rank runs its
slice of the (batch x head) units and its kernel writes the result into both ranks' full-size buffers
(`sharding.GatheredOutput`, `sla_fwd_gather`: plain stores to the peer's memory mapped with CUDA IPC). Afterwards
every rank must hold, bit for bit, what an unsharded forward of all units gives. NCCL runs without NVLS; nothing
here binds memory to a multicast object. The single-GPU form of the same kernel path is
tests/test_attention_gpu.py::test_forward_writes_its_output_to_gather_destinations."""
import os
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, n_units, L, D, quantized):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    import sla_b200
    from sla_b200 import sharding
    dev = torch.device("cuda", rank)
    g = torch.Generator().manual_seed(123)
    q, k, v = (torch.randn(1, n_units, L, D, generator=g).bfloat16().to(dev) for _ in range(3))
    m = (sla_b200.SageSparseLinearAttention(D, 0.2) if quantized else sla_b200.SparseLinearAttention(D, 0.2)).to(dev)
    with torch.no_grad():
        m.proj_l.weight.copy_((torch.randn(D, D, generator=g) * 0.05).to(dev))
        m.proj_l.bias.copy_((torch.randn(D, generator=g) * 0.05).to(dev))
        ref = m(q, k, v)[0]                                  # all units on this GPU
        lo, hi = sharding.unit_range(n_units, rank, world)
        out = sharding.GatheredOutput(n_units, L, D, torch.bfloat16, dev)
        out.full.fill_(-3.0)
        dist.barrier()
        o = m(q[:, lo:hi].contiguous(), k[:, lo:hi].contiguous(), v[:, lo:hi].contiguous(), gather=out)
        out.wait()
    assert torch.equal(o[0], ref[lo:hi]), "the local slice differs from the unsharded forward"
    assert torch.equal(out.full, ref), f"rank {rank}: the gathered buffer differs from the unsharded forward"
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("n_units,quantized", [(4, False), (3, False), (3, True)])
def test_forward_is_its_own_all_gather_on_two_gpus(n_units, quantized):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    mp.spawn(_worker, args=(2, 29650 + n_units + 10 * quantized, n_units, 1500, 128, quantized), nprocs=2, join=True)
