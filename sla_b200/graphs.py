"""CUDA-graph capture of a module's forward and backward.

Every launch of this library goes to the caller's stream, or to a second stream that forks from it and joins it
again inside the same forward (the linear-branch state, next to the block map), and nothing synchronises (the top-k
count comes from the shapes, utils.py:61-62), so a whole forward + backward of ``SparseLinearAttention`` can be captured once and
replayed: about twenty kernel launches, the workspace allocations and the Python glue between them collapse into
two graph launches per step. That matters for short sequences, where the step is launch-bound.

    fast = graphed(module, q, k, v)      # q, k, v: sample inputs (requires_grad as in training)
    o = fast(q, k, v); o.backward(do)    # same results as module(q, k, v)

Inputs of later calls must have the sample's shapes, dtypes and requires_grad flags (a CUDA graph replays fixed
launches), exactly as for ``torch.cuda.make_graphed_callables``, which does the capture.
"""
from __future__ import annotations

import torch


def graphed(module: torch.nn.Module, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, warmup: int = 3):
    if not (q.is_cuda and k.is_cuda and v.is_cuda):
        raise RuntimeError("graphed() needs CUDA tensors")
    sample = tuple(t.detach().clone().requires_grad_(t.requires_grad) for t in (q, k, v))
    return torch.cuda.make_graphed_callables(module, sample, num_warmup_iters=warmup)
