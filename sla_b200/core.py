"""Module level: the reference's two nn.Modules with unchanged constructor / forward signatures.

SparseLinearAttention      <- sparse_linear_attention/core.py:24-105
SageSparseLinearAttention  <- SageSLA/core.py:33-163

Parameters keep the reference's names, shapes and dtype (``proj_l.weight`` (D,D) fp32,
``proj_l.bias`` (D) fp32, zero-initialised), so reference checkpoints load unchanged.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from . import ops

_FEATURES = ("elu", "relu", "softmax")

# Forking to a second stream costs two cross-stream waits per forward (some tens of microseconds when the step is
# launch-bound) and gains the smaller of the two overlapped parts: measured on B200 it loses at 8 MB per tensor
# (0.150 vs 0.116 ms forward) and wins at 100 MB (0.624 vs 0.660 ms).
_OVERLAP_MIN_BYTES = 32 << 20


def _want_overlap(setting, k):
    if setting is None:
        return k.numel() * 2 >= _OVERLAP_MIN_BYTES
    return bool(setting)


class SparseLinearAttention(nn.Module):
    def __init__(self, head_dim, topk, feature_map="softmax", BLKQ=64, BLKK=64, use_bf16=True,
                 tie_feature_map_qk=True, linear_scope="all"):
        R"""
        Args:
            head_dim: dimension of each head (64 or 128).
            topk: ratio of keys selected for sparse attention, shared across all queries.
            feature_map: feature map for linear attention, one of ['elu', 'relu', 'softmax'].
            BLKQ: block size for query (64 or 128).
            BLKK: block size for key (64).
            use_bf16: bfloat16 (default) or float16 computation; the cast is done inside the module.
            tie_feature_map_qk: kept for signature compatibility; q and k always share the map type
                (in the reference both choices select the same function, core.py:43-60).
            linear_scope: not in the reference. "all" (default) is the reference's behaviour: the linear
                branch sums over every token (core.py:92-96). "unselected" sums, for each query block, over
                the KV blocks that block did not select (the scope drawn in assets/overview_of_SLA.png).
        """
        super().__init__()
        self.dtype = torch.bfloat16 if use_bf16 else torch.float16
        self.topk = topk
        self.BLKQ = BLKQ
        self.BLKK = BLKK
        self.proj_l = nn.Linear(head_dim, head_dim, dtype=torch.float32)
        if feature_map not in _FEATURES:
            raise NotImplementedError(f"Not supported feature map {feature_map}.")
        self.feature_map = feature_map
        self.tie_feature_map_qk = tie_feature_map_qk
        if linear_scope not in ("all", "unselected"):
            raise NotImplementedError(f"Not supported linear scope {linear_scope}.")
        self.linear_scope = linear_scope
        self.impl_flags = ops.FLAG_LINEAR_UNSELECTED if linear_scope == "unselected" else 0
        # run the linear-branch state next to the block-mask prediction: True, False, or None = when it pays
        self.overlap_linear_state = None
        self.init_weights_()

    def init_weights_(self):
        with torch.no_grad():
            nn.init.zeros_(self.proj_l.weight)
            nn.init.zeros_(self.proj_l.bias)

    def predict_block_map(self, q, k, with_column_lists=True):
        R"""Block-mask prediction alone (utils.py:55-67), on q and k as given (core.py:83). The result can be
        handed to `forward(..., block_map=...)` any number of times, e.g. over several steps of a diffusion sampler,
        or computed once outside a timed loop as the reference's benchmark does (evaluate/bench_kernel.py:79).
        `with_column_lists`: also build the per-KV-block lists a backward needs. `.pack16()` halves its size."""
        return ops.block_map(q.contiguous(), k.contiguous(), self.topk, self.BLKQ, self.BLKK,
                             want_cols=with_column_lists)

    def norm_rope_and_predict(self, q, k, gain_q=None, gain_k=None, rope_cos=None, rope_sin=None, eps=1e-6,
                              interleaved=True, with_column_lists=True, inplace=False):
        R"""Not in the reference: the layer's per-head RMS norm and rotary embedding of q and k fused with the first
        pass of the mask prediction (`ops.qk_norm_rope_pool` + `ops.block_map_pooled`), for callers that would otherwise
        run those as separate passes over q and k in front of `forward`. q, k: (B, H, L, D) in this module's compute
        dtype. Returns (q_out, k_out, block_map): call ``forward(q_out, k_out, v, block_map=block_map)``. Forward only
        (no autograd through the norm and the rotation)."""
        q_out, k_out, pooled = ops.qk_norm_rope_pool(q.contiguous(), k.contiguous(), gain_q, gain_k, rope_cos, rope_sin,
                                                     eps, interleaved, self.BLKQ, self.BLKK, inplace)
        return q_out, k_out, ops.block_map_pooled(pooled, self.topk, want_cols=with_column_lists)

    def forward(self, q, k, v, return_sparsity=False, block_map=None, gather=None):
        R"""
        Args:
            q, k, v: (B, H, L, D) CUDA tensors (any float dtype; output has q's dtype).
            return_sparsity: also return topk / N_BLOCKS, the kept fraction of KV blocks.
            block_map: not in the reference. A map from `predict_block_map` (or its packed form) to use instead of
                predicting one from this call's q and k.
            gather: not in the reference. A `sharding.GatheredOutput`: the result is written into this rank's slice of
                its full-size buffer and, by the same kernel, into every peer GPU's buffer (q, k, v must then be in
                the module's compute dtype and hold exactly this rank's units as (1, U, L, D)).
        """
        dtype = q.dtype
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        need_grad = torch.is_grad_enabled() and (
            q.requires_grad or k.requires_grad or v.requires_grad or self.proj_l.weight.requires_grad)
        bm = None
        if block_map is not None:
            bm = block_map.unpack() if isinstance(block_map, ops.PackedBlockMap) else block_map
            mb = (q.shape[2] + self.BLKQ - 1) // self.BLKQ
            if tuple(bm.lut.shape) != (q.shape[0], q.shape[1], mb, bm.topk) or bm.lut.device != q.device:
                raise ValueError("block_map was predicted for another shape, block size or device")
        # The linear-branch state needs k, v and proj_l only and the block map q and k only: the state kernels go to
        # a second stream and run next to the (latency-bound) mask prediction; both join before the attention kernel.
        kc, vc = k.to(self.dtype), v.to(self.dtype)
        prep = None
        if bm is None and _want_overlap(self.overlap_linear_state, k) and self.linear_scope == "all":
            nb = (k.shape[2] + self.BLKK - 1) // self.BLKK
            side = ops.side_stream(q.device)
            prep = ops.prepare_linear(kc, vc, self.proj_l.weight, self.proj_l.bias, ops.topk_count(nb, self.topk),
                                      self.BLKQ, self.BLKK, self.feature_map, self.impl_flags, stream=side)
        if bm is None:
            bm = ops.block_map(q, k, self.topk, self.BLKQ, self.BLKK, want_cols=need_grad)  # on the given dtype
        if prep is not None:
            torch.cuda.current_stream(q.device).wait_stream(side)
        q, k, v = q.to(self.dtype), kc, vc
        out, gather_ptrs = None, None
        if gather is not None:
            if dtype != self.dtype:
                raise TypeError("gather= needs inputs in the module's compute dtype")
            out, gather_ptrs = gather.local_view(q.shape), gather.peer_pointers()
        o = ops.sla_attention(q, k, v, self.proj_l.weight, self.proj_l.bias, bm, self.BLKQ, self.BLKK,
                              self.feature_map, self.impl_flags, prep, out, gather_ptrs)
        o = o.to(dtype)
        if return_sparsity:
            return o, bm.topk / bm.n_blocks
        return o


class SageSparseLinearAttention(nn.Module):
    def __init__(self, head_dim, topk, feature_map="softmax", use_bf16=True, tie_feature_map_qk=True,
                 BLKQ=128, BLKK=64):
        R"""Quantized forward (INT8 QK^T, FP8 PV). Same arguments as the reference; BLKQ/BLKK are
        accepted because the reference's README passes them, and must be 128/64."""
        super().__init__()
        if BLKQ != 128 or BLKK != 64:
            raise ValueError("SageSLA only supports BLKQ=128 and BLKK=64")
        self.dtype = torch.bfloat16 if use_bf16 else torch.float16
        self.topk = topk
        self.proj_l = nn.Linear(head_dim, head_dim, dtype=torch.float32)
        if feature_map not in _FEATURES:
            raise NotImplementedError(f"Not supported feature map {feature_map}.")
        self.feature_map = feature_map
        self.overlap_prepare = None        # True, False, or None = when it pays
        self.init_weights_()

    def init_weights_(self):
        with torch.no_grad():
            nn.init.zeros_(self.proj_l.weight)
            nn.init.zeros_(self.proj_l.bias)

    def forward(self, q, k, v, return_sparsity=False, gather=None):
        R"""As the reference's forward; `gather` (not in the reference): a `sharding.GatheredOutput`, see
        `SparseLinearAttention.forward` (under torch.no_grad(), inputs in the module's compute dtype)."""
        dtype = q.dtype
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        assert q.size(-1) in [64, 128], "headdim should be in [64, 128]."
        # quantization pre-passes and linear-branch state on a second stream next to the block-mask prediction
        qc, kc, vc = q.to(self.dtype), k.to(self.dtype), v.to(self.dtype)
        prep = None
        if _want_overlap(self.overlap_prepare, k):
            side = ops.side_stream(q.device)
            with torch.no_grad():
                prep = ops.sage_prepare(qc, kc, vc, self.proj_l.weight, self.proj_l.bias,
                                        ops.topk_count((k.shape[2] + 63) // 64, self.topk), self.feature_map,
                                        stream=side)
        bm = ops.block_map(q, k, self.topk, 128, 64)
        if prep is not None:
            torch.cuda.current_stream(q.device).wait_stream(side)
        # differentiable through the linear branch and proj_l only (SageSLA/core.py:148-158), like the reference
        out, gather_ptrs = None, None
        if gather is not None:
            if dtype != self.dtype:
                raise TypeError("gather= needs inputs in the module's compute dtype")
            out, gather_ptrs = gather.local_view(qc.shape), gather.peer_pointers()
        o = ops.sage_sla_attention(qc, kc, vc, self.proj_l.weight, self.proj_l.bias, bm, self.feature_map, prep=prep,
                                   out=out, gather_ptrs=gather_ptrs)
        o = o.to(dtype)
        if return_sparsity:
            return o, bm.topk / bm.n_blocks
        return o
