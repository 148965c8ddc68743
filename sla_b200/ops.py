"""Operator level of sla_b200: the reference's L1 names on top of the C-ABI library.

* ``get_block_map(q, k, topk_ratio, BLKQ, BLKK) -> (sparse_map, lut, topk)`` mirrors
  sparse_linear_attention/utils.py:55-67 (int8 map, int64 LUT, python int).
* ``_attention.apply(q, k, v, sparse_map, lut, topk, BLOCK_M, BLOCK_N, qk_scale=None)`` mirrors the
  autograd.Function of sparse_linear_attention/kernel.py:240-320.
* ``block_map`` / ``sla_attention`` are the fused forms the modules use (int32 LUT, column lists for
  the backward, linear branch + proj_l inside the kernels).

PyTorch is used for device memory, streams and autograd bookkeeping only; all arithmetic happens in
libsla_b200.so. Nothing here falls back to PyTorch math.
"""
from __future__ import annotations

import ctypes as C
import os
from dataclasses import dataclass
from typing import Optional

import torch

from . import _lib
from ._lib import SlaShape, check, lib

# SLA_B200_CHECK=1: after every fused forward / backward call synchronise the device and raise if a bounded
# device-side wait of a tcgen05 kernel ran out (otherwise poll with `_lib.raise_on_device_error()` once per step).
_CHECK_EVERY_CALL = os.environ.get("SLA_B200_CHECK", "0") == "1"


def _check_device():
    if _CHECK_EVERY_CALL and not torch.cuda.is_current_stream_capturing():
        _lib.raise_on_device_error()


_DT = {torch.bfloat16: _lib.SLA_BF16, torch.float16: _lib.SLA_FP16, torch.float32: _lib.SLA_FP32}


def _p(t: Optional[torch.Tensor]):
    return None if t is None else C.c_void_p(t.data_ptr())


def _stream(t: torch.Tensor):
    return C.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


def _require_cuda(*ts: torch.Tensor):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise RuntimeError("sla_b200 operators need CUDA tensors (there is no CPU path)")


def make_shape(B, H, L, D, BLKQ, BLKK, topk, dtype=torch.bfloat16, feature="softmax", flags=0,
               qk_scale: Optional[float] = None) -> SlaShape:
    if feature not in _lib.PHI:
        raise NotImplementedError(f"Not supported feature map {feature}.")
    return SlaShape(B, H, L, D, BLKQ, BLKK, topk, _DT[dtype], _lib.PHI[feature], flags,
                    0.0 if qk_scale is None else float(qk_scale))


def _workspace(shape: SlaShape, op: int, device) -> torch.Tensor:
    n = int(lib.sla_workspace_bytes(C.byref(shape), op))
    return torch.empty(max(n, 256), dtype=torch.uint8, device=device)


@dataclass
class BlockMap:
    """Result of block-mask prediction in the library's own format."""
    lut: torch.Tensor                     # (B,H,M_BLOCKS,topk) int32, ascending per row
    topk: int
    n_blocks: int
    sparse_map: Optional[torch.Tensor]    # (B,H,M_BLOCKS,N_BLOCKS) int8
    col_offsets: Optional[torch.Tensor]   # (B,H,N_BLOCKS+1) int32
    col_index: Optional[torch.Tensor]     # (B,H,M_BLOCKS*topk) int32


    def pack16(self) -> "PackedBlockMap":
        """A copy with 16-bit block indices, for keeping the map across calls at half the bytes."""
        if max(self.n_blocks, self.lut.shape[-2]) > 65536:
            raise ValueError("block indices do not fit 16 bits")
        return PackedBlockMap(_convert_index(self.lut, 16), self.topk, self.n_blocks,
                              self.col_offsets, None if self.col_index is None else _convert_index(self.col_index, 16))


@dataclass
class PackedBlockMap:
    """`BlockMap` with unsigned 16-bit indices (stored in int16 tensors); `unpack()` gives the form the operators
    read. The 0/1 map is not kept: the LUT and the column lists describe the same set."""
    lut16: torch.Tensor
    topk: int
    n_blocks: int
    col_offsets: Optional[torch.Tensor]
    col_index16: Optional[torch.Tensor]

    def unpack(self) -> BlockMap:
        return BlockMap(_convert_index(self.lut16, 32), self.topk, self.n_blocks, None, self.col_offsets,
                        None if self.col_index16 is None else _convert_index(self.col_index16, 32))


def _convert_index(t: torch.Tensor, dst_bits: int) -> torch.Tensor:
    _require_cuda(t)
    t = t.contiguous()
    src_bits = 32 if t.dtype == torch.int32 else 16
    out = torch.empty(t.shape, dtype=torch.int16 if dst_bits == 16 else torch.int32, device=t.device)
    check(lib.sla_index_convert(_p(t), src_bits, _p(out), dst_bits, t.numel(), _stream(t)))
    return out


def block_map(q: torch.Tensor, k: torch.Tensor, topk_ratio: float, BLKQ: int = 64, BLKK: int = 64,
              want_map: bool = False, want_cols: bool = False) -> BlockMap:
    _require_cuda(q, k)
    assert q.is_contiguous() and k.is_contiguous()
    if q.dtype not in _DT or k.dtype != q.dtype:
        raise TypeError(f"unsupported dtype {q.dtype}")
    B, H, L, D = q.shape
    mb, nb = (L + BLKQ - 1) // BLKQ, (L + BLKK - 1) // BLKK
    topk = _lib.topk_count(nb, topk_ratio)
    shape = SlaShape(B, H, L, D, BLKQ, BLKK, topk, _lib.SLA_BF16, 0, 0, 0.0)
    dev = q.device
    lut = torch.empty((B, H, mb, max(topk, 0)), dtype=torch.int32, device=dev)
    smap = torch.empty((B, H, mb, nb), dtype=torch.int8, device=dev) if (want_map or want_cols) else None
    co = torch.empty((B, H, nb + 1), dtype=torch.int32, device=dev) if want_cols else None
    ci = torch.empty((B, H, mb * max(topk, 0)), dtype=torch.int32, device=dev) if want_cols else None
    ws = _workspace(shape, _lib.OP_BLOCK_MAP, dev)
    check(lib.sla_block_map(C.byref(shape), _DT[q.dtype], _p(q), _p(k), _p(lut), _p(smap), _p(co), _p(ci),
                            _p(ws), ws.numel(), _stream(q)))
    return BlockMap(lut, topk, nb, smap, co, ci)


@dataclass
class PooledSums:
    """Per-block column sums of q and k left by `qk_norm_rope_pool` (fp32, the library's own layout)."""
    buf: torch.Tensor
    shape: tuple          # (B, H, L, D)
    dtype: torch.dtype
    BLKQ: int
    BLKK: int


def qk_norm_rope_pool(q, k, gain_q=None, gain_k=None, rope_cos=None, rope_sin=None, eps: float = 1e-6,
                      interleaved: bool = True, BLKQ: int = 64, BLKK: int = 64, inplace: bool = False):
    """The step in front of the operator in a DiT attention layer -- per-head RMS norm with a learned gain, then the
    rotary embedding -- in one pass over q and k that also takes the block sums the mask prediction needs.
    q, k: (B, H, L, D) bf16/fp16; gains: (D,) fp32 or None; rope_cos, rope_sin: (L, D/2) fp32 or None; pairs are
    (x[2i], x[2i+1]) when `interleaved`, else (x[i], x[i + D/2]). Returns (q_out, k_out, PooledSums); hand the last to
    `block_map_pooled`."""
    _require_cuda(q, k, gain_q, gain_k, rope_cos, rope_sin)
    assert q.is_contiguous() and k.is_contiguous() and q.shape == k.shape and q.dtype == k.dtype
    if q.dtype not in (torch.bfloat16, torch.float16):
        raise TypeError("qk_norm_rope_pool takes bf16 or fp16 tensors")
    B, H, L, D = q.shape
    f32 = lambda t: None if t is None else t.detach().to(torch.float32).contiguous()
    gain_q, gain_k, rope_cos, rope_sin = f32(gain_q), f32(gain_k), f32(rope_cos), f32(rope_sin)
    if rope_cos is not None and tuple(rope_cos.shape) != (L, D // 2):
        raise ValueError("rope tables must be (L, D/2)")
    shape = SlaShape(B, H, L, D, BLKQ, BLKK, 1, _DT[q.dtype], 0, 0, 0.0)
    q_out, k_out = (q, k) if inplace else (torch.empty_like(q), torch.empty_like(k))
    sums = torch.empty(int(lib.sla_pooled_sums_bytes(C.byref(shape))), dtype=torch.uint8, device=q.device)
    check(lib.sla_qk_norm_rope_pool(C.byref(shape), _p(q), _p(k), _p(gain_q), _p(gain_k), _p(rope_cos), _p(rope_sin),
                                    float(eps), 1 if interleaved else 0, _p(q_out), _p(k_out), _p(sums), sums.numel(),
                                    _stream(q)))
    return q_out, k_out, PooledSums(sums, (B, H, L, D), q.dtype, BLKQ, BLKK)


def block_map_pooled(pooled: PooledSums, topk_ratio: float, want_map: bool = False, want_cols: bool = False) -> BlockMap:
    """Mask prediction from the block sums of `qk_norm_rope_pool`: no further pass over q or k. One rounding point
    differs from `block_map` (see sla_block_map_pooled in the header), so rows whose k-th and (k+1)-th scores are
    within rounding of each other can select differently."""
    B, H, L, D = pooled.shape
    BLKQ, BLKK = pooled.BLKQ, pooled.BLKK
    mb, nb = (L + BLKQ - 1) // BLKQ, (L + BLKK - 1) // BLKK
    topk = _lib.topk_count(nb, topk_ratio)
    shape = SlaShape(B, H, L, D, BLKQ, BLKK, topk, _DT[pooled.dtype], 0, 0, 0.0)
    dev = pooled.buf.device
    lut = torch.empty((B, H, mb, max(topk, 0)), dtype=torch.int32, device=dev)
    smap = torch.empty((B, H, mb, nb), dtype=torch.int8, device=dev) if (want_map or want_cols) else None
    co = torch.empty((B, H, nb + 1), dtype=torch.int32, device=dev) if want_cols else None
    ci = torch.empty((B, H, mb * max(topk, 0)), dtype=torch.int32, device=dev) if want_cols else None
    ws = _workspace(shape, _lib.OP_BLOCK_MAP, dev)
    check(lib.sla_block_map_pooled(C.byref(shape), _p(pooled.buf), _p(lut), _p(smap), _p(co), _p(ci), _p(ws), ws.numel(),
                                   torch.cuda.current_stream(dev).cuda_stream))
    return BlockMap(lut, topk, nb, smap, co, ci)


def column_lists(sparse_map: torch.Tensor, L: int, BLKQ: int, BLKK: int, topk: int):
    """Per-KV-block query-block lists from a 0/1 block map (for maps made elsewhere)."""
    _require_cuda(sparse_map)
    B, H, mb, nb = sparse_map.shape
    shape = SlaShape(B, H, L, 64, BLKQ, BLKK, topk, _lib.SLA_BF16, 0, 0, 0.0)
    co = torch.empty((B, H, nb + 1), dtype=torch.int32, device=sparse_map.device)
    ci = torch.empty((B, H, mb * topk), dtype=torch.int32, device=sparse_map.device)
    check(lib.sla_column_lists(C.byref(shape), _p(sparse_map.contiguous()), _p(co), _p(ci), _stream(sparse_map)))
    return co, ci


def get_block_map(q, k, topk_ratio, BLKQ=64, BLKK=64):
    """Drop-in for sparse_linear_attention.utils.get_block_map (utils.py:55-67): returns
    (sparse_map int8, lut int64, topk). The LUT rows are sorted ascending (the reference's order is
    unspecified). The tensors remember the library-format twin (int32 LUT, column lists) so that a
    following ``_attention.apply`` does not rebuild them."""
    bm = block_map(q, k, topk_ratio, BLKQ, BLKK, want_map=True, want_cols=True)
    lut64 = bm.lut.to(torch.int64)
    lut64._sla_block_map = bm
    bm.sparse_map._sla_block_map = bm
    return bm.sparse_map, lut64, bm.topk


class _attention(torch.autograd.Function):
    """Drop-in for sparse_linear_attention.kernel._attention (kernel.py:240-320).

    ``_attention.impl_flags`` (class attribute, default 0) is OR-ed into the shape's flags: set it to
    ``_lib.FLAG_LEGACY_MMA`` to force the mma.sync kernels."""

    impl_flags = 0

    @staticmethod
    def forward(ctx, q, k, v, k_block_id, lut, topk, BLOCK_M, BLOCK_N, qk_scale=None):
        assert q.is_contiguous() and k.is_contiguous() and v.is_contiguous()
        assert k_block_id.is_contiguous() and lut.is_contiguous()
        assert BLOCK_M == 64 or BLOCK_M == 128
        assert BLOCK_N == 64
        _require_cuda(q, k, v, lut)
        B, H, L, D = q.shape
        bm = getattr(lut, "_sla_block_map", None)
        lut32 = bm.lut if bm is not None else lut.to(torch.int32)
        shape = make_shape(B, H, L, D, BLOCK_M, BLOCK_N, topk, q.dtype,
                           flags=_lib.FLAG_SPARSE_ONLY | _attention.impl_flags, qk_scale=qk_scale)
        o_s = torch.empty_like(v)
        lse = torch.empty(q.shape[:-1], device=q.device, dtype=torch.float32)
        check(lib.sla_sparse_fwd(C.byref(shape), _p(q), _p(k), _p(v), _p(lut32), _p(o_s), _p(lse), _stream(q)))
        ctx.save_for_backward(q, k, v, k_block_id, lut32, lse, o_s)
        ctx.sla_shape = shape
        ctx.sla_bm = bm
        return o_s

    @staticmethod
    def backward(ctx, do_s):
        q, k, v, k_block_id, lut32, lse, o_s = ctx.saved_tensors
        do_s = do_s.contiguous()
        shape = ctx.sla_shape
        bm = ctx.sla_bm
        if bm is not None and bm.col_offsets is not None:
            co, ci = bm.col_offsets, bm.col_index
        else:
            co, ci = column_lists(k_block_id, shape.L, shape.BLKQ, shape.BLKK, shape.topk)
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        ws = _workspace(shape, _lib.OP_SPARSE_BWD, q.device)
        check(lib.sla_sparse_bwd(C.byref(shape), _p(q), _p(k), _p(v), _p(o_s), _p(lse), _p(do_s), _p(lut32),
                                 _p(co), _p(ci), _p(dq), _p(dk), _p(dv), _p(ws), ws.numel(), _stream(q)))
        return dq, dk, dv, None, None, None, None, None, None


FLAG_LINEAR_UNSELECTED = _lib.FLAG_LINEAR_UNSELECTED
topk_count = _lib.topk_count


@dataclass
class LinearPrep:
    """What `prepare_linear` left for `sla_attention`: the linear-branch state and the forward workspace."""
    lin_state: torch.Tensor
    ws: torch.Tensor
    key: tuple


_side_streams = {}


def side_stream(device) -> torch.cuda.Stream:
    """One extra stream per device for work that runs next to the block-mask prediction."""
    idx = torch.device(device).index
    if idx is None:
        idx = torch.cuda.current_device()
    if idx not in _side_streams:
        _side_streams[idx] = torch.cuda.Stream(device=idx)
    return _side_streams[idx]


def prepare_linear(k, v, weight, bias, L_blocks_topk: int, BLKQ=64, BLKK=64, feature="softmax",
                   impl_flags: int = 0, stream: Optional[torch.cuda.Stream] = None) -> LinearPrep:
    """The part of the forward that needs k, v and proj_l only (core.py:91,93-94): the linear-branch state
    H, z and H W^T. With `stream` given it is launched there, after everything already queued on the current
    stream, so that it overlaps the block-mask prediction the caller launches next; the caller joins with
    ``torch.cuda.current_stream().wait_stream(stream)`` before `sla_attention(..., prep=...)`. Buffers are
    allocated on the current stream (they are used there afterwards)."""
    _require_cuda(k, v, weight)
    B, H, L, D = k.shape
    shape = make_shape(B, H, L, D, BLKQ, BLKK, L_blocks_topk, k.dtype, feature, flags=impl_flags)
    dev = k.device
    lin_state = torch.empty((B, H, 2 * D * D + D), dtype=k.dtype, device=dev)
    ws = _workspace(shape, _lib.OP_FWD, dev)
    w, b = weight.detach(), (bias.detach() if bias is not None else None)
    if stream is not None:
        stream.wait_stream(torch.cuda.current_stream(dev))
        handle = C.c_void_p(stream.cuda_stream)
    else:
        handle = _stream(k)
    check(lib.sla_fwd_prepare(C.byref(shape), _p(k), _p(v), _p(w), _p(b), _p(lin_state), _p(ws), ws.numel(), handle))
    return LinearPrep(lin_state, ws, (B, H, L, D, BLKQ, BLKK, L_blocks_topk, k.dtype, feature, impl_flags))


class _SLAFused(torch.autograd.Function):
    """core.py:88-100 (sparse branch + feature maps + linear branch + proj_l + sum) as one operator."""

    @staticmethod
    def forward(ctx, q, k, v, weight, bias, bm: BlockMap, BLKQ, BLKK, feature, need_grad, impl_flags, prep,
                out=None, gather_ptrs=None):
        B, H, L, D = q.shape
        shape = make_shape(B, H, L, D, BLKQ, BLKK, bm.topk, q.dtype, feature, flags=impl_flags)
        dev = q.device
        if out is not None:
            if tuple(out.shape) != tuple(q.shape) or out.dtype != q.dtype or not out.is_contiguous():
                raise ValueError("`out` must be a contiguous tensor of q's shape and dtype")
            o = out
        else:
            o = torch.empty_like(q)
        o_s = torch.empty_like(q) if need_grad else None
        lse = torch.empty((B, H, L), dtype=torch.float32, device=dev)
        if prep is not None:
            if prep.key != (B, H, L, D, BLKQ, BLKK, bm.topk, q.dtype, feature, impl_flags):
                raise ValueError("prepare_linear was called for another shape or configuration")
            lin_state, ws = prep.lin_state, prep.ws
            fwd_shape = make_shape(B, H, L, D, BLKQ, BLKK, bm.topk, q.dtype, feature,
                                   flags=impl_flags | _lib.FLAG_STATE_READY)
        else:
            lin_state = torch.empty((B, H, 2 * D * D + D), dtype=q.dtype, device=dev)
            ws = _workspace(shape, _lib.OP_FWD, dev)
            fwd_shape = shape
        if gather_ptrs:
            dst = (C.c_void_p * len(gather_ptrs))(*[int(x) for x in gather_ptrs])
            check(lib.sla_fwd_gather(C.byref(fwd_shape), _p(q), _p(k), _p(v), _p(bm.lut), _p(weight), _p(bias), _p(o),
                                     _p(o_s), _p(lse), _p(lin_state), _p(ws), ws.numel(), dst, len(gather_ptrs),
                                     _stream(q)))
        else:
            check(lib.sla_fwd(C.byref(fwd_shape), _p(q), _p(k), _p(v), _p(bm.lut), _p(weight), _p(bias), _p(o), _p(o_s),
                              _p(lse), _p(lin_state), _p(ws), ws.numel(), _stream(q)))
        _check_device()
        if need_grad:
            ctx.save_for_backward(q, k, v, o_s, lse, lin_state, weight, bm.lut, bm.col_offsets, bm.col_index)
            ctx.sla_shape = shape
            ctx.has_bias = bias is not None
        return o

    @staticmethod
    def backward(ctx, d_o):
        q, k, v, o_s, lse, lin_state, weight, lut, co, ci = ctx.saved_tensors
        shape = ctx.sla_shape
        d_o = d_o.contiguous()
        D = shape.D
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        dw = torch.empty((D, D), dtype=torch.float32, device=q.device)
        db = torch.empty((D,), dtype=torch.float32, device=q.device)
        ws = _workspace(shape, _lib.OP_BWD, q.device)
        check(lib.sla_bwd(C.byref(shape), _p(q), _p(k), _p(v), _p(o_s), _p(lse), _p(d_o), _p(lut), _p(co), _p(ci),
                          _p(weight), _p(lin_state), _p(dq), _p(dk), _p(dv), _p(dw), _p(db), _p(ws), ws.numel(),
                          _stream(q)))
        _check_device()
        return dq, dk, dv, dw, (db if ctx.has_bias else None), None, None, None, None, None, None, None, None, None


def sla_attention(q, k, v, weight, bias, bm: BlockMap, BLKQ=64, BLKK=64, feature="softmax",
                  impl_flags: int = 0, prep: Optional[LinearPrep] = None, out: Optional[torch.Tensor] = None,
                  gather_ptrs=None):
    """o = o_s + proj_l(o_l) for q, k, v already in the 16-bit compute dtype. `prep`: the result of
    `prepare_linear` on the same k, v, weight, bias (already joined into the current stream). `out`: write the
    result there instead of into a new tensor. `gather_ptrs`: up to 8 device addresses (this process's view) of
    further (B, H, L, D) blocks the kernel's epilogue also writes the result to, e.g. this rank's place in every peer
    GPU's full-size output (`sharding.GatheredOutput`)."""
    _require_cuda(q, k, v, weight)
    need_grad = torch.is_grad_enabled() and any(
        t is not None and t.requires_grad for t in (q, k, v, weight, bias))
    if need_grad and bm.col_offsets is None:
        raise RuntimeError("the block map was built without column lists (want_cols=True) but a backward is needed")
    return _SLAFused.apply(q, k, v, weight, bias, bm, BLKQ, BLKK, feature, need_grad, impl_flags, prep, out,
                           gather_ptrs)


def sage_prepare(q, k, v, weight, bias, topk: int, feature="softmax", sparse_only: bool = False,
                 stream: Optional[torch.cuda.Stream] = None) -> LinearPrep:
    """What the quantized forward needs besides the block map (linear-branch state, INT8 q and k, e4m3 v), launched
    on `stream` (after everything already queued on the current stream) so that it overlaps the block-mask
    prediction; join with ``torch.cuda.current_stream().wait_stream(stream)`` before
    `sage_sla_attention(..., prep=...)`."""
    _require_cuda(q, k, v, weight)
    B, H, L, D = q.shape
    flags = _lib.FLAG_SPARSE_ONLY if sparse_only else 0
    shape = make_shape(B, H, L, D, 128, 64, topk, q.dtype, feature, flags=flags)
    lin_state = torch.empty((B, H, 2 * D * D + D), dtype=q.dtype, device=q.device)
    ws = _workspace(shape, _lib.OP_SAGE_FWD, q.device)
    w, b = weight.detach(), (bias.detach() if bias is not None else None)
    if stream is not None:
        stream.wait_stream(torch.cuda.current_stream(q.device))
        handle = C.c_void_p(stream.cuda_stream)
    else:
        handle = _stream(q)
    check(lib.sage_sla_prepare(C.byref(shape), _p(q), _p(k), _p(v), _p(w), _p(b), _p(lin_state), _p(ws), ws.numel(),
                               handle))
    return LinearPrep(lin_state, ws, (B, H, L, D, 128, 64, topk, q.dtype, feature, flags))


class _SageFused(torch.autograd.Function):
    """SageSLA/core.py:100-158 as one operator. As in the reference the quantized sparse branch has no backward
    (SageSLA/core.py:114-146 calls a forward-only kernel), while the linear branch and proj_l after it
    (SageSLA/core.py:148-158) are differentiable: the backward returns their gradients for q, k, v, W and b."""

    @staticmethod
    def forward(ctx, q, k, v, weight, bias, bm, feature, prep):
        o, lin_state = _sage_forward(q, k, v, weight, bias, bm, feature, False, prep)
        B, H, L, D = q.shape
        ctx.save_for_backward(q, k, v, lin_state, weight)
        ctx.sla_shape = make_shape(B, H, L, D, 128, 64, bm.topk, q.dtype, feature, flags=_lib.FLAG_LINEAR_ONLY)
        ctx.has_bias = bias is not None
        return o

    @staticmethod
    def backward(ctx, d_o):
        q, k, v, lin_state, weight = ctx.saved_tensors
        shape = ctx.sla_shape
        d_o = d_o.contiguous()
        D = shape.D
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        dw = torch.empty((D, D), dtype=torch.float32, device=q.device)
        db = torch.empty((D,), dtype=torch.float32, device=q.device)
        ws = _workspace(shape, _lib.OP_BWD, q.device)
        check(lib.sla_bwd(C.byref(shape), _p(q), _p(k), _p(v), None, None, _p(d_o), None, None, None, _p(weight),
                          _p(lin_state), _p(dq), _p(dk), _p(dv), _p(dw), _p(db), _p(ws), ws.numel(), _stream(q)))
        _check_device()
        return dq, dk, dv, dw, (db if ctx.has_bias else None), None, None, None


def sage_sla_attention(q, k, v, weight, bias, bm: BlockMap, feature="softmax", sparse_only: bool = False,
                       prep: Optional[LinearPrep] = None, out: Optional[torch.Tensor] = None, gather_ptrs=None):
    """SageSLA/core.py:100-158: quantized sparse branch + linear branch + proj_l.
    ``sparse_only`` returns the quantized sparse branch alone (the o_s of SageSLA/core.py:114). When a gradient is
    required it flows through the linear branch and proj_l only, as in the reference. `out`, `gather_ptrs`: as in
    `sla_attention` (forward without gradient only)."""
    _require_cuda(q, k, v, weight)
    need_grad = not sparse_only and torch.is_grad_enabled() and any(
        t is not None and t.requires_grad for t in (q, k, v, weight, bias))
    if need_grad:
        if out is not None or gather_ptrs:
            raise NotImplementedError("out= / gather_ptrs= of the quantized forward need torch.no_grad()")
        return _SageFused.apply(q, k, v, weight, bias, bm, feature, prep)
    return _sage_forward(q, k, v, weight, bias, bm, feature, sparse_only, prep, out, gather_ptrs)[0]


def _sage_forward(q, k, v, weight, bias, bm, feature, sparse_only, prep, out=None, gather_ptrs=None):
    B, H, L, D = q.shape
    flags = _lib.FLAG_SPARSE_ONLY if sparse_only else 0
    if out is not None:
        if tuple(out.shape) != tuple(q.shape) or out.dtype != q.dtype or not out.is_contiguous():
            raise ValueError("`out` must be a contiguous tensor of q's shape and dtype")
        o = out
    else:
        o = torch.empty_like(q)
    if prep is not None:
        if prep.key != (B, H, L, D, 128, 64, bm.topk, q.dtype, feature, flags):
            raise ValueError("sage_prepare was called for another shape or configuration")
        lin_state, ws = prep.lin_state, prep.ws
        flags |= _lib.FLAG_STATE_READY
    shape = make_shape(B, H, L, D, 128, 64, bm.topk, q.dtype, feature, flags=flags)
    if prep is None:
        lin_state = torch.empty((B, H, 2 * D * D + D), dtype=q.dtype, device=q.device)
        ws = _workspace(shape, _lib.OP_SAGE_FWD, q.device)
    if gather_ptrs:
        dst = (C.c_void_p * len(gather_ptrs))(*[int(x) for x in gather_ptrs])
        check(lib.sage_sla_fwd_gather(C.byref(shape), _p(q), _p(k), _p(v), _p(bm.lut), _p(weight), _p(bias), _p(o),
                                      _p(lin_state), _p(ws), ws.numel(), dst, len(gather_ptrs), _stream(q)))
    else:
        check(lib.sage_sla_fwd(C.byref(shape), _p(q), _p(k), _p(v), _p(bm.lut), _p(weight), _p(bias), _p(o),
                               _p(lin_state), _p(ws), ws.numel(), _stream(q)))
    _check_device()
    return o, lin_state
