"""Generate the golden fixtures in this directory from the reference implementation itself.

Run once, in a container that has a checkout of the reference (thu-ml/SLA); SLA_REFERENCE_DIR names it:

    SLA_REFERENCE_DIR=<path to the reference checkout> python tests/golden/make_golden.py

The reference (thu-ml/SLA) only has Triton GPU kernels. They are executed here, unmodified, on
the CPU through Triton's interpreter (TRITON_INTERPRET=1). Two things outside the reference are
adjusted, neither of which changes its arithmetic:
  * the interpreter's ``create_dot``, element-wise ``binary_op`` and ``ReduceOps.sum`` act on the
    raw uint16 storage of bfloat16 operands; they are patched to widen bf16 to fp32 first (and,
    for the latter two, round the result back to bf16); fp16/fp32 operands take the original
    route;
  * core.py:98 opens ``torch.amp.autocast('cuda')`` which is a no-op without a GPU, so ``proj_l`` is
    wrapped in the equivalent CPU autocast region (same dtype, only around that one call).
Everything stored in the .npz files is either an input drawn from a seeded generator or an output
of reference code (`get_block_map`, `mean_pool`, `_attention.forward/backward`,
`SparseLinearAttention.forward` + autograd).
"""
import os
import sys

os.environ["TRITON_INTERPRET"] = "1"
REF = os.environ.get("SLA_REFERENCE_DIR")
if not REF or not os.path.isdir(REF):
    sys.exit("set SLA_REFERENCE_DIR to a checkout of the reference (thu-ml/SLA)")
sys.path.insert(0, REF)

import numpy as np
import torch

import triton.language as tl
from triton.runtime import interpreter as _interp

_orig_dot = _interp.InterpreterBuilder.create_dot


def _bf16_to_f32(a):
    return (a.astype(np.uint32) << 16).view(np.float32)


def _create_dot(self, a, b, d, input_precision, max_num_imprecise_acc):
    if a.dtype == tl.bfloat16 or b.dtype == tl.bfloat16:
        ad = _bf16_to_f32(a.data) if a.dtype == tl.bfloat16 else a.data.astype(np.float32)
        bd = _bf16_to_f32(b.data) if b.dtype == tl.bfloat16 else b.data.astype(np.float32)
        return _interp.TensorHandle(np.matmul(ad, bd, dtype=d.data.dtype) + d.data, d.dtype.scalar)
    return _orig_dot(self, a, b, d, input_precision, max_num_imprecise_acc)


_interp.InterpreterBuilder.create_dot = _create_dot

_orig_binary = _interp.InterpreterBuilder.binary_op


def _f32_to_bf16(x):
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)  # round to nearest even


def _binary_op(self, lhs, rhs, op):
    # element-wise arithmetic on two bf16 tensors (kernel.py:104, o_s * do_s): widen, apply, round
    if lhs.dtype.scalar == tl.bfloat16 and rhs.dtype.scalar == tl.bfloat16:
        out = op(_bf16_to_f32(lhs.data), _bf16_to_f32(rhs.data))
        if out.dtype == np.float32:
            return _interp.TensorHandle(_f32_to_bf16(out), tl.bfloat16)
    return _orig_binary(self, lhs, rhs, op)


_interp.InterpreterBuilder.binary_op = _binary_op

_orig_sum = _interp.ReduceOps.sum


def _reduce_sum(self, input):
    # tl.sum over a bf16 tensor (kernel.py:104): widen, sum in fp32, round once to bf16
    if input.dtype.scalar == tl.bfloat16:
        out = np.sum(_bf16_to_f32(input.handle.data), axis=self.axis, keepdims=self.keep_dims)
        return self.to_tensor(_f32_to_bf16(out), input.dtype)
    return _orig_sum(self, input)


_interp.ReduceOps.sum = _reduce_sum

from sparse_linear_attention import SparseLinearAttention  # noqa: E402
from sparse_linear_attention.kernel import _attention  # noqa: E402
from sparse_linear_attention.utils import get_block_map, mean_pool  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))
DT = {"fp32": torch.float32, "bf16": torch.bfloat16, "fp16": torch.float16}


def pack(t: torch.Tensor) -> np.ndarray:
    """16-bit floats are stored as their raw int16 bit patterns (numpy has no bfloat16)."""
    t = t.detach().contiguous()
    if t.dtype in (torch.bfloat16, torch.float16):
        return t.view(torch.int16).numpy()
    return t.numpy()


def save(name, **arrs):
    path = os.path.join(HERE, name + ".npz")
    np.savez_compressed(path, **arrs)
    print(f"{name}: {os.path.getsize(path) / 1024:.0f} KiB")


class _Ctx:
    """Stand-in for the autograd context so forward's saved tensors (lse, o_s) can be read."""

    def save_for_backward(self, *t):
        self.saved_tensors = t


def block_map_case(name, dtype, B, H, L, D, BLKQ, BLKK, ratio, seed, store_inputs=True):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(B, H, L, D, generator=g).to(DT[dtype])
    k = (torch.randn(B, H, L, D, generator=g) + 0.5 * torch.randn(1, H, 1, D, generator=g)).to(DT[dtype])
    sparse_map, lut, topk = get_block_map(q, k, ratio, BLKQ, BLKK)
    # the score the top-k was taken on, recomputed with the same reference ops (utils.py:56-59)
    arg_k = k - torch.mean(k, dim=-2, keepdim=True)
    pq, pk = mean_pool(q, BLKQ), mean_pool(arg_k, BLKK)
    score = pq @ pk.transpose(-1, -2)
    arrs = dict(meta=np.array([B, H, L, D, BLKQ, BLKK, topk, seed]), ratio=np.array(ratio),
                dtype=np.array(dtype), sparse_map=sparse_map.numpy(),
                lut=torch.sort(lut, dim=-1).values.numpy().astype(np.int32),
                pooled_q=pack(pq), pooled_k=pack(pk), score=pack(score))
    if store_inputs:
        arrs.update(q=pack(q), k=pack(k))
    save(name, **arrs)


def attention_case(name, dtype, B, H, L, D, BLKQ, BLKK, ratio, seed):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(B, H, L, D, generator=g).to(DT[dtype])
    k = torch.randn(B, H, L, D, generator=g).to(DT[dtype])
    v = torch.randn(B, H, L, D, generator=g).to(DT[dtype])
    do = torch.randn(B, H, L, D, generator=g).to(DT[dtype])
    sparse_map, lut, topk = get_block_map(q, k, ratio, BLKQ, BLKK)
    ctx = _Ctx()
    o_s = _attention.forward(ctx, q, k, v, sparse_map, lut, topk, BLKQ, BLKK)
    lse = ctx.saved_tensors[5]
    dq, dk, dv = _attention.backward(ctx, do)[:3]
    save(name, meta=np.array([B, H, L, D, BLKQ, BLKK, topk, seed]), dtype=np.array(dtype),
         q=pack(q), k=pack(k), v=pack(v), do=pack(do), sparse_map=sparse_map.numpy(),
         lut=torch.sort(lut, dim=-1).values.numpy().astype(np.int32),
         o_s=pack(o_s), lse=lse.numpy(), dq=pack(dq), dk=pack(dk), dv=pack(dv))


def module_case(name, in_dtype, use_bf16, feature, B, H, L, D, BLKQ, BLKK, ratio, seed,
                backward=True, store_inputs=True, canonical_seed=False):
    comp = torch.bfloat16 if use_bf16 else torch.float16
    if canonical_seed:
        # the CPU-runnable configuration: torch.manual_seed(seed); q, k, v = randn in that order,
        # then W ~ N(0, 0.02), b = 0
        torch.manual_seed(seed)
        q = torch.randn(B, H, L, D)
        k = torch.randn(B, H, L, D)
        v = torch.randn(B, H, L, D)
        w = torch.randn(D, D) * 0.02
        bias = torch.zeros(D)
        do = None
    else:
        g = torch.Generator().manual_seed(seed)
        q = torch.randn(B, H, L, D, generator=g)
        k = torch.randn(B, H, L, D, generator=g)
        v = torch.randn(B, H, L, D, generator=g)
        w = torch.randn(D, D, generator=g) * 0.05
        bias = torch.randn(D, generator=g) * 0.05
        do = torch.randn(B, H, L, D, generator=g).to(DT[in_dtype])
    q, k, v = (t.to(DT[in_dtype]).requires_grad_(backward) for t in (q, k, v))
    attn = SparseLinearAttention(D, ratio, feature, BLKQ, BLKK, use_bf16=use_bf16)
    with torch.no_grad():
        attn.proj_l.weight.copy_(w)
        attn.proj_l.bias.copy_(bias)
    inner = attn.proj_l.forward

    def proj_autocast(x):
        with torch.amp.autocast("cpu", dtype=comp):
            return inner(x)

    attn.proj_l.forward = proj_autocast
    o, sparsity = attn(q, k, v, return_sparsity=True)
    arrs = dict(meta=np.array([B, H, L, D, BLKQ, BLKK, 0, seed]), ratio=np.array(ratio),
                in_dtype=np.array(in_dtype), compute=np.array("bf16" if use_bf16 else "fp16"),
                feature=np.array(feature), w=w.numpy(), bias=bias.numpy(), o=pack(o),
                sparsity=np.array(sparsity))
    if store_inputs:
        arrs.update(q=pack(q), k=pack(k), v=pack(v))
    if backward:
        o.backward(do)
        arrs.update(do=pack(do), dq=pack(q.grad), dk=pack(k.grad), dv=pack(v.grad),
                    dw=attn.proj_l.weight.grad.numpy(), db=attn.proj_l.bias.grad.numpy())
    save(name, **arrs)


if __name__ == "__main__":
    torch.set_num_threads(8)
    # --- block map -------------------------------------------------------------------------
    block_map_case("blockmap_fp32_c1shape", "fp32", 1, 2, 1024, 64, 64, 64, 0.25, 0)
    block_map_case("blockmap_bf16_ragged", "bf16", 1, 2, 520, 64, 64, 64, 0.3, 11)
    block_map_case("blockmap_bf16_blkq128", "bf16", 1, 1, 1000, 128, 128, 64, 0.2, 12)
    block_map_case("blockmap_fp16_small", "fp16", 2, 1, 200, 64, 64, 64, 0.5, 13)
    # --- sparse attention forward + backward -----------------------------------------------
    attention_case("attn_fp32_d64", "fp32", 1, 2, 200, 64, 64, 64, 0.5, 21)
    attention_case("attn_fp16_d64", "fp16", 1, 2, 200, 64, 64, 64, 0.5, 22)
    attention_case("attn_bf16_d128", "bf16", 1, 1, 328, 128, 64, 64, 0.34, 23)
    attention_case("attn_bf16_blkq128", "bf16", 1, 1, 400, 64, 128, 64, 0.3, 24)
    attention_case("attn_fp32_blkq128_d128", "fp32", 1, 1, 300, 128, 128, 64, 0.4, 25)
    # --- whole module ------------------------------------------------------------------------
    module_case("module_c1", "fp32", True, "softmax", 1, 2, 1024, 64, 64, 64, 0.25, 0,
                backward=False, store_inputs=False, canonical_seed=True)
    module_case("module_bf16_softmax", "bf16", True, "softmax", 1, 2, 264, 64, 64, 64, 0.4, 31)
    module_case("module_fp16_relu", "fp16", False, "relu", 1, 1, 200, 128, 64, 64, 0.5, 32)
    module_case("module_fp32in_elu_blkq128", "fp32", True, "elu", 1, 1, 300, 64, 128, 64, 0.4, 33)
