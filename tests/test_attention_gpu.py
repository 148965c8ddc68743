"""GPU parity of the sparse branch (`_attention` forward/backward through the C ABI) against the
reference's golden vectors and the CPU oracle. Floating point: cosine >= 0.999 and relative L1 <= 1e-2
(the bar for 16-bit outputs); LSE within 2e-3 absolute (log2 units)."""
import numpy as np
import pytest
import torch

from helpers import DT, assert_close_parity, load_golden, unpack

pytestmark = pytest.mark.gpu

ATTN = ["attn_fp16_d64", "attn_bf16_d128", "attn_bf16_blkq128"]


def _run(q, k, v, do, smap, lut64, topk, BLKQ, BLKK):
    from sla_b200 import ops
    qg, kg, vg = (t.cuda().requires_grad_(True) for t in (q, k, v))
    o = ops._attention.apply(qg, kg, vg, smap.cuda(), lut64.cuda(), topk, BLKQ, BLKK)
    o.backward(do.cuda())
    return o.detach().cpu(), qg.grad.cpu(), kg.grad.cpu(), vg.grad.cpu()


@pytest.mark.parametrize("name", ATTN)
def test_attention_vs_reference_golden(name):
    g = load_golden(name)
    B, H, L, D, BLKQ, BLKK, topk, _ = g["meta"].tolist()
    dt = DT[str(g["dtype"])]
    q, k, v, do = (unpack(g[n], dt) for n in ("q", "k", "v", "do"))
    smap = torch.from_numpy(g["sparse_map"])
    lut64 = torch.from_numpy(g["lut"].astype(np.int64))
    o, dq, dk, dv = _run(q, k, v, do, smap, lut64, topk, BLKQ, BLKK)
    assert_close_parity(o.float(), unpack(g["o_s"], dt).float(), what=name + ".o_s")
    for mine, n in ((dq, "dq"), (dk, "dk"), (dv, "dv")):
        assert_close_parity(mine.float(), unpack(g[n], dt).float(), what=f"{name}.{n}")


@pytest.mark.parametrize("name", ["attn_fp32_d64", "attn_fp32_blkq128_d128"])
def test_attention_vs_fp32_reference_golden(name):
    """The reference kernel run on fp32 tensors is a rounding-free target: the bf16 kernels fed with
    bf16-rounded copies of the same inputs must stay within 16-bit tolerance of it."""
    g = load_golden(name)
    B, H, L, D, BLKQ, BLKK, topk, _ = g["meta"].tolist()
    q, k, v, do = (unpack(g[n], torch.float32).bfloat16() for n in ("q", "k", "v", "do"))
    smap = torch.from_numpy(g["sparse_map"])
    lut64 = torch.from_numpy(g["lut"].astype(np.int64))
    o, dq, dk, dv = _run(q, k, v, do, smap, lut64, topk, BLKQ, BLKK)
    assert_close_parity(o.float(), torch.from_numpy(g["o_s"]), cos_min=0.999, l1_max=2e-2, what=name + ".o_s")
    for mine, n in ((dq, "dq"), (dk, "dk"), (dv, "dv")):
        assert_close_parity(mine.float(), torch.from_numpy(g[n]), cos_min=0.999, l1_max=3e-2, what=f"{name}.{n}")


@pytest.mark.parametrize("dtype,B,H,L,D,BLKQ,ratio", [
    (torch.bfloat16, 1, 2, 1024, 128, 64, 0.25),
    (torch.bfloat16, 2, 1, 1000, 64, 128, 0.3),
    (torch.float16, 1, 1, 65, 64, 64, 1.0),
    (torch.bfloat16, 1, 1, 64, 128, 64, 1.0),
    (torch.bfloat16, 1, 1, 127, 128, 128, 0.5),
    (torch.bfloat16, 1, 1, 2000, 128, 64, 0.04),
])
def test_attention_vs_oracle(dtype, B, H, L, D, BLKQ, ratio):
    from oracle import sla_oracle as O
    from sla_b200 import ops
    g = torch.Generator().manual_seed(L * 7 + D)
    q, k, v, do = (torch.randn(B, H, L, D, generator=g).to(dtype) for _ in range(4))
    smap, lut, topk = O.get_block_map(q, k, ratio, BLKQ, 64)
    o_ref, lse_ref = O.sparse_fwd_gather(q, k, v, lut, BLKQ, 64, emulate=dtype)
    dq_r, dk_r, dv_r, delta_r = O.sparse_bwd_dense(q.float(), k.float(), v.float(), o_ref.float(), lse_ref,
                                                    do.float(), smap, BLKQ, 64)
    qg, kg, vg = (t.cuda().requires_grad_(True) for t in (q, k, v))
    o = ops._attention.apply(qg, kg, vg, smap.cuda(), lut.cuda(), topk, BLKQ, 64)
    o.backward(do.cuda())
    assert_close_parity(o.detach().cpu().float(), o_ref.float(), cos_min=0.9995, l1_max=6e-3, what="o_s")
    assert_close_parity(qg.grad.cpu().float(), dq_r, what="dq")
    assert_close_parity(kg.grad.cpu().float(), dk_r, what="dk")
    assert_close_parity(vg.grad.cpu().float(), dv_r, what="dv")


def test_lse_and_dense_limit():
    """topk_ratio = 1 selects every block: the operator must equal dense softmax attention, and its LSE
    the log2-sum-exp of the scaled scores (kernel.py:58,81)."""
    from sla_b200 import ops
    import ctypes as C
    from sla_b200._lib import check, lib
    g = torch.Generator().manual_seed(3)
    B, H, L, D = 1, 2, 520, 128
    q, k, v = (torch.randn(B, H, L, D, generator=g).bfloat16().cuda() for _ in range(3))
    bm = ops.block_map(q, k, 1.0, 64, 64)
    assert bm.topk == 9
    shape = ops.make_shape(B, H, L, D, 64, 64, bm.topk, torch.bfloat16, flags=1)
    o = torch.empty_like(q)
    lse = torch.empty(B, H, L, dtype=torch.float32, device="cuda")
    check(lib.sla_sparse_fwd(C.byref(shape), q.data_ptr(), k.data_ptr(), v.data_ptr(), bm.lut.data_ptr(),
                             o.data_ptr(), lse.data_ptr(), torch.cuda.current_stream().cuda_stream))
    s = (q.float() @ k.float().transpose(-1, -2)) * (D ** -0.5)
    ref = torch.softmax(s, -1) @ v.float()
    assert_close_parity(o.float().cpu(), ref.cpu(), cos_min=0.9995, l1_max=6e-3, what="dense limit")
    lse_ref = torch.logsumexp(s, -1) * 1.4426950408889634
    assert float((lse - lse_ref).abs().max()) < 2e-3


def test_lut_order_only_changes_rounding():
    from sla_b200 import ops
    g = torch.Generator().manual_seed(9)
    q, k, v = (torch.randn(1, 1, 1024, 64, generator=g).bfloat16().cuda() for _ in range(3))
    smap, lut, topk = ops.get_block_map(q, k, 0.5, 64, 64)
    a = ops._attention.apply(q, k, v, smap, lut, topk, 64, 64)
    perm = torch.randperm(topk, generator=g)
    b = ops._attention.apply(q, k, v, smap, lut[..., perm.cuda()].contiguous(), topk, 64, 64)
    assert_close_parity(a.float().cpu(), b.float().cpu(), cos_min=0.99999, l1_max=3e-3, what="lut order")


def test_reference_asserts_are_kept():
    from sla_b200 import ops
    q = torch.randn(1, 1, 128, 64, device="cuda").bfloat16()
    smap, lut, topk = ops.get_block_map(q, q, 0.5, 64, 64)
    with pytest.raises(AssertionError):
        ops._attention.apply(q, q, q, smap, lut, topk, 32, 64)     # kernel.py:247
    with pytest.raises(AssertionError):
        ops._attention.apply(q, q, q, smap, lut, topk, 64, 128)    # kernel.py:248
    with pytest.raises(AssertionError):
        ops._attention.apply(q.transpose(-1, -2), q, q, smap, lut, topk, 64, 64)  # kernel.py:243


@pytest.mark.parametrize("fused,D,BLKQ,L", [(False, 128, 64, 1000), (True, 128, 64, 1100), (True, 64, 128, 777)])
def test_forward_writes_its_output_to_gather_destinations(fused, D, BLKQ, L):
    """sla_fwd_gather: the epilogue's extra copies of the output, here into three other buffers of the same GPU
    standing in for peer GPUs' memory (two of them slices at an offset inside larger buffers, as a rank's place in
    a full-size output is). Every copy must equal o bit for bit, memory around the slices must stay untouched, and
    o itself must equal what sla_fwd gives."""
    import ctypes as C
    from sla_b200 import _lib, ops
    from sla_b200._lib import check, lib
    g = torch.Generator(device="cuda").manual_seed(L + D)
    B, H = 1, 2
    q, k, v = (torch.randn(B, H, L, D, generator=g, device="cuda").bfloat16() for _ in range(3))
    bm = ops.block_map(q, k, 0.25, BLKQ, 64)
    W = torch.randn(D, D, generator=g, device="cuda") * 0.05
    bias = torch.randn(D, generator=g, device="cuda") * 0.05
    flags = 0 if fused else _lib.FLAG_SPARSE_ONLY
    shape = ops.make_shape(B, H, L, D, BLKQ, 64, bm.topk, torch.bfloat16, "softmax", flags=flags)
    lse = torch.empty(B, H, L, dtype=torch.float32, device="cuda")
    lin_state = torch.empty(B, H, 2 * D * D + D, dtype=torch.bfloat16, device="cuda")
    ws = ops._workspace(shape, _lib.OP_FWD, "cuda")
    st = torch.cuda.current_stream().cuda_stream
    n = B * H * L * D

    def call(o, dst):
        arr = (C.c_void_p * len(dst))(*dst) if dst else None
        check(lib.sla_fwd_gather(C.byref(shape), q.data_ptr(), k.data_ptr(), v.data_ptr(), bm.lut.data_ptr(),
                                 W.data_ptr(), bias.data_ptr(), o.data_ptr(), None, lse.data_ptr(), lin_state.data_ptr(),
                                 ws.data_ptr(), ws.numel(), arr, len(dst), st))

    o_ref = torch.empty_like(q)
    check(lib.sla_fwd(C.byref(shape), q.data_ptr(), k.data_ptr(), v.data_ptr(), bm.lut.data_ptr(), W.data_ptr(),
                      bias.data_ptr(), o_ref.data_ptr(), None, lse.data_ptr(), lin_state.data_ptr(), ws.data_ptr(),
                      ws.numel(), st))
    o = torch.empty_like(q)
    plain = torch.full((n,), -7.0, dtype=torch.bfloat16, device="cuda")
    big1 = torch.full((3 * n,), -7.0, dtype=torch.bfloat16, device="cuda")
    big2 = torch.full((2 * n + 64,), -7.0, dtype=torch.bfloat16, device="cuda")
    call(o, [plain.data_ptr(), big1.data_ptr() + 2 * n, big2.data_ptr() + 2 * (n + 64)])
    torch.cuda.synchronize()
    assert torch.equal(o, o_ref)
    flat = o.flatten()
    assert torch.equal(plain, flat)
    assert torch.equal(big1[n:2 * n], flat) and bool((big1[:n] == -7.0).all()) and bool((big1[2 * n:] == -7.0).all())
    assert torch.equal(big2[n + 64:], flat) and bool((big2[:n + 64] == -7.0).all())
    # more than eight destinations, or the mma.sync kernels, are refused before anything is launched
    nine = (C.c_void_p * 9)(*([plain.data_ptr()] * 9))
    rc = lib.sla_fwd_gather(C.byref(shape), q.data_ptr(), k.data_ptr(), v.data_ptr(), bm.lut.data_ptr(), W.data_ptr(),
                            bias.data_ptr(), o.data_ptr(), None, lse.data_ptr(), lin_state.data_ptr(), ws.data_ptr(),
                            ws.numel(), nine, 9, st)
    assert rc == -10
