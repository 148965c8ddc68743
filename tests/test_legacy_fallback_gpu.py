"""The mma.sync kernels (`SLA_FLAG_LEGACY_MMA`) are the fallback for shapes whose block lists do not fit the
tcgen05 kernels' shared memory. Both ways into them are tested against the CPU oracle with the bars of the
tcgen05 path (cosine >= 0.999, relative L1 <= 1e-2; 2e-2 for dW, db): the flag on small shapes, and a shape that
takes the fallback by itself (M_BLOCKS above the dK/dV kernel's list budget at D = 128)."""
import ctypes as C

import pytest
import torch

from helpers import assert_close_parity

pytestmark = pytest.mark.gpu


def _path(B, H, L, D, BLKQ, topk, op, flags=0):
    from sla_b200 import _lib, ops
    shape = ops.make_shape(B, H, L, D, BLKQ, 64, topk, torch.bfloat16, flags=flags)
    return _lib.lib.sla_kernel_path(C.byref(shape), op)


@pytest.mark.parametrize("dtype,B,H,L,D,BLKQ,ratio", [
    (torch.bfloat16, 1, 2, 1024, 128, 64, 0.25),
    (torch.bfloat16, 2, 1, 1000, 64, 128, 0.3),
    (torch.float16, 1, 1, 65, 64, 64, 1.0),
    (torch.bfloat16, 1, 1, 127, 128, 128, 0.5),
])
def test_attention_with_legacy_flag(dtype, B, H, L, D, BLKQ, ratio, monkeypatch):
    from oracle import sla_oracle as O
    from sla_b200 import _lib, ops
    monkeypatch.setattr(ops._attention, "impl_flags", _lib.FLAG_LEGACY_MMA)
    g = torch.Generator().manual_seed(L * 7 + D)
    q, k, v, do = (torch.randn(B, H, L, D, generator=g).to(dtype) for _ in range(4))
    smap, lut, topk = O.get_block_map(q, k, ratio, BLKQ, 64)
    assert _path(B, H, L, D, BLKQ, topk, _lib.OP_SPARSE_BWD, _lib.FLAG_LEGACY_MMA) == 1
    o_ref, lse_ref = O.sparse_fwd_gather(q, k, v, lut, BLKQ, 64, emulate=dtype)
    dq_r, dk_r, dv_r, _ = O.sparse_bwd_dense(q.float(), k.float(), v.float(), o_ref.float(), lse_ref, do.float(),
                                             smap, BLKQ, 64)
    qg, kg, vg = (t.cuda().requires_grad_(True) for t in (q, k, v))
    o = ops._attention.apply(qg, kg, vg, smap.cuda(), lut.cuda(), topk, BLKQ, 64)
    o.backward(do.cuda())
    assert_close_parity(o.detach().cpu().float(), o_ref.float(), cos_min=0.9995, l1_max=6e-3, what="o_s")
    assert_close_parity(qg.grad.cpu().float(), dq_r, what="dq")
    assert_close_parity(kg.grad.cpu().float(), dk_r, what="dk")
    assert_close_parity(vg.grad.cpu().float(), dv_r, what="dv")


@pytest.mark.parametrize("B,H,L,D,BLKQ,ratio,feat,fp16", [
    (1, 2, 320, 128, 64, 1.0, "softmax", False),
    (1, 1, 700, 64, 64, 0.3, "relu", True),
    (2, 2, 1025, 128, 128, 0.2, "elu", False),
    (1, 1, 2049, 64, 128, 0.08, "softmax", False),
    (1, 1, 1300, 128, 128, 0.3, "relu", True),
])
def test_module_with_legacy_flag(B, H, L, D, BLKQ, ratio, feat, fp16):
    """Whole module on the mma.sync kernels: sparse forward with the fused read-out, both linear backward
    passes (dq; dk, dv) and the mma.sync sparse backward that adds to them."""
    import sla_b200
    from oracle import sla_oracle as O
    from sla_b200 import _lib
    dt = torch.float16 if fp16 else torch.bfloat16
    g = torch.Generator().manual_seed(1000 * L + D + BLKQ)
    q, k, v, do = (torch.randn(B, H, L, D, generator=g).to(dt) for _ in range(4))
    w = torch.randn(D, D, generator=g) * 0.05
    b = torch.randn(D, generator=g) * 0.05
    m = sla_b200.SparseLinearAttention(D, ratio, feat, BLKQ, 64, use_bf16=not fp16).cuda()
    m.impl_flags |= _lib.FLAG_LEGACY_MMA
    with torch.no_grad():
        m.proj_l.weight.copy_(w)
        m.proj_l.bias.copy_(b)
    qg, kg, vg = (t.cuda().requires_grad_(True) for t in (q, k, v))
    o = m(qg, kg, vg)
    o.backward(do.cuda())
    o_ref, parts = O.sla_forward(q, k, v, w, b, ratio, feat, BLKQ, 64, dt, return_parts=True)
    assert_close_parity(o.detach().float().cpu(), o_ref.float(), what="o")
    qd, kd, vd = (t.double().requires_grad_(True) for t in (q, k, v))
    wd, bd = w.double().requires_grad_(True), b.double().requires_grad_(True)
    O.sla_forward_fp(qd, kd, vd, wd, bd, parts["sparse_map"], feat, BLKQ, 64).backward(do.double())
    assert_close_parity(qg.grad.float().cpu(), qd.grad, what="dq")
    assert_close_parity(kg.grad.float().cpu(), kd.grad, what="dk")
    assert_close_parity(vg.grad.float().cpu(), vd.grad, what="dv")
    assert_close_parity(m.proj_l.weight.grad.cpu(), wd.grad, l1_max=2e-2, what="dw")
    assert_close_parity(m.proj_l.bias.grad.cpu(), bd.grad, l1_max=2e-2, what="db")


def test_backward_falls_back_by_itself_on_long_sequences():
    """L = 98,500 at BLKQ = 64, D = 128 has 1,540 query blocks: a KV block's column list may then be too long
    for the tcgen05 dK/dV kernel's shared memory, so the backward takes the mma.sync kernels without being
    asked, while the forward stays on tcgen05. Checked against the oracle's block-gather evaluation and its
    autograd (fp32) on one head."""
    import sla_b200
    from oracle import sla_oracle as O
    from sla_b200 import _lib
    B, H, L, D, BLKQ, ratio = 1, 1, 98500, 128, 64, 0.008
    nb = (L + 63) // 64
    topk = O.topk_count(nb, ratio)
    assert _path(B, H, L, D, BLKQ, topk, _lib.OP_FWD) == 0
    assert _path(B, H, L, D, BLKQ, topk, _lib.OP_BWD) == 1
    assert _path(B, H, 98000, D, BLKQ, topk, _lib.OP_BWD) == 0
    g = torch.Generator().manual_seed(98500)
    q, k, v, do = (torch.randn(B, H, L, D, generator=g).bfloat16() for _ in range(4))
    w = torch.randn(D, D, generator=g) * 0.05
    b = torch.randn(D, generator=g) * 0.05
    m = sla_b200.SparseLinearAttention(D, ratio, "softmax", BLKQ, 64).cuda()
    with torch.no_grad():
        m.proj_l.weight.copy_(w)
        m.proj_l.bias.copy_(b)
    qg, kg, vg = (t.cuda().requires_grad_(True) for t in (q, k, v))
    o = m(qg, kg, vg)
    o.backward(do.cuda())
    _, lut, _ = O.get_block_map(q, k, ratio, BLKQ, 64)
    qf, kf, vf = (t.float().requires_grad_(True) for t in (q, k, v))
    wf, bf = w.clone().requires_grad_(True), b.clone().requires_grad_(True)
    o_ref = O.sla_forward_gather_fp(qf, kf, vf, wf, bf, lut, "softmax", BLKQ, 64)
    o_ref.backward(do.float())
    assert_close_parity(o.detach().float().cpu(), o_ref.detach(), what="o")
    assert_close_parity(qg.grad.float().cpu(), qf.grad, what="dq")
    assert_close_parity(kg.grad.float().cpu(), kf.grad, what="dk")
    assert_close_parity(vg.grad.float().cpu(), vf.grad, what="dv")
    assert_close_parity(m.proj_l.weight.grad.cpu(), wf.grad, l1_max=2e-2, what="dw")
    assert_close_parity(m.proj_l.bias.grad.cpu(), bf.grad, l1_max=2e-2, what="db")
