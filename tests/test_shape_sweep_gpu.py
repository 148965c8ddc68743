"""Edge shapes through the whole module (forward + backward through the C ABI) against the CPU oracle and its
autograd: sequence lengths around the 64- and 128-row tile boundaries, one block, every block selected
(topk ratio 1), odd union-list lengths, both block sizes, both head dimensions, fp16 and bf16, all feature maps,
several (batch, head) units. Tolerance as everywhere: cosine >= 0.999, relative L1 <= 1e-2 (2e-2 for dW, db)."""
import pytest
import torch

from helpers import assert_close_parity

pytestmark = pytest.mark.gpu

CASES = [
    # B, H, L,    D,   BLKQ, ratio, feature,   fp16
    (1, 1, 63,   64,  64,  1.0,  "softmax", False),   # a single ragged block
    (1, 1, 64,   128, 128, 1.0,  "relu",    False),   # half a 128-row tile
    (2, 1, 65,   128, 64,  0.5,  "elu",     False),   # two blocks, the second with one row; topk 1 of 2
    (1, 2, 129,  64,  128, 0.7,  "softmax", True),    # 128-row tiles with one row in the second
    (1, 1, 191,  128, 64,  0.34, "softmax", False),   # topk 1 of 3: union lists of length 1 or 2 (odd -> padded pair)
    (1, 2, 320,  128, 64,  1.0,  "softmax", False),   # every block selected: union == either list
    (1, 1, 700,  64,  64,  0.3,  "relu",    True),    # topk 3 of 11
    (2, 2, 1025, 128, 128, 0.2,  "elu",     False),   # 9 query tiles, 17 KV blocks, last of each ragged
    (1, 3, 1536, 128, 64,  0.13, "softmax", False),   # topk 3 of 24, three heads
    (1, 1, 2049, 64,  128, 0.08, "softmax", False),   # topk 2 of 33
    (1, 2, 900,  128, 64,  0.25, "softmax", True),    # fp16 at head dim 128 (tcgen05 linear backward in fp16)
    (1, 1, 1300, 128, 128, 0.3,  "relu",    True),    # same, relu feature map, three row chunks in the linear passes
]


@pytest.mark.parametrize("B,H,L,D,BLKQ,ratio,feat,fp16", CASES)
def test_module_forward_backward_edge_shapes(B, H, L, D, BLKQ, ratio, feat, fp16):
    import sla_b200
    from oracle import sla_oracle as O
    dt = torch.float16 if fp16 else torch.bfloat16
    g = torch.Generator().manual_seed(1000 * L + D + BLKQ)
    q, k, v, do = (torch.randn(B, H, L, D, generator=g).to(dt) for _ in range(4))
    w = torch.randn(D, D, generator=g) * 0.05
    b = torch.randn(D, generator=g) * 0.05
    m = sla_b200.SparseLinearAttention(D, ratio, feat, BLKQ, 64, use_bf16=not fp16).cuda()
    with torch.no_grad():
        m.proj_l.weight.copy_(w)
        m.proj_l.bias.copy_(b)
    qg, kg, vg = (t.cuda().requires_grad_(True) for t in (q, k, v))
    o = m(qg, kg, vg)
    o.backward(do.cuda())
    for t in (o, qg.grad, kg.grad, vg.grad, m.proj_l.weight.grad, m.proj_l.bias.grad):
        assert torch.isfinite(t.float()).all()
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
