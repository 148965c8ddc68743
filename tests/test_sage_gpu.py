"""GPU checks of the SageSLA quantized forward (sage_sla_fwd through the C ABI / module).
The reference's quantized kernels live in the un-vendored spas_sage_attn package, so parity at that
boundary is unpinned; the checks are (i) against this repository's CPU restatement of the same
quantization recipe, (ii) against the un-quantized 16-bit path (cosine >= 0.995, the bar for the
quantized path), (iii) the whole module against the oracle module forward."""
import pytest
import torch

from helpers import assert_close_parity, cos_sim

pytestmark = pytest.mark.gpu


def _inputs(B, H, L, D, seed, k_offset=0.0):
    g = torch.Generator().manual_seed(seed)
    q, k, v = (torch.randn(B, H, L, D, generator=g) for _ in range(3))
    k = k + k_offset * torch.randn(1, H, 1, D, generator=g)
    return q.bfloat16(), k.bfloat16(), v.bfloat16()


@pytest.mark.parametrize("B,H,L,ratio,koff,D", [(1, 2, 1000, 0.3, 0.0, 128), (2, 1, 2500, 0.1, 2.0, 128),
                                                (1, 1, 128, 1.0, 0.5, 128), (1, 1, 1104, 0.25, 1.0, 128),
                                                (1, 2, 1000, 0.3, 0.5, 64), (2, 1, 1931, 0.15, 1.0, 64)])
def test_sage_sparse_branch(B, H, L, ratio, koff, D):
    from oracle import sla_oracle as O
    from sla_b200 import ops
    q, k, v = _inputs(B, H, L, D, L, koff)
    w = torch.zeros(D, D, device="cuda")
    bm = ops.block_map(q.cuda(), k.cuda(), ratio, 128, 64)
    got = ops.sage_sla_attention(q.cuda(), k.cuda(), v.cuda(), w, None, bm, sparse_only=True).float().cpu()
    lut = bm.lut.cpu().long()
    ref_q = O.sage_sparse_fwd(q, k, v, lut, 128, 64, p_scale=32.0)
    ref_f, _ = O.sparse_fwd_gather(q, k, v, lut, 128, 64)
    assert torch.isfinite(got).all()
    # The kernel lets the running maximum in the exponent lag the true one by up to 2^3 before it rescales O, so
    # its e4m3 rounding points differ from the oracle's (exact maximum): the two quantized results agree to
    # about sqrt(2) x the quantization noise, and the kernel must be as close to the un-quantized result as the
    # oracle's recipe is.
    assert_close_parity(got, ref_q, cos_min=0.999, l1_max=5e-2, what="vs quantized oracle")
    assert cos_sim(got, ref_f) >= 0.995, "vs un-quantized sparse attention"
    from helpers import rel_l1
    assert rel_l1(got, ref_f) <= 1.1 * rel_l1(ref_q, ref_f) + 2e-3, (rel_l1(got, ref_f), rel_l1(ref_q, ref_f))


@pytest.mark.parametrize("D,feature", [(128, "softmax"), (64, "softmax"), (64, "elu")])
def test_sage_module_matches_oracle_and_16bit_module(D, feature):
    import sla_b200
    from oracle import sla_oracle as O
    B, H, L = 1, 2, 1500
    q, k, v = _inputs(B, H, L, D, 7, 1.0)
    g = torch.Generator().manual_seed(3)
    w, b = torch.randn(D, D, generator=g) * 0.05, torch.randn(D, generator=g) * 0.05
    sage = sla_b200.SageSparseLinearAttention(D, 0.2, feature).cuda()
    full = sla_b200.SparseLinearAttention(D, 0.2, feature, BLKQ=128, BLKK=64).cuda()
    for m in (sage, full):
        with torch.no_grad():
            m.proj_l.weight.copy_(w)
            m.proj_l.bias.copy_(b)
    with torch.no_grad():
        o_sage, sp = sage(q.cuda(), k.cuda(), v.cuda(), return_sparsity=True)
        o_full = full(q.cuda(), k.cuda(), v.cuda())
    assert o_sage.dtype == torch.bfloat16 and sp == 4 / 24
    ref = O.sla_forward(q, k, v, w, b, 0.2, feature, 128, 64, torch.bfloat16)
    assert cos_sim(o_sage.float().cpu(), ref.float()) >= 0.995
    assert cos_sim(o_sage.float().cpu(), o_full.float().cpu()) >= 0.995


def test_sage_rejects_other_block_sizes_and_head_dims():
    import sla_b200
    with pytest.raises(ValueError):
        sla_b200.SageSparseLinearAttention(128, 0.2, BLKQ=64, BLKK=64)
    m = sla_b200.SageSparseLinearAttention(32, 0.5).cuda()
    x = torch.randn(1, 1, 256, 32, device="cuda").bfloat16()
    with pytest.raises(AssertionError):      # SageSLA/core.py:112
        m(x, x, x)


def test_sage_prepare_on_side_stream_changes_nothing():
    """The module runs sage_sla_prepare (quantized copies + linear-branch state) on a second stream next to the
    block map and calls sage_sla_fwd with SLA_FLAG_STATE_READY: same kernels, bit-identical output."""
    import sla_b200
    q, k, v = _inputs(1, 2, 1300, 128, 21, 1.0)
    m = sla_b200.SageSparseLinearAttention(128, 0.25, "softmax").cuda()
    with torch.no_grad():
        m.proj_l.weight.copy_(torch.randn(128, 128, generator=torch.Generator().manual_seed(2)) * 0.05)
    outs = []
    for overlap in (True, False):
        m.overlap_prepare = overlap
        with torch.no_grad():
            outs.append(m(q.cuda(), k.cuda(), v.cuda()))
        torch.cuda.synchronize()
    assert torch.equal(outs[0], outs[1])


@pytest.mark.parametrize("D,feature,L", [(128, "softmax", 1500), (64, "relu", 1100), (128, "elu", 777)])
def test_sage_module_backward_is_the_linear_branch(D, feature, L):
    """In the reference only the quantized o_s is a constant of the graph (SageSLA/core.py:114-146); the linear
    branch and proj_l after it (SageSLA/core.py:148-158) are ordinary autograd ops. The module's gradients must
    equal the oracle autograd (fp64) of  proj_l(calc_linear(phi(q), phi(k), v))  alone."""
    import sla_b200
    from oracle import sla_oracle as O
    B, H = 1, 2
    q, k, v = _inputs(B, H, L, D, L + 1, 0.5)
    g = torch.Generator().manual_seed(L)
    do = torch.randn(B, H, L, D, generator=g).bfloat16()
    w, b = torch.randn(D, D, generator=g) * 0.05, torch.randn(D, generator=g) * 0.05
    m = sla_b200.SageSparseLinearAttention(D, 0.2, feature).cuda()
    with torch.no_grad():
        m.proj_l.weight.copy_(w)
        m.proj_l.bias.copy_(b)
    qg, kg, vg = (t.cuda().requires_grad_(True) for t in (q, k, v))
    o = m(qg, kg, vg)
    with torch.no_grad():
        o_nograd = m(q.cuda(), k.cuda(), v.cuda())
    assert torch.equal(o.detach(), o_nograd)
    o.backward(do.cuda())
    qd, kd, vd = (t.double().requires_grad_(True) for t in (q, k, v))
    wd, bd = w.double().requires_grad_(True), b.double().requires_grad_(True)
    o_l = O.calc_linear(O.feature_map(qd, feature), O.feature_map(kd, feature), vd)
    (o_l @ wd.t() + bd).backward(do.double())
    assert_close_parity(qg.grad.float().cpu(), qd.grad, what="dq")
    assert_close_parity(kg.grad.float().cpu(), kd.grad, what="dk")
    assert_close_parity(vg.grad.float().cpu(), vd.grad, what="dv")
    assert_close_parity(m.proj_l.weight.grad.cpu(), wd.grad, l1_max=2e-2, what="dw")
    assert_close_parity(m.proj_l.bias.grad.cpu(), bd.grad, l1_max=2e-2, what="db")


@pytest.mark.parametrize("D,L", [(128, 1100), (64, 900)])
def test_sage_forward_writes_its_output_to_gather_destinations(D, L):
    """sage_sla_fwd_gather on one GPU: two other buffers stand in for peer GPUs' memory (one of them a slice at an
    offset inside a larger buffer). Each copy must equal o bit for bit, o must equal what sage_sla_fwd gives, and
    memory around the slice must stay untouched."""
    from sla_b200 import ops
    B, H = 1, 2
    q, k, v = (t.cuda() for t in _inputs(B, H, L, D, L, 0.5))
    g = torch.Generator().manual_seed(L)
    w = (torch.randn(D, D, generator=g) * 0.05).cuda()
    b = (torch.randn(D, generator=g) * 0.05).cuda()
    bm = ops.block_map(q, k, 0.25, 128, 64)
    with torch.no_grad():
        ref = ops.sage_sla_attention(q, k, v, w, b, bm)
        n = q.numel()
        plain = torch.full((n,), -7.0, dtype=torch.bfloat16, device="cuda")
        big = torch.full((3 * n,), -7.0, dtype=torch.bfloat16, device="cuda")
        o = ops.sage_sla_attention(q, k, v, w, b, bm, gather_ptrs=[plain.data_ptr(), big.data_ptr() + 2 * n])
    torch.cuda.synchronize()
    assert torch.equal(o, ref)
    assert torch.equal(plain, ref.flatten())
    assert torch.equal(big[n:2 * n], ref.flatten()) and bool((big[:n] == -7.0).all()) and bool((big[2 * n:] == -7.0).all())
