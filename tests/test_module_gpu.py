"""GPU parity of the whole module (SparseLinearAttention forward + backward through the C ABI)
against the reference's golden vectors and the CPU oracle; tolerance cosine >= 0.999, relL1 <= 1e-2."""
import numpy as np
import pytest
import torch

from helpers import DT, assert_close_parity, load_golden, unpack

pytestmark = pytest.mark.gpu

MODULE = ["module_bf16_softmax", "module_fp16_relu", "module_fp32in_elu_blkq128"]


def _module(D, ratio, feat, BLKQ, BLKK, use_bf16, w, b):
    import sla_b200
    m = sla_b200.SparseLinearAttention(D, ratio, feat, BLKQ, BLKK, use_bf16=use_bf16).cuda()
    with torch.no_grad():
        m.proj_l.weight.copy_(w)
        m.proj_l.bias.copy_(b)
    return m


@pytest.mark.parametrize("name", MODULE)
def test_module_vs_reference_golden(name):
    g = load_golden(name)
    B, H, L, D, BLKQ, BLKK, _, _ = g["meta"].tolist()
    in_dt = DT[str(g["in_dtype"])]
    use_bf16 = str(g["compute"]) == "bf16"
    m = _module(D, float(g["ratio"]), str(g["feature"]), BLKQ, BLKK, use_bf16,
                torch.from_numpy(g["w"]), torch.from_numpy(g["bias"]))
    q, k, v = (unpack(g[n], in_dt).cuda().requires_grad_(True) for n in ("q", "k", "v"))
    o, sparsity = m(q, k, v, return_sparsity=True)
    assert o.dtype == in_dt and sparsity == float(g["sparsity"])
    assert_close_parity(o.detach().float().cpu(), unpack(g["o"], in_dt).float(), what=name + ".o")
    o.backward(unpack(g["do"], in_dt).cuda())
    for t, n in ((q, "dq"), (k, "dk"), (v, "dv")):
        assert t.grad.dtype == in_dt
        assert_close_parity(t.grad.float().cpu(), unpack(g[n], in_dt).float(), what=f"{name}.{n}")
    assert_close_parity(m.proj_l.weight.grad.cpu(), torch.from_numpy(g["dw"]), l1_max=2e-2, what=name + ".dw")
    assert_close_parity(m.proj_l.bias.grad.cpu(), torch.from_numpy(g["db"]), l1_max=2e-2, what=name + ".db")


def test_module_c1_configuration():
    """B=1,H=2,L=1024,D=64 fp32 inputs from seed 0, BLKQ=BLKK=64, topk=0.25, softmax, W~N(0,0.02)."""
    g = load_golden("module_c1")
    torch.manual_seed(0)
    q, k, v = torch.randn(1, 2, 1024, 64), torch.randn(1, 2, 1024, 64), torch.randn(1, 2, 1024, 64)
    w = torch.randn(64, 64) * 0.02
    m = _module(64, 0.25, "softmax", 64, 64, True, w, torch.zeros(64))
    with torch.no_grad():
        o = m(q.cuda(), k.cuda(), v.cuda())
    assert o.dtype == torch.float32
    assert_close_parity(o.cpu(), torch.from_numpy(g["o"]), what="c1.o")


def test_zero_init_means_sparse_only():
    """proj_l is zero-initialised (core.py:64-67): a fresh module returns exactly the sparse branch."""
    import sla_b200
    from sla_b200 import ops
    g = torch.Generator().manual_seed(2)
    q, k, v = (torch.randn(1, 2, 1000, 128, generator=g).bfloat16().cuda() for _ in range(3))
    m = sla_b200.SparseLinearAttention(128, 0.2).cuda()
    with torch.no_grad():
        o = m(q, k, v)
    smap, lut, topk = ops.get_block_map(q, k, 0.2, 64, 64)
    o_s = ops._attention.apply(q, k, v, smap, lut, topk, 64, 64)
    assert torch.equal(o, o_s)


@pytest.mark.parametrize("feat,D,BLKQ,L", [("softmax", 128, 64, 1536), ("relu", 64, 128, 1100), ("elu", 128, 128, 900)])
def test_module_vs_oracle_autograd(feat, D, BLKQ, L):
    from oracle import sla_oracle as O
    g = torch.Generator().manual_seed(L)
    B, H = 1, 2
    q, k, v, do = (torch.randn(B, H, L, D, generator=g).bfloat16() for _ in range(4))
    w = torch.randn(D, D, generator=g) * 0.05
    b = torch.randn(D, generator=g) * 0.05
    m = _module(D, 0.3, feat, BLKQ, 64, True, w, b)
    qg, kg, vg = (t.cuda().requires_grad_(True) for t in (q, k, v))
    o = m(qg, kg, vg)
    o.backward(do.cuda())
    o_ref, parts = O.sla_forward(q, k, v, w, b, 0.3, feat, BLKQ, 64, torch.bfloat16, return_parts=True)
    assert_close_parity(o.detach().float().cpu(), o_ref.float(), what="o")
    qd, kd, vd = (t.double().requires_grad_(True) for t in (q, k, v))
    wd, bd = w.double().requires_grad_(True), b.double().requires_grad_(True)
    O.sla_forward_fp(qd, kd, vd, wd, bd, parts["sparse_map"], feat, BLKQ, 64).backward(do.double())
    assert_close_parity(qg.grad.float().cpu(), qd.grad, what="dq")
    assert_close_parity(kg.grad.float().cpu(), kd.grad, what="dk")
    assert_close_parity(vg.grad.float().cpu(), vd.grad, what="dv")
    assert_close_parity(m.proj_l.weight.grad.cpu(), wd.grad, l1_max=2e-2, what="dw")
    assert_close_parity(m.proj_l.bias.grad.cpu(), bd.grad, l1_max=2e-2, what="db")


def test_determinism_and_readme_shape():
    """README usage shape (B=2,H=4,L=4096,D=128, topk=0.2): runs, is bitwise repeatable, finite."""
    import sla_b200
    from sla_b200 import synthetic
    w = synthetic.WORKLOADS["c2"]
    q, k, v, do = synthetic.make_inputs(w, "cuda")
    W, b = synthetic.make_proj(w, "cuda")
    m = _module(128, 0.2, "softmax", 64, 64, True, W, b)
    outs = []
    for _ in range(2):
        qg, kg, vg = (t.clone().requires_grad_(True) for t in (q, k, v))
        o = m(qg, kg, vg)
        o.backward(do)
        outs.append((o.detach(), qg.grad, kg.grad, vg.grad))
        m.proj_l.weight.grad = None
    for a, bb in zip(*outs):
        assert torch.isfinite(a.float()).all() and torch.equal(a, bb)


def test_full_size_linearity_in_v_c3_head():
    """Full-size property on one L=32760 head: the operator is linear in V for a fixed block map, and
    with V = const every output row equals that constant (softmax rows sum to one)."""
    from sla_b200 import ops, synthetic
    w = synthetic.WORKLOADS["c3"]
    q, k, v, _ = synthetic.make_inputs(w, "cuda", units=[3], with_do=False)
    smap, lut, topk = ops.get_block_map(q, k, w.topk, 64, 64)
    ones = torch.full_like(v, 0.5)
    o1 = ops._attention.apply(q, k, ones, smap, lut, topk, 64, 64)
    assert float((o1.float() - 0.5).abs().max()) < 4e-3
    a = ops._attention.apply(q, k, v, smap, lut, topk, 64, 64).float()
    b = ops._attention.apply(q, k, (2 * v), smap, lut, topk, 64, 64).float()
    assert_close_parity(b.cpu(), (2 * a).cpu(), cos_min=0.99999, l1_max=1e-3, what="linearity")


@pytest.mark.parametrize("feat,D,BLKQ,L,ratio", [("softmax", 128, 64, 2000, 0.1), ("relu", 64, 128, 1100, 0.25),
                                                 ("elu", 128, 128, 900, 0.2), ("softmax", 64, 64, 1024, 0.25)])
def test_unselected_scope_vs_oracle(feat, D, BLKQ, L, ratio):
    """linear_scope='unselected' (not in the reference's code: unpinned; checked against the CPU restatement,
    which sums per-block states over the blocks a query block did not select). The linear part alone
    (o - o_s) must agree too, so proj_l is given weights large enough for it to matter."""
    import sla_b200
    from oracle import sla_oracle as O
    g = torch.Generator().manual_seed(L + D)
    B, H = 1, 2
    q, k, v = (torch.randn(B, H, L, D, generator=g).bfloat16() for _ in range(3))
    w = torch.randn(D, D, generator=g) / D ** 0.5
    b = torch.randn(D, generator=g) * 0.05
    m = sla_b200.SparseLinearAttention(D, ratio, feat, BLKQ, 64, linear_scope="unselected").cuda()
    with torch.no_grad():
        m.proj_l.weight.copy_(w)
        m.proj_l.bias.copy_(b)
        o = m(q.cuda(), k.cuda(), v.cuda()).float().cpu()
    o_ref, parts = O.sla_forward(q, k, v, w, b, ratio, feat, BLKQ, 64, linear_scope="unselected", return_parts=True)
    assert_close_parity(o, o_ref.float(), what="unselected.o")
    lin, lin_ref = o - parts["o_s"].float(), o_ref.float() - parts["o_s"].float()
    assert_close_parity(lin, lin_ref, cos_min=0.995, l1_max=5e-2, what="unselected.linear_part")
    # and it differs from the all-token scope (the test would pass vacuously otherwise)
    o_all = O.sla_forward(q, k, v, w, b, ratio, feat, BLKQ, 64, linear_scope="all").float()
    assert (o_all - o_ref.float()).abs().mean() > 5 * (o - o_ref.float()).abs().mean()


@pytest.mark.parametrize("fork", [False, True])
def test_forward_is_cuda_graph_capturable(fork):
    """The whole forward (block map, linear state, fused tcgen05 kernel) enqueues on the caller's stream, or on a
    second stream that forks from it and joins it again (fork=True), and never synchronises (the top-k count comes
    from shapes, utils.py:61-62), so it can be captured into a CUDA graph; the replay must reproduce the eager
    result bit for bit."""
    import sla_b200
    g = torch.Generator().manual_seed(11)
    q, k, v = (torch.randn(1, 2, 2048, 128, generator=g).bfloat16().cuda() for _ in range(3))
    m = sla_b200.SparseLinearAttention(128, 0.1).cuda()
    m.overlap_linear_state = fork
    with torch.no_grad():
        m.proj_l.weight.copy_(torch.randn(128, 128, generator=g) * 0.05)
        eager = m(q, k, v)
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            m(q, k, v)                      # warm-up on the side stream (function attributes, symbol lookups)
        torch.cuda.current_stream().wait_stream(s)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            out = m(q, k, v)
        out.zero_()
        graph.replay()
        torch.cuda.synchronize()
    assert torch.equal(out, eager)


def test_graphed_forward_backward_matches_eager():
    """Forward AND backward captured into CUDA graphs (sla_b200.graphed) reproduce the eager results. The graphed
    module is captured before anything else touches its parameters (autograd nodes created earlier on another
    stream would break the capture); a twin module with the same weights gives the eager results."""
    import sla_b200
    g = torch.Generator().manual_seed(12)
    q, k, v, do = (torch.randn(2, 2, 1024, 128, generator=g).bfloat16().cuda() for _ in range(4))
    w = torch.randn(128, 128, generator=g) * 0.05
    m_graph = sla_b200.SparseLinearAttention(128, 0.2).cuda()
    m_eager = sla_b200.SparseLinearAttention(128, 0.2).cuda()
    m_graph.overlap_linear_state = True     # the fork to the second stream is captured too
    with torch.no_grad():
        m_graph.proj_l.weight.copy_(w)
        m_eager.proj_l.weight.copy_(w)
    qg, kg, vg = (t.clone().requires_grad_(True) for t in (q, k, v))
    fast = sla_b200.graphed(m_graph, qg, kg, vg)
    m_graph.proj_l.weight.grad = m_graph.proj_l.bias.grad = None
    og = fast(qg, kg, vg)
    og.backward(do)
    qe, ke, ve = (t.clone().requires_grad_(True) for t in (q, k, v))
    oe = m_eager(qe, ke, ve)
    oe.backward(do)
    torch.cuda.synchronize()
    assert torch.equal(og, oe)
    for a, b in ((qg.grad, qe.grad), (kg.grad, ke.grad), (vg.grad, ve.grad),
                 (m_graph.proj_l.weight.grad, m_eager.proj_l.weight.grad)):
        assert torch.equal(a, b)


@pytest.mark.parametrize("D,BLKQ,L,feat", [(128, 64, 1500, "softmax"), (64, 128, 1000, "elu")])
def test_linear_state_on_side_stream_changes_nothing(D, BLKQ, L, feat):
    """The module launches the linear-branch state (sla_fwd_prepare) on a second stream next to the block map and
    calls sla_fwd with SLA_FLAG_STATE_READY: same kernels on the same data, so forward and gradients are
    bit-identical to the single-stream order."""
    import sla_b200
    g = torch.Generator().manual_seed(11)
    q, k, v, do = (torch.randn(1, 2, L, D, generator=g).bfloat16().cuda() for _ in range(4))
    m2 = sla_b200.SparseLinearAttention(D, 0.2, feat, BLKQ, 64).cuda()
    res = {}
    for overlap in (True, False):
        m2.overlap_linear_state = overlap
        with torch.no_grad():
            m2.proj_l.weight.copy_(torch.randn(D, D, generator=torch.Generator().manual_seed(5)) * 0.05)
            m2.proj_l.bias.fill_(0.01)
        m2.zero_grad()
        qg, kg, vg = (t.clone().requires_grad_(True) for t in (q, k, v))
        o = m2(qg, kg, vg)
        o.backward(do)
        torch.cuda.synchronize()
        res[overlap] = (o.detach(), qg.grad, kg.grad, vg.grad, m2.proj_l.weight.grad.clone(), m2.proj_l.bias.grad.clone())
    for a, b in zip(res[True], res[False]):
        assert torch.equal(a, b)


def test_block_map_reuse_and_packed_form():
    """A map predicted once (`predict_block_map`) and handed back to `forward` gives the bits of a forward that
    predicts it itself, forward and backward, also after a round trip through the 16-bit packed form; a map for
    another shape is refused."""
    import sla_b200
    g = torch.Generator().manual_seed(17)
    B, H, L, D = 1, 2, 2100, 128
    q, k, v, do = (torch.randn(B, H, L, D, generator=g).bfloat16().cuda() for _ in range(4))
    m = _module(D, 0.15, "softmax", 64, 64, True, torch.randn(D, D, generator=g) * 0.05,
                torch.randn(D, generator=g) * 0.05)

    def run(**kw):
        a, b, c = (t.clone().requires_grad_(True) for t in (q, k, v))
        o = m(a, b, c, **kw)
        o.backward(do)
        out = (o.detach(), a.grad, b.grad, c.grad, m.proj_l.weight.grad.clone())
        m.proj_l.weight.grad = m.proj_l.bias.grad = None
        return out

    ref = run()
    bm = m.predict_block_map(q, k)
    packed = bm.pack16()
    assert packed.lut16.dtype == torch.int16 and packed.lut16.numel() == bm.lut.numel()
    assert torch.equal(packed.unpack().lut, bm.lut) and torch.equal(packed.unpack().col_index, bm.col_index)
    for kw in (dict(block_map=bm), dict(block_map=packed)):
        for a, r in zip(run(**kw), ref):
            assert torch.equal(a, r)
    with torch.no_grad():
        o2, sp = m(q, k, v, return_sparsity=True, block_map=m.predict_block_map(q, k, with_column_lists=False))
    assert torch.equal(o2, ref[0]) and sp == bm.topk / bm.n_blocks
    with pytest.raises(ValueError):
        m(q[:, :1], k[:, :1], v[:, :1], block_map=bm)


@pytest.mark.parametrize("feat,D,BLKQ,L,ratio,fp16", [
    ("softmax", 128, 64, 2000, 0.1, False), ("relu", 64, 128, 1100, 0.25, False), ("elu", 128, 128, 900, 0.2, False),
    ("softmax", 64, 64, 1024, 0.25, True), ("softmax", 128, 64, 320, 1.0, False), ("relu", 128, 64, 191, 0.34, False)])
def test_unselected_scope_backward_vs_oracle_autograd(feat, D, BLKQ, L, ratio, fp16):
    """Gradients of linear_scope='unselected' (unpinned: no reference code has this scope) against the fp64
    autograd of the CPU restatement, which sums per-block states over the blocks a query block did not select.
    proj_l is given weights large enough for the linear branch to carry a fair share of every gradient. The case
    with ratio 1 selects every block: the branch is then defined as 0 and only the bias gradient flows through it."""
    import sla_b200
    from oracle import sla_oracle as O
    dt = torch.float16 if fp16 else torch.bfloat16
    g = torch.Generator().manual_seed(3 * L + D)
    B, H = 1, 2
    q, k, v, do = (torch.randn(B, H, L, D, generator=g).to(dt) for _ in range(4))
    w = torch.randn(D, D, generator=g) / D ** 0.5
    b = torch.randn(D, generator=g) * 0.05
    m = sla_b200.SparseLinearAttention(D, ratio, feat, BLKQ, 64, use_bf16=not fp16, linear_scope="unselected").cuda()
    with torch.no_grad():
        m.proj_l.weight.copy_(w)
        m.proj_l.bias.copy_(b)
    qg, kg, vg = (t.cuda().requires_grad_(True) for t in (q, k, v))
    o = m(qg, kg, vg)
    o.backward(do.cuda())
    smap, _, _ = O.get_block_map(q, k, ratio, BLKQ, 64)
    qd, kd, vd = (t.double().requires_grad_(True) for t in (q, k, v))
    wd, bd = w.double().requires_grad_(True), b.double().requires_grad_(True)
    o_ref = O.sla_forward_fp(qd, kd, vd, wd, bd, smap, feat, BLKQ, 64, linear_scope="unselected")
    o_ref.backward(do.double())
    assert_close_parity(o.detach().float().cpu(), o_ref.detach(), what="o")
    assert_close_parity(qg.grad.float().cpu(), qd.grad, what="dq")
    assert_close_parity(kg.grad.float().cpu(), kd.grad, what="dk")
    assert_close_parity(vg.grad.float().cpu(), vd.grad, what="dv")
    assert_close_parity(m.proj_l.weight.grad.cpu(), wd.grad, l1_max=2e-2, what="dw")
    assert_close_parity(m.proj_l.bias.grad.cpu(), bd.grad, l1_max=2e-2, what="db")
    # the linear branch's own share of the gradients (total minus the sparse-only operator's)
    from sla_b200 import ops
    bm = ops.block_map(q.cuda(), k.cuda(), ratio, BLKQ, 64, want_map=True, want_cols=True)
    q2, k2, v2 = (t.cuda().requires_grad_(True) for t in (q, k, v))
    ops._attention.apply(q2, k2, v2, bm.sparse_map, bm.lut.long(), bm.topk, BLKQ, 64).backward(do.cuda())
    q3, k3, v3 = (t.double().requires_grad_(True) for t in (q, k, v))
    O.sparse_fwd_dense(q3, k3, v3, smap, BLKQ, 64)[0].backward(do.double())
    if ratio < 1.0:
        for n, a, a_s, r, r_s in (("dq", qg.grad, q2.grad, qd.grad, q3.grad), ("dk", kg.grad, k2.grad, kd.grad, k3.grad),
                                  ("dv", vg.grad, v2.grad, vd.grad, v3.grad)):
            # a difference of two 16-bit tensors: it carries the rounding of the (larger) totals
            assert_close_parity((a.float() - a_s.float()).cpu(), r - r_s, cos_min=0.98, l1_max=2e-1,
                                what=f"linear share of {n}")
