"""Property tests (hypothesis) of the C-ABI operators on randomly drawn shapes: sizes around the 64- and 128-row
tile boundaries, both head dimensions, both query block sizes, any top-k ratio. They check what must hold for every
input rather than parity on one: the structure of the block map (row length, strict ascent, range, the three
representations describing one set, invariance to a constant added to every key: utils.py:56), and of the sparse
branch (a convex combination of the selected V rows: constant V in, the same constant out; linear in V; gradients
finite; dV of a block nobody selected is zero)."""
import pytest
import torch

hypothesis = pytest.importorskip("hypothesis")
from hypothesis import HealthCheck, given, settings, strategies as st

pytestmark = pytest.mark.gpu

SETTINGS = dict(max_examples=12, deadline=None, derandomize=True,
                suppress_health_check=[HealthCheck.too_slow, HealthCheck.data_too_large])

shapes = st.tuples(st.integers(1, 2), st.integers(1, 3), st.integers(65, 1400), st.sampled_from([64, 128]),
                   st.sampled_from([64, 128]), st.floats(0.05, 1.0), st.sampled_from(["bf16", "fp16", "fp32"]),
                   st.integers(0, 2 ** 20))
DT = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}


@settings(**SETTINGS)
@given(shapes)
def test_block_map_structure(case):
    from sla_b200 import ops
    B, H, L, D, BLKQ, ratio, dts, seed = case
    g = torch.Generator(device="cuda").manual_seed(seed)
    dt = DT[dts]
    q = torch.randn(B, H, L, D, generator=g, device="cuda").to(dt)
    k = (torch.randn(B, H, L, D, generator=g, device="cuda") + 0.5).to(dt)
    mb, nb = (L + BLKQ - 1) // BLKQ, (L + 63) // 64
    topk = ops.topk_count(nb, ratio)
    if topk < 1:
        return
    bm = ops.block_map(q, k, ratio, BLKQ, 64, want_map=True, want_cols=True)
    lut = bm.lut
    assert bm.topk == topk and tuple(lut.shape) == (B, H, mb, topk)
    assert int(lut.min()) >= 0 and int(lut.max()) < nb
    if topk > 1:
        assert bool((lut[..., 1:] > lut[..., :-1]).all())
    ref_map = torch.zeros_like(bm.sparse_map).scatter_(-1, lut.long(), 1)
    assert torch.equal(bm.sparse_map, ref_map)
    counts = bm.sparse_map.sum(dim=-2).int()
    assert torch.equal(counts, bm.col_offsets[..., 1:] - bm.col_offsets[..., :-1])
    assert bool((bm.col_offsets[..., 0] == 0).all()) and bool((bm.col_offsets[..., -1] == mb * topk).all())
    co, ci = bm.col_offsets.cpu(), bm.col_index.cpu()
    smap = bm.sparse_map.cpu()
    for j in {0, nb // 2, nb - 1}:
        rows = ci[0, 0, int(co[0, 0, j]):int(co[0, 0, j + 1])]
        assert torch.equal(rows.long(), smap[0, 0, :, j].nonzero().flatten())
    # determinism
    again = ops.block_map(q, k, ratio, BLKQ, 64)
    assert torch.equal(again.lut, lut)
    if dt == torch.float32 and topk < nb:
        # smoothing removes a constant key offset up to fp32 rounding: nearly every row keeps its set
        shifted = ops.block_map(q, k + 2.0 * torch.randn(1, H, 1, D, generator=g, device="cuda"), ratio, BLKQ, 64).lut
        assert float((shifted == lut).all(-1).float().mean()) > 0.9


@settings(**SETTINGS)
@given(shapes)
def test_sparse_branch_is_a_convex_combination(case):
    from sla_b200 import ops
    B, H, L, D, BLKQ, ratio, dts, seed = case
    dt = torch.float16 if dts == "fp16" else torch.bfloat16
    g = torch.Generator(device="cuda").manual_seed(seed)
    q, k, v, v2, do = (torch.randn(B, H, L, D, generator=g, device="cuda").to(dt) for _ in range(5))
    nb = (L + 63) // 64
    if ops.topk_count(nb, ratio) < 1:
        return
    smap, lut, topk = ops.get_block_map(q, k, ratio, BLKQ, 64)
    f = lambda vv: ops._attention.apply(q, k, vv, smap, lut, topk, BLKQ, 64).float()
    # rows of P sum to one: a constant V comes out unchanged (up to the rounding of P and of the output)
    const = torch.full_like(v, 0.75)
    assert float((f(const) - 0.75).abs().max()) < 0.75 * 2.0 ** -6
    # linear in V
    a, b, ab = f(v), f(v2), f((v.float() + v2.float()).to(dt))
    scale = float((a.abs() + b.abs()).mean())
    assert float((ab - a - b).abs().mean()) < 0.02 * scale
    # gradients: finite; a KV block no query block selected receives no dV
    qg, kg, vg = (t.clone().requires_grad_(True) for t in (q, k, v))
    ops._attention.apply(qg, kg, vg, smap, lut, topk, BLKQ, 64).backward(do)
    for t in (qg.grad, kg.grad, vg.grad):
        assert bool(torch.isfinite(t.float()).all())
    unused = (smap.sum(dim=-2) == 0)                     # (B, H, nb)
    if bool(unused.any()):
        rows = unused.repeat_interleave(64, dim=-1)[..., :L]
        assert float(vg.grad.float()[rows].abs().max()) == 0.0
        assert float(kg.grad.float()[rows].abs().max()) == 0.0
