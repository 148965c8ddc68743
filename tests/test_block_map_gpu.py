"""GPU parity of block-mask prediction (sla_block_map through the C ABI) against the golden
fixtures produced by the reference and against the CPU oracle. Integer outputs: bit-exact, score
ties at the k-th boundary excepted (torch.topk's tie-breaking is unspecified, utils.py:63)."""
import numpy as np
import pytest
import torch

from helpers import DT, load_golden, unpack

pytestmark = pytest.mark.gpu

BLOCKMAP = ["blockmap_fp32_c1shape", "blockmap_bf16_ragged", "blockmap_bf16_blkq128", "blockmap_fp16_small"]


def _check_against(score, lut_gpu, lut_ref, strict):
    from oracle import sla_oracle as O
    ident, tie, bad = O.lut_rows_equal_up_to_ties(score, lut_gpu.cpu().long(), lut_ref.long())
    assert bad == 0, f"{bad} rows differ beyond ties ({ident} identical, {tie} tie-only)"
    if strict:
        assert tie == 0
    return ident, tie


@pytest.mark.parametrize("name", BLOCKMAP)
def test_block_map_vs_reference_golden(name):
    from sla_b200 import ops
    g = load_golden(name)
    B, H, L, D, BLKQ, BLKK, topk, _ = g["meta"].tolist()
    dt = DT[str(g["dtype"])]
    q, k = unpack(g["q"], dt).cuda(), unpack(g["k"], dt).cuda()
    bm = ops.block_map(q, k, float(g["ratio"]), BLKQ, BLKK, want_map=True, want_cols=True)
    assert bm.topk == topk
    lut = bm.lut.cpu()
    assert bool((lut[..., 1:] > lut[..., :-1]).all()), "LUT rows must be strictly ascending"
    score = unpack(g["score"], dt)
    _check_against(score, lut, torch.from_numpy(g["lut"].astype(np.int64)), strict=(dt == torch.float32))
    # the 0/1 map and the column lists describe the same set as the LUT
    smap = bm.sparse_map.cpu()
    ref_map = torch.zeros_like(smap).scatter_(-1, lut.long(), 1)
    assert torch.equal(smap, ref_map)
    co, ci = bm.col_offsets.cpu(), bm.col_index.cpu()
    mb, nb = smap.shape[-2:]
    for b in range(B):
        for h in range(H):
            assert int(co[b, h, 0]) == 0 and int(co[b, h, nb]) == mb * topk
            for j in range(nb):
                rows = ci[b, h, int(co[b, h, j]):int(co[b, h, j + 1])]
                assert torch.equal(rows.long(), smap[b, h, :, j].nonzero().flatten())
    # compat wrapper returns the reference's types
    m2, lut64, tk = ops.get_block_map(q, k, float(g["ratio"]), BLKQ, BLKK)
    assert m2.dtype == torch.int8 and lut64.dtype == torch.int64 and tk == topk
    assert torch.equal(lut64.cpu(), lut.long())


@pytest.mark.parametrize("dtype,B,H,L,D,BLKQ,BLKK,ratio", [
    (torch.bfloat16, 1, 2, 4096, 128, 64, 64, 0.2),
    (torch.bfloat16, 1, 1, 5000, 64, 128, 64, 0.1),
    (torch.float16, 2, 1, 777, 128, 64, 64, 0.3),
    (torch.float32, 1, 1, 1500, 128, 128, 64, 0.15),
    (torch.bfloat16, 1, 1, 64, 64, 64, 64, 1.0),
    (torch.bfloat16, 1, 1, 65, 64, 64, 64, 0.5),
])
def test_block_map_vs_oracle(dtype, B, H, L, D, BLKQ, BLKK, ratio):
    from oracle import sla_oracle as O
    from sla_b200 import ops
    g = torch.Generator().manual_seed(L + D)
    q = torch.randn(B, H, L, D, generator=g).to(dtype)
    k = (torch.randn(B, H, L, D, generator=g) + 0.3).to(dtype)
    bm = ops.block_map(q.cuda(), k.cuda(), ratio, BLKQ, BLKK)
    smap, lut, topk = O.get_block_map(q, k, ratio, BLKQ, BLKK)
    assert bm.topk == topk
    score = O.pooled_scores(q, k, BLKQ, BLKK)
    _check_against(score, bm.lut, lut, strict=False)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("ratio", [0.6, 0.75, 0.95])
def test_negative_tied_kth_score(dtype, ratio):
    """The k-th largest pooled score is negative and tied: every KV block appears four times, so each score
    value occurs at least four times in a row, and with K-mean smoothing (utils.py:56) most of a row's scores at
    these ratios lie below zero. Every row must still select exactly topk blocks (utils.py:63), the 0/1 map and
    the column lists must describe the same sets, and the sets must equal the oracle's up to ties."""
    from oracle import sla_oracle as O
    from sla_b200 import ops
    g = torch.Generator().manual_seed(11)
    B, H, D, BLK, nuniq, rep = 1, 2, 64, 64, 9, 4
    q = torch.randn(B, H, nuniq * rep * BLK, D, generator=g).to(dtype)
    kb = torch.randn(B, H, nuniq, BLK, D, generator=g)
    k = kb.repeat(1, 1, rep, 1, 1).reshape(B, H, nuniq * rep * BLK, D).to(dtype)
    bm = ops.block_map(q.cuda(), k.cuda(), ratio, BLK, BLK, want_map=True, want_cols=True)
    nb = mb = nuniq * rep
    topk = O.topk_count(nb, ratio)
    assert bm.topk == topk
    lut = bm.lut.cpu()
    assert bool((lut[..., 1:] > lut[..., :-1]).all()) and int(lut.min()) >= 0 and int(lut.max()) < nb
    smap = bm.sparse_map.cpu()
    assert bool((smap.sum(-1) == topk).all()), "a row selected more or fewer than topk blocks"
    assert torch.equal(smap, torch.zeros_like(smap).scatter_(-1, lut.long(), 1))
    co = bm.col_offsets.cpu()
    assert bool((co[..., 0] == 0).all()) and bool((co[..., nb] == mb * topk).all())
    assert torch.equal(smap.sum(dim=-2).int(), co[..., 1:] - co[..., :-1])
    score = O.pooled_scores(q, k, BLK, BLK)
    kth = torch.sort(score.float(), dim=-1, descending=True).values[..., topk - 1]
    assert float((kth < 0).float().mean()) > 0.5, "the case must exercise negative k-th scores"
    _, lut_ref, _ = O.get_block_map(q, k, ratio, BLK, BLK)
    _check_against(score, lut, lut_ref, strict=False)


def test_smooth_k_invariance():
    """Adding a constant vector to every key leaves the selected set unchanged (utils.py:56)."""
    from sla_b200 import ops
    g = torch.Generator().manual_seed(5)
    q = torch.randn(1, 2, 2048, 64, generator=g)
    k = torch.randn(1, 2, 2048, 64, generator=g)
    a = ops.block_map(q.cuda(), k.cuda(), 0.25, 64, 64).lut
    b = ops.block_map(q.cuda(), (k + 3.0 * torch.randn(1, 2, 1, 64, generator=g)).cuda(), 0.25, 64, 64).lut
    same = (a == b).all(dim=-1).float().mean().item()
    assert same > 0.98  # fp32: only rounding-level near-ties may move


def test_full_size_properties_c3():
    """Full-size (L=32760, D=128, 12 heads, topk=25 of 512) size-independent properties: row length,
    strict ascent (=> no duplicates), range, determinism, and column lists that transpose the LUT."""
    from sla_b200 import ops, synthetic
    w = synthetic.WORKLOADS["c3"]
    q, k, _, _ = synthetic.make_inputs(w, "cuda", units=[0, 5], with_do=False)
    bm = ops.block_map(q, k, w.topk, w.BLKQ, w.BLKK, want_map=True, want_cols=True)
    assert bm.topk == 25 and bm.lut.shape == (1, 2, 512, 25)
    lut = bm.lut
    assert bool((lut[..., 1:] > lut[..., :-1]).all()) and int(lut.min()) >= 0 and int(lut.max()) < 512
    bm2 = ops.block_map(q, k, w.topk, w.BLKQ, w.BLKK, want_cols=True)
    assert torch.equal(bm2.lut, lut) and torch.equal(bm2.col_index, bm.col_index)
    assert int(bm.sparse_map.sum()) == 2 * 512 * 25
    counts = bm.sparse_map.sum(dim=-2).int()
    assert torch.equal(counts, (bm.col_offsets[..., 1:] - bm.col_offsets[..., :-1]))
