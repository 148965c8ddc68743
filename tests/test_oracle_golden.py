"""Pin the CPU oracle against fixtures produced by the reference implementation itself
(tests/golden/make_golden.py). Runs without a GPU."""
import numpy as np
import pytest
import torch

from oracle import sla_oracle as O
from helpers import DT, assert_close_parity, load_golden, unpack

BLOCKMAP = ["blockmap_fp32_c1shape", "blockmap_bf16_ragged", "blockmap_bf16_blkq128", "blockmap_fp16_small"]
ATTN = ["attn_fp32_d64", "attn_fp16_d64", "attn_bf16_d128", "attn_bf16_blkq128", "attn_fp32_blkq128_d128"]
MODULE = ["module_bf16_softmax", "module_fp16_relu", "module_fp32in_elu_blkq128"]


@pytest.mark.parametrize("name", BLOCKMAP)
def test_block_map_matches_reference(name):
    g = load_golden(name)
    B, H, L, D, BLKQ, BLKK, topk, _ = g["meta"].tolist()
    dt = DT[str(g["dtype"])]
    q, k = unpack(g["q"], dt), unpack(g["k"], dt)
    # pooled means: same rounding points -> identical up to fp32 summation order (<= 1 ulp)
    arg_k = k - torch.mean(k, dim=-2, keepdim=True)
    pq, pk = O.mean_pool(q, BLKQ), O.mean_pool(arg_k, BLKK)
    ulp = {torch.float32: 2e-6, torch.bfloat16: 2 ** -7, torch.float16: 2 ** -10}[dt]
    for mine, ref in ((pq, unpack(g["pooled_q"], dt)), (pk, unpack(g["pooled_k"], dt))):
        err = (mine.float() - ref.float()).abs()
        assert bool((err <= ulp * ref.float().abs() + 3e-7).all())
    sparse_map, lut, tk = O.get_block_map(q, k, float(g["ratio"]), BLKQ, BLKK)
    assert tk == topk
    assert O.topk_count(sparse_map.shape[-1], float(g["ratio"])) == topk
    ref_lut = torch.from_numpy(g["lut"].astype(np.int64))
    score = unpack(g["score"], dt)
    ident, tie, bad = O.lut_rows_equal_up_to_ties(score, lut, ref_lut)
    assert bad == 0, f"{bad} rows differ beyond score ties ({ident} identical, {tie} tie-only)"
    if dt == torch.float32:
        assert tie == 0 and torch.equal(sparse_map, torch.from_numpy(g["sparse_map"]))


@pytest.mark.parametrize("name", ATTN)
def test_sparse_attention_matches_reference(name):
    g = load_golden(name)
    B, H, L, D, BLKQ, BLKK, topk, _ = g["meta"].tolist()
    dt = DT[str(g["dtype"])]
    q, k, v, do = (unpack(g[n], dt) for n in ("q", "k", "v", "do"))
    lut = torch.from_numpy(g["lut"].astype(np.int64))
    smap = torch.from_numpy(g["sparse_map"])
    ref_o, ref_lse = unpack(g["o_s"], dt).float(), torch.from_numpy(g["lse"])
    emu = None if dt == torch.float32 else dt
    o_g, lse_g = O.sparse_fwd_gather(q, k, v, lut, BLKQ, BLKK, emulate=emu)
    o_d, lse_d = O.sparse_fwd_dense(q.float(), k.float(), v.float(), smap, BLKQ, BLKK)
    # the two oracle evaluations agree with each other and with the reference kernel
    tol = 2e-5 if dt == torch.float32 else 2e-2
    assert float((o_d - ref_o).abs().max()) <= tol
    assert float((o_g.float() - ref_o).abs().max()) <= tol
    assert float((lse_d - ref_lse).abs().max()) <= 1e-4
    assert float((lse_g - ref_lse).abs().max()) <= 1e-4
    # backward
    dq, dk, dv, _ = O.sparse_bwd_dense(q.float(), k.float(), v.float(), ref_o, ref_lse, do.float(),
                                       smap, BLKQ, BLKK)
    for mine, n in ((dq, "dq"), (dk, "dk"), (dv, "dv")):
        ref = unpack(g[n], dt).float()
        if dt == torch.float32:
            assert float((mine - ref).abs().max()) <= 5e-5 * max(1.0, float(ref.abs().max())), n
        else:
            assert_close_parity(mine, ref, cos_min=0.9995, l1_max=8e-3, what=f"{name}.{n}")


@pytest.mark.parametrize("name", MODULE)
def test_module_forward_backward_matches_reference(name):
    g = load_golden(name)
    B, H, L, D, BLKQ, BLKK, _, _ = g["meta"].tolist()
    in_dt, comp = DT[str(g["in_dtype"])], DT[str(g["compute"])]
    feat = str(g["feature"])
    q, k, v, do = (unpack(g[n], in_dt) for n in ("q", "k", "v", "do"))
    w, b = torch.from_numpy(g["w"]), torch.from_numpy(g["bias"])
    o, parts = O.sla_forward(q, k, v, w, b, float(g["ratio"]), feat, BLKQ, BLKK, comp, return_parts=True)
    ref_o = unpack(g["o"], in_dt)
    assert o.dtype == ref_o.dtype
    assert float(g["sparsity"]) == parts["topk"] / parts["sparse_map"].shape[-1]
    assert_close_parity(o.float(), ref_o.float(), cos_min=0.9999, l1_max=8e-3, what=name + ".o")
    # gradients: autograd through the rounding-free evaluation with the same (fixed) block map
    qc, kc, vc = (t.to(comp).double().requires_grad_(True) for t in (q, k, v))
    wd, bd = w.double().requires_grad_(True), b.double().requires_grad_(True)
    out = O.sla_forward_fp(qc, kc, vc, wd, bd, parts["sparse_map"], feat, BLKQ, BLKK)
    out.backward(do.double())
    for mine, n in ((qc.grad, "dq"), (kc.grad, "dk"), (vc.grad, "dv")):
        assert_close_parity(mine, unpack(g[n], in_dt).float(), cos_min=0.999, l1_max=1e-2, what=f"{name}.{n}")
    assert_close_parity(wd.grad, torch.from_numpy(g["dw"]), cos_min=0.999, l1_max=2e-2, what=name + ".dw")
    assert_close_parity(bd.grad, torch.from_numpy(g["db"]), cos_min=0.999, l1_max=2e-2, what=name + ".db")


def test_module_c1_configuration():
    """The reference's CPU-runnable configuration: B=1,H=2,L=1024,D=64 fp32 inputs from seed 0,
    BLKQ=BLKK=64, topk=0.25, softmax feature map, W ~ N(0, 0.02), b = 0."""
    g = load_golden("module_c1")
    torch.manual_seed(0)
    q, k, v = torch.randn(1, 2, 1024, 64), torch.randn(1, 2, 1024, 64), torch.randn(1, 2, 1024, 64)
    w = torch.randn(64, 64) * 0.02
    assert torch.equal(w, torch.from_numpy(g["w"]))
    o = O.sla_forward(q, k, v, w, torch.zeros(64), 0.25, "softmax", 64, 64, torch.bfloat16)
    assert o.dtype == torch.float32
    assert_close_parity(o, torch.from_numpy(g["o"]), cos_min=0.9999, l1_max=8e-3, what="c1.o")


def test_linear_scope_unselected_reduces_to_all_when_nothing_selected():
    torch.manual_seed(3)
    q, k, v = (torch.randn(1, 1, 130, 64) for _ in range(3))
    cq, ck = O.feature_map(q, "softmax"), O.feature_map(k, "softmax")
    smap = torch.zeros(1, 1, 3, 3, dtype=torch.int8)
    a = O.calc_linear_unselected(cq, ck, v, smap, 64, 64)
    b = O.calc_linear(cq, ck, v)
    assert float((a - b).abs().max()) < 1e-5


def test_sage_oracle_close_to_unquantized():
    torch.manual_seed(5)
    q, k, v = (torch.randn(1, 2, 300, 64).bfloat16() for _ in range(3))
    k = (k.float() + 2.0).bfloat16()  # a large common offset: K-mean smoothing must absorb it
    smap, lut, _ = O.get_block_map(q, k, 0.5, 128, 64)
    ref, _ = O.sparse_fwd_gather(q, k, v, lut, 128, 64)
    got = O.sage_sparse_fwd(q, k, v, lut, 128, 64)
    assert_close_parity(got, ref.float(), cos_min=0.995, l1_max=6e-2, what="sage")
