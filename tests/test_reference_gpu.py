"""On-GPU parity against the UNMODIFIED reference package (its Triton kernels), installed under
baseline/_ref. Same inputs, same parameters: LUT equal as per-row sets up to score ties, outputs and
gradients within cosine >= 0.999 / relative L1 <= 1e-2. Skipped when baseline/_ref is absent."""
import importlib.util
import os
import sys

import pytest
import torch

from helpers import assert_close_parity

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_DIR = os.path.join(ROOT, "baseline", "_ref", "sparse_linear_attention")


def _reference():
    if not os.path.isdir(REF_DIR):
        pytest.skip("baseline/_ref not installed")
    if "sla_reference" in sys.modules:
        return sys.modules["sla_reference"]
    spec = importlib.util.spec_from_file_location("sla_reference", os.path.join(REF_DIR, "__init__.py"),
                                                  submodule_search_locations=[REF_DIR])
    mod = importlib.util.module_from_spec(spec)
    sys.modules["sla_reference"] = mod
    spec.loader.exec_module(mod)
    return mod


@pytest.mark.parametrize("wl,units", [("c2", None), ("c3", [0])])
def test_module_matches_reference_triton(wl, units):
    import sla_b200
    from oracle import sla_oracle as O
    from sla_b200 import ops, synthetic
    ref = _reference()
    from sla_reference.utils import get_block_map as ref_block_map
    w = synthetic.WORKLOADS[wl]
    q, k, v, do = synthetic.make_inputs(w, "cuda", units=units)
    W, b = synthetic.make_proj(w, "cuda", std=0.05)
    b = b + 0.01
    mine = sla_b200.SparseLinearAttention(w.D, w.topk, w.feature, w.BLKQ, w.BLKK).cuda()
    theirs = ref.SparseLinearAttention(w.D, w.topk, w.feature, w.BLKQ, w.BLKK).cuda()
    for m in (mine, theirs):
        with torch.no_grad():
            m.proj_l.weight.copy_(W)
            m.proj_l.bias.copy_(b)
    # block map: sets per row, ties excepted
    _, lut_ref, topk_ref = ref_block_map(q, k, w.topk, w.BLKQ, w.BLKK)
    bm = ops.block_map(q, k, w.topk, w.BLKQ, w.BLKK)
    assert bm.topk == topk_ref
    score = O.pooled_scores(q.cpu(), k.cpu(), w.BLKQ, w.BLKK)
    ident, tie, bad = O.lut_rows_equal_up_to_ties(score, bm.lut.cpu().long(), lut_ref.cpu().long(), ulps=2)
    total = ident + tie + bad
    assert bad <= 0.002 * total, f"LUT rows differing beyond ties: {bad}/{total} (tie-only {tie})"
    res = []
    for m in (mine, theirs):
        qg, kg, vg = (t.clone().requires_grad_(True) for t in (q, k, v))
        o = m(qg, kg, vg)
        o.backward(do)
        res.append((o.detach().float().cpu(), qg.grad.float().cpu(), kg.grad.float().cpu(), vg.grad.float().cpu(),
                    m.proj_l.weight.grad.cpu(), m.proj_l.bias.grad.cpu()))
    names = ("o", "dq", "dk", "dv", "dW", "db")
    for n, a, r in zip(names, *res):
        l1 = 3e-2 if n in ("dW", "db") else 1e-2
        assert_close_parity(a, r, cos_min=0.999, l1_max=l1, what=f"{wl}.{n}")
