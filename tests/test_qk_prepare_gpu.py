"""The fused step in front of the operator (per-head RMS norm + rotary embedding of q and k, with the block sums of
the mask prediction taken in the same pass) against plain PyTorch fp32 math, and the mask predicted from those sums
against the one `block_map` predicts from the stored tensors. No reference code exists for this step (it lives in the
caller of the reference's module), so the checks are: outputs equal to the fp32 formula rounded once (at most one
unit in the last place apart where the fp32 sums are ordered differently); block sums equal to a pooling pass over the
stored output; selected sets equal to the exact path's except on rows whose k-th and (k+1)-th scores are within
rounding of each other; and the module output with either mask within the 16-bit bar."""
import pytest
import torch

from helpers import assert_close_parity

pytestmark = pytest.mark.gpu


def _rope_tables(L, D, device):
    pos = torch.arange(L, device=device, dtype=torch.float32)[:, None]
    inv = 10000.0 ** (-torch.arange(D // 2, device=device, dtype=torch.float32) / (D // 2))
    return torch.cos(pos * inv), torch.sin(pos * inv)


def _torch_norm_rope(x, gain, cos, sin, eps, interleaved):
    xf = x.float()
    if gain is not None:
        xf = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * gain
    if cos is not None:
        if interleaved:
            a, b = xf[..., 0::2], xf[..., 1::2]
            xf = torch.stack([a * cos - b * sin, a * sin + b * cos], dim=-1).flatten(-2)
        else:
            h = xf.shape[-1] // 2
            a, b = xf[..., :h], xf[..., h:]
            xf = torch.cat([a * cos - b * sin, b * cos + a * sin], dim=-1)
    return xf.to(x.dtype)


@pytest.mark.parametrize("dtype,B,H,L,D,BLKQ,interleaved,norm,rope", [
    (torch.bfloat16, 1, 2, 2000, 128, 64, True, True, True),
    (torch.bfloat16, 2, 1, 1100, 64, 128, False, True, True),
    (torch.float16, 1, 2, 777, 128, 128, False, False, True),
    (torch.bfloat16, 1, 1, 640, 64, 64, True, True, False),
])
def test_fused_norm_rope_pool(dtype, B, H, L, D, BLKQ, interleaved, norm, rope):
    from sla_b200 import ops
    g = torch.Generator(device="cuda").manual_seed(L + D)
    q = torch.randn(B, H, L, D, generator=g, device="cuda").to(dtype)
    k = (torch.randn(B, H, L, D, generator=g, device="cuda") * 1.5 + 0.2).to(dtype)
    gq = (1.0 + 0.1 * torch.randn(D, generator=g, device="cuda")) if norm else None
    gk = (1.0 + 0.1 * torch.randn(D, generator=g, device="cuda")) if norm else None
    cos, sin = _rope_tables(L, D, "cuda") if rope else (None, None)
    q2, k2, pooled = ops.qk_norm_rope_pool(q, k, gq, gk, cos, sin, 1e-6, interleaved, BLKQ, 64)
    for got, x, gain in ((q2, q, gq), (k2, k, gk)):
        ref = _torch_norm_rope(x, gain, cos, sin, 1e-6, interleaved)
        diff = (got.float() - ref.float()).abs()
        ulp = torch.maximum(ref.float().abs(), torch.tensor(1e-3, device="cuda")) * (2.0 ** -7 if dtype == torch.bfloat16 else 2.0 ** -10)
        assert bool((diff <= ulp).all()), "more than one unit in the last place from the fp32 formula"
        assert float((diff > 0).float().mean()) < 0.02
    # the block sums are those of the stored rows
    mb, nb = (L + BLKQ - 1) // BLKQ, (L + 63) // 64
    nq = B * H * mb * D
    raw = pooled.buf.view(torch.float32)
    qsum = raw[:nq].view(B, H, mb, D)
    off = ((nq * 4 + 255) // 256 * 256) // 4
    ksum = raw[off:off + B * H * nb * D].view(B, H, nb, D)
    for sums, x, blk, n in ((qsum, q2, BLKQ, mb), (ksum, k2, 64, nb)):
        xp = torch.nn.functional.pad(x.float(), (0, 0, 0, n * blk - L)).view(B, H, n, blk, D).sum(3)
        assert torch.allclose(sums, xp, rtol=1e-5, atol=1e-4)
    # the mask from the sums against the mask from the tensors
    ratio = 0.2
    bm_fast = ops.block_map_pooled(pooled, ratio, want_map=True, want_cols=True)
    bm_exact = ops.block_map(q2, k2, ratio, BLKQ, 64, want_map=True, want_cols=True)
    assert bm_fast.topk == bm_exact.topk
    same_rows = (bm_fast.lut == bm_exact.lut).all(-1).float().mean().item()
    overlap = (bm_fast.sparse_map & bm_exact.sparse_map).sum().item() / bm_exact.sparse_map.sum().item()
    assert same_rows >= 0.9 and overlap >= 0.995, (same_rows, overlap)
    assert bool((bm_fast.sparse_map.sum(-1) == bm_fast.topk).all())
    assert int(bm_fast.col_offsets[..., -1].min()) == mb * bm_fast.topk


def test_module_with_fused_front_end():
    import sla_b200
    g = torch.Generator(device="cuda").manual_seed(5)
    B, H, L, D = 1, 2, 3000, 128
    q, k, v = (torch.randn(B, H, L, D, generator=g, device="cuda").bfloat16() for _ in range(3))
    gain = 1.0 + 0.1 * torch.randn(D, generator=g, device="cuda")
    cos, sin = _rope_tables(L, D, "cuda")
    m = sla_b200.SparseLinearAttention(D, 0.1).cuda()
    with torch.no_grad():
        m.proj_l.weight.copy_(torch.randn(D, D, generator=g, device="cuda") * 0.05)
        q2, k2, bm = m.norm_rope_and_predict(q, k, gain, gain, cos, sin)
        o_fast = m(q2, k2, v, block_map=bm)
        o_exact = m(q2, k2, v)
    assert_close_parity(o_fast.float().cpu(), o_exact.float().cpu(), what="module output, fused front end")
