"""CPU oracle for the SLA attention hot path. TEST INFRASTRUCTURE ONLY.

A plain-PyTorch (CPU) restatement of the algorithm in thu-ml/SLA. Only the test-suite, the
smoke check and the CPU-baseline leg of the benchmark may import this module; the product package
never does and has no CPU fallback.

Parity status: PINNED. `tests/golden/make_golden.py` imports the reference package itself, runs its
Triton kernels under the Triton CPU interpreter, and commits the inputs/outputs as fixtures;
`tests/test_oracle_golden.py` checks every function below against those fixtures.
The SageSLA quantized sparse branch is the exception: its arithmetic lives in the un-vendored
third-party package `spas_sage_attn` (github.com/thu-ml/SpargeAttn, unpinned git HEAD, called from
SageSLA/core.py:20-28,105-144), so `sage_sparse_fwd` below restates this library's own quantization
recipe and is "parity unpinned" at that boundary; it is checked against the un-quantized path only.

Each function cites the reference lines it follows (paths relative to the reference project root).
Two modes are offered where it matters:
  * ``emulate=<torch dtype>``: intermediates are rounded where the reference rounds them
    (bf16/fp16 tensors between ops, fp32 accumulation inside an op);
  * ``emulate=None``: everything in the dtype given (fp32/fp64), no intermediate rounding.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.nn.functional as F

LOG2E = 1.4426950408889634  # kernel.py:58


# ----------------------------------------------------------------------------------------------
# Block-mask prediction (sparse_linear_attention/utils.py:21-67)
# ----------------------------------------------------------------------------------------------
def mean_pool(x: torch.Tensor, blk: int) -> torch.Tensor:
    """Per-block column mean. utils.py:21-52: the tile is summed in fp32 over its valid rows,
    divided by the number of valid rows ``nx`` (tail block: L - idx*BLK, utils.py:38) and rounded
    to x.dtype on store (utils.py:40)."""
    B, H, L, D = x.shape
    nb = (L + blk - 1) // blk
    pad = nb * blk - L
    xf = x.float()
    if pad:
        xf = F.pad(xf, (0, 0, 0, pad))
    s = xf.view(B, H, nb, blk, D).sum(dim=3)
    nx = torch.full((nb,), float(blk))
    if pad:
        nx[-1] = float(blk - pad)
    return (s / nx.view(1, 1, nb, 1)).to(x.dtype)


def topk_count(n_blocks: int, topk_ratio: float) -> int:
    """utils.py:61-62: ``min(K, int(topk_ratio * K))`` in Python (double) arithmetic."""
    return min(n_blocks, int(topk_ratio * n_blocks))


def pooled_scores(q: torch.Tensor, k: torch.Tensor, blkq: int, blkk: int) -> torch.Tensor:
    """utils.py:56-59. K is smoothed by its per-head column mean (rounded to k.dtype, as
    torch.mean and the subtraction both return k.dtype), both tensors are mean-pooled, and the
    pooled score matrix is a matmul whose result is rounded to the input dtype."""
    arg_k = k - torch.mean(k, dim=-2, keepdim=True)
    pq = mean_pool(q, blkq)
    pk = mean_pool(arg_k, blkk)
    # fp32 accumulation, then one rounding to the input dtype (what a bf16/fp16 GEMM returns)
    return (pq.float() @ pk.float().transpose(-1, -2)).to(q.dtype)


def select_topk(score: torch.Tensor, topk: int) -> torch.Tensor:
    """Per-row top-k as index sets. utils.py:63 uses ``torch.topk(sorted=False)`` whose order and
    tie-breaking are unspecified; this oracle fixes both: larger score first, lower index wins a
    tie, and the selected indices are returned in ascending order (int64)."""
    sc = score.float()
    # stable descending sort == ties resolved towards the lower index
    order = torch.sort(sc, dim=-1, descending=True, stable=True).indices[..., :topk]
    return torch.sort(order, dim=-1).values


def get_block_map(q, k, topk_ratio: float, BLKQ: int = 64, BLKK: int = 64):
    """utils.py:55-67 -> (sparse_map int8 (B,H,M_BLOCKS,N_BLOCKS), lut int64 (B,H,M_BLOCKS,topk),
    topk). The LUT is sorted ascending (the reference's is unordered)."""
    score = pooled_scores(q, k, BLKQ, BLKK)
    n_blocks = score.shape[-1]
    topk = topk_count(n_blocks, topk_ratio)
    lut = select_topk(score, topk)
    sparse_map = torch.zeros(score.shape, dtype=torch.int8)
    sparse_map.scatter_(-1, lut, 1)
    return sparse_map, lut, topk


def lut_rows_equal_up_to_ties(score: torch.Tensor, lut_a: torch.Tensor, lut_b: torch.Tensor,
                              ulps: int = 1):
    """Compare two LUTs as per-row sets. Rows may differ only in members whose score is within
    ``ulps`` units-in-the-last-place (of score.dtype) of the row's k-th largest score.
    Returns (n_rows_identical, n_rows_tie_only, n_rows_bad)."""
    sc = score.float().reshape(-1, score.shape[-1])
    a = lut_a.reshape(sc.shape[0], -1).long()
    b = lut_b.reshape(sc.shape[0], -1).long()
    topk = a.shape[-1]
    ident = tie = bad = 0
    kth = torch.sort(sc, dim=-1, descending=True).values[:, topk - 1]
    eps = {torch.bfloat16: 2.0 ** -8, torch.float16: 2.0 ** -11}.get(score.dtype, 2.0 ** -22)
    for r in range(sc.shape[0]):
        sa, sb = set(a[r].tolist()), set(b[r].tolist())
        if sa == sb:
            ident += 1
            continue
        diff = list(sa ^ sb)
        tol = ulps * eps * max(abs(float(kth[r])), 1e-30) * 2.0
        if all(abs(float(sc[r, j]) - float(kth[r])) <= tol for j in diff):
            tie += 1
        else:
            bad += 1
    return ident, tie, bad


# ----------------------------------------------------------------------------------------------
# Sparse branch (sparse_linear_attention/kernel.py)
# ----------------------------------------------------------------------------------------------
def _expand_mask(sparse_map: torch.Tensor, L: int, blkq: int, blkk: int) -> torch.Tensor:
    m = sparse_map.bool().repeat_interleave(blkq, dim=2).repeat_interleave(blkk, dim=3)
    return m[:, :, :L, :L]


def sparse_fwd_dense(q, k, v, sparse_map, BLKQ, BLKK, qk_scale=None):
    """Dense-masked evaluation of kernel.py:21-82: softmax over the keys of the selected blocks
    (keys >= L never participate, kernel.py:57-62), scale D**-0.5 (kernel.py:251-252).
    Returns (o_s, lse) with lse = m + log2(l) in log2 units of the scaled score (kernel.py:58,81).
    Computed in q.dtype (use fp32/fp64 inputs)."""
    B, H, L, D = q.shape
    if qk_scale is None:
        qk_scale = D ** -0.5
    mask = _expand_mask(sparse_map, L, BLKQ, BLKK)
    s = (q @ k.transpose(-1, -2)) * (qk_scale * LOG2E)
    s = s.masked_fill(~mask, float("-inf"))
    m = s.max(dim=-1, keepdim=True).values
    p = torch.exp2(s - m)
    l = p.sum(dim=-1, keepdim=True)
    o = (p @ v) / l
    lse = (m + torch.log2(l)).squeeze(-1)
    return o, lse


def sparse_fwd_gather(q, k, v, lut, BLKQ, BLKK, qk_scale=None, emulate=None):
    """Block-gather evaluation following the loop of kernel.py:50-82 one LUT row at a time
    (vectorised over the topk entries of a row). With ``emulate`` (bf16/fp16) P is rounded to that
    dtype before P.V (kernel.py:71) and o_s is rounded on store (kernel.py:79); accumulation stays
    fp32. Unlike the streaming kernel the row maximum is taken over all selected keys at once,
    which changes results only at fp32 rounding level."""
    B, H, L, D = q.shape
    if qk_scale is None:
        qk_scale = D ** -0.5
    mb = (L + BLKQ - 1) // BLKQ
    nb = (L + BLKK - 1) // BLKK
    topk = lut.shape[-1]
    qf, kf, vf = q.float(), k.float(), v.float()
    padk = nb * BLKK - L
    if padk:
        kf = F.pad(kf, (0, 0, 0, padk))
        vf = F.pad(vf, (0, 0, 0, padk))
    kb = kf.view(B, H, nb, BLKK, D)
    vb = vf.view(B, H, nb, BLKK, D)
    o = torch.zeros(B, H, L, D)
    lse = torch.zeros(B, H, L)
    key_pos = torch.arange(nb * BLKK).view(nb, BLKK)
    for b in range(B):
        for h in range(H):
            for i in range(mb):
                r0, r1 = i * BLKQ, min(L, (i + 1) * BLKQ)
                idx = lut[b, h, i].long()
                ks = kb[b, h, idx].reshape(topk * BLKK, D)
                vs = vb[b, h, idx].reshape(topk * BLKK, D)
                valid = (key_pos[idx].reshape(-1) < L)
                s = (qf[b, h, r0:r1] @ ks.t()) * (qk_scale * LOG2E)
                s = s.masked_fill(~valid[None, :], float("-inf"))
                m = s.max(dim=-1, keepdim=True).values
                p = torch.exp2(s - m)
                l = p.sum(dim=-1, keepdim=True)
                if emulate is not None:
                    p = p.to(emulate).float()
                o[b, h, r0:r1] = (p @ vs) / l
                lse[b, h, r0:r1] = (m + torch.log2(l)).squeeze(-1)
    if emulate is not None:
        o = o.to(emulate)
    return o, lse


def sparse_bwd_dense(q, k, v, o_s, lse, do_s, sparse_map, BLKQ, BLKK, qk_scale=None):
    """Backward of the sparse branch as the reference defines it:
    delta = rowsum(o_s * do_s) (kernel.py:102-105); P = exp2(S*scale*log2e - lse), zero for keys
    >= L (kernel.py:155-157); dP = dO V^T; dS = P*(dP - delta) (kernel.py:160-161);
    dQ = dS K * scale (kernel.py:163-164); dV = P^T dO (kernel.py:220); dK = dS^T Q * scale
    (kernel.py:225,236). fp32/fp64 dense evaluation; returns (dq, dk, dv, delta)."""
    B, H, L, D = q.shape
    if qk_scale is None:
        qk_scale = D ** -0.5
    mask = _expand_mask(sparse_map, L, BLKQ, BLKK)
    delta = (o_s * do_s).sum(dim=-1)
    s = (q @ k.transpose(-1, -2)) * (qk_scale * LOG2E)
    p = torch.exp2(s - lse.unsqueeze(-1))
    p = torch.where(mask, p, torch.zeros_like(p))
    dp = do_s @ v.transpose(-1, -2)
    ds = p * (dp - delta.unsqueeze(-1))
    dq = (ds @ k) * qk_scale
    dk = (ds.transpose(-1, -2) @ q) * qk_scale
    dv = p.transpose(-1, -2) @ do_s
    return dq, dk, dv, delta


# ----------------------------------------------------------------------------------------------
# Linear branch, projection and the module forward (sparse_linear_attention/core.py)
# ----------------------------------------------------------------------------------------------
def feature_map(x: torch.Tensor, name: str) -> torch.Tensor:
    """core.py:43-57: 'elu' -> elu(x)+1, 'relu' -> relu(x), 'softmax' -> softmax over D.
    The result keeps x.dtype (bf16/fp16 inputs give rounded outputs, core.py:90-91)."""
    if name == "elu":
        return F.elu(x) + 1
    if name == "relu":
        return F.relu(x)
    if name == "softmax":
        return F.softmax(x, dim=-1)
    raise NotImplementedError(f"Not supported feature map {name}.")


def calc_linear(cq, ck, v):
    """core.py:92-96 verbatim semantics: H = ck^T v, z = sum_L ck, o_l = cq H / (1e-5 + cq.z).
    All tokens contribute to H and z. Every op returns the operand dtype, so 16-bit inputs give
    the reference's rounding points."""
    kvsum = ck.transpose(-1, -2) @ v
    ksum = torch.sum(ck, dim=-2, keepdim=True)
    return (cq @ kvsum) / (1e-5 + (cq * ksum).sum(dim=-1, keepdim=True))


def calc_linear_unselected(cq, ck, v, sparse_map, BLKQ, BLKK):
    """The paper's scope (assets/overview_of_SLA.png, right panel): for query block i the state is
    summed over the KV blocks NOT selected for i. Evaluated in fp32, or in fp64 when the inputs are fp64;
    differentiable (the block map is a constant), and defined as 0 when every block is selected."""
    B, H, L, D = cq.shape
    mb, nb = sparse_map.shape[-2:]
    dt = torch.float64 if cq.dtype == torch.float64 else torch.float32
    padk = nb * BLKK - L
    ckf, vf = ck.to(dt), v.to(dt)
    if padk:
        ckf = F.pad(ckf, (0, 0, 0, padk))
        vf = F.pad(vf, (0, 0, 0, padk))
    ckb = ckf.view(B, H, nb, BLKK, D)
    vb = vf.view(B, H, nb, BLKK, D)
    h = ckb.transpose(-1, -2) @ vb                    # (B,H,nb,D,D)
    z = ckb.sum(dim=3)                                # (B,H,nb,D)
    unsel = (1 - sparse_map.to(dt))                   # (B,H,mb,nb)
    Hi = torch.einsum("bhmn,bhnde->bhmde", unsel, h)
    zi = torch.einsum("bhmn,bhnd->bhmd", unsel, z)
    cqf = cq.to(dt)
    if bool((unsel.sum(-1) == 0).all()):
        return torch.zeros(B, H, L, D, dtype=dt) + 0.0 * cqf
    rows = []
    for i in range(mb):
        r0, r1 = i * BLKQ, min(L, (i + 1) * BLKQ)
        num = cqf[:, :, r0:r1] @ Hi[:, :, i]
        den = 1e-5 + (cqf[:, :, r0:r1] * zi[:, :, i].unsqueeze(2)).sum(-1, keepdim=True)
        rows.append(num / den)
    return torch.cat(rows, dim=2)


def sla_forward(q, k, v, weight, bias, topk_ratio, feature="softmax", BLKQ=64, BLKK=64,
                compute_dtype=torch.bfloat16, linear_scope="all", return_parts=False):
    """SparseLinearAttention.forward, core.py:69-105: block map on the ORIGINAL dtype (core.py:83),
    q/k/v cast to the compute dtype (core.py:85-87), sparse branch, feature maps rounded to the
    compute dtype (core.py:90-91), linear branch, proj_l under autocast (weights and bias used in
    the compute dtype, fp32 accumulation, rounded output; core.py:98-99), sum and cast back
    (core.py:100)."""
    in_dtype = q.dtype
    sparse_map, lut, topk = get_block_map(q, k, topk_ratio, BLKQ, BLKK)
    qc, kc, vc = q.to(compute_dtype), k.to(compute_dtype), v.to(compute_dtype)
    o_s, lse = sparse_fwd_gather(qc, kc, vc, lut, BLKQ, BLKK, emulate=compute_dtype)
    cq = feature_map(qc, feature).contiguous().to(compute_dtype)
    ck = feature_map(kc, feature).contiguous().to(compute_dtype)
    if linear_scope == "all":
        o_l = calc_linear(cq, ck, vc)
    else:
        o_l = calc_linear_unselected(cq, ck, vc, sparse_map, BLKQ, BLKK).to(compute_dtype)
    wl = weight.to(compute_dtype).float()
    o_p = o_l.float() @ wl.t()
    if bias is not None:
        o_p = o_p + bias.to(compute_dtype).float()
    o_p = o_p.to(compute_dtype)
    o = (o_s + o_p).to(in_dtype)
    if return_parts:
        return o, dict(sparse_map=sparse_map, lut=lut, topk=topk, o_s=o_s, lse=lse, o_l=o_l,
                       cq=cq, ck=ck)
    return o


def sla_forward_fp(q, k, v, weight, bias, sparse_map, feature="softmax", BLKQ=64, BLKK=64,
                   linear_scope="all"):
    """Differentiable, rounding-free evaluation of core.py:88-100 for a FIXED block map (no
    gradient flows through the top-k, core.py:83). Used with torch.autograd (fp32/fp64) as the
    gradient oracle for dq, dk, dv, dW, db."""
    o_s, _ = sparse_fwd_dense(q, k, v, sparse_map, BLKQ, BLKK)
    cq, ck = feature_map(q, feature), feature_map(k, feature)
    if linear_scope == "all":
        o_l = calc_linear(cq, ck, v)
    else:
        o_l = calc_linear_unselected(cq, ck, v, sparse_map, BLKQ, BLKK)
    return o_s + o_l @ weight.t() + bias


# ----------------------------------------------------------------------------------------------
# SageSLA quantized sparse branch (own recipe; third-party boundary unpinned, see module header)
# ----------------------------------------------------------------------------------------------
E4M3_MAX = 448.0


def quant_int8_per_block(x: torch.Tensor, blk: int):
    """Symmetric abs-max INT8 per (b,h,block of ``blk`` rows): scale = amax/127, round-to-nearest-
    even. Returns (int8 tensor (B,H,L,D), fp32 scale (B,H,nblocks)). Call site facts:
    SageSLA/core.py:105-108 (per-block Q at 128 rows, per-block K at 64 rows, K minus its mean)."""
    B, H, L, D = x.shape
    nb = (L + blk - 1) // blk
    pad = nb * blk - L
    xf = x.float()
    if pad:
        xf = F.pad(xf, (0, 0, 0, pad))
    xb = xf.view(B, H, nb, blk, D)
    amax = xb.abs().amax(dim=(3, 4))
    scale = torch.clamp(amax, min=1e-8) / 127.0
    qx = torch.round(xb / scale[..., None, None]).clamp(-127, 127)
    return qx.view(B, H, nb * blk, D)[:, :, :L].to(torch.int8), scale


def quant_e4m3_per_channel(v: torch.Tensor, target: float = E4M3_MAX):
    """FP8 e4m3 V with one fp32 scale per (b,h,d): scale = amax_L|v| / target (call site:
    SageSLA/core.py:127-129). Returns (fp8 tensor, scale (B,H,D))."""
    amax = v.float().abs().amax(dim=-2)
    scale = torch.clamp(amax, min=1e-8) / target
    v8 = (v.float() / scale.unsqueeze(-2)).to(torch.float8_e4m3fn)
    return v8, scale


def sage_sparse_fwd(q, k, v, lut, BLKQ=128, BLKK=64, qk_scale=None, p_scale: float = E4M3_MAX):
    """Quantized sparse branch: S = (Q_i8 K_i8^T) * sq_i * sk_j * scale * log2e with
    K smoothed by its per-head mean before quantization (SageSLA/core.py:102,108; the row-constant
    term q.km cancels in the softmax); online softmax in fp32; P in [0,1] is multiplied by
    ``p_scale``, rounded to e4m3 and multiplied with e4m3 V (fp32 accumulation); the result is
    divided by p_scale, multiplied by the per-channel V scale and normalised by the fp32 row sum of
    the UNQUANTIZED P. Evaluated one LUT row at a time with the global row maximum."""
    B, H, L, D = q.shape
    if qk_scale is None:
        qk_scale = D ** -0.5
    km = k.float().mean(dim=-2, keepdim=True)
    q8, sq = quant_int8_per_block(q, BLKQ)
    k8, sk = quant_int8_per_block((k.float() - km).to(k.dtype), BLKK)
    v8, sv = quant_e4m3_per_channel(v)
    mb = (L + BLKQ - 1) // BLKQ
    nb = (L + BLKK - 1) // BLKK
    topk = lut.shape[-1]
    padk = nb * BLKK - L
    k8f, v8f = k8.float(), v8.float()
    if padk:
        k8f = F.pad(k8f, (0, 0, 0, padk))
        v8f = F.pad(v8f, (0, 0, 0, padk))
    kb = k8f.view(B, H, nb, BLKK, D)
    vb = v8f.view(B, H, nb, BLKK, D)
    key_pos = torch.arange(nb * BLKK).view(nb, BLKK)
    o = torch.zeros(B, H, L, D)
    for b in range(B):
        for h in range(H):
            for i in range(mb):
                r0, r1 = i * BLKQ, min(L, (i + 1) * BLKQ)
                idx = lut[b, h, i].long()
                ks = kb[b, h, idx].reshape(topk * BLKK, D)
                vs = vb[b, h, idx].reshape(topk * BLKK, D)
                valid = key_pos[idx].reshape(-1) < L
                kscale = sk[b, h, idx].repeat_interleave(BLKK)
                s = (q8[b, h, r0:r1].float() @ ks.t()) * (sq[b, h, i] * kscale[None, :]) \
                    * (qk_scale * LOG2E)
                s = s.masked_fill(~valid[None, :], float("-inf"))
                m = s.max(dim=-1, keepdim=True).values
                p = torch.exp2(s - m)
                l = p.sum(dim=-1, keepdim=True)
                p8 = (p * p_scale).to(torch.float8_e4m3fn).float()
                o[b, h, r0:r1] = (p8 @ vs) / (l * p_scale) * sv[b, h][None, :]
    return o


# ----------------------------------------------------------------------------------------------
# Block-gather evaluation of the whole module, differentiable (the timed CPU baseline)
# ----------------------------------------------------------------------------------------------
def sla_forward_gather_fp(q, k, v, weight, bias, lut, feature="softmax", BLKQ=64, BLKK=64, qk_scale=None):
    """core.py:88-100 for a fixed LUT in the dtype given (fp32), vectorised over the query blocks of
    one head at a time: K/V blocks are gathered per LUT row (kernel.py:55-76), the softmax is taken
    over the gathered keys, and the linear branch (core.py:90-96) and proj_l (core.py:98-99) follow.
    Differentiable with torch.autograd; cost is proportional to the selected pairs, so it is usable
    at full sequence length on the host cores."""
    B, H, L, D = q.shape
    if qk_scale is None:
        qk_scale = D ** -0.5
    mb = (L + BLKQ - 1) // BLKQ
    nb = (L + BLKK - 1) // BLKK
    topk = lut.shape[-1]
    padq, padk = mb * BLKQ - L, nb * BLKK - L
    key_pos = torch.arange(nb * BLKK).view(nb, BLKK)
    outs = []
    for b in range(B):
        row = []
        for h in range(H):
            qh, kh, vh = q[b, h], k[b, h], v[b, h]
            qb = F.pad(qh, (0, 0, 0, padq)).view(mb, BLKQ, D)
            kb = F.pad(kh, (0, 0, 0, padk)).view(nb, BLKK, D)
            vb = F.pad(vh, (0, 0, 0, padk)).view(nb, BLKK, D)
            idx = lut[b, h].long()                                   # (mb, topk)
            ks = kb[idx].reshape(mb, topk * BLKK, D)
            vs = vb[idx].reshape(mb, topk * BLKK, D)
            valid = (key_pos[idx].reshape(mb, 1, topk * BLKK) < L)
            s = torch.bmm(qb, ks.transpose(1, 2)) * qk_scale
            s = s.masked_fill(~valid, float("-inf"))
            o_s = torch.bmm(torch.softmax(s, dim=-1), vs).reshape(mb * BLKQ, D)[:L]
            cq, ck = feature_map(qh, feature), feature_map(kh, feature)
            o_l = calc_linear(cq, ck, vh)
            row.append(o_s + o_l @ weight.t() + bias)
        outs.append(torch.stack(row))
    return torch.stack(outs)
