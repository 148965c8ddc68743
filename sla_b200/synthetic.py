"""Seeded synthetic workloads with the shapes and value distributions of the benchmark configurations.

They stand in for video-diffusion attention inputs: no dataset is read. Two families:

* ``randn``: q, k, v (and dO) ~ N(0, 1) from one seed (the small configurations and the reference's
  own kernel benchmark, evaluate/bench_kernel.py:62-65).
* ``grid3d``: tokens are the cells of a (T, H, W) latent grid. q and k get a positional term
  ``f(n) P`` added to 0.5*N(0,1) noise, where f(n) holds sin/cos of the three grid coordinates at 32
  frequencies per axis (theta_i = 10000^(-i/32)) and P is a fixed Gaussian 192 x D matrix (seed 1234,
  scaled by 1/sqrt(192)) shared by q and k, so that nearby tokens score high and the block scores are
  structured like attention maps of video models. v, dO ~ N(0, 1).

Every (batch, head) unit has its own noise seed (1000*cfg + 131*b + h), so any sharding of the units
over GPUs sees identical data.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Tuple

import torch


@dataclass(frozen=True)
class Workload:
    name: str
    cfg: int
    B: int
    H: int
    L: int
    D: int
    BLKQ: int
    BLKK: int
    topk: float
    feature: str = "softmax"
    dtype: torch.dtype = torch.bfloat16
    in_dtype: torch.dtype = torch.bfloat16
    grid: Optional[Tuple[int, int, int]] = None   # None -> plain randn
    seed: int = 0
    backward: bool = True
    quantized: bool = False

    @property
    def units(self) -> int:
        return self.B * self.H

    @property
    def m_blocks(self) -> int:
        return (self.L + self.BLKQ - 1) // self.BLKQ

    @property
    def n_blocks(self) -> int:
        return (self.L + self.BLKK - 1) // self.BLKK

    @property
    def topk_blocks(self) -> int:
        return min(self.n_blocks, int(self.topk * self.n_blocks))

    # ---- algorithmic work (per whole workload) ----
    def dense_equiv_flops(self, backward: bool) -> float:
        f = 4.0 * self.B * self.H * float(self.L) ** 2 * self.D   # evaluate/bench_kernel.py:93-94
        return f * 3.5 if backward else f                        # fwd + 2.5x bwd (bench_kernel.py:97-98)

    def sparse_flops(self, backward: bool) -> float:
        pair = 2.0 * self.BLKQ * self.BLKK * self.D
        pairs = float(self.B * self.H * self.m_blocks * self.topk_blocks)
        return pairs * pair * (7 if backward else 2)

    def linear_flops(self, backward: bool) -> float:
        f = self.B * self.H * 3 * 2.0 * self.L * self.D * self.D
        return f * 3 if backward else f

    def io_bytes(self, backward: bool) -> float:
        t = float(self.B * self.H * self.L * self.D * 2)
        return t * (4 + 8) if backward else t * 4


WORKLOADS = {
    "c1": Workload("c1", 1, 1, 2, 1024, 64, 64, 64, 0.25, in_dtype=torch.float32, seed=0, backward=False),
    "c2": Workload("c2", 2, 2, 4, 4096, 128, 64, 64, 0.2, seed=1),
    "c3": Workload("c3", 3, 1, 12, 32760, 128, 64, 64, 0.05, grid=(21, 30, 52)),
    "c4": Workload("c4", 4, 1, 40, 75600, 128, 128, 64, 0.05, grid=(21, 45, 80), backward=False, quantized=True),
    "c5": Workload("c5", 5, 1, 16, 131072, 64, 128, 64, 0.05, feature="relu", grid=(32, 64, 64)),
    "refbench": Workload("refbench", 6, 2, 16, 32760, 128, 128, 64, 0.05, seed=42),
    "tiny": Workload("tiny", 9, 1, 2, 1000, 64, 64, 64, 0.25, grid=(5, 10, 20)),
    # 2 of c3's 12 heads: the same kernels and per-CTA work on 130 MB of tensors, sized for profiler captures
    "c3s": Workload("c3s", 3, 1, 2, 32760, 128, 64, 64, 0.05, grid=(21, 30, 52)),
    # 8 of c4's 40 heads: the same kernels and per-CTA work on 0.6 GB of inputs, sized for profiler captures
    "c4s": Workload("c4s", 4, 1, 8, 75600, 128, 128, 64, 0.05, grid=(21, 45, 80), backward=False, quantized=True),
}


def _positional_features(L: int, grid: Tuple[int, int, int], device) -> torch.Tensor:
    T, Hh, Ww = grid
    assert T * Hh * Ww >= L
    n = torch.arange(L, device=device)
    coords = [(n // (Hh * Ww)).float(), ((n // Ww) % Hh).float(), (n % Ww).float()]
    theta = 10000.0 ** (-torch.arange(32, device=device, dtype=torch.float32) / 32.0)
    feats = []
    for c in coords:
        ang = c[:, None] * theta[None, :]
        feats.append(torch.stack([torch.sin(ang), torch.cos(ang)], dim=-1).reshape(L, 64))
    return torch.cat(feats, dim=-1)  # (L, 192)


def _projection(D: int, device) -> torch.Tensor:
    g = torch.Generator(device="cpu").manual_seed(1234)
    return (torch.randn(192, D, generator=g) / (192 ** 0.5)).to(device)


def make_unit(w: Workload, unit: int, device, with_do: bool = True):
    """q, k, v, dO of one (batch, head) unit, shape (L, D), in w.in_dtype."""
    b, h = divmod(unit, w.H)
    g = torch.Generator(device=device).manual_seed(1000 * w.cfg + 131 * b + h)
    shape = (w.L, w.D)
    q = torch.randn(shape, generator=g, device=device)
    k = torch.randn(shape, generator=g, device=device)
    v = torch.randn(shape, generator=g, device=device)
    do = torch.randn(shape, generator=g, device=device) if with_do else None
    if w.grid is not None:
        pos = _positional_features(w.L, w.grid, device) @ _projection(w.D, device)
        q = 0.5 * q + pos
        k = 0.5 * k + pos
    out = [t.to(w.in_dtype) for t in (q, k, v)]
    out.append(do.to(w.in_dtype) if with_do else None)
    return out


def make_inputs(w: Workload, device, units: Optional[List[int]] = None, with_do: bool = True):
    """Tensors (1, U, L, D) holding the listed units (default: all B*H units as (B, H, L, D))."""
    if w.grid is None and units is None:
        # one seed for the whole tensor, drawn in the order q, k, v, dO
        g = torch.Generator(device="cpu").manual_seed(w.seed)
        shape = (w.B, w.H, w.L, w.D)
        ts = [torch.randn(shape, generator=g) for _ in range(4 if with_do else 3)]
        ts = [t.to(w.in_dtype).to(device) for t in ts]
        return ts + ([None] if not with_do else [])
    ids = list(range(w.units)) if units is None else units
    parts = [make_unit(w, u, device, with_do) for u in ids]
    stack = lambda i: None if parts[0][i] is None else torch.stack([p[i] for p in parts])
    q, k, v, do = (stack(i) for i in range(4))
    if units is None:
        rs = lambda t: None if t is None else t.view(w.B, w.H, w.L, w.D)
    else:
        rs = lambda t: None if t is None else t.view(1, len(ids), w.L, w.D)
    return [rs(q), rs(k), rs(v), rs(do)]


def make_proj(w: Workload, device, std: float = 0.02):
    """proj_l parameters W ~ N(0, std^2), b = 0 (seeded); the module's own init is all zeros."""
    g = torch.Generator(device="cpu").manual_seed(7 + w.cfg)
    return (torch.randn(w.D, w.D, generator=g) * std).to(device), torch.zeros(w.D, device=device)
