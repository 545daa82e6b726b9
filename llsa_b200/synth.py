"""Seeded synthetic inputs for the LLSA attention shapes (host side, numpy).

The reference measures on FFHQ images and `torch.randn` tensors
(test_kernel.py:41-43); neither a dataset nor the reference is needed here:
these generators produce tensors of the same shapes and value distribution.

All draws come from numpy's PCG64 (`default_rng(seed)`), which is bit-stable
across machines, so the same seed gives the same bytes on the build box and
on the GPU box.  Tokens are laid out in the repo's quad-tree (Morton) order
(models/rope_dit_transformer_2d.py:714-732).
"""
from __future__ import annotations

import math
from typing import Dict, Optional

import numpy as np
import torch

__all__ = ["morton_perm", "gaussian_qkv", "correlated_qkv", "rope_table_2d", "CONFIGS", "make_config_inputs"]


def morton_perm(side: int):
    """perm[r*side+c] = Morton code (column bits even, row bits odd); returns (perm, inv_perm)."""
    bits = int(round(math.log2(side)))
    assert 1 << bits == side, "grid side must be a power of two"
    r, c = np.meshgrid(np.arange(side), np.arange(side), indexing="ij")
    code = np.zeros((side, side), dtype=np.int64)
    for i in range(bits):
        code |= ((c >> i) & 1) << (2 * i)
        code |= ((r >> i) & 1) << (2 * i + 1)
    perm = code.reshape(-1)
    inv = np.empty_like(perm)
    inv[perm] = np.arange(side * side)
    return perm, inv


def _normal(rng, shape):
    return rng.standard_normal(shape, dtype=np.float32)


def gaussian_qkv(seed: int, B: int, H: int, N: int, D: int, n_tensors: int = 4, dtype=torch.float32):
    """n_tensors iid N(0,1) tensors [B,H,N,D] drawn in order from one generator
    (q, k, v, upstream grad), generated in fp32 then cast."""
    rng = np.random.default_rng(seed)
    return [torch.from_numpy(_normal(rng, (B, H, N, D))).to(dtype) for _ in range(n_tensors)]


def _low_freq_basis(side: int, inv_perm: np.ndarray) -> np.ndarray:
    """The 4 lowest non-constant 2-D cosine modes on the side x side grid, unit
    RMS each, listed in Morton token order: [4, side*side] fp32."""
    y = (np.arange(side, dtype=np.float64) + 0.5) / side
    c1 = np.cos(np.pi * y)
    c2 = np.cos(2 * np.pi * y)
    one = np.ones(side)
    modes = [np.outer(c1, one), np.outer(one, c1), np.outer(c1, c1), np.outer(c2, one) + np.outer(one, c2)]
    out = []
    for m in modes:
        m = m / np.sqrt(np.mean(m * m))
        out.append(m.reshape(-1)[inv_perm])        # token n sits at row-major position inv_perm[n]
    return np.stack(out).astype(np.float32)


def correlated_qkv(seed: int, B: int, H: int, N: int, D: int, n_tensors: int = 4, amp: float = 0.5,
                   dtype=torch.bfloat16, correlated=(True, True, True, False)):
    """N(0,1) plus `amp` times a smooth low-frequency 2-D field per (b,h,channel):
    a random combination (N(0,1) coefficients, normalised to unit RMS) of the 4
    lowest cosine modes of the sqrt(N) x sqrt(N) grid, so that block similarity
    is spatially correlated.  The upstream grad (4th tensor) stays iid."""
    side = int(round(math.sqrt(N)))
    assert side * side == N
    _, inv = morton_perm(side)
    basis = torch.from_numpy(_low_freq_basis(side, inv))            # [4, N]
    rng = np.random.default_rng(seed)
    out = []
    for i in range(n_tensors):
        x = torch.from_numpy(_normal(rng, (B, H, N, D)))
        if i < len(correlated) and correlated[i]:
            coef = torch.from_numpy(_normal(rng, (B, H, D, 4))) * 0.5   # 4 unit-RMS modes -> unit RMS field
            x += amp * torch.einsum("bhdm,mn->bhnd", coef, basis)
        out.append(x.to(dtype))
    return out


def rope_table_2d(side: int, axes_dim=(32, 32), theta: float = 10000.0, morton: bool = True,
                  dtype=torch.float32) -> torch.Tensor:
    """The [N, D] sin/cos table the model builds for a side x side image at
    patch size 1 (rope_dit_transformer_2d.py:71-109,153-173): even columns sin,
    odd columns cos; row-axis frequencies first, then column-axis; positions in
    Morton order when `morton`; computed in fp64 then cast."""
    r, c = np.meshgrid(np.arange(side, dtype=np.float64), np.arange(side, dtype=np.float64), indexing="ij")
    ids = np.stack([r.reshape(-1), c.reshape(-1)], -1)
    if morton:
        _, inv = morton_perm(side)
        ids = ids[inv]                              # the model permutes ids with its forward perm = inv_perm (:168-170, :846-849)
    parts = []
    for a, dim in enumerate(axes_dim):
        omega = 1.0 / (theta ** (np.arange(0, dim, 2, dtype=np.float64) / dim))
        ang = ids[:, a, None] * omega[None, :]
        parts.append(np.stack([np.sin(ang), np.cos(ang)], -1).reshape(-1, dim))
    return torch.from_numpy(np.concatenate(parts, -1)).to(dtype)


# The attention shapes of the five benchmark configurations (config 4 is a
# whole-model training step whose attention shape equals config 3's).
CONFIGS: Dict[str, dict] = {
    "cfg1": dict(op="llsa_l1", dtype=torch.float32, B=1, H=2, N=1024, D=64, seed=0, correlated=False, rope=False),
    "cfg2": dict(op="llsa_l1", dtype=torch.bfloat16, B=4, H=6, N=4096, D=64, seed=2, correlated=True, rope=True),
    "cfg3": dict(op="llsa_l2", dtype=torch.bfloat16, B=8, H=6, N=16384, D=64, seed=3, correlated=True, rope=False),
    "cfg5": dict(op="llsa_l2", dtype=torch.bfloat16, B=1, H=6, N=262144, D=64, seed=5, correlated=True, rope=False),
}


def make_config_inputs(name: str, B: Optional[int] = None, H: Optional[int] = None):
    """(q, k, v, do, rope_table_or_None) on the host for a named configuration;
    B/H override the batch/head counts (used to shard or to bound CPU work)."""
    c = CONFIGS[name]
    B = c["B"] if B is None else B
    H = c["H"] if H is None else H
    if c["correlated"]:
        q, k, v, do = correlated_qkv(c["seed"], B, H, c["N"], c["D"], dtype=c["dtype"])
    else:
        q, k, v, do = gaussian_qkv(c["seed"], B, H, c["N"], c["D"], dtype=c["dtype"])
    table = None
    if c["rope"]:
        table = rope_table_2d(int(round(math.sqrt(c["N"]))), dtype=c["dtype"])
    return q, k, v, do, table
