"""A self-contained rope-DiT: the caller of llsa_l1 / llsa_l2 in SingleZombie/LLSA, restated in plain PyTorch.

What it mirrors (models/rope_dit_transformer_2d.py of the reference; the diffusers layers that file leans on are
restated here from their published definitions, since diffusers is not a dependency):

  RopeDiTTransformer2DModel (:735-1058)  pixel-space DiT: 1x1 patch embedding, Morton token permutation in and out
                                          (:714-732, :933-936, :1001-1003), N adaLN-zero blocks, adaLN output head
  RopeTransformerBlock (:357-711)         adaLN-zero (:295-337): every block owns a timestep embedder
                                          (Timesteps(256, flip_sin_to_cos, shift 1) -> Linear, SiLU, Linear),
                                          LayerNorm(eps 1e-6, no affine), attention, gated residual, LayerNorm(eps 1e-5,
                                          no affine) modulated, GELU(tanh) MLP x4, gated residual
  RopeAttnProcessor (:112-260)            q, k, v projections -> [B,H,N,D] views of [B,N,H,D] storage -> RMSNorm on q, k
                                          -> 2-D RoPE (table per grid size, Morton-permuted positions) -> attention
                                          ("pixel": dense; "sparse_l1": llsa_l1; "sparse_l2": llsa_l2) -> to_out

The default configuration is configs/models/model_rope_dit_S_128_rms_llsa_l2.json: 12 layers, 6 heads x 64,
128 x 128 x 3 input at patch size 1 (16384 tokens), axes_dims_rope (32, 32), qk RMSNorm, sparse_l2 with top-8.
Weights are randomly initialised (structural, not weight, parity).  `fused_rope=True` rotates q and k inside the
pooling pass (llsa_l1_rope / llsa_l2_rope); False calls my_rope_fn first, exactly as the reference's processor does.
The "pixel" attention type runs on any device (it is what the CPU tests use); the sparse types need a B200.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import synth

__all__ = ["RopeDiT", "timestep_embedding"]


def timestep_embedding(t: torch.Tensor, dim: int = 256, max_period: float = 10000.0) -> torch.Tensor:
    """Sinusoidal embedding with the cosine half first and frequencies exp(-ln(max_period) * i / (dim/2 - 1)):
    Timesteps(num_channels=256, flip_sin_to_cos=True, downscale_freq_shift=1) as the reference builds it
    (rope_dit_transformer_2d.py:266-267)."""
    half = dim // 2
    freqs = torch.exp(-math.log(max_period) * torch.arange(half, dtype=torch.float32, device=t.device) / (half - 1))
    args = t.float()[:, None] * freqs[None, :]
    return torch.cat([torch.cos(args), torch.sin(args)], dim=-1)


class TimestepEmbedder(nn.Module):
    def __init__(self, dim: int):
        super().__init__()
        self.linear_1 = nn.Linear(256, dim)
        self.linear_2 = nn.Linear(dim, dim)

    def forward(self, t: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
        return self.linear_2(F.silu(self.linear_1(timestep_embedding(t).to(dtype))))


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-5):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(dim))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        var = x.float().pow(2).mean(-1, keepdim=True)
        return (x.float() * torch.rsqrt(var + self.eps)) * self.weight


class RopeAttention(nn.Module):
    """Attention + RopeAttnProcessor.__call__ (rope_dit_transformer_2d.py:186-260)."""

    def __init__(self, dim: int, heads: int, head_dim: int, attn_type: str, topk: int, block_size: int, qk_norm: bool, fused_rope: bool):
        super().__init__()
        inner = heads * head_dim
        self.heads, self.head_dim = heads, head_dim
        self.attn_type, self.topk, self.block_size, self.fused_rope = attn_type, topk, block_size, fused_rope
        self.to_q = nn.Linear(dim, inner)
        self.to_k = nn.Linear(dim, inner)
        self.to_v = nn.Linear(dim, inner)
        self.norm_q = RMSNorm(head_dim) if qk_norm else None
        self.norm_k = RMSNorm(head_dim) if qk_norm else None
        self.to_out = nn.Linear(inner, dim)

    def forward(self, x: torch.Tensor, rope_table: torch.Tensor) -> torch.Tensor:
        B, N, _ = x.shape
        q = self.to_q(x).view(B, N, self.heads, self.head_dim).transpose(1, 2)     # [B,H,N,D] view of [B,N,H,D] storage
        k = self.to_k(x).view(B, N, self.heads, self.head_dim).transpose(1, 2)
        v = self.to_v(x).view(B, N, self.heads, self.head_dim).transpose(1, 2)
        dt = q.dtype
        table = rope_table.to(dt)
        if self.norm_q is not None and self.fused_rope and self.attn_type != "pixel" and q.is_cuda:
            # q / k RMSNorm, rotation and pooling in one pass over q and k (rope_dit_transformer_2d.py:215-251)
            from . import ops
            bs, t = self.block_size, self.topk
            if self.attn_type == "sparse_l1":
                o = ops.llsa_l1_rms_rope(q, k, v, self.norm_q.weight, self.norm_k.weight, table, self.norm_q.eps, t, bs)
            else:
                o = ops.llsa_l2_rms_rope(q, k, v, self.norm_q.weight, self.norm_k.weight, table, self.norm_q.eps, t, t, bs)
            o = o.transpose(1, 2).reshape(B, N, self.heads * self.head_dim).to(dt)
            return self.to_out(o)
        if self.norm_q is not None:
            q, k = self.norm_q(q).to(dt), self.norm_k(k).to(dt)
        if self.attn_type == "pixel":
            q, k = _rope_eager(q, table), _rope_eager(k, table)
            o = F.scaled_dot_product_attention(q, k, v, dropout_p=0.0, is_causal=False)
        else:
            from . import ops
            bs, t = self.block_size, self.topk
            if self.fused_rope:
                o = ops.llsa_l1_rope(q, k, v, table, t, bs) if self.attn_type == "sparse_l1" else ops.llsa_l2_rope(q, k, v, table, t, t, bs)
            else:
                q, k = ops.my_rope_fn(q, table), ops.my_rope_fn(k, table)
                o = ops.llsa_l1(q, k, v, t, bs) if self.attn_type == "sparse_l1" else ops.llsa_l2(q, k, v, t, t, bs)
        o = o.transpose(1, 2).reshape(B, N, self.heads * self.head_dim).to(dt)
        return self.to_out(o)


def _rope_eager(x: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    """Interleaved-pair rotation (triton/rope.py:37-47): even table columns sin, odd columns cos."""
    sn, cs = table[:, 0::2], table[:, 1::2]
    xe, xo = x[..., 0::2], x[..., 1::2]
    return torch.stack([cs * xe - sn * xo, sn * xe + cs * xo], dim=-1).flatten(-2).to(x.dtype)


class RopeDiTBlock(nn.Module):
    def __init__(self, dim: int, heads: int, head_dim: int, attn_type: str, topk: int, block_size: int, qk_norm: bool, fused_rope: bool):
        super().__init__()
        self.emb = TimestepEmbedder(dim)
        self.ada = nn.Linear(dim, 6 * dim)
        self.norm1 = nn.LayerNorm(dim, elementwise_affine=False, eps=1e-6)
        self.attn = RopeAttention(dim, heads, head_dim, attn_type, topk, block_size, qk_norm, fused_rope)
        self.norm2 = nn.LayerNorm(dim, elementwise_affine=False, eps=1e-5)
        self.ff_in = nn.Linear(dim, 4 * dim)
        self.ff_out = nn.Linear(4 * dim, dim)

    def forward(self, x: torch.Tensor, t: torch.Tensor, rope_table: torch.Tensor) -> torch.Tensor:
        mod = self.ada(F.silu(self.emb(t, x.dtype)))
        shift_msa, scale_msa, gate_msa, shift_mlp, scale_mlp, gate_mlp = mod.chunk(6, dim=1)
        h = self.norm1(x) * (1 + scale_msa[:, None]) + shift_msa[:, None]
        x = gate_msa.unsqueeze(1) * self.attn(h, rope_table) + x
        h = self.norm2(x) * (1 + scale_mlp[:, None]) + shift_mlp[:, None]
        h = self.ff_out(F.gelu(self.ff_in(h), approximate="tanh"))
        return gate_mlp.unsqueeze(1) * h + x


class RopeDiT(nn.Module):
    def __init__(self, heads: int = 6, head_dim: int = 64, layers: int = 12, in_channels: int = 3, out_channels: Optional[int] = 3,
                 sample_size: int = 128, axes_dims_rope=(32, 32), attn_type: str = "sparse_l2", sparse_topk: int = 8,
                 sparse_block_size: int = 16, qk_norm: bool = True, token_permutation: bool = True, fused_rope: bool = True):
        super().__init__()
        assert attn_type in ("pixel", "sparse_l1", "sparse_l2")
        assert sum(axes_dims_rope) == head_dim
        dim = heads * head_dim
        self.dim, self.sample_size, self.token_permutation = dim, sample_size, token_permutation
        self.axes_dims_rope = tuple(axes_dims_rope)
        self.out_channels = in_channels if out_channels is None else out_channels
        self.proj_in = nn.Conv2d(in_channels, dim, kernel_size=1, stride=1)
        self.blocks = nn.ModuleList([RopeDiTBlock(dim, heads, head_dim, attn_type, sparse_topk, sparse_block_size, qk_norm, fused_rope)
                                     for _ in range(layers)])
        self.norm_out = nn.LayerNorm(dim, elementwise_affine=False, eps=1e-6)
        self.proj_out_1 = nn.Linear(dim, 2 * dim)
        self.proj_out_2 = nn.Linear(dim, self.out_channels)
        self._tables = {}

    def _grid(self, side: int, device):
        """(forward permutation, backward permutation, RoPE table) of a side x side token grid."""
        key = (side, str(device))
        if key not in self._tables:
            perm, inv = synth.morton_perm(side)
            table = synth.rope_table_2d(side, axes_dim=self.axes_dims_rope, morton=self.token_permutation, dtype=torch.float32)
            self._tables[key] = (torch.from_numpy(inv).to(device), torch.from_numpy(perm).to(device), table.to(device))
        return self._tables[key]

    def forward(self, x: torch.Tensor, timestep: torch.Tensor) -> torch.Tensor:
        """x [B, C, S, S], timestep [B] -> prediction [B, out_channels, S, S]."""
        B, _, S, _ = x.shape
        fwd, bwd, table = self._grid(S, x.device)
        h = self.proj_in(x).reshape(B, self.dim, S * S).transpose(1, 2)
        if self.token_permutation:
            h = h[:, fwd, :]
        timestep = timestep.expand(B)
        for blk in self.blocks:
            h = blk(h, timestep, table)
        if self.token_permutation:
            h = h[:, bwd, :]
        cond = self.blocks[0].emb(timestep, h.dtype)
        shift, scale = self.proj_out_1(F.silu(cond)).chunk(2, dim=1)
        h = self.norm_out(h) * (1 + scale[:, None]) + shift[:, None]
        h = self.proj_out_2(h)
        return h.transpose(1, 2).reshape(B, self.out_channels, S, S)
