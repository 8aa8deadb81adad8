"""Unbounded differential attention in plain PyTorch.

Only here so that the adapters' ``bounded=False`` mode constructs and runs (training-style full
causal attention with an O(L) cache, upstream ``src/coda_gqa_l/baseline.py:22-147``).  It is not
part of the accelerated path and uses no custom kernel.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from .primitives import HeadwiseRMSNorm, RotaryEmbedding


def _rotate_pairs(x, c, s):
    out = torch.empty_like(x)
    xe, xo = x[..., 0::2], x[..., 1::2]
    out[..., 0::2] = xe * c - xo * s
    out[..., 1::2] = xe * s + xo * c
    return out


def _rope(x, cos, sin, interleaved):
    L, half = cos.shape
    c, s = cos.view(1, 1, L, half), sin.view(1, 1, L, half)
    if interleaved:
        return _rotate_pairs(x, c, s)
    return x * torch.cat([c, c], -1) + torch.cat([-x[..., half:], x[..., :half]], -1) * torch.cat([s, s], -1)


class CoDAGQA(nn.Module):
    def __init__(self, *, embed_dim: int, num_heads: int, num_kv_heads: int, rope_base: float = 10_000.0,
                 lambda_init_bias: float = -6.0, theta_init: float = math.pi / 2, eps: float = 1e-6,
                 head_norm_mode: str = "full", rope_interleaved: bool = True):
        super().__init__()
        if embed_dim % num_heads != 0:
            raise ValueError("embed_dim must be divisible by num_heads.")
        if num_heads % num_kv_heads != 0:
            raise ValueError("num_heads must be divisible by num_kv_heads (GQA constraint).")
        self.embed_dim, self.num_heads, self.num_kv_heads = embed_dim, num_heads, num_kv_heads
        self.head_dim = embed_dim // num_heads
        if self.head_dim % 2 != 0:
            raise ValueError("head_dim must be even (required by RoPE + pairwise rotations).")
        H, Hkv, Dh = num_heads, num_kv_heads, self.head_dim
        self.q_proj = nn.Linear(embed_dim, H * Dh, bias=False)
        self.k_proj = nn.Linear(embed_dim, Hkv * Dh, bias=False)
        self.v_proj = nn.Linear(embed_dim, Hkv * Dh, bias=False)
        self.theta = nn.Parameter(torch.full((H, Dh // 2), theta_init))
        self.lambda_proj = nn.Linear(embed_dim, H, bias=True)
        nn.init.constant_(self.lambda_proj.bias, lambda_init_bias)
        self.rope = RotaryEmbedding(Dh, base=rope_base)
        self.head_norm_mode = head_norm_mode
        if head_norm_mode == "full":
            self.head_norm = HeadwiseRMSNorm(Dh, eps=eps)
        elif head_norm_mode == "identity":
            self.head_norm = nn.Identity()
        else:
            raise ValueError(f"head_norm_mode must be 'full' or 'identity', got {head_norm_mode!r}")
        self.rope_interleaved = bool(rope_interleaved)
        self.o_proj = nn.Linear(H * Dh, embed_dim, bias=False)

    def forward(self, x: torch.Tensor, *, is_causal: bool = True, attention_mask: Optional[torch.Tensor] = None,
                past_key_value: Optional[Tuple[torch.Tensor, torch.Tensor]] = None):
        B, L, D = x.shape
        H, Hkv, Dh = self.num_heads, self.num_kv_heads, self.head_dim
        split = lambda y, n: y.view(B, L, n, Dh).transpose(1, 2)  # noqa: E731
        q, k, v = split(self.q_proj(x), H), split(self.k_proj(x), Hkv), split(self.v_proj(x), Hkv)
        off = 0 if past_key_value is None else past_key_value[0].size(2)
        t = torch.arange(off, off + L, device=x.device, dtype=self.rope.inv_freq.dtype)
        ang = torch.outer(t, self.rope.inv_freq)
        cos, sin = ang.cos().to(q.dtype), ang.sin().to(q.dtype)
        q, k = _rope(q, cos, sin, self.rope_interleaved), _rope(k, cos, sin, self.rope_interleaved)
        if past_key_value is not None:
            k, v = torch.cat([past_key_value[0], k], 2), torch.cat([past_key_value[1], v], 2)
        G = H // Hkv
        kx, vx = k.repeat_interleave(G, 1), v.repeat_interleave(G, 1)
        lam = torch.sigmoid(self.lambda_proj(x)).transpose(1, 2).unsqueeze(-1)
        half = Dh // 2
        ct = torch.cos(self.theta).to(q.dtype).view(1, H, 1, half)
        st = torch.sin(self.theta).to(q.dtype).view(1, H, 1, half)
        causal = is_causal if attention_mask is None else False
        sig = F.scaled_dot_product_attention(q, kx, vx, attn_mask=attention_mask, is_causal=causal)
        noise = F.scaled_dot_product_attention(_rotate_pairs(q, ct, st), kx, vx, attn_mask=attention_mask, is_causal=causal)
        out = self.head_norm(sig - lam * noise)
        return self.o_proj(out.transpose(1, 2).contiguous().view(B, L, D)), (k, v)
