"""Small modules kept for interface and checkpoint compatibility with upstream
``src/coda_gqa_l/primitives.py``.  The arithmetic they describe runs inside the CUDA kernels;
these classes only own the parameters / buffers the kernels read."""
from __future__ import annotations

import torch
import torch.nn as nn


class HeadwiseRMSNorm(nn.Module):
    """Owner of the per-dimension scale of the head norm (upstream primitives.py:15-27).

    ``forward`` is provided for completeness (plain tensor ops on whatever device x lives on);
    the attention kernels apply the same formula in their epilogue."""

    def __init__(self, head_dim: int, eps: float = 1e-6):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(head_dim))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        var = x.pow(2).mean(dim=-1, keepdim=True)
        return x * torch.rsqrt(var + self.eps) * self.weight


class RotaryEmbedding(nn.Module):
    """Owner of ``inv_freq`` (upstream primitives.py:30-55).

    ``inv_freq`` is a non-persistent buffer exactly as upstream, so ``module.to(dtype)`` casts it;
    the kernels evaluate the angles in that buffer's dtype to reproduce upstream's numbers."""

    def __init__(self, head_dim: int, base: float = 10_000.0):
        super().__init__()
        if head_dim % 2 != 0:
            raise ValueError("RoPE requires even head_dim.")
        self.base = float(base)
        inv_freq = 1.0 / (base ** (torch.arange(0, head_dim, 2).float() / head_dim))
        self.register_buffer("inv_freq", inv_freq, persistent=False)
