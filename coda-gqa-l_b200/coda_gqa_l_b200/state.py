"""Inference state of one bounded-cache layer.

Field names and meanings follow upstream ``src/coda_gqa_l/state.py:12-54`` so that code written
against the upstream dataclass (serialisation helpers, adapters, tests) keeps working.  The
tensors of a state created by ``CoDAGQALandmarkPerf2.init_state`` are views into ONE contiguous
per-layer allocation (the slot arena): K plane, V plane, then the routing caches and the small
metadata planes, so that a layer's whole state is one HBM range.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, Optional

import torch


@dataclass
class CoDAGQALandmarkStatePerf2:
    """Mutable state for one layer.  Buffer layout along the slot axis: [recent W | exact Me | summary Ms]."""

    k_buf: torch.Tensor       # (B, Hkv, Lbuf, Dh) keys, RoPE already applied
    v_buf: torch.Tensor       # (B, Hkv, Lbuf, Dh)
    allowed: torch.Tensor     # (B, Lbuf) bool, True = slot holds valid data

    g_recent: torch.Tensor    # (B, W) float32 write gate of each ring slot
    recent_idx: int           # next ring slot to evict once the ring is full
    recent_filled: int        # occupied ring slots (<= W)

    mem_last_exact: torch.Tensor  # (B, Me) int64 LRU stamps

    pos: int                  # absolute position of the next token

    active_exact: int = 0
    active_summary: int = 0

    _exact_v_norm: Optional[torch.Tensor] = field(default=None, repr=False)   # (B,Hkv,Me,Dh)
    _sum_lf_k_norm: Optional[torch.Tensor] = field(default=None, repr=False)  # (B,Hkv,Ms,Dh/2)

    metrics: Optional[Dict[str, Any]] = field(default=None, repr=False)

    # The single allocation the tensors above are carved from (None for states built field by field).
    _arena: Optional[torch.Tensor] = field(default=None, repr=False, compare=False)
    # int32 (B, 16) routing-event record the cache-write kernels fill when metrics or bank expansion are on
    _events: Optional[torch.Tensor] = field(default=None, repr=False, compare=False)

    def __getstate__(self):
        """Pickle / ``torch.save`` support: the arena's planes have different dtypes over one storage,
        which the serialiser refuses, so every tensor is saved as its own copy and the arena is dropped."""
        d = dict(self.__dict__)
        d["_arena"] = None
        d["_events"] = None
        for k, v in d.items():
            if torch.is_tensor(v):
                d[k] = v.detach().clone()
        return d

    def __setstate__(self, d):
        self.__dict__.update(d)


def _align(n: int, a: int = 256) -> int:
    return (n + a - 1) // a * a


def arena_layout(B: int, Hkv: int, Dh: int, W: int, Me: int, Ms: int, esize: int):
    """Byte offsets of each plane inside the per-layer arena, and the total size.

    Order: k_buf, v_buf, exact_v_norm, sum_lf_k_norm, g_recent, mem_last_exact, allowed.
    Every plane starts on a 256-byte boundary (TMA needs 16; 256 keeps planes sector-aligned).
    """
    Lbuf = W + Me + Ms
    lfd = Dh - Dh // 2
    sizes = [
        ("k_buf", B * Hkv * Lbuf * Dh * esize),
        ("v_buf", B * Hkv * Lbuf * Dh * esize),
        ("exact_v_norm", B * Hkv * Me * Dh * esize),
        ("sum_lf_k_norm", B * Hkv * Ms * lfd * esize),
        ("g_recent", B * W * 4),
        ("mem_last_exact", B * Me * 8),
        ("allowed", B * Lbuf),
    ]
    off, out = 0, {}
    for name, nbytes in sizes:
        out[name] = (off, nbytes)
        off = _align(off + nbytes)
    return out, max(off, 256)


def allocate_state(B: int, Hkv: int, Dh: int, W: int, Me: int, Ms: int,
                   device, dtype: torch.dtype) -> CoDAGQALandmarkStatePerf2:
    """Zero-initialised state whose tensors are views into one arena allocation."""
    esize = torch.tensor([], dtype=dtype).element_size()
    lay, total = arena_layout(B, Hkv, Dh, W, Me, Ms, esize)
    arena = torch.zeros(total, dtype=torch.uint8, device=device)
    Lbuf, lfd = W + Me + Ms, Dh - Dh // 2

    def view(name, dt, shape):
        off, nbytes = lay[name]
        return arena[off:off + nbytes].view(dt).view(shape)

    return CoDAGQALandmarkStatePerf2(
        k_buf=view("k_buf", dtype, (B, Hkv, Lbuf, Dh)),
        v_buf=view("v_buf", dtype, (B, Hkv, Lbuf, Dh)),
        allowed=view("allowed", torch.bool, (B, Lbuf)),
        g_recent=view("g_recent", torch.float32, (B, W)),
        recent_idx=0, recent_filled=0,
        mem_last_exact=view("mem_last_exact", torch.int64, (B, Me)),
        pos=0,
        _exact_v_norm=view("exact_v_norm", dtype, (B, Hkv, Me, Dh)) if Me > 0 else None,
        _sum_lf_k_norm=view("sum_lf_k_norm", dtype, (B, Hkv, Ms, lfd)) if Ms > 0 else None,
        _arena=arena,
    )
