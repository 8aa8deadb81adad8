"""Moving, copying and importing layer states.

The three helpers mirror upstream ``src/coda_gqa_l/neural_db.py:30-82`` (they define which
attributes a serialisable state exposes); ``state_from_fields`` packs any object with those
attributes (an upstream state, a CPU-staged state) into a fresh arena on a CUDA device.
"""
from __future__ import annotations

import torch

from .state import CoDAGQALandmarkStatePerf2, allocate_state

_TENSORS = ("k_buf", "v_buf", "allowed", "g_recent", "mem_last_exact", "_exact_v_norm", "_sum_lf_k_norm")


def state_from_fields(src, device, dtype: torch.dtype = None) -> CoDAGQALandmarkStatePerf2:
    """New arena-backed state on ``device`` holding a copy of ``src``'s fields."""
    dtype = src.k_buf.dtype if dtype is None else dtype
    B, Hkv, Lbuf, Dh = src.k_buf.shape
    W = src.g_recent.shape[1]
    Me = src.mem_last_exact.shape[1]
    Ms = Lbuf - W - Me
    st = allocate_state(B, Hkv, Dh, W, Me, Ms, torch.device(device), dtype)
    for name in _TENSORS:
        s, d = getattr(src, name, None), getattr(st, name)
        if s is not None and d is not None:
            d.copy_(s.to(device=d.device, dtype=d.dtype))
    st.recent_idx, st.recent_filled, st.pos = int(src.recent_idx), int(src.recent_filled), int(src.pos)
    st.active_exact, st.active_summary = int(src.active_exact), int(src.active_summary)
    st.metrics = dict(src.metrics) if getattr(src, "metrics", None) is not None else None
    return st


def _rebuild(state, fn) -> CoDAGQALandmarkStatePerf2:
    opt = lambda t: None if t is None else fn(t)  # noqa: E731
    return CoDAGQALandmarkStatePerf2(
        k_buf=fn(state.k_buf), v_buf=fn(state.v_buf), allowed=fn(state.allowed), g_recent=fn(state.g_recent),
        recent_idx=state.recent_idx, recent_filled=state.recent_filled, mem_last_exact=fn(state.mem_last_exact),
        pos=state.pos, active_exact=state.active_exact, active_summary=state.active_summary,
        _exact_v_norm=opt(state._exact_v_norm), _sum_lf_k_norm=opt(state._sum_lf_k_norm),
        metrics=dict(state.metrics) if state.metrics is not None else None)


def _state_to_cpu(state) -> CoDAGQALandmarkStatePerf2:
    """CPU copy of every tensor field, for ``torch.save`` (upstream neural_db.py:30-46)."""
    return _rebuild(state, lambda t: t.detach().to("cpu", copy=True))


def _deep_copy_state(state) -> CoDAGQALandmarkStatePerf2:
    """Independent clone on the same device (upstream neural_db.py:66-82)."""
    if state.k_buf.is_cuda:
        return state_from_fields(state, state.k_buf.device)
    return _rebuild(state, lambda t: t.clone())


def _state_to_device(state, device, dtype: torch.dtype) -> None:
    """Move a state's tensors in place (upstream neural_db.py:49-63); K/V take ``dtype``, gates and
    the two routing caches become float32 as upstream does (the compute methods narrow the caches
    back to the K/V dtype on first use, which is lossless for values that came from that dtype)."""
    state.k_buf = state.k_buf.to(device=device, dtype=dtype)
    state.v_buf = state.v_buf.to(device=device, dtype=dtype)
    state.allowed = state.allowed.to(device=device)
    state.g_recent = state.g_recent.to(device=device, dtype=torch.float32)
    state.mem_last_exact = state.mem_last_exact.to(device=device)
    if state._exact_v_norm is not None:
        state._exact_v_norm = state._exact_v_norm.to(device=device, dtype=torch.float32)
    if state._sum_lf_k_norm is not None:
        state._sum_lf_k_norm = state._sum_lf_k_norm.to(device=device, dtype=torch.float32)
    if hasattr(state, "_arena"):
        state._arena = None
