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


# ---------------------------------------------------------------------------------------------------------
# Wire format: one blob per layer state = fixed header + the arena bytes as they lie in HBM.
#
# Upstream persists states by pickling the dataclass tensor by tensor (neural_db.py:286-308,
# demo/library.py:28-56).  The arena is already one contiguous allocation, so a state can be shipped with a
# single device->host copy and restored with a single host->device copy, no per-tensor work and no pickle.
#
#   offset  size  field
#   0       8     magic  b"CODAB2S\0"
#   8       4     version (1)
#   12      4     dtype code (0 = float32, 1 = bfloat16)
#   16      24    B, Hkv, Dh, W, Me, Ms            (6 x int32)
#   40      24    pos (int64), recent_idx, recent_filled, active_exact, active_summary (4 x int32)
#   64      8     arena bytes (uint64)
#   72      56    reserved (zero)
#   128     ...   arena (layout: state.arena_layout)
#
# All integers little-endian.  The blob round-trips to and from upstream's dataclass through
# ``state_from_fields`` / the dataclass fields of the restored state.
WIRE_MAGIC = b"CODAB2S\x00"
WIRE_VERSION = 1
WIRE_HEADER_BYTES = 128
_WIRE_DTYPES = {torch.float32: 0, torch.bfloat16: 1}


def state_to_bytes(state: CoDAGQALandmarkStatePerf2) -> bytes:
    """Serialise an arena-backed state (any device) into one blob; states without an arena (CPU copies,
    upstream objects) are packed into one first."""
    import struct
    if getattr(state, "_arena", None) is None:
        if not torch.cuda.is_available():
            raise RuntimeError("state_to_bytes: the state has no arena and no CUDA device is available to pack it")
        state = state_from_fields(state, "cuda")
    dt = state.k_buf.dtype
    if dt not in _WIRE_DTYPES:
        raise ValueError(f"state_to_bytes: unsupported dtype {dt}")
    B, Hkv, Lbuf, Dh = state.k_buf.shape
    W, Me = state.g_recent.shape[1], state.mem_last_exact.shape[1]
    Ms = Lbuf - W - Me
    arena = state._arena.detach().to("cpu").contiguous()
    head = struct.pack("<8sII6iq4iQ", WIRE_MAGIC, WIRE_VERSION, _WIRE_DTYPES[dt], B, Hkv, Dh, W, Me, Ms,
                       int(state.pos), int(state.recent_idx), int(state.recent_filled),
                       int(state.active_exact), int(state.active_summary), arena.numel())
    return head.ljust(WIRE_HEADER_BYTES, b"\x00") + arena.numpy().tobytes()


def state_from_bytes(blob: bytes, device) -> CoDAGQALandmarkStatePerf2:
    """Restore a state from ``state_to_bytes`` output onto ``device`` (one host->device copy)."""
    import struct
    from .state import arena_layout
    if len(blob) < WIRE_HEADER_BYTES or blob[:8] != WIRE_MAGIC:
        raise ValueError("state_from_bytes: not a coda-b200 state blob")
    (_, version, dcode, B, Hkv, Dh, W, Me, Ms, pos, ridx, rfill, ae, asum, nbytes) = struct.unpack(
        "<8sII6iq4iQ", blob[:struct.calcsize("<8sII6iq4iQ")])
    if version != WIRE_VERSION:
        raise ValueError(f"state_from_bytes: version {version} not supported (this build reads {WIRE_VERSION})")
    dtype = {v: k for k, v in _WIRE_DTYPES.items()}.get(dcode)
    if dtype is None:
        raise ValueError(f"state_from_bytes: unknown dtype code {dcode}")
    esize = torch.tensor([], dtype=dtype).element_size()
    _, total = arena_layout(B, Hkv, Dh, W, Me, Ms, esize)
    if nbytes != total or len(blob) != WIRE_HEADER_BYTES + nbytes:
        raise ValueError("state_from_bytes: arena size does not match the header's dimensions")
    st = allocate_state(B, Hkv, Dh, W, Me, Ms, torch.device(device), dtype)
    host = torch.frombuffer(bytearray(blob[WIRE_HEADER_BYTES:]), dtype=torch.uint8)
    st._arena.copy_(host)
    st.pos, st.recent_idx, st.recent_filled = int(pos), int(ridx), int(rfill)
    st.active_exact, st.active_summary = int(ae), int(asum)
    return st
