"""Bounded-cache differential attention on B200.

``CoDAGQALandmarkPerf2`` keeps the constructor, parameter names and the methods
``init_state / prefill_chunked / step / attend_step / cache_bytes / reset_metrics`` of upstream
``src/coda_gqa_l/attention.py:72-760``; the state object keeps the upstream field names.  The
projections are PyTorch GEMMs; everything between them (RoPE, noise-query rotation, gate and
lambda sigmoids, the two-stream attention with its subtraction/RMSNorm epilogue, candidate
selection, bank routing, ring maintenance) runs in the sm_100a kernels of libcoda_b200.so, reached
through the C ABI of include/coda_b200.h.  There is no other compute path: tensors must be CUDA
tensors in float32 or bfloat16, and the module must be in eval mode.
"""
from __future__ import annotations

import ctypes as C
import math
from typing import Dict, Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import _lib
from ._lib import LayerCfg, RingPos, StatePtrs, check, lib
from .primitives import HeadwiseRMSNorm, RotaryEmbedding
from .state import CoDAGQALandmarkStatePerf2, allocate_state

__all__ = ["CoDAGQALandmarkPerf2", "CoDAGQALandmarkStatePerf2"]

_DT = {torch.float32: _lib.CODA_F32, torch.bfloat16: _lib.CODA_BF16}
_GEMM_WS: Dict[torch.device, torch.Tensor] = {}      # split-K workspace of the projection GEMM, one per device


METRIC_KEYS = ("exact_hits", "exact_inserts", "exact_overwrites", "exact_fill_ratio", "summary_updates",
               "summary_inserts", "summary_fill_ratio", "tokens_gated_out", "total_evictions", "exact_frustrated",
               "summary_frustrated", "active_exact", "active_summary", "expansions_exact", "expansions_summary")


def new_metrics(active_exact: int, active_summary: int) -> Dict[str, object]:
    """The counters a state carries when ``collect_metrics`` is on (upstream attention.py:319-336)."""
    m: Dict[str, object] = {k: 0 for k in METRIC_KEYS}
    m["exact_fill_ratio"] = 0.0
    m["summary_fill_ratio"] = 0.0
    m["active_exact"], m["active_summary"] = int(active_exact), int(active_summary)
    return m


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream(device: Optional[torch.device] = None) -> int:
    """Handle of the current CUDA stream (of ``device``, default the current device)."""
    if _raw_stream is not None:
        idx = device.index if device is not None and device.index is not None else torch.cuda.current_device()
        return _raw_stream(idx)
    return torch.cuda.current_stream(device).cuda_stream


_SIDE_STREAMS: dict = {}


def _side_stream_for(device: torch.device) -> "torch.cuda.Stream":
    """One extra stream per device for work that runs beside the current stream (kept for the process)."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    st = _SIDE_STREAMS.get(idx)
    if st is None:
        st = _SIDE_STREAMS[idx] = torch.cuda.Stream(device=idx)
    return st


def _p(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


class CoDAGQALandmarkPerf2(nn.Module):
    """Differential attention (signal minus lambda-gated, theta-rotated noise stream) over a
    bounded per-layer state: a W-slot ring of recent tokens, an Me-slot exact landmark bank with
    LRU replacement and an Ms-slot summary bank of EMA prototypes."""

    def __init__(
        self,
        *,
        embed_dim: int,
        num_heads: int,
        num_kv_heads: int,
        window: int,
        num_landmarks_exact: int,
        num_landmarks_summary: int,
        rope_base: float = 10_000.0,
        lambda_init_bias: float = -6.0,
        theta_init: float = math.pi / 2,
        write_policy: str = "gated",
        write_gate_init_bias: float = -2.0,
        write_gate_threshold_exact: float = 0.10,
        write_gate_threshold_summary: float = 0.05,
        exact_match_threshold: float = 0.90,
        exact_novelty_threshold: float = 0.70,
        exact_refresh_on_hit: bool = False,
        exact_candidates_per_block: int = 8,
        summary_eta_init_logit: float = -3.0,
        summary_candidates_per_block: int = 64,
        summary_overwrite_on_insert: bool = True,
        min_landmarks_exact: Optional[int] = None,
        max_landmarks_exact: Optional[int] = None,
        min_landmarks_summary: Optional[int] = None,
        max_landmarks_summary: Optional[int] = None,
        expansion_t_max: int = 1_000_000,
        mem_init: str = "random_normal",
        mask_unused_memory: bool = True,
        detach_evicted: bool = True,
        eps: float = 1e-6,
        collect_metrics: bool = False,
        head_norm_mode: str = "full",
        rope_interleaved: bool = True,
    ):
        super().__init__()
        # validation messages as upstream attention.py:143-157,176-181,233
        if embed_dim % num_heads != 0:
            raise ValueError("embed_dim must be divisible by num_heads")
        if num_heads % num_kv_heads != 0:
            raise ValueError("num_heads must be divisible by num_kv_heads")
        if window <= 0:
            raise ValueError("window must be positive")
        if num_landmarks_exact < 0 or num_landmarks_summary < 0:
            raise ValueError("num_landmarks_* must be non-negative")
        self.embed_dim = int(embed_dim)
        self.num_heads = int(num_heads)
        self.num_kv_heads = int(num_kv_heads)
        self.head_dim = self.embed_dim // self.num_heads
        if self.head_dim % 2 != 0:
            raise ValueError("head_dim must be even (RoPE requirement)")
        self.lf_start = self.head_dim // 2
        self.lf_dim = self.head_dim - self.lf_start
        self.energy_scale = math.sqrt(self.head_dim / self.lf_dim)
        self.window = int(window)

        me, ms = int(num_landmarks_exact), int(num_landmarks_summary)
        self.Me_min = int(min_landmarks_exact) if min_landmarks_exact is not None else me
        self.Me_max = int(max_landmarks_exact) if max_landmarks_exact is not None else me
        self.Ms_min = int(min_landmarks_summary) if min_landmarks_summary is not None else ms
        self.Ms_max = int(max_landmarks_summary) if max_landmarks_summary is not None else ms
        self.expansion_t_max = int(expansion_t_max)
        if self.Me_min > self.Me_max:
            raise ValueError(f"min_landmarks_exact ({self.Me_min}) > max ({self.Me_max})")
        if self.Ms_min > self.Ms_max:
            raise ValueError(f"min_landmarks_summary ({self.Ms_min}) > max ({self.Ms_max})")
        if self.Me_min < 0 or self.Ms_min < 0:
            raise ValueError("min_landmarks_* must be non-negative")
        self.Me, self.Ms = self.Me_max, self.Ms_max
        self.Lbuf = self.window + self.Me + self.Ms

        # Parameters are created in upstream's order (attention.py:189-234) so that the same
        # torch.manual_seed gives the same default weights.
        H, Hkv, Dh = self.num_heads, self.num_kv_heads, self.head_dim
        self.q_proj = nn.Linear(self.embed_dim, H * Dh, bias=False)
        self.k_proj = nn.Linear(self.embed_dim, Hkv * Dh, bias=False)
        self.v_proj = nn.Linear(self.embed_dim, Hkv * Dh, bias=False)
        self.theta = nn.Parameter(torch.full((H, Dh // 2), float(theta_init)))
        self.lambda_proj = nn.Linear(self.embed_dim, H, bias=True)
        nn.init.constant_(self.lambda_proj.bias, float(lambda_init_bias))
        self.write_policy = write_policy
        self.write_proj = nn.Linear(self.embed_dim, 1, bias=True)
        nn.init.zeros_(self.write_proj.weight)
        nn.init.constant_(self.write_proj.bias, float(write_gate_init_bias))
        self.write_gate_threshold_exact = float(write_gate_threshold_exact)
        self.write_gate_threshold_summary = float(write_gate_threshold_summary)
        self.exact_match_threshold = float(exact_match_threshold)
        self.exact_novelty_threshold = float(exact_novelty_threshold)
        self.exact_refresh_on_hit = bool(exact_refresh_on_hit)
        self.exact_candidates_per_block = int(max(0, exact_candidates_per_block))
        self.summary_eta_logit = nn.Parameter(torch.full((Hkv,), float(summary_eta_init_logit)))
        self.summary_candidates_per_block = int(max(0, summary_candidates_per_block))
        self.summary_overwrite_on_insert = bool(summary_overwrite_on_insert)
        self.mem_init = mem_init
        self.mask_unused_memory = bool(mask_unused_memory)
        self.detach_evicted = bool(detach_evicted)
        self.collect_metrics = bool(collect_metrics)
        self.rope_interleaved = bool(rope_interleaved)
        self.rope_base = float(rope_base)
        self.rope = RotaryEmbedding(Dh, base=float(rope_base))
        self.head_norm_mode = head_norm_mode
        if head_norm_mode == "full":
            self.head_norm = HeadwiseRMSNorm(Dh, eps=eps)
        elif head_norm_mode == "identity":
            self.head_norm = nn.Identity()
        else:
            raise ValueError(f"head_norm_mode must be 'full' or 'identity', got {head_norm_mode!r}")
        self.eps = float(eps)
        self.o_proj = nn.Linear(H * Dh, self.embed_dim, bias=False)

        self._cfg_cache: Dict[tuple, LayerCfg] = {}
        self._const_cache: Dict[tuple, tuple] = {}
        self._scratch: Dict[tuple, torch.Tensor] = {}
        self._fused = None
        self._fused_ptrs = []
        self._wt = None
        # When set to a list, every attention launch appends (Lq, start_event, end_event) to it.
        self.kernel_timers = None
        self._qrec = None
        # False forces the shape-generic kernels even where a tuned one exists (used by tests).
        self.use_tuned_kernels = True
        # Output projection of a decode step through this library's own skinny GEMM (coda_b200_skinny_gemm: weight rows
        # through a TMA ring, a CTA pair per 64 rows splitting K, residual in the epilogue) instead of the vendor GEMM
        # + add.  On by default where the shape is supported: in the captured step of the 7B shape the two are at
        # parity (1.290 against 1.287 ms per step, three runs each), and on the eager path it is one host call fewer.
        self.use_skinny_gemm_kernel = True
        # The fused INPUT projection on the same kernel family (coda_b200_skinny_gemm_bias).  The eager fast path uses
        # it whenever use_skinny_gemm_kernel is on (one host call instead of a tensor-library call: 1.47 against
        # 1.67 ms per 32-layer step); inside the captured step the vendor GEMM is 0.9 % faster at the 7B shape (1.205
        # against 1.216 ms per step, three runs each), so the general path takes the own kernel only when this is set.
        self.use_skinny_in_proj = False
        # The decode step's two projections (at most 64 rows, bfloat16) on this library's tcgen05 GEMM
        # (coda_b200_proj_gemm: weight rows as the MMA's M, K split over the SMs with a counter-based fix-up, bias /
        # residual in the epilogue, programmatic dependent launch) instead of the vendor GEMM (+ add).  Off by default:
        # its weight stream runs at HBM speed, but the split-K fix-up is a chain of global round trips, and at the 7B
        # shape it measures 14.8 / 13.4 us (input / output projection) against 11.8 / 10.3 us for the vendor kernels.
        self.use_own_gemm = False
        self._gemm_ok: Dict[tuple, bool] = {}
        # Second half of a split decode step (after route_launch / the stack's batched routing) as one launch:
        # the attention kernel writes the new token itself (coda_b200_decode_attend_append).
        self.fuse_append_into_attention = True
        # chunked prefill: scores and decisions of a block's routing on a second stream beside the block's attention.
        # Same results; measured slower at the 7B shape (2.27 against 2.15 ms per layer and 512-token chunk: a scoring
        # CTA and an attention CTA do not fit one SM together, so the scoring kernel takes whole SMs from the attention
        # for as long as its latency chains last), hence off.
        self.overlap_block_routing = False
        # Route the attention / cache-write / routing launches through the torch custom ops (torch.ops.coda_b200.*,
        # see torch_ops.py) instead of the ctypes binding.  Same entry points underneath, so the same bits; states
        # that report routing events (metrics, growing banks) and the fused decode-step launches stay on ctypes.
        self.use_torch_ops = False
        self._status = None

    # ------------------------------------------------------------------ state
    def init_state(self, *, batch_size: int, device, dtype: torch.dtype,
                   mem_init: Optional[str] = None) -> CoDAGQALandmarkStatePerf2:
        """Fresh state in one arena allocation (upstream attention.py:247-338).

        The bank slots are filled with N(0, 0.02^2) in upstream's order (exact K, exact V, summary
        K low-frequency band, summary V) from the generator of ``device``; a CPU device may be
        given to stage a state (e.g. to reproduce a CPU-seeded initial state) and moved with
        :func:`state_to`, but the compute methods only accept CUDA states."""
        if dtype not in _DT:
            raise RuntimeError(f"unsupported dtype {dtype}: the CUDA kernels handle float32 and bfloat16")
        B, W, Me, Ms = int(batch_size), self.window, self.Me, self.Ms
        st = allocate_state(B, self.num_kv_heads, self.head_dim, W, Me, Ms, torch.device(device), dtype)
        mode = self.mem_init if mem_init is None else mem_init
        if mode == "random_normal":
            if Me > 0:
                st.k_buf[:, :, W:W + Me, :].normal_(mean=0.0, std=0.02)
                st.v_buf[:, :, W:W + Me, :].normal_(mean=0.0, std=0.02)
            if Ms > 0:
                st.k_buf[:, :, W + Me:, self.lf_start:].normal_(mean=0.0, std=0.02)
                st.v_buf[:, :, W + Me:, :].normal_(mean=0.0, std=0.02)
        elif mode != "zeros":
            raise ValueError("mem_init must be 'zeros' or 'random_normal'")
        st.active_exact = self.Me_min if Me > 0 else 0
        st.active_summary = self.Ms_min if Ms > 0 else 0
        if Me > 0:
            st._exact_v_norm.copy_(F.normalize(st.v_buf[:, :, W:W + Me, :], dim=-1, eps=1e-6))
        if Ms > 0:
            st._sum_lf_k_norm.copy_(F.normalize(st.k_buf[:, :, W + Me:, self.lf_start:], dim=-1, eps=1e-6))
        if self.collect_metrics:
            st.metrics = new_metrics(st.active_exact, st.active_summary)
        return st

    # ------------------------------------------------------------------ plumbing
    def _require_ready(self, x: torch.Tensor, st: CoDAGQALandmarkStatePerf2) -> None:
        if self.training:
            raise RuntimeError("CoDAGQALandmarkPerf2 (B200) is inference-only: call .eval() first")
        if not self.detach_evicted:
            raise NotImplementedError("detach_evicted=False (autograd through bank updates) is not supported")
        if not x.is_cuda:
            raise RuntimeError("input must be a CUDA tensor: this implementation has no CPU path")
        if x.dtype not in _DT:
            raise RuntimeError(f"unsupported dtype {x.dtype}")
        if st.k_buf.device != x.device or st.k_buf.dtype != x.dtype:
            raise RuntimeError("state and input must share device and dtype")
        if st.k_buf.shape != (x.shape[0], self.num_kv_heads, self.Lbuf, self.head_dim):
            raise RuntimeError(f"state k_buf shape {tuple(st.k_buf.shape)} does not match this layer / batch")
        # A field that has to be replaced (non-contiguous view, a routing cache widened to fp32 by a serialisation
        # helper) no longer lives in the state's arena: the arena is dropped so that nothing snapshots or ships stale
        # bytes (capture_step then asks for an arena-backed state, state_to_bytes re-packs).
        detached = False
        for name in ("k_buf", "v_buf", "allowed", "g_recent", "mem_last_exact"):
            t = getattr(st, name)
            if not t.is_contiguous():
                setattr(st, name, t.contiguous())
                detached = True
        if st._exact_v_norm is not None and (st._exact_v_norm.dtype != x.dtype or not st._exact_v_norm.is_contiguous()):
            st._exact_v_norm = st._exact_v_norm.to(x.dtype).contiguous()
            detached = True
        if st._sum_lf_k_norm is not None and (st._sum_lf_k_norm.dtype != x.dtype or not st._sum_lf_k_norm.is_contiguous()):
            st._sum_lf_k_norm = st._sum_lf_k_norm.to(x.dtype).contiguous()
            detached = True
        if st.g_recent.dtype != torch.float32:
            st.g_recent = st.g_recent.float()
            detached = True
        if detached and getattr(st, "_arena", None) is not None:
            st._arena = None

    # ------------------------------------------------------------------ metrics / bank expansion
    @property
    def expandable(self) -> bool:
        """True when the banks start below their full size and grow under pressure."""
        return self.Me_min != self.Me_max or self.Ms_min != self.Ms_max

    def _tracked(self, st: CoDAGQALandmarkStatePerf2) -> bool:
        """Does a cache write on ``st`` have to report its routing events to the host?  (Counters and the
        growth decision are host scalars, so such a write ends with one small device-to-host read.)"""
        return self.expandable or st.metrics is not None

    def _arm_events(self, st: CoDAGQALandmarkStatePerf2) -> None:
        """Give ``st`` the int32 [B, 16] event record the cache-write kernels fill (or take it away)."""
        if not self._tracked(st):
            st._events = None
        elif st._events is None or st._events.device != st.k_buf.device or st._events.shape[0] != st.k_buf.shape[0]:
            st._events = torch.zeros((st.k_buf.shape[0], _lib.CODA_EVENT_WORDS), device=st.k_buf.device,
                                     dtype=torch.int32)

    def _log_ceiling(self, tokens_seen: int) -> Tuple[int, int]:
        """Largest active bank sizes allowed after ``tokens_seen`` tokens (upstream attention.py:344-356)."""
        if self.expansion_t_max <= 0:
            return self.Me_max, self.Ms_max
        ratio = min(math.log(1 + tokens_seen) / math.log(1 + self.expansion_t_max), 1.0)
        return (self.Me_min + int((self.Me_max - self.Me_min) * ratio),
                self.Ms_min + int((self.Ms_max - self.Ms_min) * ratio))

    def _try_expand(self, st: CoDAGQALandmarkStatePerf2, frustrated_exact: int, frustrated_summary: int) -> None:
        """Grow the active capacities under pressure, up to the logarithmic ceiling (upstream
        attention.py:358-390).  ``st.pos`` must still be the position before the write."""
        if not self.expandable or (frustrated_exact <= 0 and frustrated_summary <= 0):
            return
        ceil_e, ceil_s = self._log_ceiling(int(st.pos))
        grow_e = grow_s = 0
        if frustrated_exact > 0 and st.active_exact < ceil_e:
            grow_e = min(int(frustrated_exact), ceil_e - st.active_exact)
            st.active_exact += grow_e
        if frustrated_summary > 0 and st.active_summary < ceil_s:
            grow_s = min(int(frustrated_summary), ceil_s - st.active_summary)
            st.active_summary += grow_s
        if st.metrics is not None:
            st.metrics["active_exact"], st.metrics["active_summary"] = st.active_exact, st.active_summary
            st.metrics["expansions_exact"] += grow_e
            st.metrics["expansions_summary"] += grow_s

    def _account(self, st: CoDAGQALandmarkStatePerf2, n_evicted: int, block: bool) -> None:
        """Host side of a cache write that evicted ``n_evicted`` ring tokens per state: read the event record
        the kernel left, update the counters and grow the banks, in upstream's order (single token:
        memory_banks.py:315-337 and :416-432; block: :758-774 and :934-950).  Call before ``st.pos`` advances.

        Event words per state: [0] exact candidates gated out, [1] hits, [2] inserts, [3] overwrites,
        [4] frustrated (single token: 0/1), [5] summary updates, [6] first fills, [7] every active summary slot
        in use afterwards, [8] a summary candidate came in."""
        if n_evicted <= 0 or not self._tracked(st):
            return
        W, Me, Ms = self.window, self.Me, self.Ms
        do_e = Me > 0 and (not block or self.exact_candidates_per_block > 0)
        do_s = Ms > 0 and (not block or self.summary_candidates_per_block > 0)
        m = st.metrics
        if m is not None:
            m["total_evictions"] += int(n_evicted)
        if not (do_e or do_s):
            return
        # everything the host needs in one small tensor, hence one synchronising read
        evf = st._events.to(torch.float64)
        zero = evf.new_zeros(1)
        fill_e = st.allowed[:, W:W + Me].any(dim=0).float().mean().double().view(1) if do_e else zero
        fill_s = st.allowed[:, W + Me:].any(dim=0).float().mean().double().view(1) if do_s else zero
        # (the kernels' status word rides along: this read synchronises anyway, so an expired device-side wait
        # surfaces here instead of going unnoticed)
        stat = self._status.to(torch.float64) if self._status is not None and self._status.device == evf.device else zero
        host = torch.cat([evf.sum(dim=0), evf[:, 7].min().view(1), fill_e, fill_s, stat]).tolist()
        if int(host[-1]) != 0:
            raise RuntimeError(f"a bounded device-side wait expired in one of the tuned kernels (code {int(host[-1])}): "
                               "results since the last check are not valid")
        ev = [int(t) for t in host[:_lib.CODA_EVENT_WORDS]]
        every, fill_e, fill_s = int(host[-4]) == 1, host[-3], host[-2]
        if do_e:
            if m is not None:
                if block:
                    m["exact_overwrites"] += ev[3]
                    m["exact_frustrated"] += ev[4]
                    m["exact_fill_ratio"] = fill_e
                    m["exact_inserts"] += ev[2]
                    m["exact_hits"] += ev[1]
                    if self.write_policy != "none":
                        m["tokens_gated_out"] += ev[0]
                else:
                    if self.write_policy != "none":
                        m["tokens_gated_out"] += ev[0]
                    m["exact_hits"] += ev[1]
                    m["exact_inserts"] += ev[2]
                    m["exact_overwrites"] += ev[3]
                    m["exact_fill_ratio"] = fill_e
            # single token: one step of growth per call however many rows are under pressure
            self._try_expand(st, ev[4] if block else int(ev[4] > 0), 0)
        if do_s:
            frustrated = int(every and ev[8] > 0)
            self._try_expand(st, 0, frustrated)
            if m is not None:
                m["summary_updates"] += ev[5]
                m["summary_frustrated"] += frustrated
                if self.summary_overwrite_on_insert:
                    m["summary_inserts"] += ev[6]
                m["summary_fill_ratio"] = fill_s

    def _cfg(self, B: int, dtype: torch.dtype, st: CoDAGQALandmarkStatePerf2) -> LayerCfg:
        adt = self.rope.inv_freq.dtype
        key = (B, dtype, adt, st.active_exact, st.active_summary)
        c = self._cfg_cache.get(key)
        if c is None:
            c = LayerCfg(
                B=B, H=self.num_heads, Hkv=self.num_kv_heads, Dh=self.head_dim, W=self.window, Me=self.Me, Ms=self.Ms,
                dtype=_DT[dtype], angle_dtype=_DT.get(adt, _lib.CODA_F32) if dtype != torch.float32 else _lib.CODA_F32,
                rope_interleaved=int(self.rope_interleaved), head_norm_full=int(self.head_norm_mode == "full"),
                mask_unused=int(self.mask_unused_memory), gated=int(self.write_policy != "none"),
                refresh_on_hit=int(self.exact_refresh_on_hit), overwrite_on_insert=int(self.summary_overwrite_on_insert),
                Te=self.exact_candidates_per_block, Ts=self.summary_candidates_per_block,
                active_exact=int(st.active_exact), active_summary=int(st.active_summary),
                tau_gate_exact=self.write_gate_threshold_exact, tau_gate_summary=self.write_gate_threshold_summary,
                tau_match=self.exact_match_threshold, tau_novel=self.exact_novelty_threshold,
                eps=self.eps, energy_scale=self.energy_scale)
            self._cfg_cache[key] = c
        return c

    @staticmethod
    def _ptrs(st: CoDAGQALandmarkStatePerf2) -> StatePtrs:
        return StatePtrs(st.k_buf.data_ptr(), st.v_buf.data_ptr(), st.allowed.data_ptr(), st.g_recent.data_ptr(),
                         st.mem_last_exact.data_ptr() if st.mem_last_exact.numel() else None,
                         _p(st._exact_v_norm), _p(st._sum_lf_k_norm), _p(getattr(st, "_events", None)))

    def _consts(self, device, dtype):
        """(inv_freq fp32, cos(theta), sin(theta) in dtype, eta logits fp32, head-norm weight) cached per parameter version."""
        nw = self.head_norm.weight if self.head_norm_mode == "full" else None
        key = (device, dtype, self.theta.data_ptr(), self.theta._version, self.summary_eta_logit.data_ptr(),
               self.summary_eta_logit._version, self.rope.inv_freq.data_ptr(), _p(nw), 0 if nw is None else nw._version)
        hit = self._const_cache.get("k")
        if hit is not None and hit[0] == key:
            return hit[1]
        th = self.theta.detach()
        vals = (self.rope.inv_freq.detach().to(device=device, dtype=torch.float32).contiguous(),
                torch.cos(th).to(device=device, dtype=dtype).contiguous(),
                torch.sin(th).to(device=device, dtype=dtype).contiguous(),
                self.summary_eta_logit.detach().to(device=device, dtype=torch.float32).contiguous(),
                None if nw is None else nw.detach().to(device=device, dtype=dtype).contiguous())
        self._const_cache["k"] = (key, vals)
        return vals

    def _fused_weight(self):
        """One [q | k | v | lambda | gate | pad] weight so that the five input projections are a single GEMM.

        The individual ``nn.Linear`` parameters are re-pointed at row ranges of the fused matrix (no second
        copy of the weights; ``state_dict`` / ``load_state_dict`` keep working).  Rebuilt whenever a
        parameter no longer aliases it (after ``.to()``, or when a projection was replaced)."""
        lins = (self.q_proj, self.k_proj, self.v_proj, self.lambda_proj, self.write_proj)
        if not all(type(l) is nn.Linear for l in lins):
            return None
        f = self._fused
        w0 = self.q_proj.weight
        if f is not None and f[0].device == w0.device and f[0].dtype == w0.dtype:
            # (addresses of the row ranges were noted when the matrix was built: no slicing on the decode path)
            ok = True
            for l, (wp, bp) in zip(lins, self._fused_ptrs):
                if l.weight.data_ptr() != wp or (l.bias is not None and l.bias.data_ptr() != bp):
                    ok = False
                    break
            if ok:
                return f
        n = sum(l.out_features for l in lins)
        npad = (n + 63) // 64 * 64       # the library's skinny-GEMM kernels lose 20 % on widths that are not a multiple of 32
        W = torch.zeros((npad, self.embed_dim), device=w0.device, dtype=w0.dtype)
        b = torch.zeros((npad,), device=w0.device, dtype=w0.dtype)
        off = 0
        for l in lins:
            W[off:off + l.out_features].copy_(l.weight.data)
            l.weight.data = W[off:off + l.out_features]
            if l.bias is not None:
                b[off:off + l.out_features].copy_(l.bias.data)
                l.bias.data = b[off:off + l.out_features]
            off += l.out_features
        self._fused = (W, b)
        self._fused_ptrs = [(l.weight.data_ptr(), None if l.bias is None else l.bias.data_ptr()) for l in lins]
        return self._fused

    # GEMMs with at most this many rows (decode) read transposed copies of the weights
    SKINNY_ROWS = 64

    def _skinny_weights(self):
        """Transposed, contiguous copies ([in][out]) of the fused input weight and of ``o_proj.weight`` for the
        decode GEMMs: with a handful of rows the library's kernels for that layout stream the weights
        noticeably faster (measured on B200: 12.4 vs 14.4 us for the fused input projection, 10.3 vs 11.5 us
        for o_proj, 32 rows).  Costs a second copy of the weights; rebuilt when a weight's version counter moves
        (``load_state_dict``, optimiser steps, ``.to()``); after writing through ``.data`` call
        :meth:`refresh_weights`."""
        f = self._fused_weight()
        if f is None or type(self.o_proj) is not nn.Linear or self.o_proj.bias is not None:
            return None
        lins = (self.q_proj, self.k_proj, self.v_proj, self.lambda_proj, self.write_proj)
        key = (f[0].data_ptr(), f[0]._version, f[1]._version, self.o_proj.weight.data_ptr(), self.o_proj.weight._version,
               tuple(l.weight._version for l in lins), tuple(-1 if l.bias is None else l.bias._version for l in lins))
        wt = self._wt
        if wt is None or wt[0] != key:
            wt = (key, f[0].t().contiguous(), self.o_proj.weight.detach().t().contiguous())
            self._wt = wt
        return wt

    def refresh_weights(self) -> None:
        """Drop the derived weight copies (call after modifying parameters in a way autograd's version counters
        do not see, e.g. through ``.data``)."""
        self._wt = None

    def _gemm_workspace(self, device, nbytes: int) -> torch.Tensor:
        """Split-K workspace of coda_b200_proj_gemm: one per device for every layer of the process (the calls of a
        decode step follow one another on one stream); its head (the tile counters) starts out zero and the kernel
        leaves it zero."""
        ws = _GEMM_WS.get(device)
        if ws is None or ws.numel() < nbytes:
            ws = torch.zeros(max(nbytes, 1 << 22), dtype=torch.uint8, device=device)
            _GEMM_WS[device] = ws
        return ws

    def _own_gemm(self, x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor],
                  residual: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
        """``x @ w.T (+ bias) (+ residual)`` for the few rows of a decode step on coda_b200_proj_gemm, or None where
        that kernel does not apply (more than 64 rows, not bfloat16, K not a multiple of 64, unaligned views)."""
        B, L, K = x.shape
        rows, N = B * L, w.shape[0]
        if not (self.use_own_gemm and rows <= 64 and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.is_cuda):
            return None
        ok = self._gemm_ok.get((rows, K, N))
        if ok is None:
            ok = bool(lib.coda_b200_proj_gemm_supported(rows, K, N))
            self._gemm_ok[(rows, K, N)] = ok
        if not ok or not w.is_contiguous() or w.data_ptr() % 16:
            return None
        ws = self._gemm_ok.get(("ws", rows, K, N))
        if ws is None:
            ws = int(lib.coda_b200_proj_gemm_workspace_bytes(rows, K, N))
            self._gemm_ok[("ws", rows, K, N)] = ws
        ws = self._gemm_workspace(x.device, ws)

        def rows_of(t):                      # (tensor, row stride) of t seen as [rows, features]
            if L == 1 and t.stride(2) == 1:
                return t, t.stride(0)
            t = t if t.is_contiguous() else t.contiguous()
            return t, t.shape[-1]
        x, x_rs = rows_of(x)
        if x.data_ptr() % 16 or x_rs % 8:
            x, x_rs = x.contiguous(), K
        res_rs = 0
        if residual is not None:
            residual, res_rs = rows_of(residual)
        y = torch.empty((B, L, N), device=x.device, dtype=x.dtype)
        check(lib.coda_b200_proj_gemm(x.data_ptr(), x_rs, rows, K, w.data_ptr(), N, _p(bias), _p(residual), res_rs,
                                      y.data_ptr(), N, ws.data_ptr(), self._status_word(x.device).data_ptr(), _stream()),
              "coda_b200_proj_gemm")
        return y

    def _skinny_in(self, x: torch.Tensor, f, rows: int) -> Optional[torch.Tensor]:
        """The fused input projection of a decode step on this library's own skinny GEMM (bias in its epilogue), where
        the switch is on and the kernel covers the shape; None otherwise."""
        if not (self.use_skinny_gemm_kernel and self.use_skinny_in_proj and x.is_cuda and x.dtype == torch.bfloat16 and rows <= 32):
            return None
        W, bias = f
        K, N = W.shape[1], W.shape[0]
        ok = self._gemm_ok.get(("skinny_in", rows, K, N))
        if ok is None:
            ok = self._gemm_ok[("skinny_in", rows, K, N)] = bool(
                W.dtype == torch.bfloat16 and W.is_contiguous() and W.data_ptr() % 16 == 0 and bias.data_ptr() % 16 == 0
                and lib.coda_b200_skinny_gemm_bias_supported(rows, K, N))
        x2 = x.reshape(rows, K)
        if not ok or not x2.is_contiguous() or x2.data_ptr() % 16:
            return None
        y = torch.empty((x.shape[0], x.shape[1], N), device=x.device, dtype=x.dtype)
        check(lib.coda_b200_skinny_gemm_bias(x2.data_ptr(), rows, K, W.data_ptr(), N, bias.data_ptr(), None, 0, y.data_ptr(), N,
                                             self._status_word(x.device).data_ptr(), _stream(x.device)),
              "coda_b200_skinny_gemm_bias")
        return y

    def _decode_bundle(self, device, dtype):
        """Everything an eager decode step needs besides the state, gathered once and re-validated cheaply: the fused
        and transposed weights, the constant tables and their raw addresses.  ``step()`` is called once per layer per
        token by adapter-driven loops, where the host time of walking ``nn.Module`` attributes and rebuilding cache
        keys (~60 us per call) outweighs the kernels; the bundle is checked by module identity plus address and
        version counter of every parameter it was built from.  None where the fused layout does not apply."""
        c = self.__dict__.get("_bundle")
        mods = self._modules
        if c is not None and c["dev"] == device and c["dt"] == dtype:
            ok = all(mods[n] is m for n, m in c["mods"])
            if ok:
                for prm, ver, ptr in c["stamps"]:
                    if prm._version != ver or prm.data_ptr() != ptr:
                        ok = False
                        break
            if ok:
                return c
        f = self._fused_weight()
        wt = self._skinny_weights()
        if f is None or wt is None or f[0].device != device or f[0].dtype != dtype:
            self.__dict__["_bundle"] = None
            return None
        inv_freq, cos_t, sin_t, eta, nw = self._consts(device, dtype)
        names = ("q_proj", "k_proj", "v_proj", "lambda_proj", "write_proj", "o_proj", "head_norm", "rope")
        prms = [p for n in names[:6] for p in mods[n].parameters()] + [self.theta, self.summary_eta_logit, self.rope.inv_freq]
        if nw is not None:
            prms.append(self.head_norm.weight)
        H, Hkv, Dh = self.num_heads, self.num_kv_heads, self.head_dim
        es = f[0].element_size()
        c = dict(dev=device, dt=dtype, mods=[(n, mods[n]) for n in names], stamps=[(p, p._version, p.data_ptr()) for p in prms],
                 bias=f[1], w_in_t=wt[1], w_out_t=wt[2], npad=f[0].shape[0], nq=H * Dh, nkv=Hkv * Dh,
                 off_k=H * Dh * es, off_v=(H * Dh + Hkv * Dh) * es, off_lam=(H * Dh + 2 * Hkv * Dh) * es,
                 off_gate=(H * Dh + 2 * Hkv * Dh + H) * es, gated=self.write_policy != "none",
                 inv_freq=inv_freq.data_ptr(), cos=cos_t.data_ptr(), sin=sin_t.data_ptr(), eta=eta.data_ptr(), nw=_p(nw),
                 w_out=self.o_proj.weight.data_ptr(), n_out=self.o_proj.weight.shape[0], skinny_ok={},
                 w_in=f[0].data_ptr(), bias_ptr=f[1].data_ptr(), skinny_in_ok={},
                 keep=(inv_freq, cos_t, sin_t, eta, nw, f, wt))
        self.__dict__["_bundle"] = c
        return c

    def _step_eager_fast(self, x: torch.Tensor, st: CoDAGQALandmarkStatePerf2,
                         residual: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
        """The default decode step (write, then attend) with as little host work as the launches allow; same kernels
        and the same bits as the general path.  Returns None where it does not apply (the caller then takes the
        general path).  ``residual``: added to the result inside the output projection's GEMM call."""
        if self.use_torch_ops or self.use_own_gemm or self.kernel_timers is not None:
            return None
        if st.metrics is not None or self.Me_min != self.Me_max or self.Ms_min != self.Ms_max or not self.detach_evicted:
            return None
        B = x.shape[0]
        if B > self.SKINNY_ROWS or x.dtype != torch.bfloat16:
            return None
        dev = x.device
        bd = self._decode_bundle(dev, x.dtype)
        if bd is None:
            return None
        cfg = self._cfg(B, x.dtype, st)
        if not (self._tuned_decode(cfg) and self._fused_write_ok(cfg)):
            return None
        pc = st.__dict__.get("_pc")
        kptr = st.k_buf.data_ptr()
        if pc is None or pc[0] != kptr or pc[2] is not st._exact_v_norm or pc[3] is not st._sum_lf_k_norm:
            if not (st.k_buf.shape == (B, self.num_kv_heads, self.Lbuf, self.head_dim) and st.v_buf.shape == st.k_buf.shape
                    and st.k_buf.is_contiguous() and st.v_buf.is_contiguous() and st.allowed.is_contiguous()
                    and st.g_recent.dtype == torch.float32 and st.g_recent.is_contiguous() and st.mem_last_exact.is_contiguous()
                    and st.k_buf.dtype == x.dtype and st.k_buf.device == dev
                    and (st._exact_v_norm is None or (st._exact_v_norm.dtype == x.dtype and st._exact_v_norm.is_contiguous()))
                    and (st._sum_lf_k_norm is None or (st._sum_lf_k_norm.dtype == x.dtype and st._sum_lf_k_norm.is_contiguous()))):
                return None
            st._events = None
            pc = (kptr, self._ptrs(st), st._exact_v_norm, st._sum_lf_k_norm)
            st.__dict__["_pc"] = pc
        ptrs = pc[1]
        y = None
        if self.use_skinny_gemm_kernel:
            ok = bd["skinny_in_ok"].get(B)
            if ok is None:
                f = bd["keep"][5]
                ok = bd["skinny_in_ok"][B] = bool(f[0].is_contiguous() and f[0].data_ptr() % 16 == 0 and f[1].data_ptr() % 16 == 0
                                                  and lib.coda_b200_skinny_gemm_bias_supported(B, f[0].shape[1], f[0].shape[0]))
            x2 = x.reshape(B, -1)
            if ok and x2.is_contiguous() and x2.data_ptr() % 16 == 0:
                y = torch.empty((B, bd["npad"]), device=dev, dtype=x.dtype)
                rc = lib.coda_b200_skinny_gemm_bias(x2.data_ptr(), B, x2.shape[1], bd["w_in"], bd["npad"], bd["bias_ptr"], None, 0,
                                                    y.data_ptr(), bd["npad"], self._status_word(dev).data_ptr(), _stream(dev))
                if rc:
                    check(rc, "coda_b200_skinny_gemm_bias")
        if y is None:
            y = torch.addmm(bd["bias"], x.reshape(B, -1), bd["w_in_t"])
        base, npad = y.data_ptr(), bd["npad"]
        if base % 16:
            return None
        s = _stream(dev)
        rp = RingPos(st.pos, st.recent_idx, st.recent_filled, None)
        qrec = self._decode_records(cfg, dev)
        out = torch.empty((B, self.num_heads * self.head_dim), device=dev, dtype=x.dtype)
        status = self._status_word(dev).data_ptr()
        gate = base + bd["off_gate"] if bd["gated"] else None
        rc = lib.coda_b200_step_write_attend(
            C.byref(cfg), C.byref(ptrs), rp, base + bd["off_k"], npad, base + bd["off_v"], npad, gate, npad if gate else 0,
            bd["inv_freq"], bd["eta"], base, npad, base + bd["off_lam"], npad, bd["cos"], bd["sin"], qrec.data_ptr(),
            bd["nw"], out.data_ptr(), out.shape[1], status, s)
        if rc:
            check(rc, "coda_b200_step_write_attend")
        self.advance_host_scalars(st)
        if self.use_skinny_gemm_kernel:
            ok = bd["skinny_ok"].get(B)
            if ok is None:
                w = self.o_proj.weight
                ok = bd["skinny_ok"][B] = bool(w.is_contiguous() and w.data_ptr() % 16 == 0 and w.dtype == torch.bfloat16
                                               and lib.coda_b200_skinny_gemm_supported(B, out.shape[1], w.shape[0]))
            r2 = residual.reshape(B, -1) if residual is not None else None
            if ok and (r2 is None or (r2.is_contiguous() and r2.data_ptr() % 16 == 0)):
                N = bd["n_out"]
                y = torch.empty((B, 1, N), device=dev, dtype=x.dtype)
                rc = lib.coda_b200_skinny_gemm(out.data_ptr(), B, out.shape[1], bd["w_out"], N, _p(r2), N, y.data_ptr(), N,
                                               status, s)
                if rc:
                    check(rc, "coda_b200_skinny_gemm")
                return y
        if residual is not None:
            # an eager step is bound by the host: one call for GEMM + residual beats the faster GEMM plus a separate add
            return torch.addmm(residual.reshape(B, -1), out, bd["w_out_t"]).view(B, 1, -1)
        return torch.mm(out, bd["w_out_t"]).view(B, 1, -1)

    def _project(self, x: torch.Tensor, need_kv: bool):
        """q, k, v, lambda logits, gate logits as (B, L, features) tensors (upstream attention.py:396-410,508)."""
        f = self._fused_weight() if need_kv else None
        if f is not None:
            H, Hkv, Dh = self.num_heads, self.num_kv_heads, self.head_dim
            rows = x.shape[0] * x.shape[1]
            y = self._own_gemm(x, f[0], f[1], None)
            if y is None:
                y = self._skinny_in(x, f, rows)
            wt = self._skinny_weights() if y is None and rows <= self.SKINNY_ROWS else None
            if y is not None:
                pass
            elif wt is not None:
                y = torch.addmm(f[1], x.reshape(rows, -1), wt[1]).view(x.shape[0], x.shape[1], -1)
            else:
                y = F.linear(x, f[0], f[1])
            return self._split_fused(y)
        q = self.q_proj(x)
        k = self.k_proj(x) if need_kv else None
        v = self.v_proj(x) if need_kv else None
        lam = self.lambda_proj(x)
        gate = self.write_proj(x) if (need_kv and self.write_policy != "none") else None
        return q, k, v, lam, gate

    def _split_fused(self, y: torch.Tensor):
        """The five views (q, k, v, lambda logits, gate logits) of a fused projection output (B, L, [q|k|v|lambda|gate|pad])."""
        H, Hkv, Dh = self.num_heads, self.num_kv_heads, self.head_dim
        nq, nkv = H * Dh, Hkv * Dh
        gate = y[..., nq + 2 * nkv + H:nq + 2 * nkv + H + 1] if self.write_policy != "none" else None
        return (y[..., :nq], y[..., nq:nq + nkv], y[..., nq + nkv:nq + 2 * nkv],
                y[..., nq + 2 * nkv:nq + 2 * nkv + H], gate)

    def _prep(self, cfg, L, pos, q, k, lam_logit, gate_logit, want_gate: bool, step_dev=None):
        B = q.shape[0]
        dev, dt = q.device, q.dtype
        inv_freq, cos_t, sin_t, _, _ = self._consts(dev, dt)
        qn = torch.empty((B, L, self.num_heads * self.head_dim), device=dev, dtype=dt)
        lam = torch.empty((B, L, self.num_heads), device=dev, dtype=torch.float32)
        g = torch.empty((B, L), device=dev, dtype=torch.float32) if want_gate else None
        if self.use_torch_ops and step_dev is None:
            from . import torch_ops
            ci, cf = torch_ops.cfg_lists(cfg)
            torch_ops.load().prep(q, k, qn, lam_logit, lam, gate_logit if want_gate else None, g, inv_freq, cos_t, sin_t,
                                  int(pos), ci, cf)
            return qn, lam, g
        rp = RingPos(int(pos), 0, 0, step_dev)
        check(lib.coda_b200_prep(
            C.byref(cfg), L, rp,
            q.data_ptr(), q.stride(0), q.stride(1),
            _p(k), 0 if k is None else k.stride(0), 0 if k is None else k.stride(1),
            qn.data_ptr(),
            lam_logit.data_ptr(), lam_logit.stride(0), lam_logit.stride(1), lam.data_ptr(),
            _p(gate_logit), 0 if gate_logit is None else gate_logit.stride(0),
            0 if gate_logit is None else gate_logit.stride(1), _p(g),
            inv_freq.data_ptr(), cos_t.data_ptr(), sin_t.data_ptr(), _stream()), "coda_b200_prep")
        return qn, lam, g

    def _attend(self, cfg, st, Lq, q, qn, lam, k_blk, v_blk, out):
        _, _, _, _, nw = self._consts(q.device, q.dtype)
        ptrs = self._ptrs(st)
        timers = self.kernel_timers
        if timers is not None:                  # benchmark hook: CUDA events around the attention launch
            ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            ev0.record()
        if self.use_torch_ops:
            from . import torch_ops
            ci, cf = torch_ops.cfg_lists(cfg)
            torch_ops.load().attend(out, st.k_buf, st.v_buf, st.allowed, q, qn, lam, k_blk, v_blk, nw, ci, cf)
        else:
            self._attend_ctypes(cfg, ptrs, Lq, q, qn, lam, k_blk, v_blk, nw, out)
        if timers is not None:
            ev1.record()
            timers.append((Lq, ev0, ev1))

    def _attend_ctypes(self, cfg, ptrs, Lq, q, qn, lam, k_blk, v_blk, nw, out):
        check(lib.coda_b200_attend(
            C.byref(cfg), C.byref(ptrs), Lq,
            q.data_ptr(), q.stride(0), q.stride(1), qn.data_ptr(), qn.stride(0), qn.stride(1),
            lam.data_ptr(), lam.stride(0), lam.stride(1),
            _p(k_blk), 0 if k_blk is None else k_blk.stride(0), 0 if k_blk is None else k_blk.stride(1),
            _p(v_blk), 0 if v_blk is None else v_blk.stride(0), 0 if v_blk is None else v_blk.stride(1),
            _p(nw), out.data_ptr(), out.stride(0), out.stride(1), _stream()), "coda_b200_attend")

    def _write_one(self, cfg, st, k, v, g, rp: Optional[RingPos] = None):
        """Ring write of one token per state plus routing of the evicted one (upstream memory_banks.py:183-224).

        With ``rp`` given (CUDA-graph replay: scalars baked at capture time plus a device step counter) the
        host mirrors are left alone; the caller advances them with :meth:`advance_host_scalars`."""
        _, _, _, eta, _ = self._consts(k.device, k.dtype)
        host = rp is None
        if host:
            self._arm_events(st)
            rp = RingPos(int(st.pos), int(st.recent_idx), int(st.recent_filled), None)
        ptrs = self._ptrs(st)
        if self.use_torch_ops and host and st._events is None:
            from . import torch_ops
            ci, cf = torch_ops.cfg_lists(cfg)
            torch_ops.load().step_write(st.k_buf, st.v_buf, st.allowed, st.g_recent, st.mem_last_exact, st._exact_v_norm,
                                        st._sum_lf_k_norm, k, v, g.view(-1), eta, int(st.pos), int(st.recent_idx),
                                        int(st.recent_filled), ci, cf)
        else:
            check(lib.coda_b200_step_write(C.byref(cfg), C.byref(ptrs), rp, k.data_ptr(), k.stride(0),
                                           v.data_ptr(), v.stride(0), g.data_ptr(), eta.data_ptr(), _stream()),
                  "coda_b200_step_write")
        if host:
            self._account(st, int(st.recent_filled >= self.window), block=False)
            self.advance_host_scalars(st)

    def advance_host_scalars(self, st: CoDAGQALandmarkStatePerf2, n: int = 1) -> None:
        """Host mirror of ``n`` single-token writes: the ring fills, then the eviction pointer walks round it."""
        W = self.window
        fill = min(n, W - st.recent_filled)
        st.recent_filled += fill
        st.recent_idx = (st.recent_idx + (n - fill)) % W
        st.pos += n

    def _tuned_prefill(self, cfg) -> bool:
        ok = getattr(cfg, "_tuned_prefill", None)
        if ok is None:
            ok = bool(lib.coda_b200_prefill_attend_supported(C.byref(cfg)))
            cfg._tuned_prefill = ok
        return ok and self.use_tuned_kernels

    def _attend_block_tc(self, cfg, st, L, t0, blk, q, qn, lam, k, v, out):
        """Tensor-core prefill attention of rows t0..t0+blk of the chunk (whole-chunk tensors are passed)."""
        _, _, _, _, nw = self._consts(q.device, q.dtype)
        ptrs = self._ptrs(st)
        timers = self.kernel_timers
        if timers is not None:
            ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            ev0.record()
        if self.use_torch_ops:
            from . import torch_ops
            ci, cf = torch_ops.cfg_lists(cfg)
            torch_ops.load().prefill_attend(out, st.k_buf, st.v_buf, st.allowed, q, qn, lam, k, v, nw,
                                            self._status_word(q.device), int(t0), int(blk), ci, cf)
        else:
            check(lib.coda_b200_prefill_attend(
                C.byref(cfg), C.byref(ptrs), L, t0, blk,
                q.data_ptr(), q.stride(0), q.stride(1), qn.data_ptr(), qn.stride(0), qn.stride(1),
                lam.data_ptr(), lam.stride(0), lam.stride(1),
                k.data_ptr(), k.stride(0), k.stride(1), v.data_ptr(), v.stride(0), v.stride(1),
                _p(nw), out.data_ptr(), out.stride(0), out.stride(1),
                self._status_word(q.device).data_ptr(), _stream()), "coda_b200_prefill_attend")
        if timers is not None:
            ev1.record()
            timers.append((blk, ev0, ev1))

    def _tuned_decode(self, cfg) -> bool:
        ok = getattr(cfg, "_tuned_decode", None)
        if ok is None:
            ok = bool(lib.coda_b200_decode_attend_supported(C.byref(cfg)))
            cfg._tuned_decode = ok
        return ok and self.use_tuned_kernels

    def _status_word(self, device) -> torch.Tensor:
        if self._status is None or self._status.device != device:
            self._status = torch.zeros(1, dtype=torch.int32, device=device)
        return self._status

    def device_status(self) -> int:
        """0, or the code of a bounded device-side wait that expired in one of the tuned kernels
        (1 = producer waiting for a free tile, 2 = consumer waiting for a tile).  Synchronises."""
        return 0 if self._status is None else int(self._status.item())

    def _decode_records(self, cfg, device) -> torch.Tensor:
        """Device buffer for the per-plane decode records (prepared queries, lambda, visibility mask)."""
        n = getattr(cfg, "_rec_bytes", None)
        if n is None:
            n = int(lib.coda_b200_decode_record_bytes(C.byref(cfg)))
            cfg._rec_bytes = n
        buf = self._qrec
        if buf is None or buf.numel() < n or buf.device != device:
            buf = torch.empty(n, dtype=torch.uint8, device=device)
            self._qrec = buf
        return buf

    def _fused_write_ok(self, cfg, q: Optional[torch.Tensor] = None) -> bool:
        ok = getattr(cfg, "_fused_write", None)
        if ok is None:
            ok = bool(lib.coda_b200_step_write_fused_supported(C.byref(cfg)))
            cfg._fused_write = ok
        return ok and (q is None or q.data_ptr() % 4 == 0)

    def route_launch(self, x_dtype: torch.dtype, state: CoDAGQALandmarkStatePerf2, rp: RingPos, stream: int) -> bool:
        """First half of a decode step, on ``stream``: the token the ring is about to evict is routed into the
        banks.  It depends on the state alone, so it may run beside the projection GEMM of the same step; the
        second half is ``step_graphable(..., routed=True)`` with the same ``rp``, ordered after it.  Returns
        False (nothing launched) where the step runs as one launch."""
        cfg = self._cfg(state.k_buf.shape[0], x_dtype, state)
        if not (self._tuned_decode(cfg) and self._fused_write_ok(cfg)) or self._tracked(state):
            return False
        _, _, _, eta, _ = self._consts(state.k_buf.device, x_dtype)
        check(lib.coda_b200_step_route(C.byref(cfg), C.byref(self._ptrs(state)), rp, eta.data_ptr(), stream),
              "coda_b200_step_route")
        return True

    def _out(self, heads: torch.Tensor, residual: Optional[torch.Tensor]) -> torch.Tensor:
        """Output projection, plus ``residual`` if given."""
        B, L, HD = heads.shape
        w = self.o_proj.weight if type(self.o_proj) is nn.Linear and self.o_proj.bias is None else None
        if (self.use_skinny_gemm_kernel and w is not None and heads.is_cuda and heads.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
                and heads.is_contiguous() and w.is_contiguous() and heads.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0
                and (residual is None or (residual.is_contiguous() and residual.data_ptr() % 16 == 0))
                and lib.coda_b200_skinny_gemm_supported(B * L, HD, w.shape[0])):
            # weight rows streamed through a TMA ring, residual in the epilogue (one launch instead of GEMM + add)
            N = w.shape[0]
            y = torch.empty((B, L, N), device=heads.device, dtype=heads.dtype)
            check(lib.coda_b200_skinny_gemm(heads.data_ptr(), B * L, HD, w.data_ptr(), N, _p(residual), N, y.data_ptr(), N,
                                            self._status_word(heads.device).data_ptr(), _stream()), "coda_b200_skinny_gemm")
            return y
        if type(self.o_proj) is nn.Linear:
            y = self._own_gemm(heads, self.o_proj.weight, self.o_proj.bias, residual)
            if y is not None:
                return y
        wt = self._skinny_weights() if B * L <= self.SKINNY_ROWS else None
        if wt is not None:
            h2 = heads.reshape(B * L, HD)
            y = torch.mm(h2, wt[2])
            if residual is not None:
                # a separate small add: the library's accumulate-into-C epilogue costs this GEMM 3.6 us (13.9 vs 10.3)
                y.add_(residual.reshape(B * L, -1))
            return y.view(B, L, -1)
        if residual is None:
            return self.o_proj(heads)
        return torch.addmm(residual.reshape(B * L, -1), heads.reshape(B * L, HD), self.o_proj.weight.t()).view(B, L, -1)

    def _step_fused(self, cfg, x, state, rp: RingPos, host_update: bool, routed: bool = False,
                    residual: Optional[torch.Tensor] = None, rope_cs: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Write-then-attend decode step on the tuned kernels: two launches between the two GEMMs.  The cache
        write applies RoPE / the gate sigmoid and, where it can, also prepares the attention's queries
        (decode records); the fused attention then only streams the state.  ``routed``: the evicted token
        has been routed already (:meth:`route_launch`), only the new token is left to write."""
        B = x.shape[0]
        dev, dt = x.device, x.dtype
        q, k, v, lam_logit, gate_logit = self._project(x, need_kv=True)
        inv_freq, cos_t, sin_t, eta, nw = self._consts(dev, dt)
        if host_update:
            self._arm_events(state)
        ptrs = self._ptrs(state)
        s = _stream()
        out = torch.empty((B, 1, self.num_heads * self.head_dim), device=dev, dtype=dt)
        fused_ok = self._fused_write_ok(cfg, q)
        if routed:
            if not fused_ok:
                raise RuntimeError("routed=True needs the fused cache-write kernel")
            one = getattr(cfg, "_attend_append", None)
            if one is None:
                one = bool(lib.coda_b200_decode_attend_append_supported(C.byref(cfg)))
                cfg._attend_append = one
            if one and self.fuse_append_into_attention and q.data_ptr() % 16 == 0 and q.stride(0) % 8 == 0:
                # the attention kernel writes the new token itself: one launch between the two GEMMs
                self.decode_attend_append_launch(cfg, state, rp, (q, k, v, lam_logit, gate_logit), out, rope_cs)
                if host_update:
                    self.advance_host_scalars(state)
                return self._out(out, residual)
            qrec = self._decode_records(cfg, dev)
            check(lib.coda_b200_step_append_fused(
                C.byref(cfg), C.byref(ptrs), rp, k.data_ptr(), k.stride(0), v.data_ptr(), v.stride(0),
                _p(gate_logit), 0 if gate_logit is None else gate_logit.stride(0), inv_freq.data_ptr(),
                q.data_ptr(), q.stride(0), lam_logit.data_ptr(), lam_logit.stride(0), cos_t.data_ptr(), sin_t.data_ptr(),
                qrec.data_ptr(), s), "coda_b200_step_append_fused")
            check(lib.coda_b200_decode_attend_prepared(
                C.byref(cfg), C.byref(ptrs), qrec.data_ptr(), _p(nw), out.data_ptr(), out.stride(0),
                self._status_word(dev).data_ptr(), s), "coda_b200_decode_attend_prepared")
        elif fused_ok:
            qrec = self._decode_records(cfg, dev)
            check(lib.coda_b200_step_write_fused(
                C.byref(cfg), C.byref(ptrs), rp, k.data_ptr(), k.stride(0), v.data_ptr(), v.stride(0),
                _p(gate_logit), 0 if gate_logit is None else gate_logit.stride(0), inv_freq.data_ptr(), eta.data_ptr(),
                q.data_ptr(), q.stride(0), lam_logit.data_ptr(), lam_logit.stride(0), cos_t.data_ptr(), sin_t.data_ptr(),
                qrec.data_ptr(), s), "coda_b200_step_write_fused")
            check(lib.coda_b200_decode_attend_prepared(
                C.byref(cfg), C.byref(ptrs), qrec.data_ptr(), _p(nw), out.data_ptr(), out.stride(0),
                self._status_word(dev).data_ptr(), s), "coda_b200_decode_attend_prepared")
        else:
            check(lib.coda_b200_step_write_raw(
                C.byref(cfg), C.byref(ptrs), rp, k.data_ptr(), k.stride(0), v.data_ptr(), v.stride(0),
                _p(gate_logit), 0 if gate_logit is None else gate_logit.stride(0), inv_freq.data_ptr(), eta.data_ptr(), s),
                "coda_b200_step_write_raw")
            self.decode_attend_launch(cfg, state, rp, 0, q, lam_logit, out)
        if host_update:
            self._account(state, int(state.recent_filled >= self.window), block=False)
            self.advance_host_scalars(state)
        return self._out(out, residual)

    def decode_attend_launch(self, cfg, state, rp: RingPos, token_already_written: int, q, lam_logit, out) -> None:
        """The fused decode attention alone: raw query projection ``q`` [B, H*Dh] and lambda logits [B, H] in,
        head-normalised differential attention [B, 1, H*Dh] out (a small preparation launch, then the kernel)."""
        inv_freq, cos_t, sin_t, _, nw = self._consts(q.device, q.dtype)
        ptrs = self._ptrs(state)
        qrec = self._decode_records(cfg, q.device)
        if self.use_torch_ops and rp.step_dev is None and q.dim() == 3:
            from . import torch_ops
            ci, cf = torch_ops.cfg_lists(cfg)
            torch_ops.load().decode_attend(out, state.k_buf, state.v_buf, state.allowed, q, lam_logit, inv_freq, cos_t,
                                           sin_t, nw, qrec, self._status_word(q.device), int(rp.pos), int(rp.recent_idx),
                                           int(rp.recent_filled), int(token_already_written), ci, cf)
            return
        check(lib.coda_b200_decode_attend(
            C.byref(cfg), C.byref(ptrs), rp, token_already_written, q.data_ptr(), q.stride(0),
            lam_logit.data_ptr(), lam_logit.stride(0), inv_freq.data_ptr(), cos_t.data_ptr(), sin_t.data_ptr(),
            _p(nw), qrec.data_ptr(), out.data_ptr(), out.stride(0), self._status_word(q.device).data_ptr(), _stream()),
            "coda_b200_decode_attend")

    def decode_attend_append_launch(self, cfg, state, rp: RingPos, proj, out, rope_cs=None) -> None:
        """One launch of the decode attention kernel that also writes the step's new token (ring slot, gate, slot
        flag) from the raw projections ``proj = (q, k, v, lambda logits, gate logits)`` of :meth:`_project`; the
        token the ring evicts must have been routed before (``route_launch`` / the stack's batched routing)."""
        q, k, v, lam_logit, gate_logit = proj
        inv_freq, cos_t, sin_t, _, nw = self._consts(out.device, out.dtype)
        ptrs = self._ptrs(state)
        check(lib.coda_b200_decode_attend_append(
            C.byref(cfg), C.byref(ptrs), rp, k.data_ptr(), k.stride(0), v.data_ptr(), v.stride(0),
            _p(gate_logit), 0 if gate_logit is None else gate_logit.stride(0), inv_freq.data_ptr(),
            q.data_ptr(), q.stride(0), lam_logit.data_ptr(), lam_logit.stride(0), cos_t.data_ptr(), sin_t.data_ptr(),
            _p(rope_cs), _p(nw), out.data_ptr(), out.stride(0), self._status_word(out.device).data_ptr(), _stream()),
            "coda_b200_decode_attend_append")

    def decode_attend_prepared_launch(self, cfg, state, out) -> None:
        """One launch of the decode attention kernel on the records the last fused cache write left behind."""
        _, _, _, _, nw = self._consts(out.device, out.dtype)
        ptrs = self._ptrs(state)
        check(lib.coda_b200_decode_attend_prepared(
            C.byref(cfg), C.byref(ptrs), self._decode_records(cfg, out.device).data_ptr(), _p(nw), out.data_ptr(),
            out.stride(0), self._status_word(out.device).data_ptr(), _stream()), "coda_b200_decode_attend_prepared")

    def step_graphable(self, x: torch.Tensor, state: CoDAGQALandmarkStatePerf2, rp: RingPos,
                       routed: bool = False, residual: Optional[torch.Tensor] = None,
                       rope_cs: Optional[torch.Tensor] = None) -> torch.Tensor:
        """The default ``step`` (write, then attend) with no host-side branching on the state, so that it
        can be captured in a CUDA graph: ring scalars come from ``rp`` (values at capture time plus the device
        step counter ``rp.step_dev``).  Does not touch the Python-side scalars.  With ``residual`` the result
        is ``residual + y``; ``rope_cs``: float [head_dim] cos | sin table of this step's position from
        ``coda_b200_rope_table`` (a stack computes it once per step for all its layers)."""
        if self._tracked(state):
            raise RuntimeError("a state with metrics or expandable banks needs a host read after every cache write "
                               "and cannot be replayed from a CUDA graph: use step()")
        B = x.shape[0]
        cfg = self._cfg(B, x.dtype, state)
        if self._tuned_decode(cfg):
            return self._step_fused(cfg, x, state, rp, host_update=False, routed=routed, residual=residual,
                                    rope_cs=rope_cs)
        if routed:
            raise RuntimeError("routed=True needs the tuned decode kernels")
        q, k, v, lam_logit, gate_logit = self._project(x, need_kv=True)
        qn, lam, g = self._prep(cfg, 1, rp.pos, q, k, lam_logit, gate_logit, True, step_dev=rp.step_dev)
        self._write_one(cfg, state, k, v, g, rp=rp)
        out = torch.empty((B, 1, self.num_heads * self.head_dim), device=x.device, dtype=x.dtype)
        self._attend(cfg, state, 1, q, qn, lam, None, None, out)
        return self._out(out, residual)

    # -- a captured step whose layer boundary is one launch: output projection + next layer's input projection --
    def chain_ready(self, B: int, dtype: torch.dtype, state: CoDAGQALandmarkStatePerf2,
                    next_layer: Optional["CoDAGQALandmarkPerf2"]) -> bool:
        """Can this layer's captured decode step take its projections from the previous layer's chained launch and
        hand its own output projection, with ``next_layer``'s input projection, to one
        ``coda_b200_skinny_gemm_chain`` launch?  (bf16, the attention kernel that writes the new token itself, a plain
        bias-free output projection, a fused input weight on the next layer, shapes the kernel covers as one wave.)"""
        if dtype != torch.bfloat16 or not (self.use_tuned_kernels and self.use_skinny_gemm_kernel and self.fuse_append_into_attention):
            return False
        if self._tracked(state) or type(self.o_proj) is not nn.Linear or self.o_proj.bias is not None:
            return False
        cfg = self._cfg(B, dtype, state)
        if not (self._tuned_decode(cfg) and self._fused_write_ok(cfg) and lib.coda_b200_decode_attend_append_supported(C.byref(cfg))):
            return False
        if self._fused_weight() is None:
            return False
        if next_layer is None:
            return True
        f = next_layer._fused_weight()
        w = self.o_proj.weight
        if f is None or f[0].dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or not (f[0].is_contiguous() and w.is_contiguous()):
            return False
        if f[0].shape[1] != w.shape[0] or (f[0].data_ptr() | f[1].data_ptr() | w.data_ptr()) % 16:
            return False
        return bool(lib.coda_b200_skinny_gemm_chain_supported(B, w.shape[1], w.shape[0], f[0].shape[0]))

    def step_chained(self, h: torch.Tensor, state: CoDAGQALandmarkStatePerf2, rp: RingPos, *, rope_cs, proj_y,
                     next_layer: Optional["CoDAGQALandmarkPerf2"], gsync: torch.Tensor):
        """One layer of a captured decode step (the evicted token routed beforehand) between chained launches:
        ``proj_y`` is this layer's fused projection output as the previous layer's launch left it (None: computed
        here); the layer's output projection with the residual ``h`` and ``next_layer``'s fused input projection
        leave in one launch.  Returns ``(h + layer(h), next layer's fused projection output or None)``."""
        B = h.shape[0]
        cfg = self._cfg(B, h.dtype, state)
        proj = self._project(h, need_kv=True) if proj_y is None else self._split_fused(proj_y)
        out = torch.empty((B, 1, self.num_heads * self.head_dim), device=h.device, dtype=h.dtype)
        self.decode_attend_append_launch(cfg, state, rp, proj, out, rope_cs)
        if next_layer is None:
            return self._out(out, h), None
        W_in, bias = next_layer._fused_weight()
        w = self.o_proj.weight
        D, N = w.shape[0], W_in.shape[0]
        h_next = torch.empty((B, 1, D), device=h.device, dtype=h.dtype)
        y_next = torch.empty((B, 1, N), device=h.device, dtype=h.dtype)
        check(lib.coda_b200_skinny_gemm_chain(out.data_ptr(), B, w.shape[1], w.data_ptr(), D, h.data_ptr(), D, h_next.data_ptr(),
                                              W_in.data_ptr(), N, bias.data_ptr(), y_next.data_ptr(), N, gsync.data_ptr(),
                                              self._status_word(h.device).data_ptr(), _stream()), "coda_b200_skinny_gemm_chain")
        return h_next, y_next

    def _nothing_visible(self, st) -> bool:
        # Only an empty ring can leave every slot masked; the check costs a sync, so it is made
        # only then (upstream attention.py:485-488 returns zeros in that case).
        return self.mask_unused_memory and st.recent_filled == 0 and not bool(st.allowed.any())

    # ------------------------------------------------------------------ decode
    @torch.no_grad()
    def attend_step(self, x: torch.Tensor, state: CoDAGQALandmarkStatePerf2, *,
                    query_pos: Optional[int] = None) -> torch.Tensor:
        """Attention of one new token per state over the current slots (upstream attention.py:476-514)."""
        B, L, _ = x.shape
        assert L == 1
        self._require_ready(x, state)
        if self._nothing_visible(state):
            return torch.zeros_like(x)
        cfg = self._cfg(B, x.dtype, state)
        q, _, _, lam_logit, _ = self._project(x, need_kv=False)
        qp = state.pos if query_pos is None else int(query_pos)
        if self._tuned_decode(cfg):
            # fused kernel: raw query projection in, RoPE at qp / theta rotation / lambda sigmoid inside
            out = torch.empty((B, 1, self.num_heads * self.head_dim), device=x.device, dtype=x.dtype)
            rp = RingPos(int(qp), int(state.recent_idx), int(state.recent_filled), None)
            self.decode_attend_launch(cfg, state, rp, 0, q, lam_logit, out)
            return self._out(out, None)
        qn, lam, _ = self._prep(cfg, 1, qp, q, None, lam_logit, None, False)
        out = torch.empty_like(q)
        self._attend(cfg, state, 1, q, qn, lam, None, None, out)
        return self._out(out, None)

    @torch.no_grad()
    def step_residual(self, x: torch.Tensor, state: CoDAGQALandmarkStatePerf2) -> torch.Tensor:
        """``x + step(x)``: the residual connection of a decoder layer around the default decode step.  On the eager
        fast path the sum is taken inside the output projection's GEMM call (one rounding of the fp32 sum instead
        of two), which saves a launch and a host call per layer; elsewhere it is the plain sum."""
        B, L, _ = x.shape
        if L == 1 and not self.training and x.is_cuda and state.k_buf.shape[0] == B:
            y = self._step_eager_fast(x, state, residual=x)
            if y is not None:
                return y
        y, _ = self.step(x, state)
        return x + y

    @torch.no_grad()
    def step(self, x: torch.Tensor, state: CoDAGQALandmarkStatePerf2, *, attend: bool = True,
             write_cache: bool = True, include_current_in_attention: bool = True
             ) -> Tuple[torch.Tensor, CoDAGQALandmarkStatePerf2]:
        """One decode token per state (upstream attention.py:516-547): by default the token is written
        to the cache first and then attends over all slots, itself included."""
        B, L, _ = x.shape
        assert L == 1
        if (attend and write_cache and include_current_in_attention and not self.training and x.is_cuda
                and state.k_buf.shape[0] == B):
            y = self._step_eager_fast(x, state)
            if y is not None:
                return y, state
        self._require_ready(x, state)
        cfg = self._cfg(B, x.dtype, state)
        qp = int(state.pos)
        if attend and write_cache and include_current_in_attention and self._tuned_decode(cfg):
            rp = RingPos(qp, int(state.recent_idx), int(state.recent_filled), None)
            return self._step_fused(cfg, x, state, rp, host_update=True), state
        q, k, v, lam_logit, gate_logit = self._project(x, need_kv=write_cache)
        qn, lam, g = self._prep(cfg, 1, qp, q, k, lam_logit, gate_logit, write_cache)
        write_first = attend and include_current_in_attention and write_cache
        if write_first:
            self._write_one(cfg, state, k, v, g)
        if attend and not self._nothing_visible(state):
            out = torch.empty_like(q)
            self._attend(cfg, state, 1, q, qn, lam, None, None, out)
            y = self._out(out, None)
        else:
            y = torch.zeros_like(x)
        if write_cache and not write_first:
            self._write_one(cfg, state, k, v, g)
        return y, state

    # ------------------------------------------------------------------ prefill
    def _linearize_ring(self, st) -> None:
        """Rotate the ring so that slot 0 holds its oldest token; contents in time order are unchanged."""
        r, W = int(st.recent_idx), self.window
        if r == 0:
            return
        st.k_buf[:, :, :W, :] = torch.roll(st.k_buf[:, :, :W, :], -r, dims=2)
        st.v_buf[:, :, :W, :] = torch.roll(st.v_buf[:, :, :W, :], -r, dims=2)
        st.g_recent.copy_(torch.roll(st.g_recent, -r, dims=1))
        st.recent_idx = 0

    def _route_scratch(self, cfg, device) -> torch.Tensor:
        n = int(lib.coda_b200_route_scratch_bytes(C.byref(cfg)))
        key = (device, n)
        t = self._scratch.get(key)
        if t is None:
            t = torch.empty(n, dtype=torch.uint8, device=device)
            self._scratch[key] = t
        return t

    @torch.no_grad()
    def prefill_chunked(self, x_seq: torch.Tensor, state: CoDAGQALandmarkStatePerf2, *, block_size: int = 256,
                        write_cache: bool = True, return_outputs: bool = True
                        ) -> Tuple[Optional[torch.Tensor], CoDAGQALandmarkStatePerf2]:
        """Blockwise prefill (upstream attention.py:567-728): block j attends over
        [state after block j-1 | block j, causal], then the block is pushed through the ring and the
        tokens it evicts are routed into the banks."""
        if x_seq.shape[1] == 0:
            return (x_seq[:, :0, :].clone() if return_outputs else None), state
        y_heads = self._prefill_heads(x_seq, state, block_size, write_cache, return_outputs)
        if not return_outputs:
            return None, state
        return self.o_proj(y_heads), state

    @torch.no_grad()
    def prefill_chunked_residual(self, h: torch.Tensor, state: CoDAGQALandmarkStatePerf2, *, block_size: int = 256,
                                 inplace: bool = False) -> torch.Tensor:
        """``h + layer(h)`` over a chunk, the sum taken by the output projection itself (fp32 accumulator plus
        residual, one rounding) instead of by an add behind it.  ``inplace=True`` accumulates into ``h``'s own
        memory (a GEMM with beta = 1: no copy of the residual, no extra pass over the chunk) and returns ``h``."""
        B, L, D = h.shape
        if L == 0:
            return h
        y_heads = self._prefill_heads(h, state, block_size, True, True)
        if (inplace and h.is_contiguous() and type(self.o_proj) is nn.Linear and self.o_proj.bias is None
                and self.o_proj.weight.dtype == h.dtype):
            h.view(B * L, D).addmm_(y_heads.view(B * L, -1), self.o_proj.weight.t())
            return h
        return self._out(y_heads, h)

    def _prefill_heads(self, x_seq: torch.Tensor, state: CoDAGQALandmarkStatePerf2, block_size: int,
                       write_cache: bool, return_outputs: bool) -> Optional[torch.Tensor]:
        """The blockwise prefill up to the output projection: (B, L, H*Dh) head outputs, or None."""
        B, L, _ = x_seq.shape
        if block_size <= 0:
            raise ValueError("block_size must be positive")
        self._require_ready(x_seq, state)
        cfg = self._cfg(B, x_seq.dtype, state)
        dev, dt = x_seq.device, x_seq.dtype
        H, Hkv, Dh, W = self.num_heads, self.num_kv_heads, self.head_dim, self.window
        pos0 = int(state.pos)
        q, k, v, lam_logit, gate_logit = self._project(x_seq, need_kv=True)
        qn, lam, g = self._prep(cfg, L, pos0, q, k, lam_logit, gate_logit, True)

        block = int(block_size)
        nblk = (L + block - 1) // block
        if write_cache:
            self._linearize_ring(state)
            fill0 = int(state.recent_filled)
            gates = torch.cat([state.g_recent[:, :fill0], g], dim=1).contiguous()
            te = self.exact_candidates_per_block if self.Me > 0 else 0
            ts = self.summary_candidates_per_block if self.Ms > 0 else 0
            tmax = max(1, min(max(te, ts), block))
            cand = torch.empty((B, nblk, tmax), device=dev, dtype=torch.int32)
            ops = None
            if self.use_torch_ops and not self._tracked(state):
                from . import torch_ops
                ops = torch_ops.load()
            if max(te, ts) > 0:
                if ops is not None:
                    ops.select_candidates(cand, gates, fill0, L, block, *torch_ops.cfg_lists(cfg))
                else:
                    check(lib.coda_b200_select_candidates(C.byref(cfg), gates.data_ptr(), gates.stride(0), fill0, L, block,
                                                          cand.data_ptr(), tmax, _stream()), "coda_b200_select_candidates")
            scratch = self._route_scratch(cfg, dev)
            _, _, _, eta, _ = self._consts(dev, dt)
            self._arm_events(state)
            ptrs = self._ptrs(state)
        y_heads = torch.empty((B, L, H * Dh), device=dev, dtype=dt) if return_outputs else None
        tc_ok = (return_outputs and self._tuned_prefill(cfg) and q.data_ptr() % 16 == 0 and k.data_ptr() % 16 == 0
                 and v.data_ptr() % 16 == 0 and all(t.stride(i) % 8 == 0 for t in (q, k, v) for i in (0, 1)))

        # Scores and decisions of a block's routing read the state the block's attention reads and write nothing
        # it reads, so they run beside it on a second stream; slot updates and the ring rewrite follow both.
        overlap = (self.overlap_block_routing and return_outputs and tc_ok and write_cache and ops is None
                   and state._events is None and not torch.cuda.is_current_stream_capturing())
        if overlap:
            main = torch.cuda.current_stream(dev)
            side = _side_stream_for(dev)
            ev_state, ev_plan = torch.cuda.Event(), torch.cuda.Event()

        for j in range(nblk):
            t0 = j * block
            blk = min(block, L - t0)
            kb, vb = k[:, t0:t0 + blk], v[:, t0:t0 + blk]
            if overlap:
                fill = int(state.recent_filled)
                seen = fill0 + t0
                route_args = (C.byref(cfg), C.byref(ptrs), fill, blk, pos0 + t0,
                              kb.data_ptr(), k.stride(0), k.stride(1), vb.data_ptr(), v.stride(0), v.stride(1),
                              gates.data_ptr(), gates.stride(0), seen - fill,
                              cand[:, j].data_ptr(), cand.stride(0), eta.data_ptr(), scratch.data_ptr())
                ev_state.record(main)
                side.wait_event(ev_state)
                check(lib.coda_b200_route_block_phase(*route_args, 1, side.cuda_stream), "coda_b200_route_block_phase")
                ev_plan.record(side)
                self._attend_block_tc(cfg, state, L, t0, blk, q, qn, lam, k, v, y_heads)
                main.wait_event(ev_plan)
                check(lib.coda_b200_route_block_phase(*route_args, 2, main.cuda_stream), "coda_b200_route_block_phase")
                state.recent_filled = min(W, fill + blk)
                state.recent_idx = 0
                state.pos = pos0 + t0 + blk
                continue
            if return_outputs and tc_ok:
                self._attend_block_tc(cfg, state, L, t0, blk, q, qn, lam, k, v, y_heads)
            elif return_outputs:
                self._attend(cfg, state, blk, q[:, t0:t0 + blk], qn[:, t0:t0 + blk], lam[:, t0:t0 + blk],
                             kb, vb, y_heads[:, t0:t0 + blk])
            if write_cache:
                fill = int(state.recent_filled)
                seen = fill0 + t0
                if ops is not None:
                    ops.route_block(state.k_buf, state.v_buf, state.allowed, state.g_recent, state.mem_last_exact,
                                    state._exact_v_norm, state._sum_lf_k_norm, kb, vb, gates, cand[:, j], eta, scratch,
                                    fill, pos0 + t0, seen - fill, *torch_ops.cfg_lists(cfg))
                else:
                    check(lib.coda_b200_route_block(
                        C.byref(cfg), C.byref(ptrs), fill, blk, pos0 + t0,
                        kb.data_ptr(), k.stride(0), k.stride(1), vb.data_ptr(), v.stride(0), v.stride(1),
                        gates.data_ptr(), gates.stride(0), seen - fill,
                        cand[:, j].data_ptr(), cand.stride(0), eta.data_ptr(), scratch.data_ptr(), _stream()),
                        "coda_b200_route_block")
                if state._events is not None:
                    self._account(state, fill + blk - min(W, fill + blk), block=True)
                    cfg = self._cfg(B, dt, state)          # the banks may have grown
                state.recent_filled = min(W, fill + blk)
                state.recent_idx = 0
                state.pos = pos0 + t0 + blk
        return y_heads

    # ------------------------------------------------------------------ utility
    def cache_bytes(self, *, batch_size: int, dtype: torch.dtype) -> int:
        """State size in bytes, same accounting as upstream attention.py:734-751."""
        B, Hkv, Dh = int(batch_size), self.num_kv_heads, self.head_dim
        e = torch.tensor([], dtype=dtype).element_size()
        kv = 2 * B * Hkv * self.Lbuf * Dh * e
        exact_norm = B * Hkv * self.Me * Dh * e if self.Me > 0 else 0
        sum_norm = B * Hkv * self.Ms * self.lf_dim * e if self.Ms > 0 else 0
        return int(kv + exact_norm + sum_norm + B * self.window * 4 + B * self.Lbuf + B * self.Me * 8)

    def reset_metrics(self, state: CoDAGQALandmarkStatePerf2) -> None:
        """Zero the metrics counters of a state that carries them (upstream attention.py:753-760)."""
        if state.metrics is not None:
            for key in state.metrics:
                state.metrics[key] = 0 if isinstance(state.metrics[key], int) else 0.0
