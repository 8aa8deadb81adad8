"""CPU oracle for the bounded-cache differential-attention path.

TEST INFRASTRUCTURE ONLY.  This file is a CPU restatement (plain PyTorch tensor
arithmetic on the host) of the algorithm implemented by the upstream project's
``CoDAGQALandmarkPerf2`` (``src/coda_gqa_l/attention.py``,
``src/coda_gqa_l/memory_banks.py``, ``src/coda_gqa_l/primitives.py``).  It is the
checker that the CUDA path is compared with; nothing in the shipped package may
import it.  Only ``tests/``, ``__graft_entry__.smoke()`` and the CPU-baseline /
reference legs of ``bench.py`` use it.

Parity pin: the restatement is validated against the upstream implementation
itself (imported unmodified, accelerator flags off) by
``tests/golden/make_golden.py``; the fixtures that script writes are committed
under ``tests/golden/`` and re-checked by ``tests/test_oracle_golden.py``.

Third-party behaviour the path depends on: ``torch.topk`` on CPU (ATen; the tie
order of its selection decides which evicted tokens become bank candidates and
which free slots they take).  The oracle calls ``torch.topk`` itself, so it pins
the order of the installed torch (2.11.0 here).

Structure: a weights mapping (the module's ``state_dict``), an ``OracleConfig`` of
hyper-parameters and a mutable ``OracleState`` with the same field names as the
upstream state dataclass (``src/coda_gqa_l/state.py:12-54``).
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict, Optional

import torch

NEG_FILL = -1e9          # score given to unusable slots (memory_banks.py:264-265)
I62 = 2 ** 62            # LRU sentinel (memory_banks.py:280, 659)


# --------------------------------------------------------------------------- #
# configuration / state
# --------------------------------------------------------------------------- #
@dataclass
class OracleConfig:
    """Hyper-parameters of one layer (attention.py:89-141, defaults kept)."""

    embed_dim: int
    num_heads: int
    num_kv_heads: int
    window: int
    num_landmarks_exact: int
    num_landmarks_summary: int
    rope_base: float = 10_000.0
    write_policy: str = "gated"
    write_gate_threshold_exact: float = 0.10
    write_gate_threshold_summary: float = 0.05
    exact_match_threshold: float = 0.90
    exact_novelty_threshold: float = 0.70
    exact_refresh_on_hit: bool = False
    exact_candidates_per_block: int = 8
    summary_candidates_per_block: int = 64
    summary_overwrite_on_insert: bool = True
    mem_init: str = "random_normal"
    mask_unused_memory: bool = True
    eps: float = 1e-6
    head_norm_mode: str = "full"
    rope_interleaved: bool = True
    # dtype the RoPE angles are evaluated in.  Upstream keeps inv_freq as a module buffer
    # (primitives.py:40-41), so ``module.to(bfloat16)`` casts it and the positions
    # ``arange(..., dtype=inv_freq.dtype)`` and their product are then rounded to bf16
    # (primitives.py:51-52).  None = same as the activations.
    angle_dtype: Optional[torch.dtype] = None
    # dynamic bank expansion (attention.py:116-122,344-390): banks start at min_* active slots and grow towards
    # num_landmarks_* under pressure; None = fixed size.  collect_metrics: attention.py:319-336.
    min_landmarks_exact: Optional[int] = None
    min_landmarks_summary: Optional[int] = None
    expansion_t_max: int = 1_000_000
    collect_metrics: bool = False

    @property
    def Me_min(self) -> int:
        return self.num_landmarks_exact if self.min_landmarks_exact is None else int(self.min_landmarks_exact)

    @property
    def Ms_min(self) -> int:
        return self.num_landmarks_summary if self.min_landmarks_summary is None else int(self.min_landmarks_summary)

    @property
    def head_dim(self) -> int:
        return self.embed_dim // self.num_heads

    @property
    def lf_start(self) -> int:
        return self.head_dim // 2

    @property
    def energy_scale(self) -> float:
        # attention.py:160-162
        return math.sqrt(self.head_dim / (self.head_dim - self.lf_start))

    @property
    def Lbuf(self) -> int:
        return self.window + self.num_landmarks_exact + self.num_landmarks_summary

    @classmethod
    def from_module(cls, m) -> "OracleConfig":
        """Read the hyper-parameters off a module exposing the upstream attribute names."""
        return cls(
            embed_dim=m.embed_dim, num_heads=m.num_heads, num_kv_heads=m.num_kv_heads,
            window=m.window, num_landmarks_exact=m.Me, num_landmarks_summary=m.Ms,
            rope_base=float(getattr(m, "rope_base", 10_000.0)),
            write_policy=m.write_policy,
            write_gate_threshold_exact=m.write_gate_threshold_exact,
            write_gate_threshold_summary=m.write_gate_threshold_summary,
            exact_match_threshold=m.exact_match_threshold,
            exact_novelty_threshold=m.exact_novelty_threshold,
            exact_refresh_on_hit=m.exact_refresh_on_hit,
            exact_candidates_per_block=m.exact_candidates_per_block,
            summary_candidates_per_block=m.summary_candidates_per_block,
            summary_overwrite_on_insert=m.summary_overwrite_on_insert,
            mem_init=m.mem_init, mask_unused_memory=m.mask_unused_memory,
            eps=float(getattr(getattr(m, "head_norm", None), "eps", 1e-6)),
            head_norm_mode=m.head_norm_mode, rope_interleaved=m.rope_interleaved,
            angle_dtype=m.rope.inv_freq.dtype,
            min_landmarks_exact=getattr(m, "Me_min", None), min_landmarks_summary=getattr(m, "Ms_min", None),
            expansion_t_max=int(getattr(m, "expansion_t_max", 1_000_000)),
            collect_metrics=bool(getattr(m, "collect_metrics", False)),
        )


@dataclass
class OracleState:
    """Same fields as the upstream state (state.py:23-54)."""

    k_buf: torch.Tensor
    v_buf: torch.Tensor
    allowed: torch.Tensor
    g_recent: torch.Tensor
    recent_idx: int
    recent_filled: int
    mem_last_exact: torch.Tensor
    pos: int
    active_exact: int = 0
    active_summary: int = 0
    _exact_v_norm: Optional[torch.Tensor] = field(default=None, repr=False)
    _sum_lf_k_norm: Optional[torch.Tensor] = field(default=None, repr=False)
    metrics: Optional[dict] = field(default=None, repr=False)
    # Trace of routing decisions, appended by the bank updates (oracle-only).
    trace: Optional[list] = field(default=None, repr=False)


METRIC_KEYS = ("exact_hits", "exact_inserts", "exact_overwrites", "exact_fill_ratio", "summary_updates",
               "summary_inserts", "summary_fill_ratio", "tokens_gated_out", "total_evictions", "exact_frustrated",
               "summary_frustrated", "active_exact", "active_summary", "expansions_exact", "expansions_summary")


def new_metrics(active_exact: int, active_summary: int) -> dict:
    """The counters dict of attention.py:319-336."""
    m = {k: 0 for k in METRIC_KEYS}
    m["exact_fill_ratio"] = 0.0
    m["summary_fill_ratio"] = 0.0
    m["active_exact"], m["active_summary"] = active_exact, active_summary
    return m


def log_ceiling(cfg, tokens_seen: int):
    """Largest active bank sizes allowed after ``tokens_seen`` tokens (attention.py:344-356)."""
    Me, Ms = cfg.num_landmarks_exact, cfg.num_landmarks_summary
    if cfg.expansion_t_max <= 0:
        return Me, Ms
    ratio = min(math.log(1 + tokens_seen) / math.log(1 + cfg.expansion_t_max), 1.0)
    return cfg.Me_min + int((Me - cfg.Me_min) * ratio), cfg.Ms_min + int((Ms - cfg.Ms_min) * ratio)


def try_expand(cfg, st, frustrated_exact: int, frustrated_summary: int) -> None:
    """Grow the active capacities under pressure, up to the logarithmic ceiling (attention.py:358-390)."""
    if cfg.Me_min == cfg.num_landmarks_exact and cfg.Ms_min == cfg.num_landmarks_summary:
        return
    if frustrated_exact <= 0 and frustrated_summary <= 0:
        return
    ceil_e, ceil_s = log_ceiling(cfg, st.pos)
    grow_e = grow_s = 0
    if frustrated_exact > 0 and st.active_exact < ceil_e:
        grow_e = min(frustrated_exact, ceil_e - st.active_exact)
        st.active_exact += grow_e
    if frustrated_summary > 0 and st.active_summary < ceil_s:
        grow_s = min(frustrated_summary, ceil_s - st.active_summary)
        st.active_summary += grow_s
    if st.metrics is not None:
        st.metrics["active_exact"], st.metrics["active_summary"] = st.active_exact, st.active_summary
        st.metrics["expansions_exact"] += grow_e
        st.metrics["expansions_summary"] += grow_s


def _unit(x: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """x / max(||x||_2, eps) over the last dim (what F.normalize computes)."""
    return torch.nn.functional.normalize(x, dim=-1, eps=eps)


def init_state(cfg: OracleConfig, batch_size: int, dtype: torch.dtype,
               mem_init: Optional[str] = None) -> OracleState:
    """Fresh state; bank contents drawn in the upstream order (attention.py:271-316).

    Uses the global torch RNG, so seed with ``torch.manual_seed`` before the call.
    """
    B, Hkv, Dh, W = batch_size, cfg.num_kv_heads, cfg.head_dim, cfg.window
    Me, Ms = cfg.num_landmarks_exact, cfg.num_landmarks_summary
    k = torch.zeros(B, Hkv, cfg.Lbuf, Dh, dtype=dtype)
    v = torch.zeros(B, Hkv, cfg.Lbuf, Dh, dtype=dtype)
    mode = cfg.mem_init if mem_init is None else mem_init
    if mode == "random_normal":
        if Me > 0:
            k[:, :, W:W + Me, :].normal_(mean=0.0, std=0.02)
            v[:, :, W:W + Me, :].normal_(mean=0.0, std=0.02)
        if Ms > 0:
            k[:, :, W + Me:, cfg.lf_start:].normal_(mean=0.0, std=0.02)
            v[:, :, W + Me:, :].normal_(mean=0.0, std=0.02)
    elif mode != "zeros":
        raise ValueError("mem_init must be 'zeros' or 'random_normal'")
    st = OracleState(
        k_buf=k, v_buf=v,
        allowed=torch.zeros(B, cfg.Lbuf, dtype=torch.bool),
        g_recent=torch.zeros(B, W, dtype=torch.float32),
        recent_idx=0, recent_filled=0,
        mem_last_exact=torch.zeros(B, Me, dtype=torch.int64),
        pos=0, active_exact=cfg.Me_min if Me > 0 else 0, active_summary=cfg.Ms_min if Ms > 0 else 0,
    )
    if cfg.collect_metrics:
        st.metrics = new_metrics(st.active_exact, st.active_summary)
    if Me > 0:
        st._exact_v_norm = _unit(v[:, :, W:W + Me, :]).clone()
    if Ms > 0:
        st._sum_lf_k_norm = _unit(k[:, :, W + Me:, cfg.lf_start:]).clone()
    return st


# --------------------------------------------------------------------------- #
# projections and rotations
# --------------------------------------------------------------------------- #
def _linear(x, wts: Dict[str, torch.Tensor], name: str):
    return torch.nn.functional.linear(x, wts[name + ".weight"], wts.get(name + ".bias"))


def _rope_tables(cfg: OracleConfig, L: int, offset: int, dtype):
    """cos/sin of shape (L, Dh/2): product t*inv_freq in the angle dtype, cast to dtype (primitives.py:40-55)."""
    Dh = cfg.head_dim
    adt = dtype if cfg.angle_dtype is None else cfg.angle_dtype
    inv_freq = (1.0 / (cfg.rope_base ** (torch.arange(0, Dh, 2).float() / Dh))).to(adt)
    t = torch.arange(offset, offset + L, dtype=adt)
    ang = t[:, None] * inv_freq[None, :]
    return ang.cos().to(dtype), ang.sin().to(dtype)


def _pair_rotate(x, c, s):
    """Rotate (even, odd) pairs of the last dim by angles given as cos c / sin s (primitives.py:58-80)."""
    xe, xo = x[..., 0::2], x[..., 1::2]
    out = torch.empty_like(x)
    out[..., 0::2] = xe * c - xo * s
    out[..., 1::2] = xe * s + xo * c
    return out


def _rope(x, cos, sin, interleaved: bool):
    """x: (B, heads, L, Dh); cos/sin: (L, Dh/2) (primitives.py:83-113)."""
    L, half = cos.shape
    c, s = cos.view(1, 1, L, half), sin.view(1, 1, L, half)
    if interleaved:
        return _pair_rotate(x, c, s)
    cf, sf = torch.cat([c, c], -1), torch.cat([s, s], -1)
    swapped = torch.cat([-x[..., half:], x[..., :half]], -1)
    return x * cf + swapped * sf


def _heads(y, n, Dh):
    B, L, _ = y.shape
    return y.view(B, L, n, Dh).transpose(1, 2)


def _gate(cfg, wts, x):
    """Write gate in fp32 (attention.py:406-410)."""
    if cfg.write_policy == "none":
        return torch.ones(x.shape[0], x.shape[1], dtype=torch.float32)
    return torch.sigmoid(_linear(x, wts, "write_proj")).squeeze(-1).float()


# --------------------------------------------------------------------------- #
# attention
# --------------------------------------------------------------------------- #
def _softmax_attend(q, k, v, keep):
    """softmax(q k^T / sqrt(Dh) masked by keep) v, evaluated in fp32 and cast back.

    q: (B,H,Lq,Dh); k, v: (B,H,Lk,Dh) already expanded to query heads; keep: bool
    broadcastable to (B,H,Lq,Lk) (True = visible).
    """
    Dh = q.shape[-1]
    s = torch.matmul(q.float(), k.float().transpose(-1, -2)) * (1.0 / math.sqrt(Dh))
    s = s.masked_fill(~keep, float("-inf"))
    p = torch.softmax(s, dim=-1)
    return torch.matmul(p, v.float()).to(q.dtype)


def _diff_attend(cfg, wts, q, lam, k, v, keep):
    """Signal minus lambda-gated noise attention, then the head norm (attention.py:416-465)."""
    G = cfg.num_heads // cfg.num_kv_heads
    kx = k.repeat_interleave(G, dim=1)
    vx = v.repeat_interleave(G, dim=1)
    theta = wts["theta"]
    ct, st_ = torch.cos(theta).to(q.dtype), torch.sin(theta).to(q.dtype)
    H, half = theta.shape
    qn = _pair_rotate(q, ct.view(1, H, 1, half), st_.view(1, H, 1, half))
    out = _softmax_attend(q, kx, vx, keep) - lam * _softmax_attend(qn, kx, vx, keep)
    if cfg.head_norm_mode == "full":
        var = out.pow(2).mean(dim=-1, keepdim=True)
        out = out * torch.rsqrt(var + cfg.eps)
        out = out * wts["head_norm.weight"]
    B, H, L, Dh = out.shape
    return _linear(out.transpose(1, 2).contiguous().view(B, L, H * Dh), wts, "o_proj")


def attend_step(cfg, wts, x, st: OracleState, query_pos: Optional[int] = None):
    """Decode attention over the valid slots (attention.py:476-514)."""
    B = x.shape[0]
    if cfg.mask_unused_memory:
        if not bool(st.allowed.any()):
            return torch.zeros_like(x)
        keep = st.allowed[:, None, None, :]
    else:
        keep = torch.ones(B, 1, 1, cfg.Lbuf, dtype=torch.bool)
    qp = st.pos if query_pos is None else int(query_pos)
    cos, sin = _rope_tables(cfg, 1, qp, x.dtype)
    q = _rope(_heads(_linear(x, wts, "q_proj"), cfg.num_heads, cfg.head_dim), cos, sin, cfg.rope_interleaved)
    lam = torch.sigmoid(_linear(x, wts, "lambda_proj")).transpose(1, 2).unsqueeze(-1)
    return _diff_attend(cfg, wts, q, lam, st.k_buf, st.v_buf, keep)


# --------------------------------------------------------------------------- #
# bank updates -- single evicted token (decode)
# --------------------------------------------------------------------------- #
def _exact_one(cfg, st: OracleState, k_e, v_e, pos_e: int, gate):
    """memory_banks.py:230-337 for one evicted token per row."""
    Me, W = cfg.num_landmarks_exact, cfg.window
    if Me == 0:
        return
    B = k_e.shape[0]
    Ae = st.active_exact
    sl = slice(W, W + Me)
    used = st.allowed[:, sl]
    keep = gate >= cfg.write_gate_threshold_exact if cfg.write_policy != "none" \
        else torch.ones(B, dtype=torch.bool)
    score = torch.einsum("bhd,bhmd->bhm", _unit(v_e), st._exact_v_norm).mean(dim=1)
    if Ae < Me:
        score[:, Ae:] = NEG_FILL
    score = score.masked_fill(~used, NEG_FILL)
    best, best_i = score.max(dim=-1)
    some_used = used[:, :Ae].any(dim=-1)
    novel = (~some_used) | (best < cfg.exact_novelty_threshold)
    hit = some_used & (best >= cfg.exact_match_threshold)
    free = ~used.clone()
    if Ae < Me:
        free[:, Ae:] = False
    first_free = free.to(torch.int64).argmax(dim=-1)
    stamp = torch.where(used, st.mem_last_exact, torch.full_like(st.mem_last_exact, I62))
    if Ae < Me:
        stamp[:, Ae:] = I62
    oldest = stamp.argmin(dim=-1)
    target = torch.where(novel, torch.where(free.any(dim=-1), first_free, oldest), best_i)
    ow = (novel | hit if cfg.exact_refresh_on_hit else novel) & keep
    w = torch.zeros(B, Me, dtype=st.k_buf.dtype)
    w.scatter_(1, target.view(B, 1), ow.to(w.dtype).view(B, 1))
    w4 = w[:, None, :, None]
    mk, mv = st.k_buf[:, :, sl, :], st.v_buf[:, :, sl, :]
    mk = mk + w4 * (k_e.unsqueeze(2) - mk)
    mv = mv + w4 * (v_e.unsqueeze(2) - mv)
    st.k_buf[:, :, sl, :] = mk
    st.v_buf[:, :, sl, :] = mv
    st.allowed[:, sl] = used | w.to(torch.bool)
    st._exact_v_norm = _unit(mv)
    cur = st.mem_last_exact.gather(1, target.view(B, 1)).squeeze(1)
    st.mem_last_exact.scatter_(1, target.view(B, 1),
                               torch.where(keep, torch.full_like(cur, pos_e), cur).view(B, 1))
    if st.metrics is not None:                               # memory_banks.py:315-323
        m = st.metrics
        if cfg.write_policy != "none":
            m["tokens_gated_out"] += int((~keep).sum())
        m["exact_hits"] += int(hit.sum())
        m["exact_inserts"] += int((novel & keep).sum())
        m["exact_overwrites"] += int(ow.sum())
        m["exact_fill_ratio"] = float(st.allowed[:, sl].any(dim=0).float().mean())
    # pressure: a novel, kept token that had to evict because no active slot was free (:333-337);
    # one step of growth per call whatever the number of rows under pressure
    try_expand(cfg, st, int(bool((novel & keep & ~free.any(dim=-1)).any())), 0)
    if st.trace is not None:
        st.trace.append(("exact_one", pos_e, target.clone(), ow.clone()))


def _summary_one(cfg, wts, st: OracleState, k_e, v_e, gate):
    """memory_banks.py:343-432 for one evicted token per row."""
    Ms = cfg.num_landmarks_summary
    if Ms == 0:
        return
    B, Hkv = k_e.shape[0], cfg.num_kv_heads
    As, lf = st.active_summary, cfg.lf_start
    sl = slice(cfg.window + cfg.num_landmarks_exact, cfg.Lbuf)
    used = st.allowed[:, sl]
    dt = st.k_buf.dtype
    keep = gate >= cfg.write_gate_threshold_summary if cfg.write_policy != "none" \
        else torch.ones(B, dtype=torch.bool)
    score = torch.einsum("bhd,bhmd->bhm", _unit(k_e[..., lf:]), st._sum_lf_k_norm).mean(dim=1)
    if As < Ms:
        score[:, As:] = NEG_FILL
    target = score.argmax(dim=-1)
    eta = torch.sigmoid(wts["summary_eta_logit"]).to(dt).view(1, Hkv, 1, 1).expand(B, Hkv, 1, 1)
    if cfg.write_policy != "none":
        eta = eta * gate.to(dt).view(B, 1, 1, 1)
    fresh = None
    if cfg.summary_overwrite_on_insert:
        fresh = ~used.gather(1, target.view(B, 1)).squeeze(1)
        eta = torch.where(fresh.view(B, 1, 1, 1), torch.ones_like(eta), eta)
    eta = eta * keep.to(dt).view(B, 1, 1, 1)
    w = torch.zeros(B, Ms, dtype=dt)
    w.scatter_(1, target.view(B, 1), 1.0)
    w4 = w[:, None, :, None]
    mk, mv = st.k_buf[:, :, sl, :], st.v_buf[:, :, sl, :]
    dk = torch.zeros_like(mk)
    dk[..., lf:] = k_e[..., lf:].unsqueeze(2) * cfg.energy_scale - mk[..., lf:]
    mk = mk + eta * w4 * dk
    mv = mv + eta * w4 * (v_e.unsqueeze(2) - mv)
    st.k_buf[:, :, sl, :] = mk
    st.v_buf[:, :, sl, :] = mv
    used_after = used | (keep.view(B, 1) & w.to(torch.bool))
    st.allowed[:, sl] = used_after
    st._sum_lf_k_norm = _unit(mk[..., lf:])
    # pressure: every active slot of every row is in use and something came in (:416-420)
    frustrated = int(bool(used_after[:, :As].all()) and bool(keep.any()))
    try_expand(cfg, st, 0, frustrated)
    if st.metrics is not None:                               # memory_banks.py:423-432
        m = st.metrics
        m["summary_updates"] += int(keep.sum())
        m["summary_frustrated"] += frustrated
        if cfg.summary_overwrite_on_insert:
            m["summary_inserts"] += int((fresh & keep).sum())
        m["summary_fill_ratio"] = float(used_after.any(dim=0).float().mean())
    if st.trace is not None:
        st.trace.append(("summary_one", target.clone(), keep.clone()))


def write_one(cfg, wts, st: OracleState, k_new, v_new, g_new):
    """Ring FIFO write of one token, routing the evicted one (memory_banks.py:183-224)."""
    W = cfg.window
    if st.recent_filled < W:
        i = st.recent_filled
        st.k_buf[:, :, i, :] = k_new[:, :, 0, :]
        st.v_buf[:, :, i, :] = v_new[:, :, 0, :]
        st.g_recent[:, i] = g_new[:, 0]
        st.allowed[:, i] = True
        st.recent_filled += 1
    else:
        ev = st.recent_idx
        k_e = st.k_buf[:, :, ev, :].clone()
        v_e = st.v_buf[:, :, ev, :].clone()
        g_e = st.g_recent[:, ev].clone()
        if st.metrics is not None:
            st.metrics["total_evictions"] += 1
        _exact_one(cfg, st, k_e, v_e, st.pos - W, g_e)
        _summary_one(cfg, wts, st, k_e, v_e, g_e)
        st.k_buf[:, :, ev, :] = k_new[:, :, 0, :]
        st.v_buf[:, :, ev, :] = v_new[:, :, 0, :]
        st.g_recent[:, ev] = g_new[:, 0]
        st.recent_idx = (ev + 1) % W
    st.pos += 1


def _project_kv_at(cfg, wts, x, pos):
    k = _heads(_linear(x, wts, "k_proj"), cfg.num_kv_heads, cfg.head_dim)
    v = _heads(_linear(x, wts, "v_proj"), cfg.num_kv_heads, cfg.head_dim)
    cos, sin = _rope_tables(cfg, x.shape[1], pos, x.dtype)
    return _rope(k, cos, sin, cfg.rope_interleaved), v


def step(cfg, wts, x, st: OracleState, *, attend=True, write_cache=True,
         include_current_in_attention=True):
    """One decode token (attention.py:516-547)."""
    qp = int(st.pos)
    if attend and include_current_in_attention and write_cache:
        k, v = _project_kv_at(cfg, wts, x, qp)
        write_one(cfg, wts, st, k, v, _gate(cfg, wts, x))
        return attend_step(cfg, wts, x, st, query_pos=qp)
    y = attend_step(cfg, wts, x, st, query_pos=qp) if attend else torch.zeros_like(x)
    if write_cache:
        k, v = _project_kv_at(cfg, wts, x, qp)
        write_one(cfg, wts, st, k, v, _gate(cfg, wts, x))
    return y


# --------------------------------------------------------------------------- #
# bank updates -- block of evicted tokens (prefill)
# --------------------------------------------------------------------------- #
def _exact_block(cfg, st: OracleState, k_c, v_c, pos_c, g_c, vhat):
    """memory_banks.py:570-742 (PyTorch branch :633-697)."""
    Me, W = cfg.num_landmarks_exact, cfg.window
    B, Hkv, T, Dh = k_c.shape
    Ae = st.active_exact
    sl = slice(W, W + Me)
    used = st.allowed[:, sl]
    last = st.mem_last_exact
    keep = g_c >= cfg.write_gate_threshold_exact if cfg.write_policy != "none" \
        else torch.ones(B, T, dtype=torch.bool)
    score = torch.matmul(vhat.reshape(B * Hkv, T, Dh),
                         st._exact_v_norm.reshape(B * Hkv, Me, Dh).transpose(1, 2)
                         ).view(B, Hkv, T, Me).mean(dim=1)
    if Ae < Me:
        score[:, :, Ae:] = NEG_FILL
    score.masked_fill_(~used[:, None, :], NEG_FILL)
    best, best_i = score.max(dim=-1)
    some_used = used.any(dim=-1)
    novel = (~some_used[:, None]) | (best < cfg.exact_novelty_threshold)
    hit = some_used[:, None] & (best >= cfg.exact_match_threshold)
    novel_keep = novel & keep
    key = last.clone()
    key[~used] = -I62
    if Ae < Me:
        key[:, Ae:] = -I62
    n_lru = min(T, Ae)
    _, victims = torch.topk(key, k=n_lru, dim=1, largest=False, sorted=True)
    rank = novel_keep.to(torch.int64).cumsum(dim=1) - 1
    capped = novel_keep & (rank < Ae)
    slot = victims.gather(1, rank.clamp(min=0, max=max(n_lru - 1, 0)))
    target = torch.where(capped, slot, best_i)
    touch = keep & (~novel | capped)
    ow = keep & (capped | hit) if cfg.exact_refresh_on_hit else capped
    # LRU stamps: per slot the largest position among touching candidates (:682-697)
    for b in range(B):
        new_last = last[b].clone()
        for m in range(Me):
            sel = touch[b] & (target[b] == m)
            if bool(sel.any()):
                new_last[m] = pos_c[b][sel].max()
        last[b] = new_last
    # values: mem + sum_c ow_c (x_c - old) accumulated in candidate order (:707-717)
    mk, mv = st.k_buf[:, :, sl, :], st.v_buf[:, :, sl, :]
    gi = target[:, None, :, None].expand(B, Hkv, T, Dh)
    owf = ow.to(mk.dtype).view(B, 1, T, 1)
    dk = owf * (k_c - mk.gather(2, gi))
    dv = owf * (v_c - mv.gather(2, gi))
    mk = mk + torch.zeros_like(mk).scatter_add_(2, gi, dk)
    mv = mv + torch.zeros_like(mv).scatter_add_(2, gi, dv)
    wrote = torch.zeros(B, Me, dtype=torch.bool)
    for b in range(B):
        wrote[b, target[b][ow[b]]] = True
    st.k_buf[:, :, sl, :] = mk
    st.v_buf[:, :, sl, :] = mv
    st.allowed[:, sl] = used | wrote
    cols = wrote.any(dim=0).nonzero(as_tuple=True)[0]
    st._exact_v_norm[:, :, cols, :] = _unit(mv[:, :, cols, :])
    # pressure: novel, kept candidates beyond the active capacity (memory_banks.py:758-760)
    frustrated = int((novel_keep & ~capped).sum())
    try_expand(cfg, st, frustrated, 0)
    if st.metrics is not None:                               # memory_banks.py:763-774 (PyTorch branch)
        m = st.metrics
        m["exact_overwrites"] += int(ow.sum())
        m["exact_frustrated"] += frustrated
        m["exact_fill_ratio"] = float(st.allowed[:, sl].any(dim=0).float().mean())
        m["exact_inserts"] += int(capped.sum())
        m["exact_hits"] += int((hit & keep).sum())
        if cfg.write_policy != "none":
            m["tokens_gated_out"] += int((~keep).sum())
    if st.trace is not None:
        st.trace.append(("exact_block", pos_c.clone(), target.clone(), ow.clone(), touch.clone()))


def _summary_block(cfg, wts, st: OracleState, k_c, v_c, w_c, khat):
    """memory_banks.py:853-932."""
    Ms = cfg.num_landmarks_summary
    B, Hkv, T, Dh = k_c.shape
    As, lf = st.active_summary, cfg.lf_start
    sl = slice(cfg.window + cfg.num_landmarks_exact, cfg.Lbuf)
    used = st.allowed[:, sl]
    dt = st.k_buf.dtype
    score = torch.matmul(khat.reshape(B * Hkv, T, Dh - lf),
                         st._sum_lf_k_norm.reshape(B * Hkv, Ms, Dh - lf).transpose(1, 2)
                         ).view(B, Hkv, T, Ms).mean(dim=1)
    if As < Ms:
        score[:, :, As:] = NEG_FILL
    target = score.argmax(dim=-1)
    w = w_c.to(dt)
    cnt = torch.zeros(B, Ms, dtype=dt).scatter_add_(1, target, w)
    gi = target[:, None, :, None].expand(B, Hkv, T, Dh)
    w4 = w.view(B, 1, T, 1)
    sk = torch.zeros(B, Hkv, Ms, Dh, dtype=dt).scatter_add_(2, gi, k_c * w4)
    sv = torch.zeros(B, Hkv, Ms, Dh, dtype=dt).scatter_add_(2, gi, v_c * w4)
    eta = torch.sigmoid(wts["summary_eta_logit"]).to(dt).view(1, Hkv, 1, 1)
    c4 = cnt.view(B, 1, Ms, 1)
    got = c4 > 0
    ak, av = sk / c4.clamp_min(1e-6), sv / c4.clamp_min(1e-6)
    if cfg.summary_overwrite_on_insert:
        eta_eff = torch.where((~used).view(B, 1, Ms, 1) & got, torch.ones_like(eta), eta)
    else:
        eta_eff = eta
    mk, mv = st.k_buf[:, :, sl, :], st.v_buf[:, :, sl, :]
    dk = torch.zeros_like(ak)
    dk[..., lf:] = ak[..., lf:] * cfg.energy_scale - mk[..., lf:]
    mk = torch.where(got, mk + eta_eff * dk, mk)
    mv = torch.where(got, mv + eta_eff * (av - mv), mv)
    st.k_buf[:, :, sl, :] = mk
    st.v_buf[:, :, sl, :] = mv
    used_after = used | (cnt > 0)
    n_fresh = int(((~used) & (cnt > 0)).sum())              # before `used` (a view of allowed) is overwritten
    st.allowed[:, sl] = used_after
    cols = (cnt > 0).any(dim=0).nonzero(as_tuple=True)[0]
    if cols.numel() > 0:
        st._sum_lf_k_norm[:, :, cols, :] = _unit(mk[:, :, cols, lf:])
    # pressure: all active slots of all rows in use and candidates arriving (memory_banks.py:934-940)
    frustrated = int(bool(used_after[:, :As].all()) and bool((cnt[:, :As] > 0).any()))
    try_expand(cfg, st, 0, frustrated)
    if st.metrics is not None:                               # memory_banks.py:943-950
        m = st.metrics
        m["summary_updates"] += int((cnt > 0).sum())
        m["summary_frustrated"] += frustrated
        if cfg.summary_overwrite_on_insert:
            m["summary_inserts"] += n_fresh
        m["summary_fill_ratio"] = float(used_after.any(dim=0).float().mean())
    if st.trace is not None:
        st.trace.append(("summary_block", target.clone(), w.clone()))


def eviction_plan(W: int, ring_fill: int, blk: int):
    """(evict_len, keep_len) when ``blk`` tokens join a ring holding ``ring_fill`` (memory_banks.py:462-464)."""
    total = ring_fill + blk
    keep_len = min(W, total)
    return total - keep_len, keep_len


def write_block(cfg, wts, st: OracleState, k_blk, v_blk, g_blk, pos0: int):
    """Ring + bank update with one block (memory_banks.py:438-564)."""
    W, Me, Ms = cfg.window, cfg.num_landmarks_exact, cfg.num_landmarks_summary
    B, Hkv, blk, Dh = k_blk.shape
    n = st.recent_filled
    if n < W:
        order = torch.arange(n)
    else:
        order = (torch.arange(W) + st.recent_idx) % W
    k_cat = torch.cat([st.k_buf[:, :, order, :], k_blk], dim=2)
    v_cat = torch.cat([st.v_buf[:, :, order, :], v_blk], dim=2)
    g_cat = torch.cat([st.g_recent[:, order], g_blk.float()], dim=1)
    n_ev, n_keep = eviction_plan(W, n, blk)
    first_pos = pos0 - n
    if n_ev > 0:
        if st.metrics is not None:
            st.metrics["total_evictions"] += n_ev               # memory_banks.py:468-469
        g_e = g_cat[:, :n_ev]
        do_e = Me > 0 and cfg.exact_candidates_per_block > 0
        do_s = Ms > 0 and cfg.summary_candidates_per_block > 0
        Te = min(cfg.exact_candidates_per_block, n_ev) if do_e else 0
        Ts = min(cfg.summary_candidates_per_block, n_ev) if do_s else 0
        T = max(Te, Ts)
        if T > 0:
            # one unsorted top-k; each bank takes a prefix of that list (:486-552)
            gv, gi = torch.topk(g_e, k=T, dim=1, largest=True, sorted=False)
            ix = gi.view(B, 1, T, 1).expand(B, Hkv, T, Dh)
            k_c, v_c = k_cat[:, :, :n_ev, :].gather(2, ix), v_cat[:, :, :n_ev, :].gather(2, ix)
            pos_c = gi + first_pos
            if do_e:
                _exact_block(cfg, st, k_c[:, :, :Te], v_c[:, :, :Te], pos_c[:, :Te], gv[:, :Te],
                             _unit(v_c[:, :, :Te]))
            if do_s:
                gs = gv[:, :Ts]
                w_c = gs.to(k_c.dtype)
                if cfg.write_policy != "none":
                    w_c = torch.where(gs >= cfg.write_gate_threshold_summary, w_c, torch.zeros_like(w_c))
                _summary_block(cfg, wts, st, k_c[:, :, :Ts], v_c[:, :, :Ts], w_c,
                               _unit(k_c[:, :, :Ts, cfg.lf_start:]))
    tot = n + blk
    st.k_buf[:, :, :W, :] = 0
    st.v_buf[:, :, :W, :] = 0
    st.g_recent.zero_()
    st.allowed[:, :W] = False
    if n_keep > 0:
        st.k_buf[:, :, :n_keep, :] = k_cat[:, :, tot - n_keep:tot, :]
        st.v_buf[:, :, :n_keep, :] = v_cat[:, :, tot - n_keep:tot, :]
        st.g_recent[:, :n_keep] = g_cat[:, tot - n_keep:tot]
        st.allowed[:, :n_keep] = True
    st.recent_filled = n_keep
    st.recent_idx = 0
    st.pos = pos0 + blk


def prefill_chunked(cfg, wts, x_seq, st: OracleState, *, block_size=256, write_cache=True):
    """Blockwise prefill (attention.py:567-728): each block attends [state before block | block]."""
    B, L, _ = x_seq.shape
    if L == 0:
        return x_seq[:, :0, :].clone()
    if block_size <= 0:
        raise ValueError("block_size must be positive")
    H, Hkv, Dh = cfg.num_heads, cfg.num_kv_heads, cfg.head_dim
    p0 = int(st.pos)
    cos, sin = _rope_tables(cfg, L, p0, x_seq.dtype)
    q_all = _rope(_heads(_linear(x_seq, wts, "q_proj"), H, Dh), cos, sin, cfg.rope_interleaved)
    k_all = _rope(_heads(_linear(x_seq, wts, "k_proj"), Hkv, Dh), cos, sin, cfg.rope_interleaved)
    v_all = _heads(_linear(x_seq, wts, "v_proj"), Hkv, Dh)
    g_all = _gate(cfg, wts, x_seq)
    lam_all = torch.sigmoid(_linear(x_seq, wts, "lambda_proj")).transpose(1, 2).unsqueeze(-1)
    outs = []
    t = 0
    while t < L:
        blk = min(block_size, L - t)
        sl = slice(t, t + blk)
        prefix_ok = st.allowed if cfg.mask_unused_memory else torch.ones(B, cfg.Lbuf, dtype=torch.bool)
        tri = torch.tril(torch.ones(blk, blk, dtype=torch.bool))
        keep = torch.cat([prefix_ok[:, None, None, :].expand(B, 1, blk, cfg.Lbuf),
                          tri[None, None].expand(B, 1, blk, blk)], dim=-1)
        kk = torch.cat([st.k_buf, k_all[:, :, sl]], dim=2)
        vv = torch.cat([st.v_buf, v_all[:, :, sl]], dim=2)
        outs.append(_diff_attend(cfg, wts, q_all[:, :, sl], lam_all[:, :, sl], kk, vv, keep))
        if write_cache:
            write_block(cfg, wts, st, k_all[:, :, sl], v_all[:, :, sl], g_all[:, sl], p0 + t)
        t += blk
    return torch.cat(outs, dim=1)


def cache_bytes(cfg: OracleConfig, batch_size: int, dtype: torch.dtype) -> int:
    """attention.py:734-751."""
    e = torch.tensor([], dtype=dtype).element_size()
    B, Hkv, Dh = batch_size, cfg.num_kv_heads, cfg.head_dim
    Me, Ms = cfg.num_landmarks_exact, cfg.num_landmarks_summary
    return (2 * B * Hkv * cfg.Lbuf * Dh * e + B * Hkv * Me * Dh * e
            + B * Hkv * Ms * (Dh - cfg.lf_start) * e + 4 * B * cfg.window + B * cfg.Lbuf + 8 * B * Me)


# --------------------------------------------------------------------------- #
# synthetic inputs shared by tests and bench (seeded Gaussian mixture)
# --------------------------------------------------------------------------- #
def mixture_inputs(B: int, L: int, D: int, *, centroids: int, sigma: float, seed: int,
                   repeat_prob: float = 0.0, repeat_period: int = 0,
                   dtype=torch.float32) -> torch.Tensor:
    """Hidden states from a seeded Gaussian mixture: centroids ~ N(0,1), token = centroid + sigma*N(0,1).

    ``repeat_prob`` replaces a token by an exact copy of a uniformly chosen earlier token of the
    same row with that probability; ``repeat_period`` > 0 does so for every period-th token.
    """
    g = torch.Generator().manual_seed(seed)
    cent = torch.randn(centroids, D, generator=g)
    ids = torch.randint(0, centroids, (B, L), generator=g)
    x = cent[ids] + sigma * torch.randn(B, L, D, generator=g)
    if repeat_prob > 0.0 or repeat_period > 0:
        u = torch.rand(B, L, generator=g)
        src = (torch.rand(B, L, generator=g) * torch.arange(L).clamp_min(1)[None, :]).long()
        for t in range(1, L):
            rep = (u[:, t] < repeat_prob) if repeat_prob > 0.0 else torch.zeros(B, dtype=torch.bool)
            if repeat_period > 0 and t % repeat_period == 0:
                rep = torch.ones(B, dtype=torch.bool)
            if bool(rep.any()):
                rows = rep.nonzero(as_tuple=True)[0]
                x[rows, t] = x[rows, src[rows, t]]
    return x.to(dtype)
