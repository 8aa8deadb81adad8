"""Drop-in attention adapters (Llama-family and Eve-2) over the bounded-cache module.

Interface and defaults follow upstream ``src/coda_gqa_l/llama_adapter.py:28-420`` and
``src/coda_gqa_l/eve_adapter.py:30-465``: ``bounded=True`` routes ``forward`` to
``CoDAGQALandmarkPerf2.step`` (one token) or ``prefill_chunked`` (several) on a state the adapter
owns; ``bounded=False`` builds the plain unbounded module.  The two adapters differ in their
defaults, in how source weights are laid out and in what ``forward`` returns, so the shared state
handling lives in one base class.
"""
from __future__ import annotations

import math
import warnings
from typing import List, Optional, Tuple

import torch
import torch.nn as nn

from .attention import CoDAGQALandmarkPerf2
from .baseline import CoDAGQA
from .state import CoDAGQALandmarkStatePerf2


class _AdapterBase(nn.Module):
    """State ownership and prefill/step routing shared by the adapters."""

    bounded: bool
    block_size: int
    coda: nn.Module

    def _build(self, *, embed_dim, num_heads, num_kv_heads, bounded, rope_theta, lambda_init_bias, theta_init,
               eps, head_norm_mode, rope_interleaved, window, num_landmarks_exact, num_landmarks_summary,
               block_size, coda_kwargs):
        self.bounded = bounded
        self.block_size = block_size
        common = dict(embed_dim=embed_dim, num_heads=num_heads, num_kv_heads=num_kv_heads, rope_base=rope_theta,
                      lambda_init_bias=lambda_init_bias, theta_init=theta_init, eps=eps,
                      head_norm_mode=head_norm_mode, rope_interleaved=rope_interleaved)
        if bounded:
            self.coda = CoDAGQALandmarkPerf2(window=window, num_landmarks_exact=num_landmarks_exact,
                                             num_landmarks_summary=num_landmarks_summary, **common, **coda_kwargs)
        else:
            self.coda = CoDAGQA(**common)
        self._state: Optional[CoDAGQALandmarkStatePerf2] = None

    def _forward_unbounded(self, x: torch.Tensor) -> torch.Tensor:
        out, _ = self.coda(x, is_causal=True)
        return out

    def _forward_bounded(self, x: torch.Tensor) -> torch.Tensor:
        """One token -> ``step``; several -> ``prefill_chunked(block_size)``; the state persists
        across calls (upstream llama_adapter.py:371-383).  Upstream's training branch (a fresh
        zero-initialised state per call, llama_adapter.py:352-369) is not available: the CUDA
        module is inference-only and raises in training mode, so call ``.eval()`` after swapping."""
        B, L, _ = x.shape
        if self._state is None:
            self._state = self.coda.init_state(batch_size=B, device=x.device, dtype=x.dtype)
        if L == 1:
            y, self._state = self.coda.step(x, self._state)
        else:
            y, self._state = self.coda.prefill_chunked(x, self._state, block_size=self.block_size)
        return y

    def init_inference_state(self, batch_size: int, device, dtype: torch.dtype) -> CoDAGQALandmarkStatePerf2:
        if not self.bounded:
            raise RuntimeError("init_inference_state() requires bounded=True")
        self._state = self.coda.init_state(batch_size=batch_size, device=device, dtype=dtype)
        return self._state

    def get_state(self) -> Optional[CoDAGQALandmarkStatePerf2]:
        return self._state

    def set_state(self, state: CoDAGQALandmarkStatePerf2) -> None:
        self._state = state

    def reset_state(self) -> None:
        self._state = None

    def cache_bytes(self, *, batch_size: int, dtype: torch.dtype) -> int:
        if not self.bounded:
            raise RuntimeError("cache_bytes() requires bounded=True")
        return self.coda.cache_bytes(batch_size=batch_size, dtype=dtype)


def _copy_linear(dst_owner: nn.Module, name: str, weight: torch.Tensor, bias: Optional[torch.Tensor]) -> None:
    """Copy a projection into ``dst_owner.<name>``, swapping in a biased Linear when the source has a bias."""
    lin: nn.Linear = getattr(dst_owner, name)
    if bias is not None and lin.bias is None:
        lin = nn.Linear(lin.in_features, lin.out_features, bias=True)
        setattr(dst_owner, name, lin)
    lin.weight.data.copy_(weight)
    if bias is not None:
        lin.bias.data.copy_(bias)


class LlamaCoDAAdapter(_AdapterBase):
    """Replacement for a HuggingFace Llama / Mistral / SmolLM ``self_attn`` module.

    Defaults differ from the bare module on purpose (upstream llama_adapter.py:55-64): half-split
    RoPE pairs and no head norm, which is what pre-trained Llama-family weights expect."""

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int, bounded: bool = False,
                 rope_theta: float = 10_000.0, lambda_init_bias: float = -6.0, theta_init: float = math.pi / 2,
                 eps: float = 1e-6, head_norm_mode: str = "identity", rope_interleaved: bool = False,
                 window: int = 256, num_landmarks_exact: int = 64, num_landmarks_summary: int = 64,
                 block_size: int = 1024, **coda_kwargs):
        super().__init__()
        self.hidden_size, self.num_heads, self.num_kv_heads, self.head_dim = hidden_size, num_heads, num_kv_heads, head_dim
        self._build(embed_dim=hidden_size, num_heads=num_heads, num_kv_heads=num_kv_heads, bounded=bounded,
                    rope_theta=rope_theta, lambda_init_bias=lambda_init_bias, theta_init=theta_init, eps=eps,
                    head_norm_mode=head_norm_mode, rope_interleaved=rope_interleaved, window=window,
                    num_landmarks_exact=num_landmarks_exact, num_landmarks_summary=num_landmarks_summary,
                    block_size=block_size, coda_kwargs=coda_kwargs)

    @classmethod
    def from_llama_attention(cls, llama_attn: nn.Module, bounded: bool = False, head_norm_mode: str = "identity",
                             rope_interleaved: bool = False, **coda_kwargs) -> "LlamaCoDAAdapter":
        """Build an adapter with the q/k/v/o weights (and biases, if any) of ``llama_attn``
        (upstream llama_adapter.py:116-261)."""
        hidden = llama_attn.q_proj.in_features
        n_q = getattr(llama_attn, "num_heads", None)
        n_kv = getattr(llama_attn, "num_key_value_heads", None)
        hd = getattr(llama_attn, "head_dim", None)
        if hd is None:
            q_out = llama_attn.q_proj.out_features
            if n_q is not None:
                hd = q_out // n_q
            else:
                hd = next((c for c in (128, 64, 96, 256) if q_out % c == 0), None)
                if hd is None:
                    raise ValueError(f"Cannot infer head_dim from q_proj shape {q_out}")
        if n_q is None:
            n_q = llama_attn.q_proj.out_features // hd
        if n_kv is None:
            n_kv = llama_attn.k_proj.out_features // hd
        config = getattr(llama_attn, "config", None)
        rope_theta = getattr(config, "rope_theta", 10_000.0) if config is not None else 10_000.0
        notes = []
        if rope_interleaved is not True:
            notes.append(f"rope_interleaved={rope_interleaved} (CoDAGQA default: True)")
        if head_norm_mode != "full":
            notes.append(f"head_norm_mode={head_norm_mode!r} (CoDAGQA default: 'full')")
        if notes:
            warnings.warn("LlamaCoDAAdapter.from_llama_attention: settings differ from CoDAGQA / "
                          "CoDAGQALandmarkPerf2 defaults -- " + "; ".join(notes) + ". Weights trained with the bare "
                          "module's defaults need rope_interleaved=True and head_norm_mode='full' here.",
                          UserWarning, stacklevel=2)
        ad = cls(hidden_size=hidden, num_heads=n_q, num_kv_heads=n_kv, head_dim=hd, bounded=bounded,
                 rope_theta=rope_theta, head_norm_mode=head_norm_mode, rope_interleaved=rope_interleaved, **coda_kwargs)
        for name in ("q_proj", "k_proj", "v_proj", "o_proj"):
            src = getattr(llama_attn, name)
            _copy_linear(ad.coda, name, src.weight.data, None if src.bias is None else src.bias.data)
        return ad

    @classmethod
    def swap_llama_layers(cls, model: nn.Module, bounded: bool = False, head_norm_mode: str = "identity",
                          rope_interleaved: bool = False, **coda_kwargs) -> List["LlamaCoDAAdapter"]:
        """Replace ``self_attn`` of every block in ``model.model.layers`` (upstream llama_adapter.py:263-302)."""
        made = []
        for block in model.model.layers:
            ad = cls.from_llama_attention(block.self_attn, bounded=bounded, head_norm_mode=head_norm_mode,
                                          rope_interleaved=rope_interleaved, **coda_kwargs)
            block.self_attn = ad
            made.append(ad)
        return made

    def forward(self, hidden_states: torch.Tensor, attention_mask: object = None, position_ids: object = None,
                past_key_value: object = None, output_attentions: bool = False, use_cache: bool = False,
                cache_position: object = None, position_embeddings: object = None, **kwargs) -> Tuple[torch.Tensor, ...]:
        """Llama attention signature; everything but ``hidden_states`` is accepted and ignored (the module
        keeps its own positions and cache).  Returns ``(output, past_key_value)`` (upstream :308-336)."""
        y = self._forward_bounded(hidden_states) if self.bounded else self._forward_unbounded(hidden_states)
        return y, past_key_value

    def extra_repr(self) -> str:
        return (f"hidden_size={self.hidden_size}, num_heads={self.num_heads}, num_kv_heads={self.num_kv_heads}, "
                f"head_dim={self.head_dim}, mode={'bounded' if self.bounded else 'unbounded'}")


class Qwen3CoDAAdapter(LlamaCoDAAdapter):
    """Replacement for a HuggingFace Qwen3 ``self_attn`` module (upstream qwen3_adapter.py:25-219).

    Qwen3 attention has the Llama layout (separate q/k/v/o projections, GQA, half-split RoPE pairs), so this is
    the Llama adapter with Qwen3's ``rope_theta`` of 1e6 as the default; weights map one to one."""

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int, bounded: bool = False,
                 rope_theta: float = 1_000_000.0, lambda_init_bias: float = -6.0, theta_init: float = math.pi / 2,
                 eps: float = 1e-6, head_norm_mode: str = "identity", rope_interleaved: bool = False,
                 window: int = 256, num_landmarks_exact: int = 64, num_landmarks_summary: int = 64,
                 block_size: int = 1024, **coda_kwargs):
        super().__init__(hidden_size=hidden_size, num_heads=num_heads, num_kv_heads=num_kv_heads, head_dim=head_dim,
                         bounded=bounded, rope_theta=rope_theta, lambda_init_bias=lambda_init_bias,
                         theta_init=theta_init, eps=eps, head_norm_mode=head_norm_mode,
                         rope_interleaved=rope_interleaved, window=window, num_landmarks_exact=num_landmarks_exact,
                         num_landmarks_summary=num_landmarks_summary, block_size=block_size, **coda_kwargs)

    @classmethod
    def from_qwen3_attention(cls, qwen3_attn: nn.Module, bounded: bool = False, head_norm_mode: str = "identity",
                             rope_interleaved: bool = False, **coda_kwargs) -> "Qwen3CoDAAdapter":
        """Build an adapter with the q/k/v/o weights (and biases, if any) of ``qwen3_attn``; head counts come
        from the module's attributes or, failing that, from the projection shapes; ``rope_theta`` from its
        ``config`` when present, else 1e6 (upstream qwen3_adapter.py:79-180)."""
        hidden = qwen3_attn.q_proj.in_features
        n_q = getattr(qwen3_attn, "num_heads", None)
        n_kv = getattr(qwen3_attn, "num_key_value_heads", None)
        hd = getattr(qwen3_attn, "head_dim", None)
        if hd is None:
            q_out = qwen3_attn.q_proj.out_features
            hd = q_out // n_q if n_q is not None else next((c for c in (128, 64, 96, 256) if q_out % c == 0), None)
            if hd is None:
                raise ValueError(f"Cannot infer head_dim from q_proj shape {q_out}")
        if n_q is None:
            n_q = qwen3_attn.q_proj.out_features // hd
        if n_kv is None:
            n_kv = qwen3_attn.k_proj.out_features // hd
        config = getattr(qwen3_attn, "config", None)
        rope_theta = getattr(config, "rope_theta", 1_000_000.0) if config is not None else 1_000_000.0
        ad = cls(hidden_size=hidden, num_heads=n_q, num_kv_heads=n_kv, head_dim=hd, bounded=bounded,
                 rope_theta=rope_theta, head_norm_mode=head_norm_mode, rope_interleaved=rope_interleaved, **coda_kwargs)
        for name in ("q_proj", "k_proj", "v_proj", "o_proj"):
            src = getattr(qwen3_attn, name)
            _copy_linear(ad.coda, name, src.weight.data, None if src.bias is None else src.bias.data)
        return ad

    @classmethod
    def swap_qwen3_layers(cls, model: nn.Module, bounded: bool = False, head_norm_mode: str = "identity",
                          rope_interleaved: bool = False, **coda_kwargs) -> List["Qwen3CoDAAdapter"]:
        """Replace ``self_attn`` of every block in ``model.model.layers`` (upstream qwen3_adapter.py:182-219)."""
        made = []
        for block in model.model.layers:
            ad = cls.from_qwen3_attention(block.self_attn, bounded=bounded, head_norm_mode=head_norm_mode,
                                          rope_interleaved=rope_interleaved, **coda_kwargs)
            block.self_attn = ad
            made.append(ad)
        return made


class EveCoDAAdapter(_AdapterBase):
    """Replacement for Eve-2's ``CausalSelfAttention`` (multi-head, fused QKV projection with biases);
    ``forward(x, freqs_cis=None)`` returns the output tensor only (upstream eve_adapter.py:308-328)."""

    def __init__(self, n_embd: int, n_head: int, head_dim: int, bounded: bool = False, rope_theta: float = 10_000.0,
                 lambda_init_bias: float = -6.0, theta_init: float = math.pi / 2, eps: float = 1e-6,
                 head_norm_mode: str = "full", rope_interleaved: bool = True, window: int = 256,
                 num_landmarks_exact: int = 64, num_landmarks_summary: int = 64, block_size: int = 1024, **coda_kwargs):
        super().__init__()
        self.n_embd, self.n_head, self.head_dim = n_embd, n_head, head_dim
        self._build(embed_dim=n_embd, num_heads=n_head, num_kv_heads=n_head, bounded=bounded, rope_theta=rope_theta,
                    lambda_init_bias=lambda_init_bias, theta_init=theta_init, eps=eps, head_norm_mode=head_norm_mode,
                    rope_interleaved=rope_interleaved, window=window, num_landmarks_exact=num_landmarks_exact,
                    num_landmarks_summary=num_landmarks_summary, block_size=block_size, coda_kwargs=coda_kwargs)

    def load_eve_weights(self, *, c_attn_weight: torch.Tensor, c_attn_bias: Optional[torch.Tensor] = None,
                         c_proj_weight: torch.Tensor, c_proj_bias: Optional[torch.Tensor] = None) -> None:
        """Split a fused ``(3*n_embd, n_embd)`` QKV weight (and bias) into the q/k/v projections and copy
        the output projection (upstream eve_adapter.py:251-302)."""
        n = self.n_embd
        for i, name in enumerate(("q_proj", "k_proj", "v_proj")):
            _copy_linear(self.coda, name, c_attn_weight[i * n:(i + 1) * n, :],
                         None if c_attn_bias is None else c_attn_bias[i * n:(i + 1) * n])
        _copy_linear(self.coda, "o_proj", c_proj_weight, c_proj_bias)

    @classmethod
    def from_eve_attention(cls, eve_attn: nn.Module, bounded: bool = False, head_norm_mode: str = "full",
                           rope_interleaved: bool = True, **coda_kwargs) -> "EveCoDAAdapter":
        """Adapter carrying the weights of an Eve ``CausalSelfAttention`` (upstream eve_adapter.py:146-245)."""
        ad = cls(n_embd=eve_attn.n_embd, n_head=eve_attn.n_head, head_dim=eve_attn.head_dim, bounded=bounded,
                 head_norm_mode=head_norm_mode, rope_interleaved=rope_interleaved, **coda_kwargs)
        ca, cp = eve_attn.c_attn, eve_attn.c_proj
        ad.load_eve_weights(c_attn_weight=ca.weight.data, c_attn_bias=None if ca.bias is None else ca.bias.data,
                            c_proj_weight=cp.weight.data, c_proj_bias=None if cp.bias is None else cp.bias.data)
        return ad

    def forward(self, x: torch.Tensor, freqs_cis: object = None) -> torch.Tensor:
        return self._forward_bounded(x) if self.bounded else self._forward_unbounded(x)

    def extra_repr(self) -> str:
        s = f"n_embd={self.n_embd}, n_head={self.n_head}, head_dim={self.head_dim}, mode={'bounded' if self.bounded else 'unbounded'}"
        return s + (f", block_size={self.block_size}" if self.bounded else "")
