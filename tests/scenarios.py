"""Seeded parity scenarios shared by the golden-fixture generator and the tests.

Each scenario names a layer configuration (keyword arguments of ``CoDAGQALandmarkPerf2``),
the seeds for weights / initial state / inputs, the input distribution and a list of phases:
``("prefill", lo, hi, block_size)`` feeds tokens ``lo:hi`` of the prefill stream through
``prefill_chunked``; ``("decode", lo, hi)`` feeds tokens ``lo:hi`` of the decode stream
through ``step``.
"""

from __future__ import annotations

import torch

from oracle.coda_oracle import mixture_inputs

_SMALL = dict(embed_dim=128, num_heads=4, num_kv_heads=2, window=32,
              num_landmarks_exact=16, num_landmarks_summary=16)

SCENARIOS = {
    # BASELINE config 1: the CPU reference run (fp32, B=1, 2048 prefill in blocks of 256, 1000 steps)
    "c1": dict(
        model=dict(embed_dim=512, num_heads=8, num_kv_heads=2, window=256,
                   num_landmarks_exact=64, num_landmarks_summary=64),
        model_seed=1234, state_seed=99, B=1,
        inputs=dict(kind="mixture", centroids=256, sigma=0.3, seed=7, L=2048, Ldec=1000),
        phases=[("prefill", 0, 2048, 256), ("decode", 0, 1000)], y_stride=16,
    ),
    # small generic shape (Dh=32) with ragged blocks, B=2
    "small_b2": dict(
        model=dict(_SMALL), model_seed=42, state_seed=99, B=2,
        inputs=dict(kind="mixture", centroids=24, sigma=0.3, seed=7, L=200, Ldec=80),
        phases=[("prefill", 0, 200, 48), ("decode", 0, 80)],
    ),
    # white-noise inputs: every evicted token is novel, LRU eviction runs constantly
    "small_randn": dict(
        model=dict(_SMALL), model_seed=42, state_seed=99, B=2,
        inputs=dict(kind="randn", seed=7, L=160, Ldec=100),
        phases=[("prefill", 0, 160, 32), ("decode", 0, 100)],
    ),
    # trained-like gate: non-constant write gates, so selection order depends on values
    "gate_varied": dict(
        model=dict(_SMALL), model_seed=5, state_seed=11, B=2, random_gate=True,
        inputs=dict(kind="mixture", centroids=24, sigma=0.3, seed=3, L=300, Ldec=60),
        phases=[("prefill", 0, 300, 64), ("decode", 0, 60)],
    ),
    # Llama conventions: half-split RoPE, identity head norm, rope base 1e6, Dh=64, G=4
    "llama_like": dict(
        model=dict(embed_dim=256, num_heads=4, num_kv_heads=1, window=48, num_landmarks_exact=8,
                   num_landmarks_summary=8, rope_base=1e6, head_norm_mode="identity",
                   rope_interleaved=False),
        model_seed=8, state_seed=2, B=2,
        inputs=dict(kind="mixture", centroids=32, sigma=0.5, seed=21, L=256, Ldec=70),
        phases=[("prefill", 0, 256, 64), ("decode", 0, 70)],
    ),
    # dynamic bank expansion + metrics: banks start at 4 active slots and grow under pressure (white noise:
    # every evicted token is novel); counters collected
    "expand_metrics": dict(
        model=dict(_SMALL, min_landmarks_exact=4, min_landmarks_summary=4, expansion_t_max=2000,
                   collect_metrics=True),
        model_seed=42, state_seed=99, B=2,
        inputs=dict(kind="randn", seed=7, L=160, Ldec=100),
        phases=[("prefill", 0, 160, 32), ("decode", 0, 100)],
    ),
    # metrics on fixed-size banks, clustered inputs (hits, gated-out tokens, summary inserts)
    "metrics_only": dict(
        model=dict(_SMALL, collect_metrics=True), model_seed=5, state_seed=11, B=2, random_gate=True,
        inputs=dict(kind="mixture", centroids=24, sigma=0.3, seed=3, L=200, Ldec=60),
        phases=[("prefill", 0, 200, 48), ("decode", 0, 60)],
    ),
    # the same on a Dh=64 layer (the per-head cluster cache-write kernel) with a trained-like gate: some evicted
    # tokens are gated out, banks start at 2 / 3 active slots, three states
    "expand_dh64": dict(
        model=dict(embed_dim=256, num_heads=4, num_kv_heads=2, window=24, num_landmarks_exact=12,
                   num_landmarks_summary=10, min_landmarks_exact=2, min_landmarks_summary=3, expansion_t_max=400,
                   collect_metrics=True),
        model_seed=6, state_seed=12, B=3, random_gate=True,
        inputs=dict(kind="mixture", centroids=48, sigma=0.6, seed=13, L=96, Ldec=120),
        phases=[("prefill", 0, 96, 40), ("decode", 0, 120)],
    ),
    # block larger than the window (adapter default block 1024): evicted tokens come from the block itself
    "big_block": dict(
        model=dict(_SMALL), model_seed=42, state_seed=99, B=2,
        inputs=dict(kind="mixture", centroids=40, sigma=0.3, seed=9, L=520, Ldec=10),
        phases=[("prefill", 0, 520, 256), ("decode", 0, 10)],
    ),
    # prefill, decode (ring pointer moves), prefill again, decode again
    "interleaved": dict(
        model=dict(_SMALL), model_seed=42, state_seed=99, B=2,
        inputs=dict(kind="mixture", centroids=24, sigma=0.3, seed=13, L=200, Ldec=60),
        phases=[("prefill", 0, 70, 32), ("decode", 0, 45), ("prefill", 70, 200, 40), ("decode", 45, 60)],
    ),
    # exact repeats of earlier tokens: exact-bank hits and LRU refresh (BASELINE config 3 input style)
    "repeats": dict(
        model=dict(_SMALL, exact_refresh_on_hit=True), model_seed=42, state_seed=99, B=2,
        inputs=dict(kind="mixture", centroids=64, sigma=0.3, seed=17, L=320, Ldec=64, repeat_prob=0.10),
        phases=[("prefill", 0, 320, 64), ("decode", 0, 64)],
    ),
    # more candidates per block than any fixed staging size: one summary slot takes all 160 summary candidates of a
    # block, the exact bank takes up to 150 with refresh-on-hit and many exact repeats (several overwrites per slot)
    "many_candidates": dict(
        model=dict(_SMALL, num_landmarks_summary=1, summary_candidates_per_block=160, exact_candidates_per_block=150,
                   exact_refresh_on_hit=True),
        model_seed=42, state_seed=99, B=2, random_gate=True,
        inputs=dict(kind="mixture", centroids=12, sigma=0.3, seed=19, L=720, Ldec=40, repeat_prob=0.5),
        phases=[("prefill", 0, 720, 240), ("decode", 0, 40)],
    ),
    "policy_none": dict(
        model=dict(_SMALL, write_policy="none", summary_overwrite_on_insert=False),
        model_seed=42, state_seed=99, B=2,
        inputs=dict(kind="mixture", centroids=24, sigma=0.3, seed=7, L=160, Ldec=50),
        phases=[("prefill", 0, 160, 32), ("decode", 0, 50)],
    ),
    "no_mask_zero_init": dict(
        model=dict(_SMALL, mask_unused_memory=False, mem_init="zeros"),
        model_seed=42, state_seed=99, B=2,
        inputs=dict(kind="mixture", centroids=24, sigma=0.3, seed=7, L=100, Ldec=50),
        phases=[("prefill", 0, 100, 32), ("decode", 0, 50)],
    ),
    "exact_only": dict(
        model=dict(_SMALL, num_landmarks_summary=0), model_seed=42, state_seed=99, B=2,
        inputs=dict(kind="mixture", centroids=24, sigma=0.3, seed=7, L=160, Ldec=50),
        phases=[("prefill", 0, 160, 64), ("decode", 0, 50)],
    ),
    "summary_only": dict(
        model=dict(_SMALL, num_landmarks_exact=0), model_seed=42, state_seed=99, B=2,
        inputs=dict(kind="mixture", centroids=24, sigma=0.3, seed=7, L=160, Ldec=50),
        phases=[("prefill", 0, 160, 64), ("decode", 0, 50)],
    ),
    "window_only": dict(
        model=dict(_SMALL, num_landmarks_exact=0, num_landmarks_summary=0),
        model_seed=42, state_seed=99, B=2,
        inputs=dict(kind="randn", seed=7, L=100, Ldec=40),
        phases=[("prefill", 0, 100, 32), ("decode", 0, 40)],
    ),
    "window_1": dict(
        model=dict(_SMALL, window=1, num_landmarks_exact=4, num_landmarks_summary=4),
        model_seed=42, state_seed=99, B=1,
        inputs=dict(kind="mixture", centroids=8, sigma=0.3, seed=7, L=40, Ldec=20),
        phases=[("prefill", 0, 40, 16), ("decode", 0, 20)],
    ),
    # decode from an empty state: ring fill phase, then lowest-index-first bank fill
    "decode_only": dict(
        model=dict(_SMALL, window=4, num_landmarks_exact=8, num_landmarks_summary=8),
        model_seed=42, state_seed=99, B=2,
        inputs=dict(kind="randn", seed=7, L=0, Ldec=40),
        phases=[("decode", 0, 40)],
    ),
    # bf16 end to end (tolerance 2e-2 relative, state integers not required to match)
    "small_bf16": dict(
        model=dict(embed_dim=256, num_heads=4, num_kv_heads=2, window=64,
                   num_landmarks_exact=16, num_landmarks_summary=16),
        model_seed=42, state_seed=99, B=2, dtype="bfloat16",
        inputs=dict(kind="mixture", centroids=24, sigma=0.3, seed=7, L=256, Ldec=40),
        phases=[("prefill", 0, 256, 64), ("decode", 0, 40)],
    ),
}


# Per-layer geometries of the benchmark configurations (bf16, a few states): the shapes whose tuned kernel
# instantiations (head_dim 128 decode / prefill, batched routing) the benchmark times.  Each runs a prefill long
# enough to evict into both banks and then at least 2*W decode steps, so the ring wraps.  ``layers`` > 1 chains
# independent layers (weights seeded model_seed + i) as h <- h + layer_i(h); the fixture then holds the final h.
_C4 = dict(embed_dim=4096, num_heads=32, num_kv_heads=8, window=256, num_landmarks_exact=64,
           num_landmarks_summary=64, rope_base=1e6, head_norm_mode="identity", rope_interleaved=False)
GEOMETRY_SCENARIOS = {
    # config 4 (Mistral-7B attention shape): Dh 128, G 4, 384 slots, half-split RoPE base 1e6, block 128
    "c4_layer": dict(
        model=dict(_C4), model_seed=31, state_seed=32, B=2, dtype="bfloat16",
        inputs=dict(kind="mixture", centroids=64, sigma=0.5, seed=33, L=640, Ldec=512),
        phases=[("prefill", 0, 640, 128), ("decode", 0, 512)], y_stride=8, y_fstride=4,
    ),
    # the same geometry with the RMSNorm epilogue and non-default gate / lambda / theta / eta, two chained layers
    "c4_fullnorm_stack2": dict(
        model=dict(_C4, head_norm_mode="full"), layers=2, random_gate=True,
        model_seed=41, state_seed=42, B=2, dtype="bfloat16",
        inputs=dict(kind="mixture", centroids=64, sigma=0.5, seed=43, L=512, Ldec=520),
        phases=[("prefill", 0, 512, 128), ("decode", 0, 520)], y_stride=8, y_fstride=4,
    ),
    # config 2 (SmolLM2-135M attention shape): Dh 64, G 3, 192 slots, block 128, two chained layers
    "c2_stack2": dict(
        model=dict(embed_dim=576, num_heads=9, num_kv_heads=3, window=128, num_landmarks_exact=32,
                   num_landmarks_summary=32, head_norm_mode="identity", rope_interleaved=False),
        layers=2, model_seed=51, state_seed=52, B=4, dtype="bfloat16",
        inputs=dict(kind="mixture", centroids=64, sigma=0.3, seed=53, L=384, Ldec=256),
        phases=[("prefill", 0, 384, 128), ("decode", 0, 256)], y_stride=4,
    ),
    # config 3: the medium module defaults (interleaved RoPE, full head norm) in bf16, block 256, 10 % exact repeats
    "c3_layer": dict(
        model=dict(embed_dim=512, num_heads=8, num_kv_heads=2, window=256, num_landmarks_exact=64,
                   num_landmarks_summary=64),
        model_seed=61, state_seed=62, B=3, dtype="bfloat16",
        inputs=dict(kind="mixture", centroids=64, sigma=0.3, seed=63, L=768, Ldec=512, repeat_prob=0.10),
        phases=[("prefill", 0, 768, 256), ("decode", 0, 512)], y_stride=4,
    ),
    # config 5 (70B shape): Dh 128, G 8, 768 slots, block 256, every 20th token an exact repeat
    "c5_layer": dict(
        model=dict(embed_dim=8192, num_heads=64, num_kv_heads=8, window=512, num_landmarks_exact=128,
                   num_landmarks_summary=128, rope_base=1e6, head_norm_mode="identity", rope_interleaved=False),
        model_seed=71, state_seed=72, B=2, dtype="bfloat16",
        inputs=dict(kind="mixture", centroids=128, sigma=0.5, seed=73, L=1280, Ldec=1024, repeat_period=20),
        phases=[("prefill", 0, 1280, 256), ("decode", 0, 1024)], y_stride=16, y_fstride=8,
    ),
}


def build_inputs(sc, dtype):
    """(x_prefill [B,L,D], x_decode [B,Ldec,D]) for a scenario, on the CPU."""
    spec = sc["inputs"]
    B, D = sc["B"], sc["model"]["embed_dim"]
    L, Ld = spec["L"], spec["Ldec"]
    if spec["kind"] == "randn":
        g = torch.Generator().manual_seed(spec["seed"])
        x = torch.randn(B, L + Ld, D, generator=g).to(dtype)
    else:
        x = mixture_inputs(B, L + Ld, D, centroids=spec["centroids"], sigma=spec["sigma"],
                           seed=spec["seed"], repeat_prob=spec.get("repeat_prob", 0.0),
                           repeat_period=spec.get("repeat_period", 0), dtype=dtype)
    return x[:, :L].contiguous(), x[:, L:].contiguous()


def randomize_weights(module, seed: int) -> None:
    """Give the write gate, lambda gate, noise angles, eta and head-norm weight non-default values."""
    g = torch.Generator().manual_seed(seed + 1000)
    with torch.no_grad():
        module.write_proj.weight.copy_(torch.randn(module.write_proj.weight.shape, generator=g) * 0.08)
        module.write_proj.bias.fill_(-1.8)
        module.lambda_proj.weight.copy_(torch.randn(module.lambda_proj.weight.shape, generator=g) * 0.05)
        module.lambda_proj.bias.fill_(-1.0)
        module.theta.copy_(torch.rand(module.theta.shape, generator=g) * 3.0)
        module.summary_eta_logit.copy_(torch.randn(module.summary_eta_logit.shape, generator=g))
        if hasattr(module.head_norm, "weight"):
            module.head_norm.weight.copy_(1.0 + 0.2 * torch.randn(module.head_norm.weight.shape, generator=g))


# Adapter scenarios: a seeded stand-in for the host model's attention module (the attributes and projection
# layers the adapters' ``from_*_attention`` constructors read), the adapter keyword arguments, and a token stream.
ADAPTER_SCENARIOS = {
    # Llama adapter defaults (half-split RoPE, identity head norm), rope_theta from the module's config, banks
    # zero-initialised so that the state the adapter creates inside forward() is the same on every device
    "adapter_llama": dict(
        kind="llama", hidden=256, heads=4, kv_heads=2, head_dim=64, rope_theta=5e5, bias=False, src_seed=81,
        kwargs=dict(window=48, num_landmarks_exact=16, num_landmarks_summary=16, block_size=64, mem_init="zeros"),
        B=2, L=300, Ldec=40, input_seed=82,
    ),
    "adapter_llama_bf16": dict(
        kind="llama", hidden=512, heads=4, kv_heads=2, head_dim=128, rope_theta=1e6, bias=True, src_seed=83,
        kwargs=dict(window=64, num_landmarks_exact=16, num_landmarks_summary=16, block_size=128, mem_init="zeros"),
        B=2, L=300, Ldec=40, input_seed=84, dtype="bfloat16",
    ),
    # Eve adapter: multi-head, fused QKV projection and output projection with biases, interleaved RoPE, full head
    # norm; the state is created explicitly from a CPU seed (random-normal banks) and handed over with set_state
    "adapter_eve": dict(
        kind="eve", hidden=192, heads=3, head_dim=64, bias=True, src_seed=85,
        kwargs=dict(window=40, num_landmarks_exact=12, num_landmarks_summary=12, block_size=96),
        B=2, L=250, Ldec=40, input_seed=86, seeded_state=True, state_seed=87,
    ),
    "adapter_eve_bf16": dict(
        kind="eve", hidden=256, heads=4, head_dim=64, bias=True, src_seed=88,
        kwargs=dict(window=64, num_landmarks_exact=16, num_landmarks_summary=16, block_size=96),
        B=2, L=250, Ldec=40, input_seed=89, seeded_state=True, state_seed=90, dtype="bfloat16",
    ),
}


def fake_llama_attention(sc):
    """A module with the attributes ``LlamaCoDAAdapter.from_llama_attention`` reads from a HuggingFace attention
    block: q/k/v/o projections, head counts, head_dim and ``config.rope_theta``."""
    import types
    import torch.nn as nn
    torch.manual_seed(sc["src_seed"])
    m = nn.Module()
    D, H, Hkv, Dh = sc["hidden"], sc["heads"], sc["kv_heads"], sc["head_dim"]
    m.q_proj = nn.Linear(D, H * Dh, bias=sc["bias"])
    m.k_proj = nn.Linear(D, Hkv * Dh, bias=sc["bias"])
    m.v_proj = nn.Linear(D, Hkv * Dh, bias=sc["bias"])
    m.o_proj = nn.Linear(H * Dh, D, bias=False)
    m.num_heads, m.num_key_value_heads, m.head_dim = H, Hkv, Dh
    m.config = types.SimpleNamespace(rope_theta=sc["rope_theta"])
    return m


def fake_eve_attention(sc):
    """A module with the attributes ``EveCoDAAdapter.from_eve_attention`` reads from Eve-2's attention block:
    fused ``c_attn`` (3*n_embd x n_embd), ``c_proj``, ``n_head``, ``n_embd``, ``head_dim``."""
    import torch.nn as nn
    torch.manual_seed(sc["src_seed"])
    m = nn.Module()
    D = sc["hidden"]
    m.c_attn = nn.Linear(D, 3 * D, bias=sc["bias"])
    m.c_proj = nn.Linear(D, D, bias=sc["bias"])
    m.n_head, m.n_embd, m.head_dim = sc["heads"], D, sc["head_dim"]
    return m
