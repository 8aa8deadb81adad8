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
                           seed=spec["seed"], repeat_prob=spec.get("repeat_prob", 0.0), dtype=dtype)
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
