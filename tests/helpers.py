"""Shared test plumbing: scenario construction, state conversion and comparison metrics."""
from __future__ import annotations

import os

import torch

from oracle import coda_oracle as orc
from tests.scenarios import SCENARIOS, build_inputs, randomize_weights

GOLDEN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")

# Output tolerances of the parity contract: relative L2 error of the layer output against the
# reference implementation on the same seeded inputs.
TOL_F32 = 1e-4
TOL_BF16 = 2e-2


def rel_err(a: torch.Tensor, b: torch.Tensor) -> float:
    a, b = a.detach().double().cpu(), b.detach().double().cpu()
    return float((a - b).norm() / b.norm().clamp_min(1e-30))


def build_module(sc, dtype):
    """The B200 module with the scenario's seeded default weights, still on the CPU."""
    from coda_gqa_l_b200 import CoDAGQALandmarkPerf2
    torch.manual_seed(sc["model_seed"])
    mod = CoDAGQALandmarkPerf2(**sc["model"]).eval()
    if sc.get("random_gate"):
        randomize_weights(mod, sc["model_seed"])
    return mod.to(dtype)


def weights_of(mod):
    return {k: v.detach().clone().cpu() for k, v in mod.state_dict().items()}


def weights_checksum(wts) -> float:
    return float(sum(v.double().abs().sum() for v in wts.values()))


def oracle_state_from(st) -> orc.OracleState:
    c = lambda t: None if t is None else t.detach().clone().cpu()  # noqa: E731
    return orc.OracleState(
        k_buf=c(st.k_buf), v_buf=c(st.v_buf), allowed=c(st.allowed), g_recent=c(st.g_recent),
        recent_idx=int(st.recent_idx), recent_filled=int(st.recent_filled), mem_last_exact=c(st.mem_last_exact),
        pos=int(st.pos), active_exact=int(st.active_exact), active_summary=int(st.active_summary),
        _exact_v_norm=c(st._exact_v_norm), _sum_lf_k_norm=c(st._sum_lf_k_norm),
        metrics=None if getattr(st, "metrics", None) is None else dict(st.metrics), trace=[])


def load_golden(name):
    return torch.load(os.path.join(GOLDEN_DIR, f"{name}.pt"), weights_only=False)


__all__ = ["SCENARIOS", "build_inputs", "build_module", "weights_of", "weights_checksum", "oracle_state_from",
           "load_golden", "rel_err", "TOL_F32", "TOL_BF16", "orc"]
