"""Generate the golden fixtures under tests/golden/ from the upstream implementation.

Run where a checkout of the upstream project is available:

    python tests/golden/make_golden.py --ref <upstream checkout>      # or set CODA_GQA_L_REF

For every scenario in ``SCENARIOS`` the script
  1. builds the upstream ``CoDAGQALandmarkPerf2`` (imported unmodified, with its optional
     Triton / CUDA accelerators switched off so that the plain PyTorch path runs),
  2. runs prefill_chunked and step() on seeded inputs on the CPU,
  3. runs the CPU oracle (oracle/coda_oracle.py) on the same weights, inputs and initial
     state and checks that it reproduces the upstream result (integer/bool state bit-exact,
     floating-point state and outputs to 2e-5 relative in fp32),
  4. writes ``<scenario>.pt``: config, seeds, weight checksum, sub-sampled outputs, the final
     integer state and the routing trace.

The fixtures travel with the repository; the upstream project is not needed to use them.
"""

from __future__ import annotations

import argparse
import os
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from oracle import coda_oracle as orc  # noqa: E402
from tests.scenarios import SCENARIOS, build_inputs, randomize_weights  # noqa: E402


def _load_reference(ref_root: str):
    sys.path.insert(0, os.path.join(ref_root, "src"))
    import coda_gqa_l  # noqa: F401
    import coda_gqa_l.attention as A
    import coda_gqa_l.memory_banks as MB
    A._HAS_TRITON_FLASH = False
    A._HAS_FUSED_EPILOGUE = False
    MB._HAS_TRITON_ROUTE = False
    MB._HAS_TRITON_SUMMARY = False
    return A.CoDAGQALandmarkPerf2


def _checksum(sd) -> float:
    return float(sum(v.double().abs().sum() for v in sd.values()))


def _to_oracle_state(ref_state) -> orc.OracleState:
    return orc.OracleState(
        k_buf=ref_state.k_buf.clone(), v_buf=ref_state.v_buf.clone(),
        allowed=ref_state.allowed.clone(), g_recent=ref_state.g_recent.clone(),
        recent_idx=ref_state.recent_idx, recent_filled=ref_state.recent_filled,
        mem_last_exact=ref_state.mem_last_exact.clone(), pos=ref_state.pos,
        active_exact=ref_state.active_exact, active_summary=ref_state.active_summary,
        _exact_v_norm=None if ref_state._exact_v_norm is None else ref_state._exact_v_norm.clone(),
        _sum_lf_k_norm=None if ref_state._sum_lf_k_norm is None else ref_state._sum_lf_k_norm.clone(),
        metrics=None if getattr(ref_state, "metrics", None) is None else dict(ref_state.metrics),
        trace=[],
    )


def _rel(a, b):
    a, b = a.double(), b.double()
    return float((a - b).norm() / b.norm().clamp_min(1e-30))


def _snapshot(st):
    return {
        "allowed": st.allowed.clone(), "mem_last_exact": st.mem_last_exact.clone(),
        "g_recent": st.g_recent.clone(), "recent_idx": int(st.recent_idx),
        "recent_filled": int(st.recent_filled), "pos": int(st.pos),
        "k_abs_sum": float(st.k_buf.double().abs().sum()), "v_abs_sum": float(st.v_buf.double().abs().sum()),
        "k_bank": st.k_buf[:, :, -8:, :].clone(), "v_bank": st.v_buf[:, :, -8:, :].clone(),
        "active_exact": int(st.active_exact), "active_summary": int(st.active_summary),
        "metrics": None if getattr(st, "metrics", None) is None else dict(st.metrics),
    }


def run_scenario(name, sc, RefCls, out_dir):
    dtype = getattr(torch, sc.get("dtype", "float32"))
    kw = dict(sc["model"])
    torch.manual_seed(sc["model_seed"])
    ref = RefCls(**kw).eval()
    if sc.get("random_gate"):
        randomize_weights(ref, sc["model_seed"])
    ref = ref.to(dtype)
    wts = {k: v.detach().clone() for k, v in ref.state_dict().items()}
    cfg = orc.OracleConfig.from_module(ref)
    cfg.rope_base = float(kw.get("rope_base", 10_000.0))
    B = sc["B"]
    x_pre, x_dec = build_inputs(sc, dtype)

    torch.manual_seed(sc["state_seed"])
    rst = ref.init_state(batch_size=B, device=torch.device("cpu"), dtype=dtype)
    torch.manual_seed(sc["state_seed"])
    ost0 = orc.init_state(cfg, B, dtype)
    assert torch.equal(ost0.k_buf, rst.k_buf) and torch.equal(ost0.v_buf, rst.v_buf), "init_state RNG order"
    ost = _to_oracle_state(rst)

    tol = 2e-5 if dtype == torch.float32 else 3e-2
    ys_ref, ys_orc, snaps = [], [], []
    with torch.no_grad():
        for phase in sc["phases"]:
            kind = phase[0]
            if kind == "prefill":
                _, lo, hi, blk = phase
                y_r, rst = ref.prefill_chunked(x_pre[:, lo:hi], rst, block_size=blk)
                y_o = orc.prefill_chunked(cfg, wts, x_pre[:, lo:hi], ost, block_size=blk)
            elif kind == "decode":
                _, lo, hi = phase
                yr, yo = [], []
                for t in range(lo, hi):
                    y, rst = ref.step(x_dec[:, t:t + 1], rst)
                    yr.append(y)
                    yo.append(orc.step(cfg, wts, x_dec[:, t:t + 1], ost))
                y_r, y_o = torch.cat(yr, 1), torch.cat(yo, 1)
            else:
                raise ValueError(kind)
            r = _rel(y_o, y_r)
            assert r < tol, f"{name}: oracle output deviates from upstream in {phase}: rel {r:.3e}"
            # integer / bool state must agree exactly in fp32
            if dtype == torch.float32:
                assert torch.equal(ost.allowed, rst.allowed), f"{name}: allowed differs after {phase}"
                assert torch.equal(ost.mem_last_exact, rst.mem_last_exact), f"{name}: LRU stamps differ after {phase}"
            assert (ost.recent_idx, ost.recent_filled, ost.pos) == (rst.recent_idx, rst.recent_filled, rst.pos)
            assert (ost.active_exact, ost.active_summary) == (rst.active_exact, rst.active_summary), \
                f"{name}: active bank sizes differ after {phase}"
            if rst.metrics is not None:
                for key, val in rst.metrics.items():
                    ov = ost.metrics[key]
                    assert (abs(ov - val) < 1e-6) if isinstance(val, float) else (ov == val), \
                        f"{name}: metric {key} differs after {phase}: oracle {ov} upstream {val}"
            assert _rel(ost.k_buf, rst.k_buf) < tol and _rel(ost.v_buf, rst.v_buf) < tol, f"{name}: K/V differ"
            ys_ref.append(y_r)
            ys_orc.append(y_o)
            snaps.append(_snapshot(rst))
            print(f"  {name} {phase}: oracle-vs-upstream rel={r:.2e} "
                  f"allowed={int(rst.allowed.sum())} pos={rst.pos} ridx={rst.recent_idx}")

    stride = sc.get("y_stride", 4)
    trace = []
    for ev in ost.trace:
        trace.append(tuple(e.clone() if torch.is_tensor(e) else e for e in ev))
    # keep the fixture small: routing trace of the first 64 events only
    fixture = {
        "scenario": name, "torch": torch.__version__, "weights_abs_sum": _checksum(wts),
        "y": [y[:, ::stride].clone() for y in ys_ref], "y_stride": stride,
        "snapshots": snaps, "trace_head": trace[:64],
        "cache_bytes": ref.cache_bytes(batch_size=B, dtype=dtype),
    }
    assert fixture["cache_bytes"] == orc.cache_bytes(cfg, B, dtype)
    path = os.path.join(out_dir, f"{name}.pt")
    torch.save(fixture, path)
    print(f"  wrote {path} ({os.path.getsize(path) / 1024:.0f} KiB)")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=os.environ.get("CODA_GQA_L_REF"), help="root of the upstream checkout")
    ap.add_argument("--only", default=None)
    args = ap.parse_args()
    if not args.ref:
        ap.error("--ref (or CODA_GQA_L_REF) must point at the upstream checkout")
    RefCls = _load_reference(args.ref)
    torch.set_num_threads(max(1, os.cpu_count() or 1))
    for name, sc in SCENARIOS.items():
        if args.only and name != args.only:
            continue
        print(name)
        run_scenario(name, sc, RefCls, HERE)


if __name__ == "__main__":
    main()
