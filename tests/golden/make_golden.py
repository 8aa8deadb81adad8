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
from tests.scenarios import (ADAPTER_SCENARIOS, GEOMETRY_SCENARIOS, SCENARIOS, build_inputs,  # noqa: E402
                             fake_eve_attention, fake_llama_attention, randomize_weights)


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


def run_geometry(name, sc, RefCls, out_dir):
    """A benchmark-geometry scenario: ``layers`` independent upstream modules chained as h <- h + layer(h)
    (one layer: the fixture holds the layer output itself), bf16.  The oracle is run beside upstream on the same
    inputs and must stay within the bf16 tolerance of it; the fixture stores upstream's outputs (sub-sampled
    over tokens and features) and, per layer, the final ring scalars and slot occupancy."""
    dtype = getattr(torch, sc.get("dtype", "float32"))
    nl = int(sc.get("layers", 1))
    kw = dict(sc["model"])
    refs, wts, cfgs = [], [], []
    for i in range(nl):
        torch.manual_seed(sc["model_seed"] + i)
        ref = RefCls(**kw).eval()
        if sc.get("random_gate"):
            randomize_weights(ref, sc["model_seed"] + i)
        ref = ref.to(dtype)
        refs.append(ref)
        wts.append({k: v.detach().clone() for k, v in ref.state_dict().items()})
        cfg = orc.OracleConfig.from_module(ref)
        cfg.rope_base = float(kw.get("rope_base", 10_000.0))
        cfgs.append(cfg)
    B = sc["B"]
    x_pre, x_dec = build_inputs(sc, dtype)
    rsts, osts = [], []
    for i, ref in enumerate(refs):
        torch.manual_seed(sc["state_seed"] + i)
        rst = ref.init_state(batch_size=B, device=torch.device("cpu"), dtype=dtype)
        rsts.append(rst)
        osts.append(_to_oracle_state(rst))
    tol = 2e-5 if dtype == torch.float32 else 3e-2
    ys, snaps = [], []
    with torch.no_grad():
        for phase in sc["phases"]:
            if phase[0] == "prefill":
                _, lo, hi, blk = phase
                h_r = h_o = x_pre[:, lo:hi]
                for i in range(nl):
                    y, rsts[i] = refs[i].prefill_chunked(h_r, rsts[i], block_size=blk)
                    yo = orc.prefill_chunked(cfgs[i], wts[i], h_o, osts[i], block_size=blk)
                    h_r, h_o = (h_r + y, h_o + yo) if nl > 1 else (y, yo)
                y_r, y_o = h_r, h_o
            else:
                _, lo, hi = phase
                yr, yo_ = [], []
                for t in range(lo, hi):
                    h_r = h_o = x_dec[:, t:t + 1]
                    for i in range(nl):
                        y, rsts[i] = refs[i].step(h_r, rsts[i])
                        yo = orc.step(cfgs[i], wts[i], h_o, osts[i])
                        h_r, h_o = (h_r + y, h_o + yo) if nl > 1 else (y, yo)
                    yr.append(h_r)
                    yo_.append(h_o)
                y_r, y_o = torch.cat(yr, 1), torch.cat(yo_, 1)
            r = _rel(y_o, y_r)
            assert r < tol, f"{name}: oracle output deviates from upstream in {phase}: rel {r:.3e}"
            for rst, ost in zip(rsts, osts):
                assert (ost.recent_idx, ost.recent_filled, ost.pos) == (rst.recent_idx, rst.recent_filled, rst.pos)
            ys.append(y_r)
            snaps.append([_snapshot(rst) for rst in rsts])
            print(f"  {name} {phase}: oracle-vs-upstream rel={r:.2e} pos={rsts[0].pos} "
                  f"allowed={[int(r_.allowed.sum()) for r_ in rsts]}", flush=True)
    ts, fs = sc.get("y_stride", 4), sc.get("y_fstride", 1)
    for layer_snaps in snaps:
        for sn in layer_snaps:                      # keep the fixture small: occupancy and scalars only
            for key in ("k_bank", "v_bank", "g_recent"):
                sn.pop(key)
    fixture = {"scenario": name, "torch": torch.__version__, "weights_abs_sum": [_checksum(w) for w in wts],
               "y": [y[:, ::ts, ::fs].clone() for y in ys], "y_stride": ts, "y_fstride": fs, "snapshots": snaps,
               "cache_bytes": refs[0].cache_bytes(batch_size=B, dtype=dtype)}
    path = os.path.join(out_dir, f"{name}.pt")
    torch.save(fixture, path)
    print(f"  wrote {path} ({os.path.getsize(path) / 1024:.0f} KiB)")


def run_adapter(name, sc, ref_root, out_dir):
    """Upstream's Llama / Eve adapter (bounded=True) built from a seeded stand-in for the host model's attention
    module: one multi-token forward (-> prefill_chunked with the adapter's block size), single-token forwards
    (-> step), then get_state / set_state of a deep copy on a second adapter and more single-token forwards."""
    import copy
    from coda_gqa_l.eve_adapter import EveCoDAAdapter
    from coda_gqa_l.llama_adapter import LlamaCoDAAdapter
    dtype = getattr(torch, sc.get("dtype", "float32"))
    if sc["kind"] == "llama":
        src = fake_llama_attention(sc)
        make = lambda: LlamaCoDAAdapter.from_llama_attention(src, bounded=True, **sc["kwargs"])   # noqa: E731
    else:
        src = fake_eve_attention(sc)
        make = lambda: EveCoDAAdapter.from_eve_attention(src, bounded=True, **sc["kwargs"])       # noqa: E731
    import warnings
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        ad, ad2 = make().eval().to(dtype), make().eval().to(dtype)
    B, D = sc["B"], sc["hidden"]
    x = orc.mixture_inputs(B, sc["L"] + sc["Ldec"], D, centroids=24, sigma=0.4, seed=sc["input_seed"], dtype=dtype)
    call = (lambda a, t: a(t)[0]) if sc["kind"] == "llama" else (lambda a, t: a(t))
    with torch.no_grad():
        if sc.get("seeded_state"):
            torch.manual_seed(sc["state_seed"])
            ad.init_inference_state(B, torch.device("cpu"), dtype)
        y_pre = call(ad, x[:, :sc["L"]])
        half = sc["Ldec"] // 2
        y1 = torch.cat([call(ad, x[:, sc["L"] + t:sc["L"] + t + 1]) for t in range(half)], 1)
        ad2.set_state(copy.deepcopy(ad.get_state()))
        y2 = torch.cat([call(ad2, x[:, sc["L"] + t:sc["L"] + t + 1]) for t in range(half, sc["Ldec"])], 1)
    st = ad2.get_state()
    fixture = {"scenario": name, "torch": torch.__version__, "weights_abs_sum": _checksum(ad.coda.state_dict()),
               "y": [y_pre.clone(), y1.clone(), y2.clone()], "snapshot": _snapshot(st),
               "cache_bytes": ad.cache_bytes(batch_size=B, dtype=dtype)}
    path = os.path.join(out_dir, f"{name}.pt")
    torch.save(fixture, path)
    print(f"  {name}: pos={st.pos} allowed={int(st.allowed.sum())}; wrote {path} ({os.path.getsize(path) / 1024:.0f} KiB)")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=os.environ.get("CODA_GQA_L_REF"), help="root of the upstream checkout")
    ap.add_argument("--only", default=None, help="one scenario name")
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
    for name, sc in GEOMETRY_SCENARIOS.items():
        if args.only and name != args.only:
            continue
        print(name)
        run_geometry(name, sc, RefCls, HERE)
    for name, sc in ADAPTER_SCENARIOS.items():
        if args.only and name != args.only:
            continue
        print(name)
        run_adapter(name, sc, args.ref, HERE)


if __name__ == "__main__":
    main()
