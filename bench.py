"""Benchmark of the bounded-cache differential-attention path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (BASELINE config 4, the one the headline metric is quoted on): Mistral-7B attention shape, 32
stacked layers, embed 4096, 32 query heads / 8 KV heads, head_dim 128, RoPE base 1e6, W=256 / Me=64 / Ms=64,
bf16, random-init weights, 32 independent sequence states per GPU (256 over 8 GPUs, weak scaling), seeded
4096-centroid Gaussian-mixture hidden states (sigma 0.5).  A "step" is one decode token for every state
through all layers.  Prints ONE JSON line (rank 0).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for _p in (ROOT, os.path.join(ROOT, "coda-gqa-l_b200")):
    if _p not in sys.path:
        sys.path.insert(0, _p)

import torch  # noqa: E402

WORKLOADS = {
    # name: (layers, D, H, Hkv, W, Me, Ms, states per GPU, prefill block, mixture centroids, sigma, rope base)
    "c4_mistral7b": dict(layers=32, D=4096, H=32, Hkv=8, W=256, Me=64, Ms=64, B=32, block=128, K=4096, sigma=0.5,
                         rope_base=1e6, head_norm_mode="identity", rope_interleaved=False),
    "c2_smollm135m": dict(layers=30, D=576, H=9, Hkv=3, W=128, Me=32, Ms=32, B=512, block=128, K=1024, sigma=0.3,
                          rope_base=1e4, head_norm_mode="identity", rope_interleaved=False),
    "c3_medium": dict(layers=1, D=512, H=8, Hkv=2, W=256, Me=64, Ms=64, B=8, block=256, K=512, sigma=0.3,
                      rope_base=1e4, head_norm_mode="full", rope_interleaved=True),
}


def decode_bytes_per_state_layer(w) -> int:
    """Algorithmic HBM bytes of one decode token for one state in one layer: K+V arena read once per KV head,
    q in / out, new K/V row + one exact-slot and one summary-slot K/V write, lambda, allowed mask."""
    Dh = w["D"] // w["H"]
    Lbuf, e = w["W"] + w["Me"] + w["Ms"], 2
    return 2 * w["Hkv"] * Lbuf * Dh * e + 2 * w["H"] * Dh * e + 6 * w["Hkv"] * Dh * e + 4 * w["H"] + Lbuf


def prefill_flops_per_state_layer_block(w) -> float:
    """Causal-aware attention FLOPs of one block: 2 streams x (QK^T + PV) over Lbuf prefix slots + the block."""
    Dh, blk = w["D"] // w["H"], w["block"]
    Lbuf = w["W"] + w["Me"] + w["Ms"]
    return 8.0 * w["H"] * blk * Dh * (Lbuf + (blk + 1) / 2)


def layer_kwargs(w):
    return dict(embed_dim=w["D"], num_heads=w["H"], num_kv_heads=w["Hkv"], window=w["W"],
                num_landmarks_exact=w["Me"], num_landmarks_summary=w["Ms"], rope_base=w["rope_base"],
                head_norm_mode=w["head_norm_mode"], rope_interleaved=w["rope_interleaved"])


def mixture_on_device(B, L, D, centroids, sigma, seed, device, dtype):
    g = torch.Generator(device=device).manual_seed(seed)
    cent = torch.randn(centroids, D, generator=g, device=device)
    ids = torch.randint(0, centroids, (B, L), generator=g, device=device)
    return (cent[ids] + sigma * torch.randn(B, L, D, generator=g, device=device)).to(dtype)


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples of one GPU while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self._stop, self._t = index, [], threading.Event(), None

    def _run(self):
        while not self._stop.is_set():
            try:
                out = subprocess.run(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}",
                                      "--format=csv,noheader,nounits"], capture_output=True, text=True, timeout=5).stdout
                parts = [p.strip() for p in out.strip().split(",")]
                if len(parts) >= 6:
                    self.rows.append(parts)
            except Exception:
                pass
            self._stop.wait(0.1)

    def __enter__(self):
        self._t = threading.Thread(target=self._run, daemon=True)
        self._t.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        self._t.join(timeout=6)

    def summary(self):
        if not self.rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        mhz = sorted(float(r[0]) for r in self.rows)
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[2 + i].lower().startswith("active") for r in self.rows)]
        return {"sm_mhz": mhz[len(mhz) // 2], "sm_max_mhz": float(self.rows[0][1]), "reasons": reasons,
                "samples": len(self.rows)}


def cpu_decode_baseline(w, budget_s: float, threads: int, seed: int = 0):
    """The CPU oracle (restatement of the reference's PyTorch path) timed on the host: a bounded sample of the
    same workload -- `B` states, a couple of layers, a few decode steps after a short prefill -- scaled to
    tokens/s of the full stack (tokens/s = B*steps / (t * layers_full / layers_sampled))."""
    from oracle import coda_oracle as orc
    from coda_gqa_l_b200 import CoDAGQALandmarkPerf2
    torch.set_num_threads(threads)
    dtype = torch.bfloat16
    B = min(w["B"], 8)
    n_layers = 1
    torch.manual_seed(seed)
    mod = CoDAGQALandmarkPerf2(**layer_kwargs(w)).eval().to(dtype)
    wts = {k: v.detach() for k, v in mod.state_dict().items()}
    cfg = orc.OracleConfig.from_module(mod)
    torch.manual_seed(seed + 1)
    st = orc.init_state(cfg, B, dtype)
    x = orc.mixture_inputs(B, w["W"] + w["block"] + 64, w["D"], centroids=min(w["K"], 256), sigma=w["sigma"],
                           seed=seed + 2, dtype=dtype)
    with torch.no_grad():
        orc.prefill_chunked(cfg, wts, x[:, :w["W"] + w["block"]], st, block_size=w["block"])   # ring full, banks live
        t0 = time.perf_counter()
        orc.step(cfg, wts, x[:, -64:-63], st)                                                 # warm-up + probe
        probe = time.perf_counter() - t0
        steps = int(max(2, min(62, budget_s / max(probe, 1e-3))))
        t0 = time.perf_counter()
        for t in range(steps):
            orc.step(cfg, wts, x[:, -63 + t:-62 + t], st)
        dt = time.perf_counter() - t0
    tok_s = B * steps / (dt * w["layers"] / n_layers)
    return {"value": tok_s, "unit": "tokens/s", "cores": threads, "kind": "port",
            "sample": f"CPU oracle, bf16, {B} states x {n_layers} of {w['layers']} layers x {steps} decode steps after a "
                      f"{w['W'] + w['block']}-token prefill; scaled by layers"}


def workload_config(args, w, world):
    """The `config` object of the JSON line: the same for this arm and for the reference arm."""
    P = max(args.prefill_tokens, w["W"] + w["block"])
    P = (P + w["block"] - 1) // w["block"] * w["block"]
    D = w["D"]
    return {"workload": args.workload, "layers": w["layers"], "states_per_gpu": w["B"], "global_states": world * w["B"],
            "embed": D, "heads": w["H"], "kv_heads": w["Hkv"], "head_dim": D // w["H"], "window": w["W"],
            "exact": w["Me"], "summary": w["Ms"], "sharding": f"batch x{world}, no data-path collective",
            "launch": "eager" if args.eager else "cuda-graph replay of one stack step",
            "l2": "inputs larger than L2: each step streams every layer's state and weights (GBs) once",
            "warm_state": f"{2 * P}-token prefill in blocks of {w['block']}"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c4_mistral7b", choices=sorted(WORKLOADS))
    ap.add_argument("--layers", type=int, default=None, help="override the layer count (profiling small cases)")
    ap.add_argument("--states", type=int, default=None, help="override states per GPU (profiling small cases)")
    ap.add_argument("--prefill-tokens", type=int, default=512)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--eager", action="store_true", help="time eager launches instead of CUDA-graph replay")
    ap.add_argument("--no-split-routing", action="store_true",
                    help="route the evicted tokens inside each layer's chain instead of on a second graph branch")
    args = ap.parse_args()
    w = dict(WORKLOADS[args.workload])
    if args.layers:
        w["layers"] = args.layers
    if args.states:
        w["B"] = args.states
    K, Wm = max(1, args.steps), max(3, args.warmup)

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    cores = os.cpu_count() or 1

    if args.impl == "reference":
        # The reference's own (CPU, PyTorch) implementation of the path; rank 0 alone runs it.
        if rank != 0:
            return
        cb = cpu_decode_baseline(w, budget_s=20.0 * K / 64, threads=cores)
        print(json.dumps({
            "impl": "reference", "metric": "decode tokens/s, 7B-shape bounded attention stack", "value": cb["value"],
            "unit": "tokens/s", "n_gpus": args.gpus, "steps": K, "warmup": Wm, "ms_per_step": 1e3 * w["B"] / cb["value"],
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": workload_config(args, w, max(1, args.gpus)),
            "cpu_baseline": cb,
            "e2e": {"value": cb["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))
        return

    import torch.distributed as dist
    from coda_gqa_l_b200 import CoDAGQALandmarkPerf2, CoDAStack
    from coda_gqa_l_b200.sharding import max_over_ranks
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    dtype = torch.bfloat16

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    # ---- model + state (random-init weights of the named architecture, created on the device) ----
    layers = []
    for i in range(w["layers"]):
        torch.manual_seed(1000 + i)
        with torch.device(dev):
            layers.append(CoDAGQALandmarkPerf2(**layer_kwargs(w)).eval().to(dtype))
    stack = CoDAStack(layers)
    stack.split_routing = not args.no_split_routing
    B, D = w["B"], w["D"]
    torch.manual_seed(7 + rank)
    states = stack.init_states(batch_size=B, device=dev, dtype=dtype)
    P = max(args.prefill_tokens, w["W"] + w["block"])
    P = (P + w["block"] - 1) // w["block"] * w["block"]
    x_pre = mixture_on_device(B, 2 * P, D, w["K"], w["sigma"], 11 + rank, dev, dtype)
    x_dec = mixture_on_device(B, 2 * (K + Wm) + 8, D, w["K"], w["sigma"], 13 + rank, dev, dtype)
    x_dec_host = x_dec.cpu().pin_memory()

    # ---- prefill (brings every ring to steady state); timed as a secondary figure ----
    stack.prefill(x_pre[:, :P], states, block_size=w["block"])                  # warm-up chunk: fills every ring
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for l in stack.layers:
        l.kernel_timers = []
    e0.record()
    stack.prefill(x_pre[:, P:], states, block_size=w["block"])                  # timed chunk: same shapes, steady state
    e1.record()
    barrier()
    prefill_ms = max_over_ranks(e0.elapsed_time(e1), dev)
    pre_tokens = B * P
    att_ms = [a.elapsed_time(b) for l in stack.layers for (_, a, b) in l.kernel_timers]
    pre_kernel_ms = sum(att_ms) / max(1, len(att_ms))
    for l in stack.layers:
        l.kernel_timers = None
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except Exception:
        pass
    hbm_peak = float(peaks.get("hbm_gbs", 6650.0))
    tc_peak = float(peaks.get("bf16_tflops", 1590.0))
    peak_src = "measured" if peaks else "fallback"
    pre_tf = prefill_flops_per_state_layer_block(w) * B / (pre_kernel_ms * 1e-3) / 1e12

    # ---- decode: device-resident inputs (value) ----
    step_fn = stack.step if args.eager else stack.step_graph
    t = 0
    for _ in range(Wm):
        step_fn(x_dec[:, t:t + 1], states); t += 1
    barrier()
    with ClockSampler(local) as clocks:
        e0.record()
        for _ in range(K):
            step_fn(x_dec[:, t:t + 1], states); t += 1
        e1.record()
        barrier()
    ms = max_over_ranks(e0.elapsed_time(e1), dev)
    tok_s = world * B * K / (ms * 1e-3)

    # ---- decode end to end: host buffers in, host result out, every step ----
    out_host = torch.empty((B, 1, D), dtype=dtype).pin_memory()
    x_stage = torch.empty((B, 1, D), dtype=dtype, device=dev)
    for _ in range(3):
        x_stage.copy_(x_dec_host[:, t:t + 1], non_blocking=True)
        out_host.copy_(step_fn(x_stage, states), non_blocking=True); t += 1
    barrier()
    e0.record()
    for _ in range(K):
        x_stage.copy_(x_dec_host[:, t:t + 1], non_blocking=True)
        out_host.copy_(step_fn(x_stage, states), non_blocking=True)
        torch.cuda.current_stream(dev).synchronize(); t += 1
    e1.record()
    barrier()
    ms_e2e = max_over_ranks(e0.elapsed_time(e1), dev)
    e2e_tok_s = world * B * K / (ms_e2e * 1e-3)

    # ---- roofline of the dominant kernel (decode attention) ----
    # One CUDA graph holding one attention launch per layer (each on its own layer's state, so consecutive
    # launches never find their planes in L2 once layers * bytes_per_launch exceeds it), replayed and timed
    # with events on the launching stream; per-launch time = elapsed / launches.
    from coda_gqa_l_b200._lib import RingPos
    roof_stream = torch.cuda.Stream(dev)
    dt = dtype
    H_, Dh_ = w["H"], D // w["H"]
    q_fix = torch.randn(B, H_ * Dh_, device=dev, dtype=dt)
    lam_fix = torch.randn(B, H_, device=dev, dtype=dt)
    outs = [torch.empty(B, 1, H_ * Dh_, device=dev, dtype=dt) for _ in stack.layers]
    reps = max(1, -(-8 // len(stack.layers)))            # layer sweeps per replay (>= 8 launches per graph)
    def launch_all(prepare=False):
        for _ in range(1 if prepare else reps):
            for l, st, o in zip(stack.layers, states, outs):
                cfg = l._cfg(B, dt, st)
                if prepare:          # decode records (prepared queries + mask) of this layer's state, once
                    rp = RingPos(int(st.pos), int(st.recent_idx), int(st.recent_filled), None)
                    l.decode_attend_launch(cfg, st, rp, 1, q_fix, lam_fix, o)
                else:                # the attention kernel alone
                    l.decode_attend_prepared_launch(cfg, st, o)
    roof_stream.wait_stream(torch.cuda.current_stream(dev))
    with torch.cuda.stream(roof_stream):
        launch_all(prepare=True)
        launch_all()
        roof_graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(roof_graph, stream=roof_stream):
            launch_all()
        for _ in range(3):
            roof_graph.replay()
        r0, r1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        nrep = 10
        r0.record(roof_stream)
        for _ in range(nrep):
            roof_graph.replay()
        r1.record(roof_stream)
    roof_stream.synchronize()
    kern_ms = r0.elapsed_time(r1) / (nrep * reps * len(stack.layers))
    for l in stack.layers:
        if l.device_status() != 0:
            raise RuntimeError("decode attention reported an expired device-side wait")
    bytes_launch = decode_bytes_per_state_layer(w) * B
    achieved = bytes_launch / (kern_ms * 1e-3) / 1e9

    line = {
        "metric": "decode tokens/s, 7B-shape bounded attention stack", "value": tok_s, "unit": "tokens/s",
        "n_gpus": world, "steps": K, "warmup": Wm, "ms_per_step": ms / K, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": workload_config(args, w, world),
        "e2e": {"value": e2e_tok_s, "unit": "tokens/s", "h2d_bytes_per_step": B * D * 2, "d2h_bytes_per_step": B * D * 2,
                "ms_per_step": ms_e2e / K},
        # this repository's kernels inside the timed region: per layer the fused cache write and the decode
        # attention, plus the step-counter kernel of the captured graph (the two GEMMs per layer are library calls)
        "gpu_launches": K * ((2 if args.eager or args.no_split_routing else 1) * w["layers"] + (0 if args.eager else (1 if args.no_split_routing else 3))),
        "clocks": clocks.summary(),
        "roofline": {"kernel": "decode_attend_kernel (coda_b200_decode_attend_prepared)", "timing": "graph of back-to-back launches over all layers' states, CUDA events", "bound": "hbm", "achieved": achieved,
                     "peak": hbm_peak, "unit": "GB/s", "frac": achieved / hbm_peak, "of": peak_src,
                     "frac_of_nominal_8000": achieved / 8000.0,
                     # dram__bytes_read.sum + dram__bytes_write.sum of one launch of this kernel at this workload
                     # (ncu capture summarised under profiles/), scaled by the states processed
                     "traffic": int(round(51044000 * B / 32)) if args.workload == "c4_mistral7b" else None, "kernel_ms": kern_ms,
                     "bytes_per_launch": bytes_launch},
        "prefill": {"tokens_per_s": world * pre_tokens / (prefill_ms * 1e-3), "tokens": pre_tokens, "ms": prefill_ms,
                    "attention_kernel_ms_per_block": pre_kernel_ms, "attention_tflops": pre_tf,
                    "tensor_frac": pre_tf / tc_peak, "tensor_peak": tc_peak, "of": peak_src},
    }
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_decode_baseline(w, budget_s=15.0, threads=cores)
    # Every rank finishes its own (unsynchronised) roofline section before any rank tears the process group down:
    # a communicator destroyed while a peer still runs kernels took that peer's kernels down with it.
    barrier()
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
