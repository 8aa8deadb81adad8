"""Benchmark of the bounded-cache differential-attention path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference|reference-gpu] [--workload NAME]

Default workload (BASELINE config 4, the one the headline metric is quoted on): Mistral-7B attention shape, 32
stacked layers, embed 4096, 32 query heads / 8 KV heads, head_dim 128, RoPE base 1e6, W=256 / Me=64 / Ms=64,
bf16, random-init weights, 32 independent sequence states per GPU (256 over 8 GPUs, weak scaling), seeded
4096-centroid Gaussian-mixture hidden states (sigma 0.5).  A "step" is one decode token for every state
through all layers.  Prints ONE JSON line (rank 0).

``--impl reference`` times the reference's own PyTorch implementation of the same step on the host cores (the
unmodified upstream package from oracle/_ref when present, else this repository's CPU restatement of it);
``--impl reference-gpu`` runs that same upstream eager code on cuda:0 as a second reference line.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import re
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

WORKLOADS = {
    # layers, embed, heads, KV heads, window / exact / summary slots, states per GPU, prefill block, mixture centroids, sigma
    "c4_mistral7b": dict(layers=32, D=4096, H=32, Hkv=8, W=256, Me=64, Ms=64, B=32, block=128, K=4096, sigma=0.5,
                         rope_base=1e6, head_norm_mode="identity", rope_interleaved=False),
    "c2_smollm135m": dict(layers=30, D=576, H=9, Hkv=3, W=128, Me=32, Ms=32, B=512, block=128, K=1024, sigma=0.3,
                          rope_base=1e4, head_norm_mode="identity", rope_interleaved=False),
    "c3_medium": dict(layers=1, D=512, H=8, Hkv=2, W=256, Me=64, Ms=64, B=8, block=256, K=512, sigma=0.3,
                      rope_base=1e4, head_norm_mode="full", rope_interleaved=True),
    "c5_70b": dict(layers=80, D=8192, H=64, Hkv=8, W=512, Me=128, Ms=128, B=64, block=256, K=8192, sigma=0.5,
                   rope_base=1e6, head_norm_mode="identity", rope_interleaved=False),
}
METRIC = "decode tokens/s, bounded attention stack"


def decode_bytes_per_state_layer(w) -> int:
    """Algorithmic HBM bytes of one decode token for one state in one layer: K+V arena read once per KV head,
    q in / out, new K/V row + one exact-slot and one summary-slot K/V write, lambda, allowed mask."""
    Dh = w["D"] // w["H"]
    Lbuf, e = w["W"] + w["Me"] + w["Ms"], 2
    return 2 * w["Hkv"] * Lbuf * Dh * e + 2 * w["H"] * Dh * e + 6 * w["Hkv"] * Dh * e + 4 * w["H"] + Lbuf


def weight_bytes_per_layer(w) -> int:
    """bf16 bytes of the projection weights one decode step streams per layer: [q|k|v|lambda|gate] and o_proj."""
    Dh = w["D"] // w["H"]
    return 2 * (w["D"] * (w["H"] * Dh + 2 * w["Hkv"] * Dh + w["H"] + 1) + w["H"] * Dh * w["D"])


def prefill_flops_per_state_layer_block(w) -> float:
    """Causal-aware attention FLOPs of one block: 2 streams x (QK^T + PV) over Lbuf prefix slots + the block."""
    Dh, blk = w["D"] // w["H"], w["block"]
    Lbuf = w["W"] + w["Me"] + w["Ms"]
    return 8.0 * w["H"] * blk * Dh * (Lbuf + (blk + 1) / 2)


def layer_kwargs(w):
    return dict(embed_dim=w["D"], num_heads=w["H"], num_kv_heads=w["Hkv"], window=w["W"],
                num_landmarks_exact=w["Me"], num_landmarks_summary=w["Ms"], rope_base=w["rope_base"],
                head_norm_mode=w["head_norm_mode"], rope_interleaved=w["rope_interleaved"])


def mixture(B, L, D, centroids, sigma, seed, device, dtype):
    g = torch.Generator(device=device).manual_seed(seed)
    cent = torch.randn(centroids, D, generator=g, device=device)
    ids = torch.randint(0, centroids, (B, L), generator=g, device=device)
    return (cent[ids] + sigma * torch.randn(B, L, D, generator=g, device=device)).to(dtype)


def profiled_traffic(workload: str, variant: str):
    """(DRAM bytes per launch, states of that capture) of the decode attention kernel from the ncu summaries kept
    beside this file: a line ``bench-traffic: <workload> <variant> dram_bytes_per_launch=<N> states=<B>``."""
    folder = os.path.join(ROOT, "profiles")
    pat = re.compile(r"bench-traffic:\s*(\S+)\s+(\S+)\s+dram_bytes_per_launch=(\d+)\s+states=(\d+)")
    try:
        for name in sorted(os.listdir(folder)):
            if name.endswith((".md", ".txt")):
                for m in pat.finditer(open(os.path.join(folder, name)).read()):
                    if m.group(1) == workload and m.group(2) == variant:
                        return int(m.group(3)), int(m.group(4))
    except OSError:
        pass
    return None


class ClockSampler:
    """Clock / throttle-reason samples of one GPU while the timed region runs (read-only queries).

    Samples through NVML (every 20 ms) when the binding is importable and the device can be found by its UUID or
    index; otherwise through one ``nvidia-smi`` query per sample (each takes a few hundred ms)."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self._stop, self._t = index, [], threading.Event(), None
        self._nvml = self._handle = None
        try:
            import pynvml
            pynvml.nvmlInit()
            try:
                uuid = str(torch.cuda.get_device_properties(index).uuid)
                self._handle = pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + uuid) if not uuid.startswith("GPU-") else uuid)
            except Exception:
                self._handle = pynvml.nvmlDeviceGetHandleByIndex(index)
            self._nvml = pynvml
        except Exception:
            self._nvml = self._handle = None

    def _sample_nvml(self):
        n, h = self._nvml, self._handle
        sm = n.nvmlDeviceGetClockInfo(h, n.NVML_CLOCK_SM)
        mx = n.nvmlDeviceGetMaxClockInfo(h, n.NVML_CLOCK_SM)
        get = getattr(n, "nvmlDeviceGetCurrentClocksEventReasons", None) or n.nvmlDeviceGetCurrentClocksThrottleReasons
        r = int(get(h))
        flag = lambda bit: "Active" if r & bit else "Not Active"
        return [str(sm), str(mx), flag(n.nvmlClocksThrottleReasonHwSlowdown), flag(n.nvmlClocksThrottleReasonHwThermalSlowdown),
                flag(n.nvmlClocksThrottleReasonSwThermalSlowdown), flag(n.nvmlClocksThrottleReasonSwPowerCap)]

    def _run(self):
        while not self._stop.is_set():
            try:
                if self._nvml is not None:
                    self.rows.append(self._sample_nvml())
                else:
                    out = subprocess.run(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits"], capture_output=True, text=True, timeout=5).stdout
                    parts = [p.strip() for p in out.strip().split(",")]
                    if len(parts) >= 6:
                        self.rows.append(parts)
            except Exception:
                if self._nvml is not None:
                    self._nvml = None                       # fall back to nvidia-smi for the rest of the region
            self._stop.wait(0.02 if self._nvml is not None else 0.1)

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
                "samples": len(self.rows), "source": "nvml" if self._nvml is not None else "nvidia-smi"}


# ------------------------------------------------------------------------------------------------ reference arm
def reference_decode(w, steps: int, warmup: int, device: str, threads: int, sample_layers: int = None,
                     budget_s: float = None, region_s: float = 90.0):
    """The reference's PyTorch implementation of the decode step, timed on ``device``.

    Runs ``sample_layers`` independent layers (chained h <- h + layer(h), default seeded weights) of the workload's
    shape at the workload's states-per-GPU, each warmed by a prefill that fills its ring, for ``steps`` decode tokens
    after ``warmup`` untimed ones.  ``sample_layers=None``: as many layers of the stack as keep warm-up + timed steps
    within ``region_s`` seconds (all of them when they fit), judged from one layer's probed step time.  Tokens/s of
    the full stack = states / (seconds per sampled step x layers / sample_layers): every layer of the stack has the
    same shape and cost.  With ``budget_s`` the step count is cut instead so that the timed region stays near that
    many seconds.  Nothing of this repository's package is imported."""
    from oracle import build_ref
    torch.set_num_threads(threads)
    dtype = torch.bfloat16
    dev = torch.device(device)
    B, D = w["B"], w["D"]
    kind = "reference" if build_ref.available() else "port"
    layers, states = [], []
    if kind == "reference":
        Ref = build_ref.load()

        def add_layer(i):
            torch.manual_seed(1000 + i)
            m = Ref(**layer_kwargs(w)).eval().to(dtype).to(dev)
            torch.manual_seed(7 + i)
            layers.append(m)
            states.append(m.init_state(batch_size=B, device=dev, dtype=dtype))

        def prefill_layer(i, x):
            _, states[i] = layers[i].prefill_chunked(x, states[i], block_size=w["block"], return_outputs=False)

        def step(x):
            for i, m in enumerate(layers):
                y, states[i] = m.step(x, states[i])
                x = x + y
            return x
    else:
        import math
        from oracle import coda_oracle as orc
        from oracle.coda_oracle import OracleConfig

        def add_layer(i):
            # the module's default initialisation (upstream attention.py:189-234) restated with plain tensors
            torch.manual_seed(1000 + i)
            H, Hkv, Dh = w["H"], w["Hkv"], D // w["H"]
            lin = lambda o, n: (torch.rand(o, n) * 2 - 1) / math.sqrt(n)          # noqa: E731
            sd = {"q_proj.weight": lin(H * Dh, D), "k_proj.weight": lin(Hkv * Dh, D), "v_proj.weight": lin(Hkv * Dh, D),
                  "theta": torch.full((H, Dh // 2), math.pi / 2), "lambda_proj.weight": lin(H, D),
                  "lambda_proj.bias": torch.full((H,), -6.0), "write_proj.weight": torch.zeros(1, D),
                  "write_proj.bias": torch.full((1,), -2.0), "summary_eta_logit": torch.full((Hkv,), -3.0),
                  "o_proj.weight": lin(D, H * Dh)}
            if w["head_norm_mode"] == "full":
                sd["head_norm.weight"] = torch.ones(Dh)
            cfg = OracleConfig(embed_dim=D, num_heads=H, num_kv_heads=Hkv, window=w["W"], num_landmarks_exact=w["Me"],
                               num_landmarks_summary=w["Ms"], rope_base=w["rope_base"], head_norm_mode=w["head_norm_mode"],
                               rope_interleaved=w["rope_interleaved"], angle_dtype=dtype)
            layers.append((cfg, {k: v.to(dtype) for k, v in sd.items()}))
            torch.manual_seed(7 + i)
            states.append(orc.init_state(cfg, B, dtype))

        def prefill_layer(i, x):
            orc.prefill_chunked(layers[i][0], layers[i][1], x, states[i], block_size=w["block"])

        def step(x):
            for (c, wt), st in zip(layers, states):
                x = x + orc.step(c, wt, x, st)
            return x

    sync = (lambda: torch.cuda.synchronize(dev)) if dev.type == "cuda" else (lambda: None)
    P = (w["W"] + w["block"] + w["block"] - 1) // w["block"] * w["block"]
    x_pre = mixture(B, P, D, min(w["K"], 512), w["sigma"], 11, "cpu", dtype).to(dev)
    x_dec = mixture(B, steps + warmup + 2, D, min(w["K"], 512), w["sigma"], 13, "cpu", dtype).to(dev)
    with torch.no_grad():
        add_layer(0)
        prefill_layer(0, x_pre)                                               # ring full, banks live
        sync()
        step(x_dec[:, :1])
        sync()
        t0 = time.perf_counter()
        step(x_dec[:, 1:2])
        sync()
        probe = time.perf_counter() - t0                                      # one layer, one step
        if budget_s is not None:
            steps = int(max(2, min(steps, budget_s / max(probe, 1e-4))))
            warmup = min(warmup, 1)
        nl = sample_layers
        if nl is None:
            nl = int(max(1, min(w["layers"], region_s / ((steps + warmup) * max(probe, 1e-5)))))
        for i in range(1, nl):
            add_layer(i)
            prefill_layer(i, x_pre)
        t = 2
        for _ in range(warmup):
            step(x_dec[:, t:t + 1]); t += 1
        sync()
        t0 = time.perf_counter()
        for _ in range(steps):
            step(x_dec[:, t:t + 1]); t += 1
        sync()
        dt = time.perf_counter() - t0
    s_per_step = dt / steps
    tok_s = B / (s_per_step * w["layers"] / nl)
    where = f"{threads} host threads" if dev.type == "cpu" else torch.cuda.get_device_name(dev)
    what = "upstream CoDAGQALandmarkPerf2, PyTorch path, unmodified" if kind == "reference" else "CPU restatement of upstream (oracle)"
    return {"value": tok_s, "unit": "tokens/s", "cores": threads if dev.type == "cpu" else 0, "kind": kind,
            "sample": f"{what}, bf16, on {where}: {B} states x {nl} of {w['layers']} layers x {steps} decode steps after a "
                      f"{P}-token prefill; tokens/s scaled to the full stack by layers ({w['layers']}/{nl})",
            "steps": steps, "sample_layers": nl, "seconds_per_sampled_step": s_per_step, "seconds_timed": dt}


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
            "warm_state": f"{3 * P}-token prefill in blocks of {w['block']}"}


def reference_main(args, w, K, Wm, rank):
    """`--impl reference` (host cores) / `--impl reference-gpu` (upstream eager on cuda:0).  Rank 0 alone runs."""
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    if args.impl == "reference":
        r = reference_decode(w, K, Wm, "cpu", cores)
    else:
        r = reference_decode(w, K, Wm, "cuda:0", cores, sample_layers=w["layers"])
    # ms_per_step is the MEASURED time of one sampled step (steps x ms_per_step = the timed region); `value` scales
    # it to the full stack as stated in cpu_baseline.sample
    print(json.dumps({
        "impl": args.impl, "metric": METRIC, "value": r["value"], "unit": "tokens/s", "n_gpus": args.gpus, "steps": r["steps"],
        "warmup": Wm, "ms_per_step": 1e3 * r["seconds_per_sampled_step"], "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": workload_config(args, w, max(1, args.gpus)),
        "cpu_baseline": r, "ms_per_full_stack_step": 1e3 * r["seconds_per_sampled_step"] * w["layers"] / r["sample_layers"],
        "e2e": {"value": r["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))


# ------------------------------------------------------------------------------------------------------ our arm
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "reference-gpu"])
    ap.add_argument("--workload", default="c4_mistral7b", choices=sorted(WORKLOADS))
    ap.add_argument("--layers", type=int, default=None, help="override the layer count (profiling small cases)")
    ap.add_argument("--states", type=int, default=None, help="override states per GPU")
    ap.add_argument("--prefill-tokens", type=int, default=512)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--eager", action="store_true", help="time eager launches instead of CUDA-graph replay")
    ap.add_argument("--no-split-routing", action="store_true",
                    help="route the evicted tokens inside each layer's chain instead of in one launch per step")
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

    if args.impl != "ours":
        reference_main(args, w, K, Wm, rank)
        return

    pkg = os.path.join(ROOT, "coda-gqa-l_b200")
    if pkg not in sys.path:
        sys.path.insert(0, pkg)
    import torch.distributed as dist
    from coda_gqa_l_b200 import CoDAGQALandmarkPerf2, CoDAStack
    from coda_gqa_l_b200._lib import RingPos, check, lib
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
    # three chunks of one token stream, each a tensor of its own (a chunk arrives as a contiguous batch)
    x_pre = [c.contiguous() for c in mixture(B, 3 * P, D, w["K"], w["sigma"], 11 + rank, dev, dtype).split(P, dim=1)]
    x_dec = mixture(B, 2 * (K + Wm) + 8, D, w["K"], w["sigma"], 13 + rank, dev, dtype)
    x_dec_host = x_dec.cpu().pin_memory()

    # ---- prefill (brings every ring to steady state); timed as a secondary figure ----
    stack.prefill(x_pre[0], states, block_size=w["block"])                      # warm-up chunk: fills every ring
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    stack.prefill(x_pre[1], states, block_size=w["block"])                      # timed chunk: same shapes, steady state
    e1.record()
    barrier()
    prefill_ms = max_over_ranks(e0.elapsed_time(e1), dev)
    pre_tokens = B * P
    # the attention kernel by itself: a third chunk with events around every attention launch
    for l in stack.layers:
        l.kernel_timers = []
    stack.prefill(x_pre[2], states, block_size=w["block"])
    barrier()
    att_ms = [a.elapsed_time(b) for l in stack.layers for (_, a, b) in l.kernel_timers]
    pre_kernel_ms = sum(att_ms) / max(1, len(att_ms))
    for l in stack.layers:
        l.kernel_timers = None
    del x_pre
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
    def e2e_step(tt):
        if args.eager:
            x_stage.copy_(x_dec_host[:, tt:tt + 1], non_blocking=True)
            out_host.copy_(step_fn(x_stage, states), non_blocking=True)
        else:
            # one launch per token: the captured step with its host-to-device and device-to-host copies inside
            stack.step_graph_host(x_dec_host[:, tt:tt + 1], states)
        torch.cuda.current_stream(dev).synchronize()

    for _ in range(3):
        e2e_step(t); t += 1
    barrier()
    e0.record()
    for _ in range(K):
        e2e_step(t); t += 1
    e1.record()
    barrier()
    ms_e2e = max_over_ranks(e0.elapsed_time(e1), dev)
    e2e_tok_s = world * B * K / (ms_e2e * 1e-3)

    # ---- roofline of the dominant kernel: the decode attention AS THE TIMED STEP RUNS IT ----
    # The captured step launches decode_attend_kernel<Dh, NQ, true> (coda_b200_decode_attend_append: the attention that
    # also writes the step's new token).  Timed here as one CUDA graph holding one such launch per layer, each on its
    # own layer's state (so no launch finds its planes in L2 once layers x bytes-per-launch exceeds it), replayed and
    # timed with events on the launching stream; re-writing the same token at the same ring position is idempotent.
    # The variant without the token write (records prepared beforehand) and the step's batched routing launch are
    # timed the same way for the secondary figures.  This section runs last: it leaves the states as they are.
    roof_stream = torch.cuda.Stream(dev)
    H_, Dh_ = w["H"], D // w["H"]
    x_fix = mixture(B, 1, D, w["K"], w["sigma"], 17, dev, dtype)
    q_fix = torch.randn(B, H_ * Dh_, device=dev, dtype=dtype)
    lam_fix = torch.randn(B, H_, device=dev, dtype=dtype)
    outs = [torch.empty(B, 1, H_ * Dh_, device=dev, dtype=dtype) for _ in stack.layers]
    reps = max(1, -(-8 // len(stack.layers)))            # layer sweeps per replay (>= 8 launches per graph)
    cfgs = [l._cfg(B, dtype, st) for l, st in zip(stack.layers, states)]
    rps = [RingPos(int(st.pos), int(st.recent_idx), int(st.recent_filled), None) for st in states]
    append_ok = all(bool(lib.coda_b200_decode_attend_append_supported(C.byref(c))) and l._fused_write_ok(c)
                    for l, c in zip(stack.layers, cfgs))

    def timed_graph(body, nrep=10):
        """Mean ms per call of `body` from `nrep` replays of a graph holding `reps` calls."""
        with torch.cuda.stream(roof_stream):
            body()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=roof_stream):
                for _ in range(reps):
                    body()
            for _ in range(3):
                g.replay()
            r0, r1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            r0.record(roof_stream)
            for _ in range(nrep):
                g.replay()
            r1.record(roof_stream)
        roof_stream.synchronize()
        return r0.elapsed_time(r1) / (nrep * reps)

    roof_stream.wait_stream(torch.cuda.current_stream(dev))
    with torch.cuda.stream(roof_stream):
        projs = [l._project(x_fix, need_kv=True) for l in stack.layers]          # raw projections of one token per layer
        for l, st, c, rp, o in zip(stack.layers, states, cfgs, rps, outs):      # decode records for the prepared variant
            l.decode_attend_launch(c, st, rp, 1, q_fix, lam_fix, o)
    roof_stream.synchronize()

    def sweep_prepared():
        for l, st, c, o in zip(stack.layers, states, cfgs, outs):
            l.decode_attend_prepared_launch(c, st, o)

    # cos / sin of the token's position, computed once for all layers as the captured step does
    rope_cs = None
    if append_ok and stack._shared_rope(states, dtype):
        rope_cs = torch.empty(stack.layers[0].head_dim, dtype=torch.float32, device=dev)
        with torch.cuda.stream(roof_stream):
            check(lib.coda_b200_rope_table(C.byref(cfgs[0]), rps[0], stack.layers[0]._consts(dev, dtype)[0].data_ptr(),
                                           rope_cs.data_ptr(), roof_stream.cuda_stream), "coda_b200_rope_table")
        roof_stream.synchronize()

    def sweep_append():
        for l, st, c, rp, pr, o in zip(stack.layers, states, cfgs, rps, projs, outs):
            l.decode_attend_append_launch(c, st, rp, pr, o, rope_cs)

    nl = len(stack.layers)
    # In the step the attention lets the kernel after it (the output projection) onto SMs as they free up.  In a
    # train of attention launches that would let consecutive launches overlap, so the trains below are captured
    # with the implicit trigger at grid completion: the figure stays the duration of one launch.
    lib.coda_b200_decode_set_early_trigger(0)
    prepared_ms = timed_graph(sweep_prepared) / nl
    append_ms = timed_graph(sweep_append) / nl if append_ok else None
    route_ms = None
    plan = stack._route_plan(states, rps, dtype) if append_ok else None
    if plan is not None:
        def route_all():
            check(lib.coda_b200_step_route_batched(C.byref(plan[0]), plan[1].data_ptr(), nl, roof_stream.cuda_stream),
                  "coda_b200_step_route_batched")
        route_ms = timed_graph(route_all)
    lib.coda_b200_decode_set_early_trigger(1)
    for l in stack.layers:
        if l.device_status() != 0:
            raise RuntimeError("a tuned kernel reported an expired device-side wait")
    bytes_launch = decode_bytes_per_state_layer(w) * B
    kern_ms = append_ms if append_ms is not None else prepared_ms
    variant = "append" if append_ms is not None else "prepared"
    achieved = bytes_launch / (kern_ms * 1e-3) / 1e9
    prof = profiled_traffic(args.workload, variant)
    step_bytes = w["layers"] * (bytes_launch + weight_bytes_per_layer(w))
    roofline = {
        "kernel": (f"decode_attend_kernel<{Dh_},*,true> (coda_b200_decode_attend_append: attention + the new token's write, "
                   "the launch the timed step makes)" if variant == "append" else
                   f"decode_attend_kernel<{Dh_},*,false> (coda_b200_decode_attend_prepared)"),
        "timing": "graph of back-to-back launches over all layers' states, CUDA events on the launching stream",
        "bound": "hbm", "achieved": achieved, "peak": hbm_peak, "unit": "GB/s", "frac": achieved / hbm_peak, "of": peak_src,
        "frac_of_nominal_8000": achieved / 8000.0, "kernel_ms": kern_ms, "bytes_per_launch": bytes_launch,
        # dram__bytes_read.sum + dram__bytes_write.sum per launch of this variant from the ncu capture kept beside this
        # file, scaled by the states processed (traffic grows with the planes streamed)
        "traffic": None if prof is None else int(round(prof[0] * B / prof[1])),
        "prepared_variant": {"kernel_ms": prepared_ms, "achieved": bytes_launch / (prepared_ms * 1e-3) / 1e9,
                             "frac": bytes_launch / (prepared_ms * 1e-3) / 1e9 / hbm_peak},
        # attention + new-token write + this layer's share of the step's routing launch, same algorithmic bytes
        "with_routing": None if route_ms is None else {
            "routing_launch_ms": route_ms, "ms_per_layer": kern_ms + route_ms / nl,
            "achieved": bytes_launch / ((kern_ms + route_ms / nl) * 1e-3) / 1e9,
            "frac": bytes_launch / ((kern_ms + route_ms / nl) * 1e-3) / 1e9 / hbm_peak},
        # the whole timed step against HBM: every layer's state traffic plus its projection weights, once per step
        "whole_step": {"bytes_per_step": step_bytes, "achieved": step_bytes / (ms / K * 1e-3) / 1e9,
                       "frac": step_bytes / (ms / K * 1e-3) / 1e9 / hbm_peak},
    }

    # own output-projection GEMM: one more launch of this repository's per layer where the layers use it
    Dh_ = D // w["H"]
    own_out = all(l.use_skinny_gemm_kernel and bool(lib.coda_b200_skinny_gemm_supported(B, w["H"] * Dh_, D)) for l in stack.layers)
    per_step_launches = ((2 if args.eager or args.no_split_routing else 1) * w["layers"] + (w["layers"] if own_out else 0)
                         + (0 if args.eager else (1 if args.no_split_routing else 3)))
    line = {
        "metric": METRIC, "value": tok_s, "unit": "tokens/s",
        "n_gpus": world, "steps": K, "warmup": Wm, "ms_per_step": ms / K, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": workload_config(args, w, world),
        "chained_projections": bool(not args.eager and stack._graph is not None and stack._graph.get("chained")),
        "e2e": {"value": e2e_tok_s, "unit": "tokens/s", "h2d_bytes_per_step": B * D * 2, "d2h_bytes_per_step": B * D * 2,
                "ms_per_step": ms_e2e / K},
        # this repository's kernels inside the timed region: per layer the decode attention (which writes the new
        # token) and the output-projection GEMM, per step the batched routing, the cos/sin table and the step counter
        # (the first layer's input projection is a library call; where the stack chains its projections, the other
        # layers' input projections are the second phase of the launch that holds the output projection before them)
        "gpu_launches": K * per_step_launches,
        "clocks": clocks.summary(),
        "roofline": roofline,
        "prefill": {"tokens_per_s": world * pre_tokens / (prefill_ms * 1e-3), "tokens": pre_tokens, "ms": prefill_ms,
                    "attention_kernel_ms_per_block": pre_kernel_ms, "attention_tflops": pre_tf,
                    "tensor_frac": pre_tf / tc_peak, "tensor_peak": tc_peak, "of": peak_src},
    }
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = reference_decode(w, 64, 1, "cpu", cores, sample_layers=1, budget_s=15.0)
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
