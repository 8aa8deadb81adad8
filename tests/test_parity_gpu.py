"""GPU: the CUDA path (through the C ABI) against the CPU oracle run live on the same seeded inputs,
and against the fixtures generated from the upstream implementation.

Bar: ring scalars, `allowed` and the LRU stamps bit-exact in fp32; layer outputs within 1e-4 relative
(fp32) / 2e-2 relative (bf16) of the reference."""
import pytest
import torch

from tests.helpers import (SCENARIOS, TOL_BF16, TOL_F32, build_inputs, build_module, load_golden, oracle_state_from,
                           orc, rel_err, weights_of)

pytestmark = pytest.mark.gpu


def _same_metrics(got, want, tag):
    """Counters are integers and must agree exactly; the two fill ratios are fp32 means."""
    assert (got is None) == (want is None), f"{tag}: one side carries no metrics"
    if want is None:
        return
    assert set(got) == set(want), tag
    for key, val in want.items():
        if isinstance(val, float):
            assert abs(got[key] - val) < 1e-6, f"{tag}: {key} {got[key]} != {val}"
        else:
            assert got[key] == val, f"{tag}: {key} {got[key]} != {val}"


def _run(name, check_golden=True):
    from coda_gqa_l_b200 import state_from_fields
    sc = SCENARIOS[name]
    dtype = getattr(torch, sc.get("dtype", "float32"))
    f32 = dtype == torch.float32
    tol = TOL_F32 if f32 else TOL_BF16
    mod = build_module(sc, dtype)
    wts = weights_of(mod)
    cfg = orc.OracleConfig.from_module(mod)
    torch.manual_seed(sc["state_seed"])
    st_cpu = mod.init_state(batch_size=sc["B"], device="cpu", dtype=dtype)
    ost = oracle_state_from(st_cpu)
    mod = mod.to("cuda")
    st = state_from_fields(st_cpu, "cuda")
    x_pre, x_dec = build_inputs(sc, dtype)
    gold = load_golden(name) if check_golden else None
    for i, phase in enumerate(sc["phases"]):
        if phase[0] == "prefill":
            lo, hi, blk = phase[1:]
            y_o = orc.prefill_chunked(cfg, wts, x_pre[:, lo:hi], ost, block_size=blk)
            y, st = mod.prefill_chunked(x_pre[:, lo:hi].cuda(), st, block_size=blk)
        else:
            lo, hi = phase[1:]
            xs = x_dec.cuda()
            ys, yo = [], []
            for t in range(lo, hi):
                yy, st = mod.step(xs[:, t:t + 1], st)
                ys.append(yy)
                yo.append(orc.step(cfg, wts, x_dec[:, t:t + 1], ost))
            y, y_o = torch.cat(ys, 1), torch.cat(yo, 1)
        torch.cuda.synchronize()
        tag = f"{name} phase {i} {phase}"
        assert (st.recent_idx, st.recent_filled, st.pos) == (ost.recent_idx, ost.recent_filled, ost.pos), tag
        if f32:
            assert torch.equal(st.allowed.cpu(), ost.allowed), f"{tag}: slot occupancy differs"
            assert torch.equal(st.mem_last_exact.cpu(), ost.mem_last_exact), f"{tag}: LRU stamps differ"
            assert torch.equal(st.g_recent.cpu(), ost.g_recent) or rel_err(st.g_recent, ost.g_recent) < 1e-6, tag
        assert (st.active_exact, st.active_summary) == (ost.active_exact, ost.active_summary), f"{tag}: bank growth"
        if f32:
            _same_metrics(st.metrics, ost.metrics, f"{tag} vs oracle")
        e = rel_err(y, y_o)
        assert e < tol, f"{tag}: output rel err {e:.3e} vs oracle"
        if f32:
            assert rel_err(st.k_buf, ost.k_buf) < tol and rel_err(st.v_buf, ost.v_buf) < tol, f"{tag}: K/V"
            if ost._exact_v_norm is not None:
                assert rel_err(st._exact_v_norm, ost._exact_v_norm) < tol, tag
            if ost._sum_lf_k_norm is not None:
                assert rel_err(st._sum_lf_k_norm, ost._sum_lf_k_norm) < tol, tag
        if gold is not None:
            snap = gold["snapshots"][i]
            eg = rel_err(y[:, ::gold["y_stride"]], gold["y"][i])
            assert eg < tol, f"{tag}: output rel err {eg:.3e} vs upstream fixture"
            assert (st.recent_idx, st.recent_filled, st.pos) == (snap["recent_idx"], snap["recent_filled"], snap["pos"])
            if f32:
                assert torch.equal(st.allowed.cpu(), snap["allowed"]), f"{tag}: occupancy vs fixture"
                assert torch.equal(st.mem_last_exact.cpu(), snap["mem_last_exact"]), f"{tag}: stamps vs fixture"
                if "active_exact" in snap:
                    assert (st.active_exact, st.active_summary) == (snap["active_exact"], snap["active_summary"]), tag
                    _same_metrics(st.metrics, snap["metrics"], f"{tag} vs fixture")
    return mod, st, ost


@pytest.mark.parametrize("name", [n for n in SCENARIOS if n != "c1"])
def test_scenario_matches_oracle_and_fixture(name):
    _run(name)


def test_config1_cpu_reference_run():
    """BASELINE config 1 exactly: fp32, B=1, 2048-token prefill in blocks of 256, then 1000 decode steps."""
    _run("c1")


def test_flag_combinations_of_step():
    """attend=False writes only; write_cache=False leaves the state untouched;
    include_current_in_attention=False attends before writing (upstream attention.py:529-547)."""
    from coda_gqa_l_b200 import state_from_fields
    sc = SCENARIOS["small_b2"]
    mod = build_module(sc, torch.float32)
    wts, cfg = weights_of(mod), None
    cfg = orc.OracleConfig.from_module(mod)
    torch.manual_seed(1)
    st_cpu = mod.init_state(batch_size=2, device="cpu", dtype=torch.float32)
    ost = oracle_state_from(st_cpu)
    mod = mod.cuda()
    st = state_from_fields(st_cpu, "cuda")
    x = torch.randn(2, 90, 128, generator=torch.Generator().manual_seed(4))
    for t in range(90):
        kw = [dict(), dict(attend=False), dict(write_cache=False), dict(include_current_in_attention=False)][t % 4]
        y, st = mod.step(x[:, t:t + 1].cuda(), st, **kw)
        y_o = orc.step(cfg, wts, x[:, t:t + 1], ost, **kw)
        assert (st.pos, st.recent_idx, st.recent_filled) == (ost.pos, ost.recent_idx, ost.recent_filled)
        if float(y_o.abs().sum()) == 0.0:
            assert float(y.abs().sum()) == 0.0
        else:
            assert rel_err(y, y_o) < TOL_F32, (t, kw)
    assert torch.equal(st.allowed.cpu(), ost.allowed)
    assert torch.equal(st.mem_last_exact.cpu(), ost.mem_last_exact)


def test_prefill_without_write_and_streaming_equivalence():
    """write_cache=False leaves pos and buffers untouched; prefilling in two calls equals one call."""
    from coda_gqa_l_b200 import _deep_copy_state, state_from_fields
    sc = SCENARIOS["small_b2"]
    mod = build_module(sc, torch.float32)
    torch.manual_seed(1)
    st_cpu = mod.init_state(batch_size=2, device="cpu", dtype=torch.float32)
    mod = mod.cuda()
    x, _ = build_inputs(sc, torch.float32)
    x = x.cuda()
    a = state_from_fields(st_cpu, "cuda")
    k0 = a.k_buf.clone()
    y0, a = mod.prefill_chunked(x[:, :64], a, block_size=32, write_cache=False)
    assert a.pos == 0 and torch.equal(a.k_buf, k0) and y0.shape == (2, 64, 128)
    y1, a = mod.prefill_chunked(x, a, block_size=32)
    b = state_from_fields(st_cpu, "cuda")
    y2a, b = mod.prefill_chunked(x[:, :96], b, block_size=32)
    y2b, b = mod.prefill_chunked(x[:, 96:], b, block_size=32)
    assert torch.equal(torch.cat([y2a, y2b], 1), y1)
    assert torch.equal(a.k_buf, b.k_buf) and torch.equal(a.mem_last_exact, b.mem_last_exact) and a.pos == b.pos
    c = _deep_copy_state(a)
    none, c = mod.prefill_chunked(x[:, :40], c, block_size=16, return_outputs=False)
    assert none is None and c.pos == a.pos + 40
    empty, c = mod.prefill_chunked(x[:, :0], c)
    assert empty.shape == (2, 0, 128)
    with pytest.raises(ValueError):
        mod.prefill_chunked(x, c, block_size=0)


def test_bounded_equals_unbounded_when_window_covers_sequence():
    """Independent of the bank code: with W >= L nothing is evicted, so prefill and token-by-token decode must
    equal plain full causal differential attention with the same weights (upstream README.md:263-269)."""
    from coda_gqa_l_b200 import CoDAGQA, CoDAGQALandmarkPerf2
    torch.manual_seed(0)
    kw = dict(embed_dim=256, num_heads=4, num_kv_heads=2)
    bounded = CoDAGQALandmarkPerf2(window=320, num_landmarks_exact=8, num_landmarks_summary=8, **kw).eval()
    plain = CoDAGQA(**kw).eval()
    plain.load_state_dict({k: v for k, v in bounded.state_dict().items() if k in plain.state_dict()})
    x = torch.randn(2, 300, 256, generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        y_ref, _ = plain(x)
    bounded = bounded.cuda()
    st = bounded.init_state(batch_size=2, device="cuda", dtype=torch.float32)
    y, st = bounded.prefill_chunked(x[:, :236].cuda(), st, block_size=100)
    assert rel_err(y, y_ref[:, :236]) < TOL_F32
    ys = []
    for t in range(236, 300):
        yy, st = bounded.step(x[:, t:t + 1].cuda(), st)
        ys.append(yy)
    assert rel_err(torch.cat(ys, 1), y_ref[:, 236:]) < TOL_F32


def test_run_to_run_determinism():
    """Same inputs twice give bit-identical outputs and state: the kernels use no atomics."""
    outs = []
    for _ in range(2):
        mod, st, _ = _run("small_randn", check_golden=False)
        outs.append((st.k_buf.clone(), st.v_buf.clone(), st.mem_last_exact.clone()))
    for a, b in zip(*outs):
        assert torch.equal(a, b)


def test_rejects_cpu_tensors_and_training_mode():
    from coda_gqa_l_b200 import CoDAGQALandmarkPerf2
    mod = CoDAGQALandmarkPerf2(embed_dim=64, num_heads=2, num_kv_heads=1, window=8, num_landmarks_exact=4,
                               num_landmarks_summary=4).eval()
    st = mod.init_state(batch_size=1, device="cpu", dtype=torch.float32)
    with pytest.raises(RuntimeError):
        mod.step(torch.randn(1, 1, 64), st)
    mod = mod.cuda().train()
    st = mod.init_state(batch_size=1, device="cuda", dtype=torch.float32)
    with pytest.raises(RuntimeError):
        mod.step(torch.randn(1, 1, 64, device="cuda"), st)


@pytest.mark.parametrize("shape", [
    dict(embed_dim=512, num_heads=4, num_kv_heads=1, window=100, num_landmarks_exact=20, num_landmarks_summary=12),   # Dh 128, G 4, 132 slots
    dict(embed_dim=512, num_heads=8, num_kv_heads=1, window=256, num_landmarks_exact=64, num_landmarks_summary=64),   # Dh 64, G 8
    dict(embed_dim=384, num_heads=3, num_kv_heads=3, window=40, num_landmarks_exact=8, num_landmarks_summary=8,
         head_norm_mode="identity", rope_interleaved=False, rope_base=1e6),                                          # Dh 128, MHA
    dict(embed_dim=576, num_heads=9, num_kv_heads=3, window=128, num_landmarks_exact=32, num_landmarks_summary=32,
         head_norm_mode="identity", rope_interleaved=False),                                                         # config-2 shape
    dict(embed_dim=1024, num_heads=8, num_kv_heads=1, window=70, num_landmarks_exact=16, num_landmarks_summary=10),   # Dh 128, G 8 (two query n-tiles)
    dict(embed_dim=512, num_heads=8, num_kv_heads=2, window=40, num_landmarks_exact=24, num_landmarks_summary=16,
         min_landmarks_exact=3, min_landmarks_summary=2, expansion_t_max=300, collect_metrics=True),                  # growing banks, counters
])
def test_tuned_decode_kernel_matches_generic_kernels(shape):
    """The TMA / tensor-core decode kernel against the shape-generic kernels on identical states (bf16),
    through a prefill and 150 decode steps so that the ring wraps and both banks are live."""
    from coda_gqa_l_b200 import CoDAGQALandmarkPerf2, _deep_copy_state
    from tests.scenarios import randomize_weights
    torch.manual_seed(3)
    mod = CoDAGQALandmarkPerf2(**shape).eval()
    randomize_weights(mod, 3)
    mod = mod.to(torch.bfloat16).cuda()
    D, B = shape["embed_dim"], 3
    x = orc.mixture_inputs(B, 64 + 150, D, centroids=16, sigma=0.3, seed=5, dtype=torch.bfloat16).cuda()
    torch.manual_seed(4)
    sa = mod.init_state(batch_size=B, device="cuda", dtype=torch.bfloat16)
    _, sa = mod.prefill_chunked(x[:, :64], sa, block_size=32)
    sb = _deep_copy_state(sa)
    ya, yb = [], []
    for t in range(64, 214):
        mod.use_tuned_kernels = True
        y, sa = mod.step(x[:, t:t + 1], sa)
        ya.append(y)
        mod.use_tuned_kernels = False
        y, sb = mod.step(x[:, t:t + 1], sb)
        yb.append(y)
    assert mod.device_status() == 0
    # the cache-write kernel is the same code in both modes (raw vs pre-rotated input): state must agree exactly
    assert torch.equal(sa.allowed, sb.allowed) and torch.equal(sa.mem_last_exact, sb.mem_last_exact)
    assert torch.equal(sa.k_buf, sb.k_buf) and torch.equal(sa.v_buf, sb.v_buf)
    assert (sa.active_exact, sa.active_summary) == (sb.active_exact, sb.active_summary) and sa.metrics == sb.metrics
    if shape.get("collect_metrics"):
        assert sa.metrics["total_evictions"] > 0 and sa.active_exact > shape["min_landmarks_exact"]
    e = rel_err(torch.cat(ya, 1), torch.cat(yb, 1))
    assert e < 5e-3, f"tuned vs generic decode attention: rel err {e:.3e}"


@pytest.mark.parametrize("B,nl,steps,kw", [
    (2, 3, 40, dict(embed_dim=256, num_heads=4, num_kv_heads=2, window=24, num_landmarks_exact=8, num_landmarks_summary=8)),
    # config-4 head geometry, 192 planes (two per CTA of the attention kernel), many replays
    (24, 2, 150, dict(embed_dim=1024, num_heads=8, num_kv_heads=8, window=24, num_landmarks_exact=16, num_landmarks_summary=16)),
])
def test_graph_replay_equals_eager_steps(B, nl, steps, kw):
    """A captured stack step replayed N times gives the same states and outputs as N eager steps."""
    from coda_gqa_l_b200 import CoDAGQALandmarkPerf2, CoDAStack, _deep_copy_state
    layers = []
    for i in range(nl):
        torch.manual_seed(i)
        layers.append(CoDAGQALandmarkPerf2(**kw).eval().to(torch.bfloat16).cuda())
    stack = CoDAStack(layers)
    torch.manual_seed(9)
    sa = stack.init_states(batch_size=B, device="cuda", dtype=torch.bfloat16)
    x = orc.mixture_inputs(B, 16 + steps, kw["embed_dim"], centroids=8, sigma=0.3, seed=2, dtype=torch.bfloat16).cuda()
    stack.prefill(x[:, :16], sa, block_size=8)          # ring not yet full: replay crosses the fill -> evict boundary
    sb = [_deep_copy_state(s) for s in sa]
    outs_a, outs_b = [], []
    for t in range(16, 16 + steps):
        outs_a.append(stack.step_graph(x[:, t:t + 1], sa).clone())
        outs_b.append(stack.step(x[:, t:t + 1], sb))
    # Library GEMMs may pick another algorithm under capture, so floats are compared with the bf16 tolerance
    # and only the integer state exactly.
    for a, b in zip(sa, sb):
        assert (a.pos, a.recent_idx, a.recent_filled) == (b.pos, b.recent_idx, b.recent_filled)
        assert torch.equal(a.allowed, b.allowed) and torch.equal(a.mem_last_exact, b.mem_last_exact)
        assert rel_err(a.k_buf, b.k_buf) < TOL_BF16 and rel_err(a.v_buf, b.v_buf) < TOL_BF16
    assert rel_err(torch.cat(outs_a, 1), torch.cat(outs_b, 1)) < TOL_BF16


@pytest.mark.parametrize("shape,block,L", [
    (dict(embed_dim=512, num_heads=4, num_kv_heads=1, window=100, num_landmarks_exact=20, num_landmarks_summary=12), 128, 384),
    (dict(embed_dim=512, num_heads=8, num_kv_heads=2, window=256, num_landmarks_exact=64, num_landmarks_summary=64), 256, 768),
    (dict(embed_dim=384, num_heads=3, num_kv_heads=3, window=40, num_landmarks_exact=8, num_landmarks_summary=8,
          head_norm_mode="identity", rope_interleaved=False, rope_base=1e6), 100, 250),
    (dict(embed_dim=576, num_heads=9, num_kv_heads=3, window=128, num_landmarks_exact=32, num_landmarks_summary=32,
          head_norm_mode="identity", rope_interleaved=False), 128, 300),
    (dict(embed_dim=256, num_heads=2, num_kv_heads=1, window=64, num_landmarks_exact=16, num_landmarks_summary=16), 48, 200),
])
def test_tensor_core_prefill_matches_generic_kernel(shape, block, L):
    """The tcgen05 prefill attention against the shape-generic kernel on identical inputs and states (bf16):
    ragged last blocks, several query tiles per block, slot counts that are not multiples of the key tile,
    partly masked banks."""
    from coda_gqa_l_b200 import CoDAGQALandmarkPerf2, _deep_copy_state
    from tests.scenarios import randomize_weights
    torch.manual_seed(3)
    mod = CoDAGQALandmarkPerf2(**shape).eval()
    randomize_weights(mod, 3)
    mod = mod.to(torch.bfloat16).cuda()
    D, B = shape["embed_dim"], 2
    x = orc.mixture_inputs(B, L, D, centroids=16, sigma=0.3, seed=5, dtype=torch.bfloat16).cuda()
    torch.manual_seed(4)
    sa = mod.init_state(batch_size=B, device="cuda", dtype=torch.bfloat16)
    sb = _deep_copy_state(sa)
    mod.use_tuned_kernels = True
    ya, sa = mod.prefill_chunked(x, sa, block_size=block)
    assert mod.device_status() == 0
    mod.use_tuned_kernels = False
    yb, sb = mod.prefill_chunked(x, sb, block_size=block)
    assert torch.equal(sa.k_buf, sb.k_buf) and torch.equal(sa.allowed, sb.allowed)
    assert torch.isfinite(ya).all()
    e = rel_err(ya, yb)
    assert e < 8e-3, f"tensor-core vs generic prefill attention: rel err {e:.3e}"


@pytest.mark.gpu
@pytest.mark.parametrize("shape", [
    dict(embed_dim=512, num_heads=4, num_kv_heads=1, window=100, num_landmarks_exact=20, num_landmarks_summary=12),   # Dh 128, G 4
    dict(embed_dim=576, num_heads=9, num_kv_heads=3, window=24, num_landmarks_exact=6, num_landmarks_summary=5,
         head_norm_mode="identity", rope_interleaved=False),                                                         # Dh 64, G 3, 35 slots
])
def test_decode_records_of_fused_write_match_preparation_kernel(shape):
    """The decode records (prepared queries, lambda, visibility mask after the write) that the fused cache
    write leaves behind are bit-identical to what the stand-alone preparation computes from the state after
    the write -- while the ring fills and after it wraps."""
    from coda_gqa_l_b200 import CoDAGQALandmarkPerf2
    from coda_gqa_l_b200._lib import RingPos
    from tests.scenarios import randomize_weights
    torch.manual_seed(3)
    mod = CoDAGQALandmarkPerf2(**shape).eval()
    randomize_weights(mod, 3)
    mod = mod.to(torch.bfloat16).cuda()
    D, B = shape["embed_dim"], 3
    H, Hkv = shape["num_heads"], shape["num_kv_heads"]
    G, Dh = H // Hkv, D // H
    Lbuf = shape["window"] + shape["num_landmarks_exact"] + shape["num_landmarks_summary"]
    rows, qstr = (8 if 2 * G <= 8 else 16), Dh + 8
    rec_bytes = rows * qstr * 2 + 32 + (Lbuf + 63) // 64 * 64
    x = orc.mixture_inputs(B, 80, D, centroids=16, sigma=0.3, seed=5, dtype=torch.bfloat16).cuda()
    st = mod.init_state(batch_size=B, device="cuda", dtype=torch.bfloat16)
    _, st = mod.prefill_chunked(x[:, :8], st, block_size=8)        # ring not yet full
    out = torch.empty(B, 1, D, device="cuda", dtype=torch.bfloat16)
    for t in range(8, 80):
        xt = x[:, t:t + 1]
        cfg = mod._cfg(B, xt.dtype, st)
        q, _, _, lam_logit, _ = mod._project(xt, need_kv=True)
        y, st = mod.step(xt, st)
        fused = mod._qrec[:B * Hkv * rec_bytes].clone()
        assert fused.numel() == B * Hkv * rec_bytes
        rp = RingPos(int(st.pos), int(st.recent_idx), int(st.recent_filled), None)
        mod.decode_attend_launch(cfg, st, rp, 1, q, lam_logit, out)
        prep = mod._qrec[:B * Hkv * rec_bytes].clone()
        f, p = fused.view(B * Hkv, rec_bytes), prep.view(B * Hkv, rec_bytes)
        qf = f[:, :rows * qstr * 2].contiguous().view(torch.bfloat16).view(-1, rows, qstr)[:, :, :Dh]
        qp = p[:, :rows * qstr * 2].contiguous().view(torch.bfloat16).view(-1, rows, qstr)[:, :, :Dh]
        assert torch.equal(qf, qp), f"step {t}: prepared queries differ"
        assert torch.equal(f[:, rows * qstr * 2:], p[:, rows * qstr * 2:]), f"step {t}: lambda / mask differ"
    assert mod.device_status() == 0


@pytest.mark.gpu
def test_wire_format_restores_a_live_state():
    """A state shipped as one blob and restored continues bit-identically to the original."""
    from coda_gqa_l_b200 import CoDAGQALandmarkPerf2, state_from_bytes, state_to_bytes
    from tests.scenarios import randomize_weights
    torch.manual_seed(0)
    mod = CoDAGQALandmarkPerf2(embed_dim=256, num_heads=4, num_kv_heads=2, window=24, num_landmarks_exact=8,
                               num_landmarks_summary=8).eval()
    randomize_weights(mod, 1)
    mod = mod.to(torch.bfloat16).cuda()
    x = orc.mixture_inputs(2, 90, 256, centroids=8, sigma=0.3, seed=2, dtype=torch.bfloat16).cuda()
    st = mod.init_state(batch_size=2, device="cuda", dtype=torch.bfloat16)
    _, st = mod.prefill_chunked(x[:, :40], st, block_size=16)
    for t in range(40, 60):
        _, st = mod.step(x[:, t:t + 1], st)
    twin = state_from_bytes(state_to_bytes(st), "cuda")
    assert (twin.pos, twin.recent_idx, twin.recent_filled) == (st.pos, st.recent_idx, st.recent_filled)
    for t in range(60, 90):
        ya, st = mod.step(x[:, t:t + 1], st)
        yb, twin = mod.step(x[:, t:t + 1], twin)
        assert torch.equal(ya, yb)
    assert torch.equal(st._arena, twin._arena)


@pytest.mark.gpu
def test_decode_attention_back_to_back_replays_are_stable():
    """Thousands of back-to-back launches of the decode attention kernel (a CUDA graph, CTAs with two planes
    each, tiles landing in any order) give the same bits every time.  Guards the ring's stage ownership: each
    stage is consumed by one consumer group only, so a parity wait can never run past an unobserved phase."""
    from coda_gqa_l_b200 import CoDAGQALandmarkPerf2
    from coda_gqa_l_b200._lib import RingPos
    torch.manual_seed(0)
    B, H, Hkv, Dh = 32, 8, 8, 128                       # 256 planes on 148 SMs, 6 tiles of 64 slots per plane
    mod = CoDAGQALandmarkPerf2(embed_dim=H * Dh, num_heads=H, num_kv_heads=Hkv, window=256, num_landmarks_exact=64,
                               num_landmarks_summary=64, head_norm_mode="identity", rope_interleaved=False)
    mod = mod.eval().to(torch.bfloat16).cuda()
    st = mod.init_state(batch_size=B, device="cuda", dtype=torch.bfloat16)
    x = (torch.randn(B, 384, H * Dh, device="cuda") * 0.5).to(torch.bfloat16)
    mod.prefill_chunked(x, st, block_size=128, return_outputs=False)
    cfg = mod._cfg(B, torch.bfloat16, st)
    q = torch.randn(B, H * Dh, device="cuda", dtype=torch.bfloat16)
    lam = torch.randn(B, H, device="cuda", dtype=torch.bfloat16)
    outs = [torch.empty(B, 1, H * Dh, device="cuda", dtype=torch.bfloat16) for _ in range(4)]
    rp = RingPos(int(st.pos), int(st.recent_idx), int(st.recent_filled), None)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        mod.decode_attend_launch(cfg, st, rp, 1, q, lam, outs[0])         # writes the decode records
        torch.cuda.synchronize()
        ref = outs[0].clone()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=side):
            for o in outs:
                mod.decode_attend_prepared_launch(cfg, st, o)
        for rep in range(1500):
            g.replay()
            if rep % 500 == 499:
                torch.cuda.synchronize()
                for o in outs:
                    assert torch.equal(o, ref), f"replay {rep}: output changed"
    torch.cuda.synchronize()
    assert mod.device_status() == 0


@pytest.mark.gpu
def test_prefill_attention_repeated_launches_are_stable():
    """The tcgen05 prefill kernel on the same state and inputs, launched back to back many times (no cache
    write), returns the same bits every time: its barriers are only ever waited on by threads that follow
    their phases in order."""
    from coda_gqa_l_b200 import CoDAGQALandmarkPerf2
    torch.manual_seed(1)
    mod = CoDAGQALandmarkPerf2(embed_dim=1024, num_heads=8, num_kv_heads=2, window=256, num_landmarks_exact=64,
                               num_landmarks_summary=64, head_norm_mode="identity", rope_interleaved=False)
    mod = mod.eval().to(torch.bfloat16).cuda()
    B = 24                                               # 24 x 8 heads = 192 CTAs: more than one wave
    st = mod.init_state(batch_size=B, device="cuda", dtype=torch.bfloat16)
    x = (torch.randn(B, 512, 1024, device="cuda") * 0.5).to(torch.bfloat16)
    mod.prefill_chunked(x[:, :384], st, block_size=128, return_outputs=False)
    ref, _ = mod.prefill_chunked(x[:, 384:], st, block_size=128, write_cache=False)
    ref = ref.clone()
    for rep in range(300):
        y, _ = mod.prefill_chunked(x[:, 384:], st, block_size=128, write_cache=False)
        if rep % 50 == 49:
            assert torch.equal(y, ref), f"repeat {rep}: output changed"
    assert mod.device_status() == 0


@pytest.mark.gpu
def test_attend_step_tuned_matches_generic():
    """attend_step (attention only, no cache write) on the fused decode kernel against the generic kernels,
    at the state's own position and at an explicit query position."""
    from coda_gqa_l_b200 import CoDAGQALandmarkPerf2
    from tests.scenarios import randomize_weights
    torch.manual_seed(2)
    mod = CoDAGQALandmarkPerf2(embed_dim=512, num_heads=4, num_kv_heads=2, window=48, num_landmarks_exact=16,
                               num_landmarks_summary=8).eval()
    randomize_weights(mod, 5)
    mod = mod.to(torch.bfloat16).cuda()
    x = orc.mixture_inputs(3, 120, 512, centroids=8, sigma=0.3, seed=3, dtype=torch.bfloat16).cuda()
    st = mod.init_state(batch_size=3, device="cuda", dtype=torch.bfloat16)
    _, st = mod.prefill_chunked(x[:, :100], st, block_size=32)
    for qpos in (None, 7, 250):
        mod.use_tuned_kernels = True
        ya = mod.attend_step(x[:, 100:101], st, query_pos=qpos)
        mod.use_tuned_kernels = False
        yb = mod.attend_step(x[:, 100:101], st, query_pos=qpos)
        assert rel_err(ya, yb) < 5e-3, f"query_pos={qpos}"
    mod.use_tuned_kernels = True
    assert mod.device_status() == 0


@pytest.mark.gpu
@pytest.mark.parametrize("M,K,N,res", [(32, 4096, 4096, True), (32, 4096, 4096, False), (5, 512, 256, True), (1, 128, 64, False),
                                       (17, 2048, 6208, True),
                                       # four-way split: 128-row tiles (112-row ones would need more clusters than fit),
                                       # a ragged last tile, few rows of X
                                       (32, 4096, 4608, True), (9, 1024, 4160, True), (3, 256, 64, False)])
def test_skinny_gemm_matches_library_gemm(M, K, N, res):
    """The decode step's output projection kernels (weight rows streamed through a TMA ring, K split over a cluster of
    four CTAs or over a CTA pair, residual in the epilogue) against torch's GEMM: fp32 accumulation on both sides, so
    the results agree to bf16 rounding of the outputs."""
    import ctypes as C
    from coda_gqa_l_b200._lib import lib, check
    g = torch.Generator(device="cuda").manual_seed(M * 7 + N)
    x = (torch.randn(M, K, device="cuda", generator=g) * 0.5).to(torch.bfloat16)
    w = (torch.randn(N, K, device="cuda", generator=g) * 0.05).to(torch.bfloat16)
    r = (torch.randn(M, N, device="cuda", generator=g)).to(torch.bfloat16) if res else None
    y = torch.full((M, N), float("nan"), device="cuda", dtype=torch.bfloat16)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    assert lib.coda_b200_skinny_gemm_supported(M, K, N)
    check(lib.coda_b200_skinny_gemm(x.data_ptr(), M, K, w.data_ptr(), N, None if r is None else r.data_ptr(), N, y.data_ptr(), N,
                                    status.data_ptr(), torch.cuda.current_stream().cuda_stream), "coda_b200_skinny_gemm")
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    ref = (x.float() @ w.float().t()).to(torch.bfloat16)
    if res:
        ref = (ref.float() + r.float()).to(torch.bfloat16)
    assert torch.isfinite(y.float()).all()
    err = rel_err(y, ref)
    assert err < 4e-3, f"skinny gemm rel err {err:.3e}"
    # element-wise: within one bf16 step of the fp32 reference
    assert float((y.float() - ref.float()).abs().max()) <= 2.0 ** -7 * float(ref.float().abs().max())


@pytest.mark.gpu
@pytest.mark.parametrize("M,K,N", [(32, 4096, 6208), (7, 1024, 1088), (32, 2048, 4096), (1, 256, 64)])
def test_skinny_gemm_with_bias_matches_linear(M, K, N):
    """The fused input projection's kernel (`coda_b200_skinny_gemm_bias`: K split over clusters of four CTAs, tile
    height chosen so that the clusters fill the device, bias added to the fp32 sum) against `F.linear`."""
    from coda_gqa_l_b200._lib import lib, check
    if not lib.coda_b200_skinny_gemm_bias_supported(M, K, N):
        pytest.skip("the four-way kernel does not cover this shape on this device")
    g = torch.Generator(device="cuda").manual_seed(M + K + N)
    x = (torch.randn(M, K, device="cuda", generator=g) * 0.5).to(torch.bfloat16)
    w = (torch.randn(N, K, device="cuda", generator=g) * 0.05).to(torch.bfloat16)
    b = torch.randn(N, device="cuda", generator=g).to(torch.bfloat16)
    y = torch.full((M, N), float("nan"), device="cuda", dtype=torch.bfloat16)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    for _ in range(3):                                                    # repeated launches: same bits
        check(lib.coda_b200_skinny_gemm_bias(x.data_ptr(), M, K, w.data_ptr(), N, b.data_ptr(), None, 0, y.data_ptr(), N,
                                             status.data_ptr(), torch.cuda.current_stream().cuda_stream), "coda_b200_skinny_gemm_bias")
        torch.cuda.synchronize()
        y_prev = y.clone() if _ == 0 else y_prev
        assert torch.equal(y, y_prev)
    assert int(status.item()) == 0
    ref = (x.float() @ w.float().t() + b.float()).to(torch.bfloat16)
    assert torch.isfinite(y.float()).all()
    assert rel_err(y, ref) < 4e-3
    assert float((y.float() - ref.float()).abs().max()) <= 2.0 ** -7 * float(ref.float().abs().max())


@pytest.mark.gpu
@pytest.mark.parametrize("M,KA,NA,NB", [(32, 4096, 4096, 6208), (7, 1024, 1024, 1088), (32, 2048, 4096, 6208), (1, 256, 256, 64),
                                        (32, 512, 4096, 1024)])
def test_chained_projections_equal_the_two_separate_launches(M, KA, NA, NB):
    """`coda_b200_skinny_gemm_chain` (a layer's output projection with the residual, a barrier across the grid, the
    next layer's input projection with its bias, one launch) against the two launches it replaces: the same bits
    in both outputs, over many launches that share the barrier words, and a clean status word."""
    from coda_gqa_l_b200._lib import lib, check
    if not (lib.coda_b200_skinny_gemm_chain_supported(M, KA, NA, NB) and lib.coda_b200_skinny_gemm_bias_supported(M, NA, NB)
            and lib.coda_b200_skinny_gemm_supported(M, KA, NA)):
        pytest.skip("not covered on this device")
    g = torch.Generator(device="cuda").manual_seed(M + KA + NA + NB)
    wa = (torch.randn(NA, KA, device="cuda", generator=g) * 0.05).to(torch.bfloat16)
    wb = (torch.randn(NB, NA, device="cuda", generator=g) * 0.05).to(torch.bfloat16)
    bias = torch.randn(NB, device="cuda", generator=g).to(torch.bfloat16)
    gsync = torch.zeros(2, dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    s = torch.cuda.current_stream().cuda_stream
    for it in range(12):
        x = (torch.randn(M, KA, device="cuda", generator=g) * 0.5).to(torch.bfloat16)
        res = torch.randn(M, NA, device="cuda", generator=g).to(torch.bfloat16)
        ya = torch.full((M, NA), float("nan"), device="cuda", dtype=torch.bfloat16)
        yb = torch.full((M, NB), float("nan"), device="cuda", dtype=torch.bfloat16)
        ra, rb = torch.empty_like(ya), torch.empty_like(yb)
        check(lib.coda_b200_skinny_gemm_chain(x.data_ptr(), M, KA, wa.data_ptr(), NA, res.data_ptr(), NA, ya.data_ptr(),
                                              wb.data_ptr(), NB, bias.data_ptr(), yb.data_ptr(), NB,
                                              gsync.data_ptr(), status.data_ptr(), s), "coda_b200_skinny_gemm_chain")
        check(lib.coda_b200_skinny_gemm(x.data_ptr(), M, KA, wa.data_ptr(), NA, res.data_ptr(), NA, ra.data_ptr(), NA,
                                        status.data_ptr(), s), "coda_b200_skinny_gemm")
        check(lib.coda_b200_skinny_gemm_bias(ra.data_ptr(), M, NA, wb.data_ptr(), NB, bias.data_ptr(), None, 0, rb.data_ptr(), NB,
                                             status.data_ptr(), s), "coda_b200_skinny_gemm_bias")
        torch.cuda.synchronize()
        assert int(status.item()) == 0, f"launch {it}"
        assert torch.equal(ya, ra), f"launch {it}: first product"
        assert torch.equal(yb, rb), f"launch {it}: second product"
    assert gsync.tolist() == [0, 12]                       # every launch passed the barrier once and left the count at zero


@pytest.mark.gpu
def test_decode_step_with_own_output_gemm_matches_library_gemm():
    """`use_skinny_gemm_kernel` swaps the decode step's output projection (+ residual) for this library's kernel."""
    from coda_gqa_l_b200 import CoDAGQALandmarkPerf2, _deep_copy_state
    torch.manual_seed(2)
    mod = CoDAGQALandmarkPerf2(embed_dim=512, num_heads=4, num_kv_heads=2, window=48, num_landmarks_exact=16,
                               num_landmarks_summary=16).eval().to(torch.bfloat16).cuda()
    x = orc.mixture_inputs(4, 80, 512, centroids=12, sigma=0.3, seed=3, dtype=torch.bfloat16).cuda()
    sa = mod.init_state(batch_size=4, device="cuda", dtype=torch.bfloat16)
    _, sa = mod.prefill_chunked(x[:, :60], sa, block_size=20)
    sb = _deep_copy_state(sa)
    ya, yb = [], []
    for t in range(60, 80):
        mod.use_skinny_gemm_kernel = True
        y, sa = mod.step(x[:, t:t + 1], sa)
        ya.append(y)
        mod.use_skinny_gemm_kernel = False
        y, sb = mod.step(x[:, t:t + 1], sb)
        yb.append(y)
    assert mod.device_status() == 0
    assert torch.equal(sa.k_buf, sb.k_buf) and torch.equal(sa.allowed, sb.allowed)
    assert rel_err(torch.cat(ya, 1), torch.cat(yb, 1)) < 5e-3


@pytest.mark.gpu
@pytest.mark.parametrize("B,kw", [
    (5, dict(embed_dim=512, num_heads=8, num_kv_heads=2, window=40, num_landmarks_exact=16, num_landmarks_summary=16)),
    # 480 planes on 148 SMs: three or four planes per CTA of the attention kernel that also writes the new token
    (120, dict(embed_dim=256, num_heads=4, num_kv_heads=4, window=40, num_landmarks_exact=16, num_landmarks_summary=16)),
    (40, dict(embed_dim=1024, num_heads=8, num_kv_heads=8, window=150, num_landmarks_exact=24, num_landmarks_summary=24,
              rope_interleaved=False, head_norm_mode="identity")),
    # eight query heads per KV head (two query n-tiles, two heads per auxiliary warp), head_dim 64 and 128
    (6, dict(embed_dim=512, num_heads=8, num_kv_heads=1, window=40, num_landmarks_exact=16, num_landmarks_summary=8)),
    (3, dict(embed_dim=1024, num_heads=8, num_kv_heads=1, window=70, num_landmarks_exact=8, num_landmarks_summary=16,
             write_policy="none")),
    # half-split RoPE at head_dim 64 (two items per auxiliary thread), slot count not a multiple of 64
    (4, dict(embed_dim=256, num_heads=4, num_kv_heads=2, window=37, num_landmarks_exact=9, num_landmarks_summary=7,
             rope_interleaved=False, rope_base=1e6)),
])
def test_split_step_route_then_append_equals_single_launch_step(B, kw):
    """`coda_b200_step_route` + `coda_b200_step_append_fused` (the step in two launches, through
    `route_launch` / `step_graphable(routed=True)`) leave the state exactly as the one-launch `step()` does,
    across the fill -> evict boundary of the ring."""
    from coda_gqa_l_b200 import CoDAGQALandmarkPerf2, _deep_copy_state
    from coda_gqa_l_b200._lib import RingPos
    from tests.scenarios import randomize_weights
    torch.manual_seed(5)
    mod = CoDAGQALandmarkPerf2(**kw).eval()
    randomize_weights(mod, 5)
    mod = mod.to(torch.bfloat16).cuda()
    x = orc.mixture_inputs(B, 30 + 70, kw["embed_dim"], centroids=16, sigma=0.3, seed=8, dtype=torch.bfloat16).cuda()
    sa = mod.init_state(batch_size=B, device="cuda", dtype=torch.bfloat16)
    _, sa = mod.prefill_chunked(x[:, :30], sa, block_size=16)         # ring not yet full
    sb = _deep_copy_state(sa)
    stream = torch.cuda.current_stream().cuda_stream
    ya, yb = [], []
    for t in range(30, 100):
        xt = x[:, t:t + 1]
        rp = RingPos(int(sa.pos), int(sa.recent_idx), int(sa.recent_filled), None)
        assert mod.route_launch(xt.dtype, sa, rp, stream)
        mod.fuse_append_into_attention = t % 3 != 0        # mostly the one-launch second half, sometimes the two-launch one
        ya.append(mod.step_graphable(xt, sa, rp, routed=True))
        mod.advance_host_scalars(sa)
        y, sb = mod.step(xt, sb)
        yb.append(y)
    assert mod.device_status() == 0
    assert (sa.pos, sa.recent_idx, sa.recent_filled) == (sb.pos, sb.recent_idx, sb.recent_filled)
    assert torch.equal(sa.allowed, sb.allowed) and torch.equal(sa.mem_last_exact, sb.mem_last_exact)
    assert torch.equal(sa.k_buf, sb.k_buf) and torch.equal(sa.v_buf, sb.v_buf) and torch.equal(sa.g_recent, sb.g_recent)
    assert torch.equal(sa._exact_v_norm, sb._exact_v_norm) and torch.equal(sa._sum_lf_k_norm, sb._sum_lf_k_norm)
    assert rel_err(torch.cat(ya, 1), torch.cat(yb, 1)) < 5e-3


@pytest.mark.gpu
def test_token_writing_attention_back_to_back_replays_are_stable():
    """The attention kernel that also writes the step's new token, launched back to back on the same inputs and
    ring position (a CUDA graph of four launches, replayed 1000 times; two planes per CTA): rewriting the same
    token is idempotent, so every launch must return the same bits and leave the state as the first one did."""
    import ctypes as C
    from coda_gqa_l_b200 import CoDAGQALandmarkPerf2
    from coda_gqa_l_b200._lib import RingPos, lib, check
    torch.manual_seed(0)
    B, H, Hkv, Dh = 32, 8, 8, 128
    mod = CoDAGQALandmarkPerf2(embed_dim=H * Dh, num_heads=H, num_kv_heads=Hkv, window=256, num_landmarks_exact=64,
                               num_landmarks_summary=64)
    mod = mod.eval().to(torch.bfloat16).cuda()
    st = mod.init_state(batch_size=B, device="cuda", dtype=torch.bfloat16)
    x = (torch.randn(B, 385, H * Dh, device="cuda") * 0.5).to(torch.bfloat16)
    mod.prefill_chunked(x[:, :384], st, block_size=128, return_outputs=False)
    cfg = mod._cfg(B, torch.bfloat16, st)
    assert lib.coda_b200_decode_attend_append_supported(C.byref(cfg))
    rp = RingPos(int(st.pos), int(st.recent_idx), int(st.recent_filled), None)
    assert mod.route_launch(torch.bfloat16, st, rp, torch.cuda.current_stream().cuda_stream)
    q, k, v, lam_logit, gate_logit = mod._project(x[:, 384:385], need_kv=True)
    inv_freq, cos_t, sin_t, _, nw = mod._consts(x.device, torch.bfloat16)
    ptrs = mod._ptrs(st)
    outs = [torch.empty(B, 1, H * Dh, device="cuda", dtype=torch.bfloat16) for _ in range(4)]

    def launch(o):
        check(lib.coda_b200_decode_attend_append(
            C.byref(cfg), C.byref(ptrs), rp, k.data_ptr(), k.stride(0), v.data_ptr(), v.stride(0),
            gate_logit.data_ptr(), gate_logit.stride(0), inv_freq.data_ptr(), q.data_ptr(), q.stride(0),
            lam_logit.data_ptr(), lam_logit.stride(0), cos_t.data_ptr(), sin_t.data_ptr(), None,
            None if nw is None else nw.data_ptr(), o.data_ptr(), o.stride(0), mod._status_word(x.device).data_ptr(),
            torch.cuda.current_stream().cuda_stream), "coda_b200_decode_attend_append")

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        launch(outs[0])
        torch.cuda.synchronize()
        ref = outs[0].clone()
        k_ref, v_ref, al_ref, g_ref = st.k_buf.clone(), st.v_buf.clone(), st.allowed.clone(), st.g_recent.clone()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=side):
            for o in outs:
                launch(o)
        for rep in range(1000):
            g.replay()
            if rep % 250 == 249:
                torch.cuda.synchronize()
                for o in outs:
                    assert torch.equal(o, ref), f"replay {rep}: output changed"
    torch.cuda.synchronize()
    assert mod.device_status() == 0
    assert torch.equal(st.k_buf, k_ref) and torch.equal(st.v_buf, v_ref)
    assert torch.equal(st.allowed, al_ref) and torch.equal(st.g_recent, g_ref)


@pytest.mark.gpu
@pytest.mark.parametrize("M,K,N,bias,res", [
    (32, 4096, 6208, True, False),      # the 7B shape's fused input projection: 48.5 weight tiles, K split three ways
    (32, 4096, 4096, False, True),      # its output projection with the residual
    (64, 8192, 8192, False, True),      # 70B shape, 64 tokens (the wider token tile)
    (33, 1024, 1280, True, True),
    (5, 512, 256, True, True),
    (1, 128, 64, False, False),         # half a weight tile, two k-blocks
    (17, 576, 1000, True, False),       # K = 9 k-blocks, N not a multiple of the tile
    (8, 64, 130, True, True),           # a single k-block per tile: no tile is shared
    (32, 8192, 10368, True, False),     # 70B shape's input projection: 81 tiles, runs of ~70 k-blocks crossing tile boundaries
    (3, 4096, 128, False, True),        # one tile cut into 64 single-k-block runs
])
def test_projection_gemm_matches_library_gemm(M, K, N, bias, res):
    """The decode step's projection kernel (tcgen05, weight rows as the MMA's M, split-K over a cluster, bias and
    residual in the epilogue) against torch: fp32 accumulation on both sides, one bf16 rounding of the product (+ bias),
    a second one after the residual.  x is a row-strided view, as a slice of a longer sequence is."""
    from coda_gqa_l_b200._lib import check, lib
    g = torch.Generator(device="cuda").manual_seed(M * 7 + N)
    xs = (torch.randn(M, 3, K, device="cuda", generator=g) * 0.5).to(torch.bfloat16)
    x = xs[:, 1]                                                    # rows 3*K elements apart
    w = (torch.randn(N, K, device="cuda", generator=g) * 0.05).to(torch.bfloat16)
    b = (torch.randn(N, device="cuda", generator=g)).to(torch.bfloat16) if bias else None
    r = (torch.randn(M, N, device="cuda", generator=g)).to(torch.bfloat16) if res else None
    y = torch.full((M, N + 8), float("nan"), device="cuda", dtype=torch.bfloat16)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    assert lib.coda_b200_proj_gemm_supported(M, K, N)
    ws = torch.zeros(int(lib.coda_b200_proj_gemm_workspace_bytes(M, K, N)), dtype=torch.uint8, device="cuda")
    outs = []
    for _ in range(3):                      # again and again: the tile counters return to zero, the bits repeat
        y.fill_(float("nan"))
        check(lib.coda_b200_proj_gemm(x.data_ptr(), x.stride(0), M, K, w.data_ptr(), N, None if b is None else b.data_ptr(),
                                      None if r is None else r.data_ptr(), N, y.data_ptr(), N + 8, ws.data_ptr(), status.data_ptr(),
                                      torch.cuda.current_stream().cuda_stream), "coda_b200_proj_gemm")
        outs.append(y.clone())
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    assert int(ws[:4096].view(torch.int32).abs().sum()) == 0, "tile counters must be back at zero"
    assert torch.equal(outs[0][:, :N], outs[1][:, :N]) and torch.equal(outs[1][:, :N], outs[2][:, :N])
    ref = x.float() @ w.float().t()
    if bias:
        ref = ref + b.float()
    ref = ref.to(torch.bfloat16)
    if res:
        ref = (ref.float() + r.float()).to(torch.bfloat16)
    got = y[:, :N]
    assert torch.isnan(y[:, N:].float()).all(), "wrote past the row"
    assert torch.isfinite(got.float()).all()
    err = rel_err(got, ref)
    assert err < 4e-3, f"projection gemm rel err {err:.3e}"
    # element-wise: within one bf16 step of the fp32 reference
    assert float((got.float() - ref.float()).abs().max()) <= 2.0 ** -7 * float(ref.float().abs().max())


@pytest.mark.gpu
def test_decode_step_on_own_gemms_matches_library_gemms():
    """`use_own_gemm` swaps both projections of a decode step for coda_b200_proj_gemm; the step must agree
    with the library-GEMM step to bf16 rounding, eagerly and through a captured stack step (where the kernels chain
    as programmatic dependent launches)."""
    from coda_gqa_l_b200 import CoDAGQALandmarkPerf2, CoDAStack, _deep_copy_state
    layers = []
    for i in range(3):
        torch.manual_seed(20 + i)
        layers.append(CoDAGQALandmarkPerf2(embed_dim=1024, num_heads=8, num_kv_heads=2, window=48, num_landmarks_exact=16,
                                           num_landmarks_summary=16).eval().to(torch.bfloat16).cuda())
    stack = CoDAStack(layers)
    x = orc.mixture_inputs(6, 60 + 80, 1024, centroids=12, sigma=0.3, seed=3, dtype=torch.bfloat16).cuda()
    torch.manual_seed(4)
    sa = stack.init_states(batch_size=6, device="cuda", dtype=torch.bfloat16)
    stack.prefill(x[:, :60], sa, block_size=20)
    sb = [_deep_copy_state(s) for s in sa]
    sc_ = [_deep_copy_state(s) for s in sa]
    ya, yb, yc = [], [], []
    for t in range(60, 140):
        for l in layers:
            l.use_own_gemm = True
        ya.append(stack.step_graph(x[:, t:t + 1], sa).clone())
        yc.append(stack.step(x[:, t:t + 1], sc_))
        for l in layers:
            l.use_own_gemm = False
        yb.append(stack.step(x[:, t:t + 1], sb))
    for l in layers:
        assert l.device_status() == 0
    for a, b, c in zip(sa, sb, sc_):
        assert torch.equal(a.allowed, b.allowed) and torch.equal(c.allowed, b.allowed)
        assert rel_err(a.k_buf, b.k_buf) < 5e-3 and rel_err(c.k_buf, b.k_buf) < 5e-3
    assert rel_err(torch.cat(ya, 1), torch.cat(yb, 1)) < 1e-2
    assert rel_err(torch.cat(yc, 1), torch.cat(yb, 1)) < 1e-2


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("interleaved", [True, False])
@pytest.mark.parametrize("Dh,H,Hkv", [(128, 8, 2), (64, 9, 3), (32, 4, 2)])
@pytest.mark.parametrize("spread", [False, True])
def test_vectorised_projection_postprocessing_equals_elementwise_kernel(dtype, interleaved, Dh, H, Hkv, spread):
    """RoPE of q and k, the theta-rotated noise query and the two sigmoids: the 16-byte-vector kernel (aligned rows)
    and the element-wise kernel (here forced by rows that start 2 or 4 bytes off a 16-byte boundary) do the same
    arithmetic, so their results are bit-equal -- in bf16 the vector kernel computes on packed pairs with native
    bf16 instructions, the element-wise one in fp32 with a rounding after every operation.  ``spread`` scales every
    input element by its own power of two (2^-120 .. 2^30), so that partners of a rotation lie many binades apart and
    results fall into the subnormal range."""
    from coda_gqa_l_b200 import CoDAGQALandmarkPerf2
    from tests.scenarios import randomize_weights
    torch.manual_seed(1)
    mod = CoDAGQALandmarkPerf2(embed_dim=H * Dh, num_heads=H, num_kv_heads=Hkv, window=16, num_landmarks_exact=4,
                               num_landmarks_summary=4, rope_interleaved=interleaved, rope_base=1e6).eval()
    randomize_weights(mod, 2)
    mod = mod.to(dtype).cuda()
    B, L = 3, 37
    st = mod.init_state(batch_size=B, device="cuda", dtype=dtype)
    cfg = mod._cfg(B, dtype, st)
    g = torch.Generator(device="cuda").manual_seed(3)
    nq, nk = H * Dh, Hkv * Dh
    pad = 8 if dtype == torch.bfloat16 else 4                    # keeps every row start 16-byte aligned in the base layout
    width = (nq + nk + H + 1 + pad + 7) // 8 * 8
    outs = []
    for shift in (0, 1):                                         # shift 1: every row starts one element off alignment
        y = torch.zeros(B, L, width + 8, device="cuda", dtype=dtype)
        src = torch.randn(B, L, nq + nk + H + 1, device="cuda", generator=torch.Generator(device="cuda").manual_seed(4))
        if spread:
            e = torch.randint(-120, 31, src.shape, device="cuda", generator=torch.Generator(device="cuda").manual_seed(5))
            src = torch.ldexp(src, e)
        src = src.to(dtype)
        y[..., shift:shift + nq + nk + H + 1] = src
        q, k = y[..., shift:shift + nq], y[..., shift + nq:shift + nq + nk]
        lam_logit, gate_logit = y[..., shift + nq + nk:shift + nq + nk + H], y[..., shift + nq + nk + H:shift + nq + nk + H + 1]
        qn, lam, gate = mod._prep(cfg, L, 1000, q, k, lam_logit, gate_logit, True)
        outs.append((q.clone(), k.clone(), qn.clone(), lam.clone(), gate.clone()))
    torch.cuda.synchronize()
    for a, b, name in zip(outs[0], outs[1], ("q", "k", "q_noise", "lambda", "gate")):
        assert torch.equal(a, b), f"{name} differs between the vector and the element-wise kernel"
    assert not torch.equal(outs[0][0], outs[0][2])               # the noise rotation did something


@pytest.mark.gpu
def test_four_way_gemm_plan_keeps_its_clusters_resident():
    """The launcher of the four-way GEMM sizes its tiles from the device's own answer to "how many clusters of four
    fit at once": every planned launch is one wave, and its tiles cover all weight rows."""
    import ctypes as C
    from coda_gqa_l_b200._lib import lib
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    for K, N in ((4096, 4096), (4096, 6208), (2048, 4096), (1024, 1088), (256, 64)):
        t, c = C.c_int32(), C.c_int32()
        if not lib.coda_b200_skinny_gemm_plan(K, N, C.byref(t), C.byref(c)):
            continue
        assert t.value % 16 == 0 and 16 <= t.value <= 192
        assert c.value * t.value >= N and (c.value - 1) * t.value < N
        assert 4 * c.value <= sms
