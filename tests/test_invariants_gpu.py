"""GPU: state invariants, edge configurations and determinism of the CUDA module, restating what upstream's own
suite asserts of its PyTorch module (tests/test_invariants.py, tests/test_edge_configs.py:111-240,
tests/test_correctness.py:332-424, tests/test_determinism.py:150-275 of the upstream project), on small fp32 shapes."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu

D, H, HKV, W, ME, MS = 128, 4, 2, 32, 16, 16


def _module(**over):
    from coda_gqa_l_b200 import CoDAGQALandmarkPerf2
    kw = dict(embed_dim=D, num_heads=H, num_kv_heads=HKV, window=W, num_landmarks_exact=ME, num_landmarks_summary=MS)
    kw.update(over)
    return CoDAGQALandmarkPerf2(**kw).eval().cuda()


def _fresh(batch=1, seed=0, **over):
    torch.manual_seed(seed)
    m = _module(**over)
    return m, m.init_state(batch_size=batch, device="cuda", dtype=torch.float32)


def _x(b, n, d=D):
    return torch.randn(b, n, d, device="cuda")


def _feed(m, st, pattern, batch=1):
    """pattern: list of ("p", tokens, block) prefill calls and ("d", steps) decode runs; yields the state after each
    single call so that per-call properties can be asserted."""
    for op in pattern:
        if op[0] == "p":
            _, st = m.prefill_chunked(_x(batch, op[1], m.embed_dim), st, block_size=op[2], return_outputs=False)
            yield st
        else:
            for _ in range(op[1]):
                _, st = m.step(_x(batch, 1, m.embed_dim), st)
                yield st


@pytest.mark.parametrize("pattern", [
    [("p", 100, 64), ("d", 50)],
    [("d", 70), ("p", 45, 16), ("d", 40), ("p", 3, 8), ("d", 5)],
    [("p", 1, 64), ("p", 31, 7), ("p", 1, 1), ("d", 3), ("p", 200, 64)],
])
def test_ring_scalars_follow_the_token_count(pattern):
    """pos counts every written token; recent_filled == min(pos, W); recent_idx stays inside the ring, is 0 after a
    prefill call and walks one slot per decode step once the ring is full; the ring part of `allowed` covers exactly
    the filled slots."""
    m, st = _fresh(batch=2)
    seen, prev_idx = 0, 0
    ops = [o for op in pattern for o in ([op] if op[0] == "p" else [("d", 1)] * op[1])]
    for op, st in zip(ops, _feed(m, st, pattern, batch=2)):
        was_full = seen >= W
        seen += op[1]
        assert st.pos == seen and st.recent_filled == min(seen, W) and 0 <= st.recent_idx < W
        if op[0] == "p":
            assert st.recent_idx == 0
        else:
            assert st.recent_idx == ((prev_idx + 1) % W if was_full else prev_idx)
        prev_idx = st.recent_idx
        ring = st.allowed[:, :W]
        assert int(ring.sum()) == 2 * min(seen, W)
        if seen < W:
            assert bool(ring[:, :seen].all()) and not bool(ring[:, seen:].any())


def test_bank_occupancy_only_grows_and_is_bounded():
    """Bank slots are never released: the allowed counts of both banks are non-decreasing over prefill chunks and
    decode steps; the total never exceeds the buffer, nor the number of tokens seen."""
    m, st = _fresh(write_policy="none")
    pe = ps = 0
    for st in _feed(m, st, [("p", W, W)] * 5 + [("d", 2 * W)]):
        e, s = int(st.allowed[:, W:W + ME].sum()), int(st.allowed[:, W + ME:].sum())
        assert e >= pe and s >= ps
        pe, ps = e, s
        assert int(st.allowed.sum()) <= min(m.Lbuf, st.pos)
    assert pe > 0 and ps > 0


def test_lru_stamps_and_norm_caches_track_the_banks():
    """Used exact slots carry the (non-negative) position of the token that last touched them, unused ones keep 0;
    the two routing caches equal F.normalize of the bank rows they mirror, after block and single-token updates."""
    m, st = _fresh(batch=2, write_policy="none")
    for st in _feed(m, st, [("p", 3 * W, 16), ("d", W + 5)], batch=2):
        pass
    used = st.allowed[:, W:W + ME]
    assert bool((st.mem_last_exact[used] >= 0).all()) and bool((st.mem_last_exact[~used] == 0).all())
    assert bool((st.mem_last_exact < st.pos).all())
    want_v = F.normalize(st.v_buf[:, :, W:W + ME], dim=-1, eps=1e-6)
    want_k = F.normalize(st.k_buf[:, :, W + ME:, m.lf_start:], dim=-1, eps=1e-6)
    assert torch.allclose(st._exact_v_norm, want_v, atol=1e-5)
    assert torch.allclose(st._sum_lf_k_norm, want_k, atol=1e-5)


def test_summary_keys_keep_a_zero_high_frequency_band():
    """Only the low-frequency half of a summary key is ever blended; the other half stays exactly zero."""
    m, st = _fresh(seed=1)
    lo = W + ME
    assert float(st.k_buf[:, :, lo:, :m.lf_start].abs().max()) == 0.0
    for st in _feed(m, st, [("p", 512, 128), ("d", 40)]):
        pass
    assert bool(st.allowed[:, lo:].any())
    assert float(st.k_buf[:, :, lo:, :m.lf_start].abs().max()) == 0.0


def test_block_queries_see_the_whole_prefix():
    """Prefill attention is prefix-visible + causal inside the block (not upper-left triangular): the first query
    of a block reacts to a change of the LAST valid prefix slot."""
    from coda_gqa_l_b200 import _deep_copy_state
    m, st = _fresh(seed=2)
    _, st = m.prefill_chunked(_x(1, W), st, block_size=W, return_outputs=False)
    xb = _x(1, 32)
    y0, _ = m.prefill_chunked(xb, st, block_size=32, write_cache=False)
    bad = _deep_copy_state(st)
    last = int(bad.allowed[0].nonzero()[-1])
    bad.k_buf[:, :, last, :] += 100.0
    y1, _ = m.prefill_chunked(xb, bad, block_size=32, write_cache=False)
    assert float((y0[:, 0] - y1[:, 0]).abs().max()) > 0.01
    # ... and no query reacts to a later token of its own block
    xc = xb.clone()
    xc[:, 20:] += 3.0
    y2, _ = m.prefill_chunked(xc, st, block_size=32, write_cache=False)
    assert torch.equal(y0[:, :20], y2[:, :20]) and not torch.equal(y0[:, 20:], y2[:, 20:])


@pytest.mark.parametrize("over,prefill,steps,block", [
    (dict(num_landmarks_exact=0), 100, 20, 32),
    (dict(num_landmarks_summary=0), 100, 20, 32),
    (dict(num_landmarks_exact=0, num_landmarks_summary=0), 100, 20, 32),
    (dict(window=4), 40, 20, 16),
    (dict(window=1), 20, 10, 8),
    (dict(write_policy="none"), 100, 20, 32),
    (dict(exact_refresh_on_hit=True), 100, 20, 32),
    (dict(summary_overwrite_on_insert=False), 100, 20, 32),
    (dict(mem_init="zeros"), 100, 20, 32),
    (dict(mask_unused_memory=False), 100, 20, 32),
    (dict(window=64), 1, 3, 256),                 # a single prefill token
    (dict(), W, 5, 256),                          # exactly one window: nothing evicted yet
    (dict(), W + 1, 5, 256),                      # exactly one token evicted
    (dict(window=64), 64, 0, 1024),               # block larger than the sequence
])
def test_edge_configurations_run_clean(over, prefill, steps, block):
    """Zero-sized banks, tiny windows, policy switches and eviction-boundary lengths: right shapes, finite values,
    position advanced by exactly the tokens fed; zero-sized banks carry no routing cache."""
    m, st = _fresh(batch=2, seed=3, **over)
    assert st.k_buf.shape == (2, HKV, m.Lbuf, D // H) and st.allowed.shape == (2, m.Lbuf)
    assert st.g_recent.shape == (2, m.window) and st.mem_last_exact.shape == (2, m.Me)
    assert (st._exact_v_norm is None) == (m.Me == 0) and (st._sum_lf_k_norm is None) == (m.Ms == 0)
    y, st = m.prefill_chunked(_x(2, prefill), st, block_size=block)
    assert y.shape == (2, prefill, D) and bool(torch.isfinite(y).all()) and st.pos == prefill
    for i in range(steps):
        y, st = m.step(_x(2, 1), st)
        assert y.shape == (2, 1, D) and bool(torch.isfinite(y).all())
    assert st.pos == prefill + steps and y.dtype == torch.float32
    none, st2 = m.prefill_chunked(_x(2, 9), st, block_size=4, write_cache=False, return_outputs=False)
    assert none is None and st2.pos == prefill + steps


def test_same_seeds_same_bits_different_seeds_differ():
    """Two runs from the same seeds agree bit for bit in outputs and state (prefill with evictions, then decode);
    another input seed gives different outputs."""
    def run(model_seed, input_seed):
        torch.manual_seed(model_seed)
        m = _module()
        torch.manual_seed(99)
        st = m.init_state(batch_size=2, device="cuda", dtype=torch.float32)
        g = torch.Generator(device="cuda").manual_seed(input_seed)
        x = torch.randn(2, 200 + 64, D, device="cuda", generator=g)
        y, st = m.prefill_chunked(x[:, :200], st, block_size=64)
        ys = [y] + [m.step(x[:, t:t + 1], st)[0] for t in range(200, 264)]
        return torch.cat(ys, 1), st
    ya, sa = run(42, 7)
    yb, sb = run(42, 7)
    assert torch.equal(ya, yb)
    for f in ("k_buf", "v_buf", "allowed", "g_recent", "mem_last_exact", "_exact_v_norm", "_sum_lf_k_norm"):
        assert torch.equal(getattr(sa, f), getattr(sb, f)), f
    yc, _ = run(42, 8)
    assert not torch.equal(ya, yc)


def test_captured_step_notices_writes_made_outside_it():
    """A captured stack step bakes the ring scalars in and advances them with its own device counter.  An eager
    step (or prefill) between two replays moves the state without that counter: the next replay must capture
    again instead of overwriting the wrong ring slot.  Checked against running everything eagerly."""
    from coda_gqa_l_b200 import CoDAGQALandmarkPerf2, CoDAStack, _deep_copy_state
    kw = dict(embed_dim=256, num_heads=4, num_kv_heads=2, window=24, num_landmarks_exact=8, num_landmarks_summary=8)
    layers = []
    for i in range(2):
        torch.manual_seed(i)
        layers.append(CoDAGQALandmarkPerf2(**kw).eval().to(torch.bfloat16).cuda())
    stack = CoDAStack(layers)
    torch.manual_seed(5)
    sa = stack.init_states(batch_size=3, device="cuda", dtype=torch.bfloat16)
    x = (torch.randn(3, 120, 256, device="cuda") * 0.5).to(torch.bfloat16)
    stack.prefill(x[:, :40], sa, block_size=16)
    sb = [_deep_copy_state(s) for s in sa]
    ya, yb = [], []
    for t in range(40, 100):
        kind = "eager" if t % 7 == 3 else ("layer" if t % 11 == 5 else "graph")
        if kind == "graph":
            ya.append(stack.step_graph(x[:, t:t + 1], sa).clone())
        elif kind == "eager":
            ya.append(stack.step(x[:, t:t + 1], sa))
        else:                                   # a write through the layers themselves, behind the stack's back
            h = x[:, t:t + 1]
            for l, s in zip(stack.layers, sa):
                h = h + l.step(h, s)[0]
            ya.append(h)
        yb.append(stack.step(x[:, t:t + 1], sb))
    for a, b in zip(sa, sb):
        assert (a.pos, a.recent_idx, a.recent_filled) == (b.pos, b.recent_idx, b.recent_filled)
        assert torch.equal(a.allowed, b.allowed) and torch.equal(a.mem_last_exact, b.mem_last_exact)
    ea = (torch.cat(ya, 1).double() - torch.cat(yb, 1).double()).norm() / torch.cat(yb, 1).double().norm()
    assert float(ea) < 2e-2
    # a reloaded weight is noticed too
    sd = {k: v.clone() for k, v in stack.layers[0].state_dict().items()}
    sd["theta"] = sd["theta"] * 0.5
    stack.step_graph(x[:, 100:101], sa)
    g0 = stack._graph["graph"]
    stack.layers[0].load_state_dict(sd)
    stack.step_graph(x[:, 101:102], sa)
    assert stack._graph["graph"] is not g0


def test_a_wait_that_runs_out_reports_and_releases_the_cta():
    """The bounded wait all pipelined kernels use, on barriers nobody arrives at: the short wait gives up and
    leaves its code in the status word and the CTA's abort word; the long wait of the same CTA sees the abort
    word and leaves at once instead of polling to its own limit; the context stays usable afterwards."""
    from coda_gqa_l_b200._lib import check, lib
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    report = torch.full((5,), -1, dtype=torch.int32, device="cuda")
    check(lib.coda_b200_selftest_bounded_wait(2048, status.data_ptr(), report.data_ptr(),
                                              torch.cuda.current_stream().cuda_stream), "coda_b200_selftest_bounded_wait")
    torch.cuda.synchronize()
    r = report.tolist()
    assert int(status.item()) == 77, "the first wait to give up names itself in the status word"
    assert r[0] == 0 and r[2] == 0 and r[4] == 77
    # the second waiter was released by the abort word: it took about as long as the first, not 2048x longer
    assert r[3] <= 4 * r[1] + 100_000, r
    assert float((torch.ones(8, device="cuda") * 2).sum()) == 16.0          # the context still works
    with pytest.raises(RuntimeError):
        check(lib.coda_b200_selftest_bounded_wait(0, status.data_ptr(), report.data_ptr(), None), "selftest")


@pytest.mark.gpu
def test_host_fed_captured_step_equals_device_fed_one():
    """`step_graph_host` carries the host-to-device copy, the step and the device-to-host copy in one graph; its
    results and the states it leaves equal those of `step_graph` on a device tensor bit for bit, and replays of
    the two graphs may be mixed (they advance one device counter)."""
    from coda_gqa_l_b200 import CoDAGQALandmarkPerf2, CoDAStack, _deep_copy_state
    kw = dict(embed_dim=256, num_heads=4, num_kv_heads=2, window=24, num_landmarks_exact=8, num_landmarks_summary=8)
    layers = []
    for i in range(2):
        torch.manual_seed(i)
        layers.append(CoDAGQALandmarkPerf2(**kw).eval().to(torch.bfloat16).cuda())
    sa_stack, sb_stack = CoDAStack(layers), CoDAStack(layers)
    torch.manual_seed(6)
    sa = sa_stack.init_states(batch_size=3, device="cuda", dtype=torch.bfloat16)
    x = (torch.randn(3, 90, 256, device="cuda") * 0.5).to(torch.bfloat16)
    sa_stack.prefill(x[:, :40], sa, block_size=16)
    sb = [_deep_copy_state(s) for s in sa]
    xh = x.cpu().pin_memory()
    for t in range(40, 90):
        if t % 5 == 2:                                   # a device-fed replay in between
            ya = sa_stack.step_graph(x[:, t:t + 1], sa).clone()
        else:
            out = sa_stack.step_graph_host(xh[:, t:t + 1], sa)
            torch.cuda.current_stream().synchronize()
            assert out.device.type == "cpu" and out.is_pinned()
            ya = out.cuda()
        yb = sb_stack.step_graph(x[:, t:t + 1], sb)
        assert torch.equal(ya, yb), f"token {t}"
    for a, b in zip(sa, sb):
        assert (a.pos, a.recent_idx, a.recent_filled) == (b.pos, b.recent_idx, b.recent_filled)
        assert torch.equal(a._arena, b._arena)


@pytest.mark.gpu
def test_block_routing_beside_attention_equals_routing_after_it():
    """Chunked prefill can run the scores and decisions of a block's routing on a second stream beside the block's
    attention (`overlap_block_routing`; they read what it reads and write nothing it reads).  Outputs and states
    equal the serial order's bit for bit, over several chunks and with decode steps in between."""
    from coda_gqa_l_b200 import CoDAGQALandmarkPerf2
    kw = dict(embed_dim=512, num_heads=8, num_kv_heads=2, window=48, num_landmarks_exact=16, num_landmarks_summary=16)
    torch.manual_seed(3)
    mod = CoDAGQALandmarkPerf2(**kw).eval().to(torch.bfloat16).cuda()
    x = (torch.randn(3, 400, 512, device="cuda") * 0.5).to(torch.bfloat16)
    outs, states = [], []
    for overlap in (True, False):
        mod.overlap_block_routing = overlap
        torch.manual_seed(9)
        st = mod.init_state(batch_size=3, device="cuda", dtype=torch.bfloat16)
        ys = []
        y, st = mod.prefill_chunked(x[:, :160], st, block_size=32); ys.append(y)
        for t in range(160, 170):
            y, st = mod.step(x[:, t:t + 1], st); ys.append(y)
        y, st = mod.prefill_chunked(x[:, 170:400], st, block_size=64); ys.append(y)      # ragged last block
        torch.cuda.synchronize()
        outs.append(torch.cat(ys, 1)); states.append(st)
    mod.overlap_block_routing = False
    assert torch.equal(outs[0], outs[1])
    a, b = states
    assert (a.pos, a.recent_idx, a.recent_filled) == (b.pos, b.recent_idx, b.recent_filled)
    assert torch.equal(a._arena, b._arena)


def test_stack_prefill_with_the_residual_in_the_output_projection():
    """`CoDAStack.prefill` lets the output projection take the residual (one rounding of accumulator + residual;
    from the second layer on into the chain's own buffer).  Against the chain written out with a separate add:
    the caller's chunk is left untouched, the first layer's state is identical (its input is the same tensor),
    the outputs agree to bf16 rounding, and in fp32 the two chains are equal to accumulation order."""
    from coda_gqa_l_b200 import CoDAGQALandmarkPerf2, CoDAStack
    kw = dict(embed_dim=256, num_heads=4, num_kv_heads=2, window=24, num_landmarks_exact=8, num_landmarks_summary=8)
    for dtype, tol in ((torch.bfloat16, 3e-2), (torch.float32, 2e-5)):
        layers = []
        for i in range(3):
            torch.manual_seed(i)
            layers.append(CoDAGQALandmarkPerf2(**kw).eval().to(dtype).cuda())
        stack = CoDAStack(layers)
        torch.manual_seed(9)
        x = (torch.randn(2, 70, 256, device="cuda") * 0.5).to(dtype)
        x_before = x.clone()
        torch.manual_seed(10)                            # the banks start from N(0, 0.02^2) draws: same draws for both
        sa = stack.init_states(batch_size=2, device="cuda", dtype=dtype)
        torch.manual_seed(10)
        sb = stack.init_states(batch_size=2, device="cuda", dtype=dtype)
        ya = stack.prefill(x, sa, block_size=16)
        assert torch.equal(x, x_before)
        h = x
        for layer, st in zip(layers, sb):
            y, _ = layer.prefill_chunked(h, st, block_size=16)
            h = h + y
        for name in ("k_buf", "v_buf", "allowed", "g_recent", "mem_last_exact"):
            assert torch.equal(getattr(sa[0], name), getattr(sb[0], name)), name
        assert ya.shape == h.shape and ya.data_ptr() != x.data_ptr()
        err = (ya.float() - h.float()).abs().max().item() / h.float().abs().max().item()
        assert err < tol, (dtype, err)
        for a, b in zip(sa, sb):
            assert (a.pos, a.recent_idx, a.recent_filled) == (b.pos, b.recent_idx, b.recent_filled)


def test_captured_step_with_chained_projections_equals_the_unchained_one():
    """With `chain_projections` a layer's output projection and the next layer's input projection leave in one launch
    (two phases, a barrier across the grid between them).  Against the same stack with the two products as launches of
    their own (`use_skinny_in_proj`, so that both run this library's GEMM): the same bits in every output and state."""
    from coda_gqa_l_b200 import CoDAGQALandmarkPerf2, CoDAStack, _deep_copy_state
    kw = dict(embed_dim=256, num_heads=4, num_kv_heads=2, window=24, num_landmarks_exact=8, num_landmarks_summary=8)
    layers = []
    for i in range(4):
        torch.manual_seed(i)
        l = CoDAGQALandmarkPerf2(**kw).eval().to(torch.bfloat16).cuda()
        l.use_skinny_in_proj = True
        layers.append(l)
    sa_stack, sb_stack = CoDAStack(layers), CoDAStack(layers)
    sa_stack.chain_projections, sb_stack.chain_projections = True, False
    torch.manual_seed(6)
    sa = sa_stack.init_states(batch_size=3, device="cuda", dtype=torch.bfloat16)
    x = (torch.randn(3, 90, 256, device="cuda") * 0.5).to(torch.bfloat16)
    sa_stack.prefill(x[:, :40], sa, block_size=16)
    sb = [_deep_copy_state(s) for s in sa]
    for t in range(40, 90):
        ya = sa_stack.step_graph(x[:, t:t + 1], sa).clone()
        yb = sb_stack.step_graph(x[:, t:t + 1], sb)
        assert torch.equal(ya, yb), f"token {t}"
    assert sa_stack._graph["chained"] and not sb_stack._graph["chained"]
    assert sa_stack._graph["gsync"].tolist() == [0, 50 * 3]            # three chained launches per step, each passed its barrier
    for l in layers:
        assert l.device_status() == 0
    for a, b in zip(sa, sb):
        assert (a.pos, a.recent_idx, a.recent_filled) == (b.pos, b.recent_idx, b.recent_filled)
        assert torch.equal(a._arena, b._arena)
