"""CPU: the oracle reproduces the fixtures generated from the upstream implementation, starting
from weights and initial state rebuilt here from seeds (no upstream code needed)."""
import pytest
import torch

from tests.helpers import (SCENARIOS, build_inputs, build_module, load_golden, oracle_state_from, orc, rel_err,
                           weights_checksum, weights_of)


@pytest.mark.parametrize("name", [n for n in SCENARIOS if n != "c1"] + ["c1"])
def test_oracle_matches_golden(name):
    sc = SCENARIOS[name]
    dtype = getattr(torch, sc.get("dtype", "float32"))
    gold = load_golden(name)
    mod = build_module(sc, dtype)
    wts = weights_of(mod)
    assert abs(weights_checksum(wts) - gold["weights_abs_sum"]) <= 1e-9 * gold["weights_abs_sum"], \
        "seeded default weights differ from the ones the fixture was generated with"
    cfg = orc.OracleConfig.from_module(mod)
    assert gold["cache_bytes"] == mod.cache_bytes(batch_size=sc["B"], dtype=dtype) == orc.cache_bytes(cfg, sc["B"], dtype)
    torch.manual_seed(sc["state_seed"])
    st = oracle_state_from(mod.init_state(batch_size=sc["B"], device="cpu", dtype=dtype))
    x_pre, x_dec = build_inputs(sc, dtype)
    stride = gold["y_stride"]
    tol = 2e-5 if dtype == torch.float32 else 3e-2
    for i, phase in enumerate(sc["phases"]):
        if phase[0] == "prefill":
            y = orc.prefill_chunked(cfg, wts, x_pre[:, phase[1]:phase[2]], st, block_size=phase[3])
        else:
            y = torch.cat([orc.step(cfg, wts, x_dec[:, t:t + 1], st) for t in range(phase[1], phase[2])], 1)
        snap = gold["snapshots"][i]
        assert rel_err(y[:, ::stride], gold["y"][i]) < tol
        assert (st.recent_idx, st.recent_filled, st.pos) == (snap["recent_idx"], snap["recent_filled"], snap["pos"])
        if dtype == torch.float32:
            assert torch.equal(st.allowed, snap["allowed"])
            assert torch.equal(st.mem_last_exact, snap["mem_last_exact"])
            assert rel_err(st.k_buf[:, :, -8:], snap["k_bank"]) < tol
            assert rel_err(st.v_buf[:, :, -8:], snap["v_bank"]) < tol


def test_known_answer_c1_slots():
    """Slot-level facts measured on the upstream implementation for the config-1 shape: with the default
    constant gate the first evicting block selects positions 160,191,190,... and fills exact slots 40..47."""
    gold = load_golden("c1")
    ev = [e for e in gold["trace_head"] if e[0] == "exact_block"]
    first = ev[0]
    assert first[1][0].tolist() == [160, 191, 190, 189, 188, 187, 186, 185]
    assert first[2][0].tolist() == [44, 41, 42, 43, 46, 47, 40, 45]
    assert ev[1][1][0].tolist()[:2] == [416, 447]
    assert sorted(ev[1][2][0].tolist()) == [30, 35, 36, 37, 38, 39, 48, 49]


@pytest.mark.parametrize("name", ["c2_stack2", "c3_layer"])
def test_oracle_matches_geometry_fixture(name):
    """The benchmark-geometry fixtures (bf16, stacks chained as h <- h + layer(h)) re-derived by the oracle from
    seeds: outputs within the bf16 tolerance of upstream's, ring scalars exact."""
    from tests.scenarios import GEOMETRY_SCENARIOS
    from tests.test_geometry_gpu import _build
    sc = GEOMETRY_SCENARIOS[name]
    dtype = getattr(torch, sc["dtype"])
    gold = load_golden(name)
    mods, sts = _build(sc, dtype)
    nl = len(mods)
    wts = [weights_of(m) for m in mods]
    cfgs = [orc.OracleConfig.from_module(m) for m in mods]
    for w, want in zip(wts, gold["weights_abs_sum"]):
        assert abs(weights_checksum(w) - want) <= 1e-9 * want
    osts = [oracle_state_from(s) for s in sts]
    x_pre, x_dec = build_inputs(sc, dtype)
    ts, fs = gold["y_stride"], gold.get("y_fstride", 1)

    def through(fn, h):
        for c, w, o in zip(cfgs, wts, osts):
            y = fn(c, w, h, o)
            h = h + y if nl > 1 else y
        return h

    for i, phase in enumerate(sc["phases"]):
        if phase[0] == "prefill":
            y = through(lambda c, w, h, o: orc.prefill_chunked(c, w, h, o, block_size=phase[3]), x_pre[:, phase[1]:phase[2]])
        else:
            y = torch.cat([through(orc.step, x_dec[:, t:t + 1]) for t in range(phase[1], phase[2])], 1)
        assert rel_err(y[:, ::ts, ::fs], gold["y"][i]) < 3e-2
        for o, snap in zip(osts, gold["snapshots"][i]):
            assert (o.recent_idx, o.recent_filled, o.pos) == (snap["recent_idx"], snap["recent_filled"], snap["pos"])
