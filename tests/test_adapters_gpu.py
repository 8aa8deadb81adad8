"""GPU: the Llama and Eve adapters driven the way a host model drives them -- one multi-token forward (routed to
``prefill_chunked`` with the adapter's block size), then single-token forwards (routed to ``step``) on the state
the adapter owns, then the state handed to a second adapter with ``get_state`` / ``set_state`` -- against
fixtures produced by upstream's adapters (``src/coda_gqa_l/llama_adapter.py:342-383``,
``src/coda_gqa_l/eve_adapter.py:203-243,343-369``) on the same seeded stand-in attention modules.

Bar: fp32 outputs within 1e-4 relative, slot occupancy / LRU stamps / ring scalars bit-exact; bf16 within 2e-2."""
import warnings

import pytest
import torch

from tests.helpers import TOL_BF16, TOL_F32, load_golden, orc, rel_err
from tests.scenarios import ADAPTER_SCENARIOS, fake_eve_attention, fake_llama_attention

pytestmark = pytest.mark.gpu


def _make_pair(sc):
    """Two adapters built one after the other from ONE stand-in attention module, as the fixture generator does:
    the lambda projection keeps its random initialisation, so the second adapter's differs from the first's."""
    from coda_gqa_l_b200 import EveCoDAAdapter, LlamaCoDAAdapter
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        if sc["kind"] == "llama":
            src = fake_llama_attention(sc)
            return [LlamaCoDAAdapter.from_llama_attention(src, bounded=True, **sc["kwargs"]) for _ in range(2)]
        src = fake_eve_attention(sc)
        return [EveCoDAAdapter.from_eve_attention(src, bounded=True, **sc["kwargs"]) for _ in range(2)]


@pytest.mark.parametrize("name", list(ADAPTER_SCENARIOS))
def test_adapter_forward_matches_upstream_adapter(name):
    from coda_gqa_l_b200 import _deep_copy_state, state_from_fields
    sc = ADAPTER_SCENARIOS[name]
    dtype = getattr(torch, sc.get("dtype", "float32"))
    f32 = dtype == torch.float32
    tol = TOL_F32 if f32 else TOL_BF16
    gold = load_golden(name)
    ad, ad2 = (a.eval().to(dtype) for a in _make_pair(sc))
    got = float(sum(v.double().abs().sum() for v in ad.coda.state_dict().values()))
    assert abs(got - gold["weights_abs_sum"]) <= 1e-6 * gold["weights_abs_sum"], "adapter weights differ from upstream's"
    assert ad.cache_bytes(batch_size=sc["B"], dtype=dtype) == gold["cache_bytes"]
    if sc["kind"] == "eve" and sc["bias"]:
        assert ad.coda.q_proj.bias is not None and ad.coda.o_proj.bias is not None
    B, L, Ld = sc["B"], sc["L"], sc["Ldec"]
    x = orc.mixture_inputs(B, L + Ld, sc["hidden"], centroids=24, sigma=0.4, seed=sc["input_seed"], dtype=dtype).cuda()
    if sc.get("seeded_state"):
        # random-normal banks drawn from the CPU generator, as the fixture's were, then handed to the adapter
        torch.manual_seed(sc["state_seed"])
        st_cpu = ad.coda.init_state(batch_size=B, device="cpu", dtype=dtype)
        ad.set_state(state_from_fields(st_cpu, "cuda"))
    ad, ad2 = ad.cuda(), ad2.cuda()
    call = (lambda a, t: a(t, past_key_value="kv")) if sc["kind"] == "llama" else (lambda a, t: a(t))

    def out(r):
        if sc["kind"] == "llama":
            assert isinstance(r, tuple) and len(r) == 2 and r[1] == "kv"      # (output, past_key_value passed through)
            return r[0]
        return r

    y_pre = out(call(ad, x[:, :L]))
    assert ad.get_state().pos == L and y_pre.shape == (B, L, sc["hidden"])
    half = Ld // 2
    y1 = torch.cat([out(call(ad, x[:, L + t:L + t + 1])) for t in range(half)], 1)
    ad2.set_state(_deep_copy_state(ad.get_state()))
    y2 = torch.cat([out(call(ad2, x[:, L + t:L + t + 1])) for t in range(half, Ld)], 1)
    torch.cuda.synchronize()
    assert ad.get_state().pos == L + half            # the first adapter's state was not advanced by the second
    for tag, y, want in zip(("prefill", "steps", "steps after set_state"), (y_pre, y1, y2), gold["y"]):
        e = rel_err(y, want)
        assert e < tol, f"{name} {tag}: rel err {e:.3e} vs upstream adapter"
    st, snap = ad2.get_state(), gold["snapshot"]
    assert (st.recent_idx, st.recent_filled, st.pos) == (snap["recent_idx"], snap["recent_filled"], snap["pos"])
    if f32:
        assert torch.equal(st.allowed.cpu(), snap["allowed"]) and torch.equal(st.mem_last_exact.cpu(), snap["mem_last_exact"])
        assert rel_err(st.k_buf[:, :, -8:], snap["k_bank"]) < tol and rel_err(st.v_buf[:, :, -8:], snap["v_bank"]) < tol
    assert ad.coda.device_status() == 0 and ad2.coda.device_status() == 0
    ad.reset_state()
    assert ad.get_state() is None
