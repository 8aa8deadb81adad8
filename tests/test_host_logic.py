"""CPU: host-side behaviour of the drop-in classes (no kernel is launched)."""
import io

import pytest
import torch

from coda_gqa_l_b200 import (CoDAGQALandmarkPerf2, CoDAGQALandmarkStatePerf2, EveCoDAAdapter, LlamaCoDAAdapter, Qwen3CoDAAdapter,
                             _deep_copy_state, _state_to_cpu, _state_to_device, state_from_fields)
from coda_gqa_l_b200.state import arena_layout

KW = dict(embed_dim=128, num_heads=4, num_kv_heads=2, window=32, num_landmarks_exact=16, num_landmarks_summary=16)


def test_constructor_validation_messages():
    bad = [(dict(KW, embed_dim=130), "embed_dim must be divisible"), (dict(KW, num_kv_heads=3), "num_heads must be divisible"),
           (dict(KW, window=0), "window must be positive"), (dict(KW, num_landmarks_exact=-1), "non-negative"),
           (dict(KW, head_norm_mode="x"), "head_norm_mode"), (dict(KW, embed_dim=12, num_heads=4, num_kv_heads=2), "even"),
           (dict(KW, min_landmarks_exact=20), "min_landmarks_exact")]
    for kw, msg in bad:
        with pytest.raises(ValueError, match=msg):
            CoDAGQALandmarkPerf2(**kw)


def test_state_dict_keys_and_cache_bytes():
    m = CoDAGQALandmarkPerf2(embed_dim=512, num_heads=8, num_kv_heads=2, window=256, num_landmarks_exact=64,
                             num_landmarks_summary=64)
    assert list(m.state_dict().keys()) == [
        "theta", "summary_eta_logit", "q_proj.weight", "k_proj.weight", "v_proj.weight", "lambda_proj.weight",
        "lambda_proj.bias", "write_proj.weight", "write_proj.bias", "head_norm.weight", "o_proj.weight"]
    # values published for this shape by the upstream project
    assert m.cache_bytes(batch_size=1, dtype=torch.float32) == 444_288
    assert m.cache_bytes(batch_size=1, dtype=torch.bfloat16) == 223_104
    big = CoDAGQALandmarkPerf2(embed_dim=4096, num_heads=32, num_kv_heads=8, window=256, num_landmarks_exact=64,
                               num_landmarks_summary=64)
    assert big.cache_bytes(batch_size=1, dtype=torch.bfloat16) == 1_771_392


def test_state_is_one_arena_with_upstream_fields():
    m = CoDAGQALandmarkPerf2(**KW)
    st = m.init_state(batch_size=3, device="cpu", dtype=torch.bfloat16)
    assert st.k_buf.shape == (3, 2, 64, 32) and st.allowed.dtype == torch.bool and st.g_recent.dtype == torch.float32
    assert st.mem_last_exact.dtype == torch.int64 and st._sum_lf_k_norm.shape == (3, 2, 16, 16)
    lay, total = arena_layout(3, 2, 32, 32, 16, 16, 2)
    base = st._arena.data_ptr()
    assert st._arena.numel() == total
    for name, t in (("k_buf", st.k_buf), ("v_buf", st.v_buf), ("allowed", st.allowed), ("g_recent", st.g_recent),
                    ("mem_last_exact", st.mem_last_exact), ("exact_v_norm", st._exact_v_norm),
                    ("sum_lf_k_norm", st._sum_lf_k_norm)):
        assert t.data_ptr() - base == lay[name][0] and lay[name][0] % 256 == 0
    assert (st.pos, st.recent_idx, st.recent_filled, st.active_exact, st.active_summary) == (0, 0, 0, 16, 16)
    assert not bool(st.allowed.any()) and float(st.k_buf[:, :, :32].abs().sum()) == 0.0
    # summary keys: high-frequency half stays zero
    assert float(st.k_buf[:, :, 48:, :16].abs().sum()) == 0.0 and float(st.k_buf[:, :, 48:, 16:].abs().sum()) > 0.0
    z = m.init_state(batch_size=1, device="cpu", dtype=torch.float32, mem_init="zeros")
    assert float(z.k_buf.abs().sum()) == 0.0
    with pytest.raises(ValueError):
        m.init_state(batch_size=1, device="cpu", dtype=torch.float32, mem_init="ones")


def test_state_helpers_round_trip():
    m = CoDAGQALandmarkPerf2(**KW)
    st = m.init_state(batch_size=2, device="cpu", dtype=torch.float32)
    st.pos, st.recent_filled = 7, 7
    c = _deep_copy_state(st)
    c.k_buf.add_(1.0)
    assert not torch.equal(c.k_buf, st.k_buf) and c.pos == 7
    cpu = _state_to_cpu(st)
    buf = io.BytesIO()
    torch.save(cpu, buf)
    buf.seek(0)
    back = torch.load(buf, weights_only=False)
    assert isinstance(back, CoDAGQALandmarkStatePerf2)
    for f in ("k_buf", "v_buf", "allowed", "g_recent", "mem_last_exact", "_exact_v_norm", "_sum_lf_k_norm"):
        assert torch.equal(getattr(back, f), getattr(st, f))
    _state_to_device(back, torch.device("cpu"), torch.bfloat16)
    assert back.k_buf.dtype == torch.bfloat16 and back._exact_v_norm.dtype == torch.float32
    packed = state_from_fields(back, "cpu")
    assert packed._arena is not None and packed._exact_v_norm.dtype == torch.bfloat16 and packed.pos == 7


class _FakeLlamaAttn(torch.nn.Module):
    def __init__(self):
        super().__init__()
        self.q_proj = torch.nn.Linear(64, 64, bias=True)
        self.k_proj = torch.nn.Linear(64, 32, bias=False)
        self.v_proj = torch.nn.Linear(64, 32, bias=False)
        self.o_proj = torch.nn.Linear(64, 64, bias=False)
        self.num_heads, self.num_key_value_heads, self.head_dim = 4, 2, 16
        self.config = type("Cfg", (), {"rope_theta": 1e6})()


def test_llama_adapter_weight_copy_and_state_api():
    src = _FakeLlamaAttn()
    with pytest.warns(UserWarning):
        ad = LlamaCoDAAdapter.from_llama_attention(src, bounded=True, window=8, num_landmarks_exact=4,
                                                   num_landmarks_summary=4)
    assert ad.coda.rope_base == 1e6 and ad.coda.head_norm_mode == "identity" and not ad.coda.rope_interleaved
    assert torch.equal(ad.coda.q_proj.weight, src.q_proj.weight) and torch.equal(ad.coda.q_proj.bias, src.q_proj.bias)
    assert ad.coda.k_proj.bias is None and ad.block_size == 1024
    assert ad.get_state() is None
    st = ad.init_inference_state(2, "cpu", torch.float32)
    assert ad.get_state() is st
    ad.reset_state()
    assert ad.get_state() is None
    ad.set_state(st)
    assert ad.get_state() is st
    assert ad.cache_bytes(batch_size=2, dtype=torch.float32) == ad.coda.cache_bytes(batch_size=2, dtype=torch.float32)
    model = type("M", (torch.nn.Module,), {})()
    model.model = type("Inner", (torch.nn.Module,), {})()
    blocks = [type("Blk", (torch.nn.Module,), {})() for _ in range(2)]
    for b in blocks:
        b.self_attn = _FakeLlamaAttn()
    model.model.layers = torch.nn.ModuleList(blocks)
    with pytest.warns(UserWarning):
        ads = LlamaCoDAAdapter.swap_llama_layers(model, bounded=False)
    assert len(ads) == 2 and model.model.layers[0].self_attn is ads[0]
    y, pkv = ads[0](torch.randn(1, 5, 64), past_key_value="tok")       # unbounded mode runs on the CPU
    assert y.shape == (1, 5, 64) and pkv == "tok"
    with pytest.raises(RuntimeError):
        ads[0].cache_bytes(batch_size=1, dtype=torch.float32)


def test_eve_adapter_splits_fused_qkv():
    ad = EveCoDAAdapter(n_embd=64, n_head=4, head_dim=16, bounded=True, window=8, num_landmarks_exact=4,
                        num_landmarks_summary=4)
    w, b = torch.randn(192, 64), torch.randn(192)
    ad.load_eve_weights(c_attn_weight=w, c_attn_bias=b, c_proj_weight=torch.randn(64, 64), c_proj_bias=torch.randn(64))
    assert torch.equal(ad.coda.k_proj.weight, w[64:128]) and torch.equal(ad.coda.v_proj.bias, b[128:])
    assert ad.coda.num_kv_heads == 4 and ad.coda.head_norm_mode == "full" and ad.coda.rope_interleaved
    assert "block_size=1024" in ad.extra_repr()


def test_qwen3_adapter_defaults_and_weight_copy():
    """Qwen3 adapter = Llama adapter with rope_theta 1e6 by default (upstream qwen3_adapter.py:25-219)."""
    ad = Qwen3CoDAAdapter(hidden_size=64, num_heads=4, num_kv_heads=2, head_dim=16, bounded=True, window=8,
                          num_landmarks_exact=4, num_landmarks_summary=4)
    assert ad.coda.rope_base == 1e6 and ad.coda.head_norm_mode == "identity" and not ad.coda.rope_interleaved
    src = _FakeLlamaAttn()
    del src.config                                                     # no config: the Qwen3 default applies
    src.num_heads = None                                               # head count inferred from the projection shape
    ad = Qwen3CoDAAdapter.from_qwen3_attention(src, bounded=True, window=8, num_landmarks_exact=4,
                                               num_landmarks_summary=4)
    assert isinstance(ad, LlamaCoDAAdapter) and ad.num_heads == 4 and ad.num_kv_heads == 2 and ad.head_dim == 16
    assert ad.coda.rope_base == 1e6
    for name in ("q_proj", "k_proj", "v_proj", "o_proj"):
        assert torch.equal(getattr(ad.coda, name).weight, getattr(src, name).weight)
    assert torch.equal(ad.coda.q_proj.bias, src.q_proj.bias) and ad.coda.k_proj.bias is None
    model = type("M", (torch.nn.Module,), {})()
    model.model = type("Inner", (torch.nn.Module,), {})()
    blocks = [type("Blk", (torch.nn.Module,), {})() for _ in range(3)]
    for b in blocks:
        b.self_attn = _FakeLlamaAttn()
    model.model.layers = torch.nn.ModuleList(blocks)
    ads = Qwen3CoDAAdapter.swap_qwen3_layers(model, bounded=False)
    assert len(ads) == 3 and all(model.model.layers[i].self_attn is ads[i] for i in range(3))
    y, _ = ads[1](torch.randn(2, 3, 64))
    assert y.shape == (2, 3, 64)


def test_state_wire_format_round_trip_and_validation():
    """One blob per layer state: header + arena bytes; round trip restores every field; bad blobs are refused."""
    from coda_gqa_l_b200 import state_from_bytes, state_to_bytes
    from coda_gqa_l_b200.state import allocate_state
    from coda_gqa_l_b200.state_io import WIRE_HEADER_BYTES
    for dtype in (torch.float32, torch.bfloat16):
        st = allocate_state(2, 3, 16, 10, 4, 5, "cpu", dtype)
        g = torch.Generator().manual_seed(1)
        st.k_buf.copy_(torch.randn(st.k_buf.shape, generator=g).to(dtype))
        st.v_buf.copy_(torch.randn(st.v_buf.shape, generator=g).to(dtype))
        st._exact_v_norm.copy_(torch.randn(st._exact_v_norm.shape, generator=g).to(dtype))
        st._sum_lf_k_norm.copy_(torch.randn(st._sum_lf_k_norm.shape, generator=g).to(dtype))
        st.g_recent.copy_(torch.rand(st.g_recent.shape, generator=g))
        st.mem_last_exact.copy_(torch.randint(-1, 1000, st.mem_last_exact.shape, generator=g))
        st.allowed.copy_(torch.rand(st.allowed.shape, generator=g) > 0.5)
        st.pos, st.recent_idx, st.recent_filled, st.active_exact, st.active_summary = 12345678901, 7, 10, 4, 5
        blob = state_to_bytes(st)
        assert len(blob) == WIRE_HEADER_BYTES + st._arena.numel() and blob[:7] == b"CODAB2S"
        back = state_from_bytes(blob, "cpu")
        for name in ("k_buf", "v_buf", "allowed", "g_recent", "mem_last_exact", "_exact_v_norm", "_sum_lf_k_norm"):
            a, b = getattr(st, name), getattr(back, name)
            assert a.dtype == b.dtype and a.shape == b.shape and torch.equal(a, b), name
        assert (back.pos, back.recent_idx, back.recent_filled, back.active_exact, back.active_summary) == \
               (12345678901, 7, 10, 4, 5)
        with pytest.raises(ValueError):
            state_from_bytes(b"XXXXXXXX" + blob[8:], "cpu")
        with pytest.raises(ValueError):
            state_from_bytes(blob[:-1], "cpu")
        with pytest.raises(ValueError):
            state_from_bytes(blob[:8] + (99).to_bytes(4, "little") + blob[12:], "cpu")


def test_captured_step_key_sees_every_way_a_parameter_can_change():
    """The key a captured decode step is checked against before every replay is read through a flat tuple of the
    Parameter objects; it must still change on an in-place write, on a replaced Parameter object (directly on the
    layer and inside a sub-module), on a flipped switch, on a dtype conversion and on other states."""
    from types import SimpleNamespace
    from coda_gqa_l_b200.stack import CoDAStack
    kw = dict(embed_dim=64, num_heads=4, num_kv_heads=2, window=8, num_landmarks_exact=4, num_landmarks_summary=4)
    layers = [CoDAGQALandmarkPerf2(**kw) for _ in range(3)]
    stack = CoDAStack(layers)
    states = [SimpleNamespace(active_exact=4, active_summary=4) for _ in layers]
    key = lambda: stack._graph_key(states, torch.bfloat16)
    k = key()
    assert key() == k
    with torch.no_grad():
        layers[1].q_proj.weight.mul_(1.0)
    assert key() != k; k = key()
    with torch.no_grad():
        layers[2].summary_eta_logit.add_(0.0)
    assert key() != k; k = key()
    layers[0].theta = torch.nn.Parameter(layers[0].theta.detach().clone())
    assert key() != k; k = key()
    layers[2].o_proj.weight = torch.nn.Parameter(layers[2].o_proj.weight.detach().clone())
    assert key() != k; k = key()
    layers[1].use_skinny_in_proj = not layers[1].use_skinny_in_proj
    assert key() != k; k = key()
    stack.to(torch.float64)
    assert key() != k; k = key()
    states[1].active_exact = 2
    assert key() != k; k = key()
    assert stack._graph_key(list(states[:2]) + [SimpleNamespace(active_exact=4, active_summary=4)], torch.bfloat16) != k
    assert stack._graph_key(states, torch.float32) != k
    assert key() == k
