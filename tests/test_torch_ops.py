"""The torch custom-op layer (torch.ops.coda_b200.*): registration and schemas on CPU; on the GPU the ops against the
ctypes binding of the same C-ABI entry points (bit-equal), called directly and through a module switched to them."""
import ctypes as C

import pytest
import torch

OPS = ("prep", "attend", "decode_attend", "prefill_attend", "step_write", "select_candidates", "route_block")
# tensors each op writes: every one must carry an alias annotation in the schema
WRITES = {"prep": ("q", "k", "q_noise", "lam", "gate"), "attend": ("out",), "decode_attend": ("out", "qrec", "status"),
          "prefill_attend": ("out", "status"), "select_candidates": ("cand",),
          "step_write": ("k_buf", "v_buf", "allowed", "g_recent", "mem_last_exact", "exact_v_norm", "sum_lf_k_norm"),
          "route_block": ("k_buf", "v_buf", "allowed", "g_recent", "mem_last_exact", "exact_v_norm", "sum_lf_k_norm", "scratch")}


def test_ops_are_registered_with_mutation_annotations():
    from coda_gqa_l_b200 import torch_ops
    ns = torch_ops.load()
    for name in OPS:
        schema = getattr(ns, name).default._schema
        args = {a.name: a for a in schema.arguments}
        for w in WRITES[name]:
            assert args[w].alias_info is not None and args[w].alias_info.is_write, f"{name}: {w} is written but not annotated"
        for a in schema.arguments:
            if a.name not in WRITES[name]:
                assert a.alias_info is None, f"{name}: {a.name} is read-only but annotated"
        assert len(schema.returns) == 0


def test_ops_have_no_cpu_implementation():
    from coda_gqa_l_b200 import torch_ops
    ns = torch_ops.load()
    with pytest.raises((NotImplementedError, RuntimeError)):
        ns.select_candidates(torch.zeros(1, 1, 1, dtype=torch.int32), torch.zeros(1, 4), 0, 4, 4, [0] * 19, [0.0] * 6)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,kw", [
    (torch.float32, dict(embed_dim=128, num_heads=4, num_kv_heads=2, window=32, num_landmarks_exact=16, num_landmarks_summary=16)),
    (torch.bfloat16, dict(embed_dim=512, num_heads=4, num_kv_heads=2, window=64, num_landmarks_exact=16, num_landmarks_summary=16,
                          rope_interleaved=False, head_norm_mode="identity")),
    (torch.float32, dict(embed_dim=128, num_heads=4, num_kv_heads=2, window=32, num_landmarks_exact=16, num_landmarks_summary=16,
                         write_policy="none")),
])
def test_module_through_torch_ops_equals_module_through_ctypes(dtype, kw):
    """prefill (prep, attention, candidate selection, block routing) + decode with every flag combination of step()
    + attend_step, once through torch.ops.coda_b200.* and once through ctypes: same bits in outputs and state."""
    from coda_gqa_l_b200 import CoDAGQALandmarkPerf2, _deep_copy_state
    from tests.helpers import orc
    from tests.scenarios import randomize_weights
    torch.manual_seed(1)
    mod = CoDAGQALandmarkPerf2(**kw).eval()
    randomize_weights(mod, 1)
    mod = mod.to(dtype).cuda()
    x = orc.mixture_inputs(2, 200 + 48, kw["embed_dim"], centroids=16, sigma=0.3, seed=2, dtype=dtype).cuda()
    torch.manual_seed(3)
    sa = mod.init_state(batch_size=2, device="cuda", dtype=dtype)
    sb = _deep_copy_state(sa)
    outs = {}
    for tag, st, flag in (("ops", sa, True), ("ctypes", sb, False)):
        mod.use_torch_ops = flag
        ys = [mod.prefill_chunked(x[:, :200], st, block_size=48)[0]]
        for t in range(200, 248):
            kws = [dict(), dict(attend=False), dict(include_current_in_attention=False), dict(write_cache=False)][t % 4]
            ys.append(mod.step(x[:, t:t + 1], st, **kws)[0])
        ys.append(mod.attend_step(x[:, 100:101], st, query_pos=17))
        outs[tag] = torch.cat(ys, 1)
    assert torch.equal(outs["ops"], outs["ctypes"])
    for f in ("k_buf", "v_buf", "allowed", "g_recent", "mem_last_exact", "_exact_v_norm", "_sum_lf_k_norm"):
        assert torch.equal(getattr(sa, f), getattr(sb, f)), f
    assert (sa.pos, sa.recent_idx, sa.recent_filled) == (sb.pos, sb.recent_idx, sb.recent_filled)
    assert mod.device_status() == 0


@pytest.mark.gpu
def test_decode_attend_and_route_block_ops_called_directly():
    """torch.ops.coda_b200.decode_attend and .route_block with explicit tensors against the ctypes calls, plus the
    argument checks: wrong dtype, wrong shape, a CPU tensor and an unsupported configuration raise RuntimeError."""
    from coda_gqa_l_b200 import CoDAGQALandmarkPerf2, _deep_copy_state, torch_ops
    from coda_gqa_l_b200._lib import RingPos, check, lib
    ns = torch_ops.load()
    torch.manual_seed(0)
    B, D = 3, 512
    mod = CoDAGQALandmarkPerf2(embed_dim=D, num_heads=4, num_kv_heads=2, window=64, num_landmarks_exact=16,
                               num_landmarks_summary=16).eval().to(torch.bfloat16).cuda()
    x = (torch.randn(B, 200, D, device="cuda") * 0.5).to(torch.bfloat16)
    st = mod.init_state(batch_size=B, device="cuda", dtype=torch.bfloat16)
    mod.prefill_chunked(x[:, :128], st, block_size=64, return_outputs=False)
    cfg = mod._cfg(B, torch.bfloat16, st)
    ci, cf = torch_ops.cfg_lists(cfg)
    inv_freq, cos_t, sin_t, eta, nw = mod._consts(x.device, torch.bfloat16)

    # ---- decode attention
    q, _, _, lam_logit, _ = mod._project(x[:, 128:129], need_kv=False)
    out_a, out_b = torch.empty(B, 1, D, device="cuda", dtype=torch.bfloat16), torch.empty(B, 1, D, device="cuda", dtype=torch.bfloat16)
    qrec = torch.empty(int(lib.coda_b200_decode_record_bytes(C.byref(cfg))), dtype=torch.uint8, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    ns.decode_attend(out_a, st.k_buf, st.v_buf, st.allowed, q, lam_logit, inv_freq, cos_t, sin_t, nw, qrec, status,
                     st.pos, st.recent_idx, st.recent_filled, 0, ci, cf)
    mod.decode_attend_launch(cfg, st, RingPos(st.pos, st.recent_idx, st.recent_filled, None), 0, q, lam_logit, out_b)
    torch.cuda.synchronize()
    assert torch.equal(out_a, out_b) and int(status.item()) == 0 and bool(torch.isfinite(out_a.float()).all())
    with pytest.raises(RuntimeError, match="dtype"):
        ns.decode_attend(out_a.float(), st.k_buf, st.v_buf, st.allowed, q, lam_logit, inv_freq, cos_t, sin_t, nw, qrec, status,
                         st.pos, st.recent_idx, st.recent_filled, 0, ci, cf)
    with pytest.raises(RuntimeError, match="k_buf"):
        ns.decode_attend(out_a, st.k_buf[:, :1], st.v_buf, st.allowed, q, lam_logit, inv_freq, cos_t, sin_t, nw, qrec, status,
                         st.pos, st.recent_idx, st.recent_filled, 0, ci, cf)
    with pytest.raises(RuntimeError, match="CUDA"):
        ns.decode_attend(out_a, st.k_buf, st.v_buf, st.allowed, q, lam_logit.cpu(), inv_freq, cos_t, sin_t, nw, qrec, status,
                         st.pos, st.recent_idx, st.recent_filled, 0, ci, cf)
    ci32 = list(ci)
    ci32[7] = 0                                            # float32 is not covered by the fused decode kernel
    with pytest.raises(RuntimeError, match="not covered"):
        ns.decode_attend(out_a, st.k_buf, st.v_buf, st.allowed, q, lam_logit, inv_freq, cos_t, sin_t, nw, qrec, status,
                         st.pos, st.recent_idx, st.recent_filled, 0, ci32, cf)

    # ---- block routing
    qb, kb, vb, lam_l, gate_l = mod._project(x[:, 128:192], need_kv=True)
    qn, lam, g = mod._prep(cfg, 64, st.pos, qb, kb, lam_l, gate_l, True)
    gates = torch.cat([st.g_recent, g], dim=1).contiguous()
    cand = torch.empty(B, 1, 64, device="cuda", dtype=torch.int32)
    ns.select_candidates(cand, gates, 64, 64, 64, ci, cf)
    scratch = torch.empty(int(lib.coda_b200_route_scratch_bytes(C.byref(cfg))), dtype=torch.uint8, device="cuda")
    sa, sb = _deep_copy_state(st), _deep_copy_state(st)
    ns.route_block(sa.k_buf, sa.v_buf, sa.allowed, sa.g_recent, sa.mem_last_exact, sa._exact_v_norm, sa._sum_lf_k_norm,
                   kb, vb, gates, cand[:, 0], eta, scratch, 64, st.pos, 0, ci, cf)
    check(lib.coda_b200_route_block(
        C.byref(cfg), C.byref(mod._ptrs(sb)), 64, 64, st.pos, kb.data_ptr(), kb.stride(0), kb.stride(1), vb.data_ptr(),
        vb.stride(0), vb.stride(1), gates.data_ptr(), gates.stride(0), 0, cand[:, 0].data_ptr(), cand.stride(0),
        eta.data_ptr(), scratch.data_ptr(), torch.cuda.current_stream().cuda_stream), "coda_b200_route_block")
    torch.cuda.synchronize()
    assert torch.equal(sa._arena, sb._arena) and not torch.equal(sa.k_buf, st.k_buf)
    with pytest.raises(RuntimeError, match="scratch"):
        ns.route_block(sa.k_buf, sa.v_buf, sa.allowed, sa.g_recent, sa.mem_last_exact, sa._exact_v_norm, sa._sum_lf_k_norm,
                       kb, vb, gates, cand[:, 0], eta, scratch[:8], 64, st.pos, 0, ci, cf)
    with pytest.raises(RuntimeError, match="mem_last_exact"):
        ns.route_block(sa.k_buf, sa.v_buf, sa.allowed, sa.g_recent, sa.mem_last_exact.int(), sa._exact_v_norm,
                       sa._sum_lf_k_norm, kb, vb, gates, cand[:, 0], eta, scratch, 64, st.pos, 0, ci, cf)
