"""GPU: the allocation-free block-routing entry point.

Some callers cannot allocate device memory (a serving process whose pool is frozen, a host framework that owns
every allocation); for them ``coda_b200_route_block_noalloc`` keeps its scratch in a fixed array inside the
library.  This test drives it directly through the C ABI, twice in a row on consecutive blocks, and requires the
same state as the ordinary entry point (caller-provided scratch) produces from the same inputs.  It is collected
last so that a failure here cannot hide another test's result.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _route(mod, entry, cfg, st, fill, blk, pos0, k, v, t0, gates, seen, cand, j, eta, scratch):
    from coda_gqa_l_b200._lib import check, lib
    ptrs = mod._ptrs(st)
    kb, vb = k[:, t0:t0 + blk], v[:, t0:t0 + blk]
    args = [C.byref(cfg), C.byref(ptrs), fill, blk, pos0, kb.data_ptr(), k.stride(0), k.stride(1),
            vb.data_ptr(), v.stride(0), v.stride(1), gates.data_ptr(), gates.stride(0), seen - fill,
            cand[:, j].data_ptr(), cand.stride(0), eta.data_ptr()]
    stream = torch.cuda.current_stream().cuda_stream
    if entry == "noalloc":
        check(lib.coda_b200_route_block_noalloc(*args, stream), "coda_b200_route_block_noalloc")
    else:
        check(lib.coda_b200_route_block(*args, scratch.data_ptr(), stream), "coda_b200_route_block")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_noalloc_route_block_matches_regular_entry_point(dtype):
    from coda_gqa_l_b200 import CoDAGQALandmarkPerf2, _deep_copy_state
    from coda_gqa_l_b200._lib import lib
    from oracle.coda_oracle import mixture_inputs
    torch.manual_seed(0)
    mod = CoDAGQALandmarkPerf2(embed_dim=256, num_heads=4, num_kv_heads=2, window=32, num_landmarks_exact=8,
                               num_landmarks_summary=8).eval().to(dtype).cuda()
    B, L, block = 3, 160, 48
    x = mixture_inputs(B, L, 256, centroids=12, sigma=0.3, seed=1, dtype=dtype).cuda()
    torch.manual_seed(1)
    sa = mod.init_state(batch_size=B, device="cuda", dtype=dtype)
    _, sa = mod.prefill_chunked(x[:, :64], sa, block_size=32)          # ring full, banks live
    sb = _deep_copy_state(sa)
    cfg = mod._cfg(B, dtype, sa)
    assert lib.coda_b200_route_scratch_bytes(C.byref(cfg)) <= lib.coda_b200_route_static_scratch_bytes()

    # the same preparation prefill_chunked does: projections, RoPE, gates, candidate lists
    xs = x[:, 64:]
    Lc = xs.shape[1]
    with torch.no_grad():
        q, k, v, lam_logit, gate_logit = mod._project(xs, need_kv=True)
        _, _, g = mod._prep(cfg, Lc, int(sa.pos), q, k, lam_logit, gate_logit, True)
    fill0 = int(sa.recent_filled)
    gates = torch.cat([sa.g_recent[:, :fill0], g], dim=1).contiguous()
    nblk = (Lc + block - 1) // block
    tmax = min(max(mod.exact_candidates_per_block, mod.summary_candidates_per_block), block)
    cand = torch.empty((B, nblk, tmax), device="cuda", dtype=torch.int32)
    from coda_gqa_l_b200._lib import check
    check(lib.coda_b200_select_candidates(C.byref(cfg), gates.data_ptr(), gates.stride(0), fill0, Lc, block,
                                          cand.data_ptr(), tmax, torch.cuda.current_stream().cuda_stream), "select")
    scratch = mod._route_scratch(cfg, x.device)
    eta = mod._consts(x.device, dtype)[3]
    pos0 = int(sa.pos)
    for j in range(2):                                                  # two calls in a row
        t0, blk = j * block, min(block, Lc - j * block)
        fill = min(mod.window, fill0 + t0)
        for st, entry in ((sa, "regular"), (sb, "noalloc")):
            _route(mod, entry, cfg, st, fill, blk, pos0 + t0, k, v, t0, gates, fill0 + t0, cand, j, eta, scratch)
        torch.cuda.synchronize()
        for name in ("k_buf", "v_buf", "allowed", "g_recent", "mem_last_exact", "_exact_v_norm", "_sum_lf_k_norm"):
            assert torch.equal(getattr(sa, name), getattr(sb, name)), f"{name} differs after call {j + 1}"


def test_noalloc_rejects_configurations_beyond_the_builtin_scratch():
    from coda_gqa_l_b200 import _lib
    cfg = _lib.LayerCfg(B=100000, H=4, Hkv=2, Dh=32, W=8, Me=64, Ms=64, dtype=0, Te=8, Ts=64)
    rc = _lib.lib.coda_b200_route_block_noalloc(C.byref(cfg), None, 0, 8, 0, None, 0, 0, None, 0, 0,
                                                None, 0, 0, None, 0, None, None)
    assert rc == -3 and b"built-in buffer" in _lib.lib.coda_b200_last_error()
