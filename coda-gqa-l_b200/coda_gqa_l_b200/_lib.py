"""ctypes binding of libcoda_b200.so (the C ABI declared in include/coda_b200.h).

The library is the only compute path: if it is missing the import fails loudly instead of
falling back to another implementation.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libcoda_b200.so")

CODA_F32, CODA_BF16 = 0, 1
CODA_EVENT_WORDS = 16   # int32 words per state in the routing-event record (coda_b200.h)


class LayerCfg(C.Structure):
    """struct coda_layer_cfg"""
    _fields_ = [(n, C.c_int32) for n in (
        "B", "H", "Hkv", "Dh", "W", "Me", "Ms", "dtype", "angle_dtype", "rope_interleaved",
        "head_norm_full", "mask_unused", "gated", "refresh_on_hit", "overwrite_on_insert",
        "Te", "Ts", "active_exact", "active_summary")] + [(n, C.c_float) for n in (
        "tau_gate_exact", "tau_gate_summary", "tau_match", "tau_novel", "eps", "energy_scale")]


class StatePtrs(C.Structure):
    """struct coda_state_ptrs"""
    _fields_ = [(n, C.c_void_p) for n in (
        "k_buf", "v_buf", "allowed", "g_recent", "mem_last_exact", "exact_v_norm", "sum_lf_k_norm", "events")]


class RingPos(C.Structure):
    """struct coda_ring_pos"""
    _fields_ = [("pos", C.c_int64), ("recent_idx", C.c_int32), ("recent_filled", C.c_int32),
                ("step_dev", C.c_void_p)]


def _load() -> C.CDLL:
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} not found: build the CUDA library first (python coda-gqa-l_b200/build.py). "
            "coda_gqa_l_b200 has no fallback path.")
    lib = C.CDLL(LIB_PATH)
    vp, i32, i64, fp = C.c_void_p, C.c_int32, C.c_int64, C.c_void_p
    cfgp, stp = C.POINTER(LayerCfg), C.POINTER(StatePtrs)
    lib.coda_b200_last_error.restype = C.c_char_p
    lib.coda_b200_version.restype = C.c_int
    lib.coda_b200_prep.argtypes = [cfgp, i32, RingPos, vp, i64, i64, vp, i64, i64, vp,
                                   vp, i64, i64, fp, vp, i64, i64, fp, fp, vp, vp, vp]
    lib.coda_b200_step_write.argtypes = [cfgp, stp, RingPos, vp, i64, vp, i64, fp, fp, vp]
    lib.coda_b200_step_write_raw.argtypes = [cfgp, stp, RingPos, vp, i64, vp, i64, vp, i64, fp, fp, vp]
    lib.coda_b200_decode_attend_supported.argtypes = [cfgp]
    lib.coda_b200_decode_attend.argtypes = [cfgp, stp, RingPos, i32, vp, i64, vp, i64, fp, vp, vp, vp, vp, vp, i64, vp, vp]
    lib.coda_b200_decode_attend_prepared.argtypes = [cfgp, stp, vp, vp, vp, i64, vp, vp]
    lib.coda_b200_decode_set_early_trigger.argtypes = [i32]
    lib.coda_b200_decode_set_early_trigger.restype = None
    lib.coda_b200_decode_record_bytes.argtypes = [cfgp]
    lib.coda_b200_decode_record_bytes.restype = C.c_int64
    lib.coda_b200_step_write_fused.argtypes = [cfgp, stp, RingPos, vp, i64, vp, i64, vp, i64, fp, fp,
                                               vp, i64, vp, i64, vp, vp, vp, vp]
    lib.coda_b200_step_write_fused_supported.argtypes = [cfgp]
    lib.coda_b200_step_write_attend.argtypes = [cfgp, stp, RingPos, vp, i64, vp, i64, vp, i64, fp, fp,
                                                vp, i64, vp, i64, vp, vp, vp, vp, vp, i64, vp, vp]
    lib.coda_b200_step_route.argtypes = [cfgp, stp, RingPos, fp, vp]
    lib.coda_b200_step_route_plan_bytes.argtypes = [i32]
    lib.coda_b200_step_route_plan_bytes.restype = C.c_int64
    lib.coda_b200_step_route_plan.argtypes = [cfgp, C.POINTER(StatePtrs), C.POINTER(RingPos), C.POINTER(C.c_void_p),
                                              i32, vp, vp]
    lib.coda_b200_step_route_batched.argtypes = [cfgp, vp, i32, vp]
    lib.coda_b200_decode_attend_append_supported.argtypes = [cfgp]
    lib.coda_b200_decode_attend_append.argtypes = [cfgp, stp, RingPos, vp, i64, vp, i64, vp, i64, fp,
                                                   vp, i64, vp, i64, vp, vp, fp, vp, vp, i64, vp, vp]
    lib.coda_b200_rope_table.argtypes = [cfgp, RingPos, fp, fp, vp]
    lib.coda_b200_proj_gemm_supported.argtypes = [i32, i32, i32]
    lib.coda_b200_proj_gemm.argtypes = [vp, i64, i32, i32, vp, i32, vp, vp, i64, vp, i64, vp, vp, vp]
    lib.coda_b200_proj_gemm_workspace_bytes.argtypes = [i32, i32, i32]
    lib.coda_b200_proj_gemm_workspace_bytes.restype = C.c_int64
    lib.coda_b200_skinny_gemm_supported.argtypes = [i32, i32, i32]
    lib.coda_b200_skinny_gemm.argtypes = [vp, i32, i32, vp, i32, vp, i64, vp, i64, vp, vp]
    lib.coda_b200_skinny_gemm_bias.argtypes = [vp, i32, i32, vp, i32, vp, vp, i64, vp, i64, vp, vp]
    lib.coda_b200_skinny_gemm_bias_supported.argtypes = [i32, i32, i32]
    lib.coda_b200_skinny_gemm_plan.argtypes = [i32, i32, C.POINTER(C.c_int32), C.POINTER(C.c_int32)]
    lib.coda_b200_skinny_gemm_chain_supported.argtypes = [i32, i32, i32, i32]
    lib.coda_b200_skinny_gemm_chain.argtypes = [vp, i32, i32, vp, i32, vp, i64, vp, vp, i32, vp, vp, i64, vp, vp, vp]
    lib.coda_b200_step_append_fused.argtypes = [cfgp, stp, RingPos, vp, i64, vp, i64, vp, i64, fp,
                                                vp, i64, vp, i64, vp, vp, vp, vp]
    lib.coda_b200_prefill_attend_supported.argtypes = [cfgp]
    lib.coda_b200_prefill_attend.argtypes = [cfgp, stp, i32, i32, i32, vp, i64, i64, vp, i64, i64, fp, i64, i64,
                                             vp, i64, i64, vp, i64, i64, vp, vp, i64, i64, vp, vp]
    lib.coda_b200_attend.argtypes = [cfgp, stp, i32, vp, i64, i64, vp, i64, i64, fp, i64, i64,
                                     vp, i64, i64, vp, i64, i64, vp, vp, i64, i64, vp]
    lib.coda_b200_select_candidates.argtypes = [cfgp, fp, i64, i32, i32, i32, vp, i32, vp]
    lib.coda_b200_route_scratch_bytes.argtypes = [cfgp]
    lib.coda_b200_route_scratch_bytes.restype = i64
    lib.coda_b200_route_block.argtypes = [cfgp, stp, i32, i32, i64, vp, i64, i64, vp, i64, i64,
                                          fp, i64, i64, vp, i64, fp, vp, vp]
    lib.coda_b200_route_block_phase.argtypes = [cfgp, stp, i32, i32, i64, vp, i64, i64, vp, i64, i64,
                                                fp, i64, i64, vp, i64, fp, vp, i32, vp]
    lib.coda_b200_route_static_scratch_bytes.argtypes = []
    lib.coda_b200_route_static_scratch_bytes.restype = i64
    lib.coda_b200_route_block_noalloc.argtypes = [cfgp, stp, i32, i32, i64, vp, i64, i64, vp, i64, i64,
                                                  fp, i64, i64, vp, i64, fp, vp]
    lib.coda_b200_advance_steps.argtypes = [vp, i64, vp]
    lib.coda_b200_selftest_bounded_wait.argtypes = [i32, vp, vp, vp]
    lib.coda_b200_host_topk_f32.argtypes = [vp, i32, i32, i32, i32, vp]
    lib.coda_b200_host_topk_i64.argtypes = [vp, i32, i32, i32, i32, vp]
    for name in EXPORTS:
        fn = getattr(lib, name)
        if name not in ("coda_b200_last_error", "coda_b200_route_scratch_bytes", "coda_b200_route_static_scratch_bytes",
                        "coda_b200_decode_record_bytes", "coda_b200_decode_set_early_trigger", "coda_b200_proj_gemm_workspace_bytes"):
            fn.restype = C.c_int
    return lib


EXPORTS = (
    "coda_b200_last_error", "coda_b200_version", "coda_b200_prep", "coda_b200_step_write",
    "coda_b200_step_write_raw", "coda_b200_step_write_fused", "coda_b200_step_write_fused_supported", "coda_b200_step_write_attend",
    "coda_b200_step_route", "coda_b200_step_append_fused", "coda_b200_step_route_plan_bytes",
    "coda_b200_step_route_plan", "coda_b200_step_route_batched",
    "coda_b200_skinny_gemm_supported", "coda_b200_skinny_gemm", "coda_b200_skinny_gemm_bias", "coda_b200_skinny_gemm_bias_supported", "coda_b200_skinny_gemm_plan", "coda_b200_skinny_gemm_chain_supported", "coda_b200_skinny_gemm_chain", "coda_b200_proj_gemm_supported", "coda_b200_proj_gemm", "coda_b200_proj_gemm_workspace_bytes",
    "coda_b200_decode_attend_append_supported", "coda_b200_decode_attend_append", "coda_b200_rope_table",
    "coda_b200_decode_attend_supported", "coda_b200_decode_attend", "coda_b200_decode_attend_prepared",
    "coda_b200_decode_record_bytes", "coda_b200_decode_set_early_trigger",
    "coda_b200_prefill_attend_supported", "coda_b200_prefill_attend",
    "coda_b200_attend", "coda_b200_select_candidates", "coda_b200_route_scratch_bytes",
    "coda_b200_route_block", "coda_b200_route_block_phase", "coda_b200_route_static_scratch_bytes", "coda_b200_route_block_noalloc",
    "coda_b200_advance_steps", "coda_b200_selftest_bounded_wait", "coda_b200_host_topk_f32",
    "coda_b200_host_topk_i64",
)

lib = _load()


def check(rc: int, what: str) -> None:
    """Raise RuntimeError with the library's message when an entry point rejects a call."""
    if rc != 0:
        msg = lib.coda_b200_last_error()
        raise RuntimeError(f"{what} failed ({rc}): {msg.decode() if msg else ''}")
