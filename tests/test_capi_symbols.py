"""CPU: libcoda_b200.so loads without a GPU and exports every function include/coda_b200.h declares."""
import ctypes as C
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    names = set()
    for f in os.listdir(os.path.join(ROOT, "include")):
        if f.endswith(".h"):
            src = open(os.path.join(ROOT, "include", f)).read()
            src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
            names |= set(re.findall(r"\b(coda_b200_[a-z0-9_]+)\s*\(", src))
    return names


def test_every_declared_symbol_is_exported():
    from coda_gqa_l_b200 import _lib
    dll = C.CDLL(_lib.LIB_PATH)
    declared = _declared()
    assert len(declared) >= 10
    for name in sorted(declared):
        assert hasattr(dll, name), f"{name} declared in include/ but not exported"
    assert set(_lib.EXPORTS) <= declared
    assert dll.coda_b200_version() >= 1


def test_argument_errors_are_reported_without_a_gpu():
    """Host-side validation happens before any CUDA call, so it can be exercised on a CPU-only box."""
    from coda_gqa_l_b200 import _lib
    cfg = _lib.LayerCfg(B=0, H=4, Hkv=2, Dh=32, W=8, Me=0, Ms=0, dtype=0)
    rc = _lib.lib.coda_b200_select_candidates(C.byref(cfg), None, 0, 0, 16, 8, None, 8, None)
    assert rc == -1
    assert b"select_candidates" in _lib.lib.coda_b200_last_error()
    try:
        _lib.check(rc, "coda_b200_select_candidates")
    except RuntimeError as e:
        assert "select_candidates" in str(e)
    else:
        raise AssertionError("check() must raise")
