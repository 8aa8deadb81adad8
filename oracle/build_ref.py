"""Recipe that places an importable, UNMODIFIED copy of the upstream project's Python package under oracle/_ref/.

TEST / BENCHMARK INFRASTRUCTURE ONLY.  Nothing in the shipped package imports oracle/_ref; it exists so that the
reference arm of bench.py (``--impl reference`` / ``--impl reference-gpu``) and the ``cpu_baseline`` leg can time the
reference's own ``CoDAGQALandmarkPerf2`` instead of this repository's restatement of it.

    python oracle/build_ref.py [--ref <upstream checkout>]        # default: $CODA_GQA_L_REF, else DEFAULT_CHECKOUT below

The upstream checkout is installed with pip (no index, no dependencies) from a temporary copy -- the build writes into
its source tree and the checkout may be read-only -- into ``oracle/_ref`` (listed in .gitignore: reference sources never
enter this repository's history).  Where no checkout is available the folder is left as it is; callers fall back to
the oracle port and say so.
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
TARGET = os.path.join(HERE, "_ref")
DEFAULT_CHECKOUT = os.path.join(os.sep, "root", "reference")


def available() -> bool:
    return os.path.exists(os.path.join(TARGET, "coda_gqa_l", "attention.py"))


def build(ref_root: str | None = None, force: bool = False) -> bool:
    """Install upstream into oracle/_ref.  Returns whether an importable copy is present afterwards."""
    ref_root = ref_root or os.environ.get("CODA_GQA_L_REF") or DEFAULT_CHECKOUT
    if available() and not force:
        return True
    if not os.path.exists(os.path.join(ref_root, "pyproject.toml")):
        return available()
    with tempfile.TemporaryDirectory() as tmp:
        src = os.path.join(tmp, "upstream")
        shutil.copytree(ref_root, src, ignore=shutil.ignore_patterns(".git", "notebooks", "demo", "benchmarks", "reproduce",
                                                                      "makora", "examples", "tests", "kernels"))
        cmd = [sys.executable, "-m", "pip", "install", "--quiet", "--no-index", "--no-build-isolation", "--no-deps",
               "--upgrade", "--target", TARGET, src]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            sys.stderr.write(r.stdout + r.stderr)
            return available()
    return available()


def load():
    """Import upstream's package from oracle/_ref with its optional Triton / CUDA accelerators switched off, so that
    the plain PyTorch path -- the reference semantics -- runs on any device.  Returns the ``CoDAGQALandmarkPerf2`` class."""
    if not available():
        raise ImportError("oracle/_ref holds no upstream package: run python oracle/build_ref.py where a checkout exists")
    if TARGET not in sys.path:
        sys.path.insert(0, TARGET)
    import coda_gqa_l.attention as A
    import coda_gqa_l.memory_banks as MB
    A._HAS_TRITON_FLASH = False
    A._HAS_FUSED_EPILOGUE = False
    MB._HAS_TRITON_ROUTE = False
    MB._HAS_TRITON_SUMMARY = False
    return A.CoDAGQALandmarkPerf2


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=None)
    ap.add_argument("--force", action="store_true")
    a = ap.parse_args()
    ok = build(a.ref, a.force)
    print("oracle/_ref:", "ready" if ok else "unavailable (no upstream checkout)")
