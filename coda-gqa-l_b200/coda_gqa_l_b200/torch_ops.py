"""The torch custom-op face of the library: ``torch.ops.coda_b200.*``.

``libcoda_b200_torch.so`` (built from torch_ext/torch_binding.cpp) registers one op per C-ABI entry point of the
attention / cache-write / routing path with a ``Tensor(x!)`` annotation on everything the op writes, argument
checks that raise ``RuntimeError`` and the current CUDA stream picked up on the C++ side -- the same layering as
upstream's ``coda_kernels`` package over its epilogue kernel (kernels/coda_diff_epilogue/torch-ext/
coda_kernels/__init__.py:67-72).  The ops call the same entry points the ctypes binding calls, so results are
bit-identical; ``CoDAGQALandmarkPerf2.use_torch_ops = True`` routes a module through them.
"""
from __future__ import annotations

import os
from typing import List, Tuple

import torch

from ._lib import LayerCfg

TORCH_LIB_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "libcoda_b200_torch.so")
_loaded = False


def load():
    """Register the ops (once) and return the ``torch.ops.coda_b200`` namespace.  Raises ``ImportError`` when the
    op library has not been built (python coda-gqa-l_b200/build.py): there is nothing to fall back to."""
    global _loaded
    if not _loaded:
        if not os.path.exists(TORCH_LIB_PATH):
            raise ImportError(f"{TORCH_LIB_PATH} not found: build it first (python coda-gqa-l_b200/build.py)")
        torch.ops.load_library(TORCH_LIB_PATH)
        _loaded = True
    return torch.ops.coda_b200


def is_available() -> bool:
    return os.path.exists(TORCH_LIB_PATH)


_INT_FIELDS = tuple(n for n, t in LayerCfg._fields_[:19])
_FLOAT_FIELDS = tuple(n for n, t in LayerCfg._fields_[19:])


def cfg_lists(cfg: LayerCfg) -> Tuple[List[int], List[float]]:
    """A ``coda_layer_cfg`` as the two lists the ops take (field order of the struct)."""
    hit = getattr(cfg, "_lists", None)
    if hit is None:
        hit = ([int(getattr(cfg, n)) for n in _INT_FIELDS], [float(getattr(cfg, n)) for n in _FLOAT_FIELDS])
        cfg._lists = hit
    return hit
