"""B200-native bounded-cache differential attention (drop-in for the CoDA-GQA-L hot path).

Importing this package loads libcoda_b200.so; there is no alternative compute path.
"""
from ._lib import LIB_PATH, lib  # noqa: F401  (fails loudly when the CUDA library is missing)
from .adapters import EveCoDAAdapter, LlamaCoDAAdapter, Qwen3CoDAAdapter
from .attention import CoDAGQALandmarkPerf2
from .baseline import CoDAGQA
from .primitives import HeadwiseRMSNorm, RotaryEmbedding
from .stack import CoDAStack
from .state import CoDAGQALandmarkStatePerf2
from .state_io import (_deep_copy_state, _state_to_cpu, _state_to_device, state_from_bytes, state_from_fields,
                       state_to_bytes)

__all__ = [
    "CoDAGQALandmarkPerf2", "CoDAGQALandmarkStatePerf2", "CoDAGQA", "CoDAStack", "LlamaCoDAAdapter", "EveCoDAAdapter", "Qwen3CoDAAdapter",
    "HeadwiseRMSNorm", "RotaryEmbedding", "state_from_fields", "state_to_bytes", "state_from_bytes", "_state_to_cpu", "_state_to_device",
    "_deep_copy_state",
]
