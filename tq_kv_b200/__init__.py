"""tq_kv_b200 — a small, whole generation library for the Qwen2.5 dense
decoder on one B200: typed configuration and registry, weights by name,
layers put together from parts, a paged cache with slots, one step function,
a generation loop, samplers, hand-written CUDA kernels for sm_100a, a true
float32 path, and trace replay."""
from .api import EngineBuilder, load
from .config import named_shape, register_architecture, shape_names
from .engine import Engine, StepError, StepRow
from .engine.generate import GenerationResult, generate
from .sampling import GenerationParams

__all__ = ["Engine", "EngineBuilder", "GenerationParams", "GenerationResult", "StepError", "StepRow", "generate",
           "load", "named_shape", "register_architecture", "shape_names"]
