"""Model assembly, the step function, the generation loop, trace replay."""
from .batch import StepRow, build_step_batch
from .engine import Engine, StepError
from .model import DecoderModel

__all__ = ["DecoderModel", "Engine", "StepError", "StepRow", "build_step_batch"]
