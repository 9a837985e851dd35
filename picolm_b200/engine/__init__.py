from .engine import Engine
from .model import Model
from .step_batch import StepBatch, build_step_batch

__all__ = ["Engine", "Model", "StepBatch", "build_step_batch"]
