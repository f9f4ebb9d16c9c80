from .engine import ModelStepper, StudentEngine
from .generate import GenerationLoop, SequenceResult
from .model import Model
from .step import StepContext, build_context

__all__ = ["Model", "ModelStepper", "StudentEngine", "GenerationLoop", "SequenceResult", "StepContext", "build_context"]
