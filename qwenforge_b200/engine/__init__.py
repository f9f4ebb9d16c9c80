from .model import Model
from .step import StepContext, build_context

__all__ = ["Model", "StepContext", "build_context"]
