"""The model assembled from parts, the step function, and the generation loop."""
from .model import Model
from .engine import DeviceFault, Engine, StepError
from .generate import GenerationResult, generate, plan_batches, run_batch

__all__ = ["Model", "DeviceFault", "Engine", "StepError", "GenerationResult", "generate",
           "plan_batches", "run_batch"]
