"""Model, step function, generation loop and the runtime entry point."""
from .batch import StepBatch, StepEntry, build_batch
from .engine import Engine, StepError
from .generate import STOP, Blocked, GenerationLoop, RequestError
from .model import Model, declared_weights
from .probe import LayerProbe
from .runtime import GpuRuntime

__all__ = ["StepBatch", "StepEntry", "build_batch", "Engine", "StepError", "Model", "declared_weights",
           "GpuRuntime", "GenerationLoop", "RequestError", "Blocked", "STOP", "LayerProbe"]
