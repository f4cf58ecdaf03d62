"""The entry points: a loaded model with its cache (``Engine``), steps, generation."""
from .batch import StepEntry
from .spec import LayerSpec, ModelSpec, PartSpec, RunSpec

__all__ = ["StepEntry", "LayerSpec", "ModelSpec", "PartSpec", "RunSpec"]
