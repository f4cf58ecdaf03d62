"""Model assembly, the step function, generation and the entry points."""
from .batch import StepEntry
from .spec import LayerSpec, ModelSpec, PartSpec, RunSpec

__all__ = ["StepEntry", "LayerSpec", "ModelSpec", "PartSpec", "RunSpec"]
