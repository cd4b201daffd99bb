"""Model assembly, the step function, generation and trace replay."""
from .model import Model, expected_tensors, parse_dtype
from .step import LayerTaps, StepEntry, StepError, StepOutcome, Stepper

__all__ = ["Model", "expected_tensors", "parse_dtype", "LayerTaps", "StepEntry", "StepError", "StepOutcome", "Stepper"]
