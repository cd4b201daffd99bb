"""Decode steps as CUDA graphs (placeholder until capture is wired: runs eagerly)."""
from __future__ import annotations

from .step import Stepper


class GraphStepper(Stepper):
    pass
