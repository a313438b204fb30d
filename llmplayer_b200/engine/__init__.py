"""The model walk, the step function and the generation loop."""
from .engine import Engine
from .model import Model, expected_tensors
from .step import SequenceStep, StepContext, Workspace

__all__ = ["Engine", "Model", "SequenceStep", "StepContext", "Workspace", "expected_tensors"]
