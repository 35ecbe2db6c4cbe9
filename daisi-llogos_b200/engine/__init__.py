"""The assembled model and the step function."""
from .context import StepContext, Workspace
from .engine import Engine, StepError
from .model import DecoderModel

__all__ = ["StepContext", "Workspace", "Engine", "StepError", "DecoderModel"]
