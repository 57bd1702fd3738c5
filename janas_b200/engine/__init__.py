"""The engine: the generic decoder, the step function, the generation loop."""
from .model import DecoderModel, expected_tensors
from .engine import Engine, StepEntry, StepError, parse_dtype
from .replay import Replayer
from .session import Session, SessionError, sessions_step

__all__ = ["DecoderModel", "expected_tensors", "Engine", "StepEntry", "StepError", "parse_dtype", "Replayer",
           "Session", "SessionError", "sessions_step"]
