"""The engine: an open model with its cache, the step function, decode steps, the
generation loop, sessions and trace replay (all of them the library's, C++)."""
from .engine import Engine, PendingDecode, StepEntry, StepError, parse_dtype
from . import generate
from .generate import (GenOptions, GenStats, Request, Result, finish_reason,
                       goes_on_unless_stopped, plan_batches, tokens_needed)
from .replay import Replayer
from .session import Session, SessionError, sessions_step
from ..weights import expected_tensors

__all__ = ["Engine", "GenOptions", "GenStats", "PendingDecode", "Replayer", "Request", "Result",
           "Session", "SessionError", "StepEntry", "StepError", "expected_tensors", "finish_reason",
           "generate", "goes_on_unless_stopped", "parse_dtype", "plan_batches", "sessions_step",
           "tokens_needed"]
