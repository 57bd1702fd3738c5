"""janas_b200: a small, whole generation library for one B200.

Everything between a request's tokens and its next token: configuration and
registry (``config``), weights (``weights``), layer parts (``parts``), the
paged cache and per-sequence state (``cache``), the step function and the
generation loop (``engine``), sampling (``sampling``) and the CUDA kernels
for sm_100a (``csrc``).
"""
__version__ = "0.1.0"

from .api import (ABI_VERSION, EFAIL, EFULL, EINVAL, EMODEL, ENOMEM, EOPEN, OK, LLM, LLMError,
                  LLMParams, abi_version, open, params_default)
from .engine.generate import GenOptions, GenStats

__all__ = ["ABI_VERSION", "EFAIL", "EFULL", "EINVAL", "EMODEL", "ENOMEM", "EOPEN", "OK", "LLM",
           "LLMError", "LLMParams", "abi_version", "open", "params_default", "GenOptions",
           "GenStats"]
