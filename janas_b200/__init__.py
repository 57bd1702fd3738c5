"""janas_b200: a small, whole generation library for one B200.

Everything between a request's tokens and its next token: configuration and
registry (``config``), weights (``weights``), layer parts (``parts``), the
paged cache and per-sequence state (``cache``), the step function, the
generation loop and sessions (``engine``), and the CUDA kernels for sm_100a
(``csrc``).  All of it is one C++/CUDA library (``libjanas_b200.so``, built in
the tree at the first call) behind the C interface of
``include/janas_b200/llm.h``; the Python modules are thin wrappers over it.
"""
__version__ = "0.1.0"

from .api import (ABI_VERSION, EFAIL, EFULL, EINVAL, ELIMIT, EMODEL, ENOMEM, EOPEN, OK, LLM,
                  CacheFull, LLMError, LLMParams, abi_version, open, params_default)
from .engine.generate import GenOptions, GenStats

__all__ = ["ABI_VERSION", "EFAIL", "EFULL", "EINVAL", "ELIMIT", "EMODEL", "ENOMEM", "EOPEN", "OK",
           "LLM", "CacheFull", "LLMError", "LLMParams", "abi_version", "open", "params_default", "GenOptions",
           "GenStats"]
