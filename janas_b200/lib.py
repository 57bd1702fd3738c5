"""The compiled library (``libjanas_b200.so``) as ctypes sees it.

Everything this package does happens in that library: configuration, weights,
parts, cache, step function, generation loop and kernels are C++ and CUDA behind
the C interface of ``include/janas_b200/llm.h``.  This module loads the library
(building it at the first call), declares the interface's structs and functions,
and turns its return codes into exceptions.  The Python modules beside it are thin
wrappers over these calls.
"""
from __future__ import annotations

import ctypes
import json
import threading
from typing import Any, Dict, Optional

from .csrc import build

ABI_VERSION = 2

OK = 0
DONE = 1
EINVAL = -1   # invalid argument
ENOMEM = -2   # out of memory
EOPEN = -3    # model folder missing, unreadable, invalid
EMODEL = -4   # model not supported (architecture)
EFULL = -5    # the context or the cache is full
EBUSY = -6
ESMALL = -7   # buffer too small
EFAIL = -8    # internal failure
ELIMIT = -9   # the prompt is longer than the context

BF16 = 0
F32 = 1
MAX_STOP = 4


class LLMError(RuntimeError):
    """A call of the library that failed; ``code`` is its return code."""

    def __init__(self, code: int, message: str):
        super().__init__(message)
        self.code = code


class CacheFull(LLMError):
    """No free page or slot is left (code EFULL)."""

    def __init__(self, message: str, code: int = EFULL):
        super().__init__(code, message)


class Params(ctypes.Structure):
    _fields_ = [("size", ctypes.c_uint32), ("n_ctx", ctypes.c_uint32),
                ("max_batch", ctypes.c_uint32), ("dtype", ctypes.c_int32),
                ("device", ctypes.c_int32), ("reserved", ctypes.c_uint32),
                ("max_tokens", ctypes.c_uint64)]


class GenOptionsC(ctypes.Structure):
    _fields_ = [("size", ctypes.c_uint32), ("eos", ctypes.c_int32),
                ("temperature", ctypes.c_float), ("top_k", ctypes.c_int32),
                ("top_p", ctypes.c_float), ("min_p", ctypes.c_float), ("seed", ctypes.c_uint64),
                ("stop", ctypes.c_int32 * MAX_STOP), ("n_stop", ctypes.c_int32),
                ("reserved", ctypes.c_uint32)]


class GenStatsC(ctypes.Structure):
    _fields_ = [("size", ctypes.c_uint32), ("prompt_tokens", ctypes.c_uint32),
                ("new_tokens", ctypes.c_uint32), ("passes", ctypes.c_uint32),
                ("forced_tokens", ctypes.c_uint32), ("batches", ctypes.c_uint32),
                ("prefill_seconds", ctypes.c_double), ("decode_seconds", ctypes.c_double),
                ("sample_seconds", ctypes.c_double), ("h2d_bytes", ctypes.c_uint64),
                ("d2h_bytes", ctypes.c_uint64)]


class Piece(ctypes.Structure):
    _fields_ = [("slot", ctypes.c_int32), ("n", ctypes.c_uint32),
                ("tokens", ctypes.POINTER(ctypes.c_int32)), ("n_want", ctypes.c_uint32),
                ("want", ctypes.POINTER(ctypes.c_int32))]


PART_CALLBACK = ctypes.CFUNCTYPE(ctypes.c_void_p, ctypes.c_void_p, ctypes.c_char_p,
                                 ctypes.c_char_p)

_lock = threading.Lock()
_lib: Optional[ctypes.CDLL] = None


def _declare(L: ctypes.CDLL) -> None:
    P, I32, U32, U64 = ctypes.c_void_p, ctypes.c_int32, ctypes.c_uint32, ctypes.c_uint64
    i32p, u32p = ctypes.POINTER(ctypes.c_int32), ctypes.POINTER(ctypes.c_uint32)
    sig = {
        "jb_llm_abi_version": (I32, []),
        "jb_llm_last_error": (ctypes.c_char_p, []),
        "jb_llm_params_default": (None, [ctypes.POINTER(Params)]),
        "jb_gen_options_default": (None, [ctypes.POINTER(GenOptionsC)]),
        "jb_llm_open": (I32, [ctypes.c_char_p, ctypes.POINTER(Params), ctypes.POINTER(P)]),
        "jb_llm_open_random": (I32, [ctypes.c_char_p, U64, ctypes.POINTER(Params),
                                     ctypes.POINTER(P)]),
        "jb_llm_open_spec": (I32, [ctypes.c_char_p, ctypes.c_char_p, U64, ctypes.POINTER(Params),
                                   ctypes.POINTER(P)]),
        "jb_llm_close": (None, [P]),
        "jb_llm_info": (ctypes.c_char_p, [P]),
        "jb_llm_n_ctx": (U32, [P]),
        "jb_llm_n_vocab": (U32, [P]),
        "jb_llm_check": (I32, [P]),
        "jb_llm_slot_new": (I32, [P, i32p]),
        "jb_llm_slot_free": (I32, [P, I32]),
        "jb_llm_slot_length": (I32, [P, I32, u32p]),
        "jb_llm_slot_truncate": (I32, [P, I32, U32]),
        "jb_llm_step": (I32, [P, ctypes.POINTER(Piece), U32, P, U64]),
        "jb_llm_generate": (I32, [P, i32p, U32, U32, ctypes.POINTER(GenOptionsC), i32p, u32p, i32p,
                                  ctypes.POINTER(GenStatsC)]),
        "jb_llm_generate_batch": (I32, [P, U32, ctypes.POINTER(i32p), u32p, u32p,
                                        ctypes.POINTER(ctypes.POINTER(GenOptionsC)), i32p, u32p,
                                        i32p, ctypes.POINTER(GenStatsC)]),
        "jb_llm_session_create": (I32, [P, ctypes.POINTER(GenOptionsC), ctypes.POINTER(P)]),
        "jb_llm_session_destroy": (None, [P]),
        "jb_llm_session_set_options": (I32, [P, ctypes.POINTER(GenOptionsC)]),
        "jb_llm_session_append": (I32, [P, i32p, U32]),
        "jb_llm_session_prefill": (I32, [P]),
        "jb_llm_session_next": (I32, [P, i32p]),
        "jb_llm_sessions_step": (I32, [ctypes.POINTER(P), I32, i32p, i32p]),
        "jb_llm_session_computed": (U32, [P]),
        "jb_llm_session_length": (U32, [P]),
        "jb_llm_session_tokens": (U32, [P, ctypes.POINTER(i32p)]),
        "jb_llm_session_truncate": (I32, [P, U32]),
        "jb_llm_session_reset": (I32, [P]),
        "jb_llm_session_stats": (I32, [P, ctypes.POINTER(GenStatsC)]),
        "jb_llm_slot_sampler": (I32, [P, I32, ctypes.POINTER(GenOptionsC)]),
        "jb_llm_decode_begin": (I32, [P, i32p, U32, i32p, I32, ctypes.POINTER(P)]),
        "jb_llm_decode_end": (I32, [P, P, i32p]),
        "jb_llm_stream": (P, [P]),
        "jb_register_part": (I32, [ctypes.c_char_p, ctypes.c_char_p, PART_CALLBACK, P]),
        "jb_call": (I32, [ctypes.c_char_p, ctypes.c_char_p, ctypes.POINTER(P)]),
        "jb_free": (None, [P]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(L, name)
        fn.restype = res
        fn.argtypes = args


def lib() -> ctypes.CDLL:
    """The loaded library; compiled first when it is missing or out of date."""
    global _lib
    if _lib is None:
        with _lock:
            if _lib is None:
                path = build.library_path()
                try:
                    loaded = ctypes.CDLL(path)
                except OSError as e:
                    raise LLMError(EFAIL, f"janas_b200: cannot load {path}: {e}") from None
                _declare(loaded)
                have = loaded.jb_llm_abi_version()
                if have != ABI_VERSION:
                    raise LLMError(EFAIL, f"janas_b200: {path} has ABI version {have}, this "
                                          f"package wants {ABI_VERSION}")
                _lib = loaded
    return _lib


def loaded_library_path() -> Optional[str]:
    return _lib._name if _lib is not None else None


def last_error() -> str:
    return lib().jb_llm_last_error().decode("utf-8", "replace")


def check(code: int) -> int:
    """Raises for a negative return code; returns the code otherwise."""
    if code >= 0:
        return code
    msg = last_error()
    if code == EFULL:
        raise CacheFull(msg)
    raise LLMError(code, msg)


def call(method: str, **args: Any) -> Dict[str, Any]:
    """``jb_call``: one of the library's methods by name, JSON in and out."""
    out = ctypes.c_void_p()
    L = lib()
    code = L.jb_call(method.encode(), json.dumps(args).encode(), ctypes.byref(out))
    raw = ctypes.string_at(out.value) if out.value else b""
    L.jb_free(out)
    result = json.loads(raw.decode("utf-8")) if raw else {}
    if code < 0:
        msg = last_error()
        err = CacheFull(msg) if code == EFULL else LLMError(code, msg)
        err.detail = result
        raise err
    return result


def i32_array(values) -> ctypes.Array:
    values = list(values)
    return (ctypes.c_int32 * max(len(values), 1))(*values)
