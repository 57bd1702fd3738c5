"""Sessions: one token sequence that grows by appending tokens (a prompt, a user's
turn) and by generating them, token by token on request.

The session is the library's (``engine/generate.cpp``: Session, sessions_step), with
the reference's names and meanings (``janas_llm_session_*``,
src/llm/generate.h:88-175): ``append``, ``prefill`` (all appended tokens but the
last, which the next pass takes), ``next`` (the next token, appended to the
sequence; status 1 when the context is full), ``truncate``, ``reset``,
``set_options`` (the seed restarts the random sequence), ``computed`` / ``length`` /
``tokens``, and ``sessions_step`` for several sessions on one model.  A session
does not stop by itself at a stop token: the caller sees every token and decides.
"""
from __future__ import annotations

import ctypes
from typing import List, Optional, Sequence, Tuple

from .. import lib
from .generate import GenOptions, GenStats, options_c, stats_c

OK = 0          # a token was produced
FULL = 1        # the context is full: no further token can be fed


class SessionError(lib.LLMError, ValueError):
    """A call that cannot be served; ``code`` is the library's code for it: -1 an
    invalid argument, -5 a full context."""

    def __init__(self, message: str, code: int = -1):
        lib.LLMError.__init__(self, code, message)


def _check(code: int) -> int:
    if code in (lib.EINVAL, lib.EFULL):
        raise SessionError(lib.last_error(), code)
    return lib.check(code)


class Session:
    def __init__(self, engine, options: Optional[GenOptions] = None):
        self.engine = engine
        self.options = options or GenOptions()
        o = options_c(self.options)
        h = ctypes.c_void_p()
        _check(lib.lib().jb_llm_session_create(engine._h, ctypes.byref(o), ctypes.byref(h)))
        self._s = h

    def _h(self):
        if self._s is None:
            raise SessionError("the session is closed")
        return self._s

    @property
    def computed(self) -> int:
        """Tokens of the sequence the model has computed."""
        return int(lib.lib().jb_llm_session_computed(self._h()))

    @property
    def length(self) -> int:
        """Tokens in the sequence (appended and returned)."""
        return int(lib.lib().jb_llm_session_length(self._h()))

    def tokens(self) -> List[int]:
        p = ctypes.POINTER(ctypes.c_int32)()
        n = lib.lib().jb_llm_session_tokens(self._h(), ctypes.byref(p))
        return [p[i] for i in range(n)]

    @property
    def hist(self) -> List[int]:
        return self.tokens()

    @property
    def stats(self) -> GenStats:
        c = stats_c()
        _check(lib.lib().jb_llm_session_stats(self._h(), ctypes.byref(c)))
        return GenStats.from_c(c)

    def set_options(self, options: GenOptions) -> None:
        o = options_c(options)
        _check(lib.lib().jb_llm_session_set_options(self._h(), ctypes.byref(o)))
        self.options = options

    def append(self, tokens: Sequence[int]) -> None:
        """Appends tokens to the sequence.  Raises SessionError when the context
        cannot hold them or an id lies outside the vocabulary; nothing is changed
        then."""
        toks = [int(t) for t in tokens]
        _check(lib.lib().jb_llm_session_append(self._h(), lib.i32_array(toks), len(toks)))

    def truncate(self, n: int) -> None:
        _check(lib.lib().jb_llm_session_truncate(self._h(), int(n)))

    def reset(self) -> None:
        _check(lib.lib().jb_llm_session_reset(self._h()))

    def close(self) -> None:
        if self._s is not None:
            lib.lib().jb_llm_session_destroy(self._s)
            self._s = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def prefill(self) -> None:
        _check(lib.lib().jb_llm_session_prefill(self._h()))

    def next(self) -> Tuple[int, Optional[int]]:
        """The next token after the sequence, appended to it: (OK, token), or
        (FULL, None) when the context is full."""
        t = ctypes.c_int32()
        code = _check(lib.lib().jb_llm_session_next(self._h(), ctypes.byref(t)))
        return (FULL, None) if code == lib.DONE else (OK, t.value)


def sessions_step(engine, sessions: Sequence[Session]) -> Tuple[List[Optional[int]], List[int]]:
    """Moves several sessions of one engine on together, every weight read once for
    all of them.  Returns (tokens, status) as ``Session.next`` gives them."""
    n = len(sessions)
    for s in sessions:
        if s.engine is not engine:
            raise SessionError("a session of another engine")
    hs = (ctypes.c_void_p * max(n, 1))(*[s._h() for s in sessions])
    toks = (ctypes.c_int32 * max(n, 1))()
    status = (ctypes.c_int32 * max(n, 1))()
    _check(lib.lib().jb_llm_sessions_step(hs, n, toks, status))
    return [None if status[i] else toks[i] for i in range(n)], [status[i] for i in range(n)]
