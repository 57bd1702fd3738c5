"""Sessions: one token sequence that grows by appending tokens (a prompt, a
user's turn) and by generating them, token by token on request.

Every token is computed once: a new turn goes on from the position reached, with
the cache kept (src/llm/generate.h:88-98).  The names and meanings are those of
the reference's session interface: ``append`` (src/llm/generate.c:709-742),
``prefill`` (:744-773: all appended tokens but the last, which the next pass
takes), ``next`` (:886-900: the next token, appended to the sequence; status 1
when the context is full, an error for an empty sequence), ``truncate``
(src/llm/generate.h:160-167), ``reset``, ``set_options`` (the seed restarts the
random sequence, src/llm/generate.h:116-119), ``computed`` / ``length`` /
``tokens`` (:166-175), and ``sessions_step`` for several sessions on one model:
each one's prompt or its next token in one pass, each token drawn by its own
sampler, the tokens those each session would get alone
(src/llm/generate.c:1155-1249).  A session does not stop by itself at a stop
token: the caller sees every token and decides (``is_stop``, :699-707).

Left out, as in the rest of this library: drafts, slides of the context, saved
copies, biases, filters and log-probabilities.
"""
from __future__ import annotations

import time
from typing import List, Optional, Sequence, Tuple

from .generate import GenOptions, GenStats, _pick

OK = 0          # a token was produced
FULL = 1        # the context is full: no further token can be fed


class SessionError(ValueError):
    """A call that cannot be served; ``code`` is the reference's error code for it
    (include/janas/llm.h:43-53): -1 an invalid argument, -5 a full context."""

    def __init__(self, message: str, code: int = -1):
        super().__init__(message)
        self.code = code


class Session:
    def __init__(self, engine, options: Optional[GenOptions] = None):
        self.engine = engine
        self.vocab = engine.model.spec.vocab_size
        self.hist: List[int] = []
        self.stats = GenStats()
        self.slot: Optional[int] = engine.new_sequence()
        self.options = GenOptions()
        try:
            self.set_options(options or GenOptions())
        except Exception:
            self.close()
            raise

    # ------------------------------------------------------------ the sequence
    @property
    def computed(self) -> int:
        """Tokens of the sequence the model has computed."""
        return self.engine.length(self._slot())

    @property
    def length(self) -> int:
        """Tokens in the sequence (appended and returned)."""
        return len(self.hist)

    def tokens(self) -> List[int]:
        return list(self.hist)

    def _slot(self) -> int:
        if self.slot is None:
            raise SessionError("the session is closed")
        return self.slot

    def set_options(self, options: GenOptions) -> None:
        """New sampling settings, from the next pass on; the seed restarts the
        random sequence."""
        options.validate(self.vocab)
        self.options = options
        self.engine.cache.set_samplers([self._slot()], [options])

    def append(self, tokens: Sequence[int]) -> None:
        """Appends tokens to the sequence.  Raises SessionError when the context
        cannot hold them (it holds ``max_positions`` computed tokens and one more
        that is not fed) or an id lies outside the vocabulary; nothing is changed
        then."""
        self._slot()
        toks = [int(t) for t in tokens]
        if any(t < 0 or t >= self.vocab for t in toks):
            raise SessionError(f"a token id lies outside the vocabulary of {self.vocab}")
        if len(self.hist) + len(toks) > self.engine.max_positions + 1:
            raise SessionError(f"{len(self.hist)} + {len(toks)} tokens do not fit the context "
                               f"of {self.engine.max_positions}", code=-5)
        self.hist.extend(toks)

    def truncate(self, n: int) -> None:
        """Keeps only the first ``n`` tokens of the sequence, so that what follows
        can be appended in place of the rest.  Of the kept tokens the last one is
        computed again by the next pass (its logits are needed); where the cache
        cannot go back (a window whose pages are gone, a mixer with a state of its
        own), all of them are."""
        if not 0 <= n <= len(self.hist):
            raise SessionError(f"cannot keep {n} of {len(self.hist)} tokens")
        del self.hist[n:]
        keep = min(self.computed, max(n - 1, 0))
        if not self.engine.truncate_sequence(self._slot(), keep):
            self.engine.truncate_sequence(self._slot(), 0)

    def reset(self) -> None:
        """Back to an empty sequence."""
        self.truncate(0)

    def close(self) -> None:
        if self.slot is not None:
            self.engine.free_sequence(self.slot)
            self.slot = None

    # ---------------------------------------------------------------- passes
    def prefill(self) -> None:
        """Runs the appended tokens through the model now (``next`` does it
        anyway): all but the last, which the next pass takes."""
        n = len(self.hist) - 1 - self.computed
        if n > 0:
            t0 = time.perf_counter()
            _feed(self.engine, [(self, n, False)])
            self.stats.prompt_tokens += n
            self.stats.prefill_seconds += time.perf_counter() - t0

    def next(self) -> Tuple[int, Optional[int]]:
        """The next token after the sequence, appended to it: (OK, token), or
        (FULL, None) when the context is full."""
        tokens, status = sessions_step(self.engine, [self])
        return status[0], tokens[0]


def _feed(engine, items):
    """Runs, for each (session, count, wanted) of ``items``, the next ``count``
    tokens that the session has not computed; returns the logits of the last one
    of every item that wants them (in the items' order), or None.

    One step where the model can take it: all sequences at their start, all with
    one token, or (models whose mixers can append several tokens to a sequence
    that holds some) any mixture.  Else the sequences at their start go first,
    and the others go on token by token together."""
    import torch
    from .engine import StepEntry
    from ..parts import EXTEND

    def entries(part, counts, wants):
        return [StepEntry(s._slot(), s.hist[s.computed:s.computed + c], [c - 1] if w else [])
                for (s, _, _), c, w in zip(part, counts, wants)]

    starts = [it for it in items if it[0].computed == 0]
    others = [it for it in items if it[0].computed > 0]
    one_step = (not others or not starts) and all(c == 1 for _, c, _ in others)
    if one_step or engine.model.supports(EXTEND):
        return engine.step(entries(items, [c for _, c, _ in items], [w for _, _, w in items]))
    rows = {}
    if starts:
        lg = engine.step(entries(starts, [c for _, c, _ in starts], [w for _, _, w in starts]))
        wanted = [it for it in starts if it[2]]
        for i, it in enumerate(wanted):
            rows[id(it[0])] = lg[i]
    left = {id(s): c for s, c, _ in others}
    while any(left.values()):
        part = [it for it in others if left[id(it[0])] > 0]
        wants = [it[2] and left[id(it[0])] == 1 for it in part]
        lg = engine.step(entries(part, [1] * len(part), wants))
        k = 0
        for it, w in zip(part, wants):
            left[id(it[0])] -= 1
            if w:
                rows[id(it[0])] = lg[k]
                k += 1
    out = [rows[id(s)] for s, _, w in items if w]
    if not out:
        return None
    return torch.stack(out) if isinstance(out[0], torch.Tensor) else out


def sessions_step(engine, sessions: Sequence[Session]) -> Tuple[List[Optional[int]], List[int]]:
    """Moves several sessions of one engine on together, every weight read once
    for all of them: each one's appended tokens and its next token in one pass.
    Returns (tokens, status) as ``Session.next`` gives them, one per session.  An
    empty sequence is an error; a cache without room raises CacheFull with nothing
    changed."""
    from ..csrc import ops
    if len({id(s) for s in sessions}) != len(sessions):
        raise SessionError("a session appears twice")
    for s in sessions:
        if s.engine is not engine:
            raise SessionError("a session of another engine")
        s._slot()
        if not s.hist:
            raise SessionError("the sequence is empty")
    tokens: List[Optional[int]] = [None] * len(sessions)
    status = [OK] * len(sessions)
    live = []
    for i, s in enumerate(sessions):
        if len(s.hist) > engine.max_positions:
            status[i] = FULL
        else:
            live.append(i)
    if not live:
        return tokens, status
    t0 = time.perf_counter()
    ss = [sessions[i] for i in live]
    slots = [s._slot() for s in ss]
    sampled = any(s.options.temperature > 0 for s in ss)
    big = None
    if any(s.options.temperature > 0 and not 0 < s.options.top_k <= ops.sample_small_cap()
           for s in ss):
        big = engine.sampler_scratch(len(ss))
    counts = [len(s.hist) - s.computed for s in ss]
    if all(c == 1 and s.computed > 0 for s, c in zip(ss, counts)) and hasattr(engine, "decode"):
        got = engine.decode(slots, [s.hist[-1] for s in ss], sampled, big)
        forced = 0
    else:
        logits = _feed(engine, [(s, c, True) for s, c in zip(ss, counts)])
        got, forced = _pick(engine, logits, slots, sampled, big)
    dt = time.perf_counter() - t0
    for i, s, c, tok in zip(live, ss, counts, got):
        tokens[i] = int(tok)
        s.hist.append(int(tok))
        s.stats.new_tokens += 1
        s.stats.passes += 1
        s.stats.forced_tokens += forced if len(ss) == 1 else 0
        if c > 1:
            s.stats.prompt_tokens += c - 1
            s.stats.prefill_seconds += dt
        else:
            s.stats.decode_seconds += dt
    return tokens, status
