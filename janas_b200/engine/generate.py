"""The generation loop above the step function.

Requests (a prompt, a limit of new tokens, sampling options) are run in batches:
the prompts of a batch in one step, then one token for every sequence that is
still going, until all have ended; then the next batch, whose sequences take
the slots and pages the previous ones gave back.  A sequence ends after a stop
token (which is part of its output), at its limit of new tokens, or when the
context is full.  Once a batch has started, no request joins it.

The reference's loop is ``janas_llm_generate`` (src/llm/generate.c:1116-1144:
prompt, then tokens until a stop token or max_new; the stop token is counted:
:1136-1137; ``is_stop`` :699-707; a full context ends the sequence:
:895-896) and, for several sequences, ``janas_llm_sessions_step``
(src/llm/generate.c:1155-1249: one pass for all sessions, each token drawn by
its own sampler).  Options and statistics carry the reference's names
(``struct janas_gen_options``, ``struct janas_gen_stats``:
src/llm/generate.h:31-86).

The decisions (which requests form a batch, when a sequence ends) are plain
host code without a device, so they can be tested alone.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import List, Optional, Sequence, Tuple

import numpy as np

from ..cache.pages import PAGE, pages_for

MAX_STOP = 4  # JANAS_GEN_MAX_STOP (src/llm/generate.h:27)

FINISH_STOP = "stop"        # a stop token was generated
FINISH_LENGTH = "length"    # max_new tokens were generated
FINISH_CONTEXT = "context"  # the context is full


@dataclass
class GenOptions:
    """Sampling and stopping; all zero: greedy (src/llm/generate.h:31-63)."""

    eos: int = -1              # stop at this token, -1 for none
    temperature: float = 0.0   # 0: the most likely token
    top_k: int = 0             # keep the k most likely tokens; 0: no limit
    top_p: float = 0.0         # keep the most likely tokens up to this mass; 0 or 1: off
    min_p: float = 0.0         # drop tokens below min_p x the top probability
    seed: int = 0
    stop: Sequence[int] = ()   # more stop tokens, besides eos (at most 4)

    def validate(self, vocab: int) -> None:
        if len(self.stop) > MAX_STOP:
            raise ValueError(f"at most {MAX_STOP} stop tokens besides eos")
        if self.temperature < 0 or not 0 <= self.top_p <= 1 or not 0 <= self.min_p <= 1 \
                or self.top_k < 0:
            raise ValueError("temperature >= 0, top_k >= 0, top_p and min_p within [0, 1]")

    def stop_set(self) -> frozenset:
        s = set(int(t) for t in self.stop)
        if self.eos >= 0:
            s.add(int(self.eos))
        return frozenset(s)


@dataclass
class GenStats:
    """Counters of one call (src/llm/generate.h:65-86, the fields that apply)."""

    prompt_tokens: int = 0
    new_tokens: int = 0
    passes: int = 0             # forward passes after the prefill
    forced_tokens: int = 0      # drawn where only one candidate was left
    prefill_seconds: float = 0.0
    decode_seconds: float = 0.0
    sample_seconds: float = 0.0
    batches: int = 0
    h2d_bytes: int = 0          # step inputs copied to the device while decoding
    d2h_bytes: int = 0          # chosen tokens read back while decoding


@dataclass
class Request:
    prompt: Sequence[int]
    max_new: int
    options: GenOptions = field(default_factory=GenOptions)


@dataclass
class Result:
    tokens: List[int]
    finish: str


# ------------------------------------------------------------------ decisions
def tokens_needed(prompt_len: int, max_new: int, max_positions: int) -> int:
    """Cache tokens a request may come to hold, rounded up to whole pages.  The
    last generated token is never fed back, so it needs no place."""
    return pages_for(min(prompt_len + max(max_new - 1, 0), max_positions)) * PAGE


def plan_batches(prompt_lens: Sequence[int], max_news: Sequence[int], max_batch: int,
                 max_tokens: int, max_positions: int) -> List[List[int]]:
    """Cuts the requests, in their order, into batches of at most ``max_batch``
    whose sequences fit the cache together even if every one runs to its limit."""
    batches: List[List[int]] = []
    cur: List[int] = []
    used = 0
    for i, (p, m) in enumerate(zip(prompt_lens, max_news)):
        need = tokens_needed(p, m, max_positions)
        if need > max_tokens:
            raise ValueError(f"request {i}: {p} prompt tokens and {m} new ones need "
                             f"{need} tokens of cache, the cache has {max_tokens}")
        if cur and (len(cur) >= max_batch or used + need > max_tokens):
            batches.append(cur)
            cur, used = [], 0
        cur.append(i)
        used += need
    if cur:
        batches.append(cur)
    return batches


def finish_reason(token: int, n_generated: int, max_new: int, length: int, max_positions: int,
                  stops: frozenset) -> Optional[str]:
    """Whether a sequence ends after ``token``, its ``n_generated``-th new one;
    ``length`` is what the cache holds of it (the token itself not yet)."""
    if token in stops:
        return FINISH_STOP
    if n_generated >= max_new:
        return FINISH_LENGTH
    if length + 1 > max_positions:
        return FINISH_CONTEXT
    return None


def goes_on_unless_stopped(n_generated: int, max_new: int, length: int, max_positions: int
                           ) -> bool:
    """Whether a sequence goes on after its ``n_generated``-th new token if that is
    no stop token (``finish_reason`` with the token left open): the next step may
    then be launched before the token is known.  ``length`` is what the cache
    holds of the sequence before that token is fed."""
    return n_generated < max_new and length + 1 <= max_positions


# ----------------------------------------------------------------------- loop
def generate(engine, requests: Sequence[Request], max_batch: int = 64,
             stats: Optional[GenStats] = None) -> List[Result]:
    """Runs all requests; returns their new tokens and why each ended."""
    import torch
    from ..csrc import ops
    from .engine import StepEntry

    vocab = engine.model.spec.vocab_size
    for i, r in enumerate(requests):
        r.options.validate(vocab)
        if len(r.prompt) == 0:
            raise ValueError(f"request {i}: the prompt is empty")
        if len(r.prompt) > engine.max_positions:
            raise ValueError(f"request {i}: the prompt has {len(r.prompt)} tokens, the context "
                             f"{engine.max_positions}")
    st = stats if stats is not None else GenStats()
    results: List[Optional[Result]] = [None] * len(requests)
    plan = plan_batches([len(r.prompt) for r in requests], [r.max_new for r in requests],
                        min(max_batch, engine.cache.max_seqs), engine.cache.max_tokens,
                        engine.max_positions)
    cache = engine.cache
    for batch in plan:
        st.batches += 1
        live = [i for i in batch if requests[i].max_new > 0]
        for i in batch:
            if requests[i].max_new <= 0:
                results[i] = Result([], FINISH_LENGTH)
        if not live:
            continue
        slots = {i: engine.new_sequence() for i in live}
        try:
            sampled = any(requests[i].options.temperature > 0 for i in live)
            if sampled:
                cache.set_samplers([slots[i] for i in live], [requests[i].options for i in live])
            big = None
            if sampled and any(requests[i].options.temperature > 0 and
                               not 0 < requests[i].options.top_k <= ops.sample_small_cap()
                               for i in live):
                if hasattr(engine, "sampler_scratch"):
                    big = engine.sampler_scratch(len(live))
                else:
                    cap = 1 << (vocab - 1).bit_length()
                    big = (torch.empty((len(live), cap), dtype=torch.int64, device=engine.device),
                           torch.empty((len(live), cap), dtype=torch.float32,
                                       device=engine.device))
            out = {i: [] for i in live}
            stops = {i: requests[i].options.stop_set() for i in live}

            t0 = time.perf_counter()
            st.prompt_tokens += sum(len(requests[i].prompt) for i in live)
            logits = engine.step([StepEntry(slots[i], requests[i].prompt,
                                            [len(requests[i].prompt) - 1]) for i in live])
            toks, forced = _pick(engine, logits, [slots[i] for i in live], sampled, big)
            now = time.perf_counter()
            st.prefill_seconds += now - t0
            active = list(live)
            # Decode steps are launched one ahead where the engine can feed a step
            # the tokens of the step before it on the device: while step t runs,
            # step t + 1 is already queued behind it, and the host reads t's tokens
            # meanwhile.  That is done only when every sequence is sure to go on
            # unless it draws a stop token; one that does has run one step too many,
            # which changes nothing for the others, and the loop then takes the
            # remaining sequences' tokens from that step before it goes on.
            ahead_ok = bool(getattr(engine, "decodes_ahead", False))
            ahead = None            # the step under way beyond ``toks``, and its rows
            ahead_rows: List[int] = []
            while True:
                st.forced_tokens += forced
                forced = 0
                nxt, feed = [], []
                for i, tok in zip(active, toks):
                    out[i].append(int(tok))
                    st.new_tokens += 1
                    held = engine.length(slots[i]) - (1 if ahead is not None else 0)
                    why = finish_reason(int(tok), len(out[i]), requests[i].max_new, held,
                                        engine.max_positions, stops[i])
                    if why is None:
                        nxt.append(i)
                        feed.append(int(tok))
                    else:
                        results[i] = Result(out[i], why)
                        engine.free_sequence(slots.pop(i))
                ended = len(nxt) != len(active)
                active = nxt
                t0 = time.perf_counter()
                if ahead is not None and (ended or not active):
                    # the step under way ran with sequences that have ended: the
                    # others' tokens are good
                    got = engine.decode_end(ahead)
                    st.passes += 1
                    st.d2h_bytes += 4 * len(ahead_rows)
                    st.decode_seconds += time.perf_counter() - t0
                    toks = [got[ahead_rows.index(i)] for i in active]
                    ahead = None
                    if not active:
                        break
                    continue
                if not active:
                    break
                h2d0 = getattr(engine, "h2d_bytes", 0)
                cur_slots = [slots[i] for i in active]
                if ahead is not None:
                    cur, ahead = ahead, None
                elif ahead_ok:
                    cur = engine.decode_begin(cur_slots, feed, sampled, big)
                else:
                    cur = None
                    toks, forced = _decode(engine, cur_slots, feed, sampled, big)
                if cur is not None:
                    if all(goes_on_unless_stopped(len(out[i]) + 1, requests[i].max_new,
                                                  engine.length(slots[i]), engine.max_positions)
                           for i in active):
                        ahead = engine.decode_begin(cur_slots, None, sampled, big)
                        ahead_rows = list(active)
                    toks = engine.decode_end(cur)
                st.passes += 1
                st.decode_seconds += time.perf_counter() - t0
                st.h2d_bytes += getattr(engine, "h2d_bytes", 0) - h2d0
                st.d2h_bytes += 4 * len(active)
        finally:
            for s in slots.values():
                engine.free_sequence(s)
    return results  # type: ignore[return-value]


def _decode(engine, slots: List[int], tokens: List[int], sampled: bool, big
            ) -> Tuple[np.ndarray, int]:
    """One decode step and the choice of the next tokens; returns them on the
    host (and how many draws had one candidate only, where that is counted)."""
    if hasattr(engine, "decode"):
        return engine.decode(slots, tokens, sampled, big), 0
    from .engine import StepEntry
    logits = engine.step([StepEntry(s, [t], [0]) for s, t in zip(slots, tokens)])
    return _pick(engine, logits, slots, sampled, big)


def _pick(engine, logits, slots: List[int], sampled: bool, big) -> Tuple[np.ndarray, int]:
    """One token per row of logits, on the device; returns them on the host."""
    import torch
    from ..csrc import ops

    cache = engine.cache
    if not sampled:
        return ops.sample(logits).cpu().numpy(), 0
    row_slot = torch.tensor(slots, dtype=torch.int32).to(engine.device, non_blocking=True)
    forced = torch.zeros(len(slots), dtype=torch.int32, device=engine.device)
    toks = ops.sample(logits, row_slot=row_slot, temperature=cache.temperature,
                      top_k=cache.top_k, top_p=cache.top_p, min_p=cache.min_p, rng=cache.rng,
                      big_keys=None if big is None else big[0],
                      big_probs=None if big is None else big[1], forced=forced)
    toks = toks.cpu().numpy()
    if (toks < 0).any():
        raise RuntimeError("the sampler had no scratch for a row with top_k off")
    return toks, int(forced.sum().item())
