"""Generation options and counters, the loop's decisions, and the loop itself, as
the library has them (``engine/generate.cpp``).

The names are the reference's (``struct janas_gen_options``, ``struct
janas_gen_stats``: src/llm/generate.h:31-86).  ``generate`` runs requests through
an open engine; the decision functions answer without a device.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass, field
from typing import List, Optional, Sequence

from .. import lib

MAX_STOP = lib.MAX_STOP  # JANAS_GEN_MAX_STOP (src/llm/generate.h:27)

FINISH_STOP = "stop"        # a stop token was generated
FINISH_LENGTH = "length"    # max_new tokens were generated
FINISH_CONTEXT = "context"  # the context is full
_FINISH = {1: FINISH_STOP, 2: FINISH_LENGTH, 3: FINISH_CONTEXT}


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

    def validate(self, vocab: int = 0) -> None:
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


def options_c(o: Optional[GenOptions]) -> lib.GenOptionsC:
    """The options as the C interface's struct."""
    c = lib.GenOptionsC()
    lib.lib().jb_gen_options_default(ctypes.byref(c))
    if o is None:
        return c
    o.validate()
    c.eos, c.temperature, c.top_k = int(o.eos), float(o.temperature), int(o.top_k)
    c.top_p, c.min_p, c.seed = float(o.top_p), float(o.min_p), int(o.seed) & (2 ** 64 - 1)
    c.n_stop = len(o.stop)
    for i, t in enumerate(o.stop):
        c.stop[i] = int(t)
    return c


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

    @staticmethod
    def from_c(c: lib.GenStatsC) -> "GenStats":
        return GenStats(c.prompt_tokens, c.new_tokens, c.passes, c.forced_tokens, c.prefill_seconds,
                        c.decode_seconds, c.sample_seconds, c.batches, c.h2d_bytes, c.d2h_bytes)


def stats_c() -> lib.GenStatsC:
    c = lib.GenStatsC()
    c.size = ctypes.sizeof(lib.GenStatsC)
    return c


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
    """Cache tokens a request may come to hold, rounded up to whole pages."""
    return lib.call("gen.tokens_needed", prompt_len=prompt_len, max_new=max_new,
                    max_positions=max_positions)["tokens"]


def plan_batches(prompt_lens: Sequence[int], max_news: Sequence[int], max_batch: int,
                 max_tokens: int, max_positions: int) -> List[List[int]]:
    """Cuts the requests, in their order, into batches of at most ``max_batch``
    whose sequences fit the cache together even if every one runs to its limit."""
    return lib.call("gen.plan_batches", prompt_lens=list(prompt_lens), max_news=list(max_news),
                    max_batch=max_batch, max_tokens=max_tokens,
                    max_positions=max_positions)["batches"]


def finish_reason(token: int, n_generated: int, max_new: int, length: int, max_positions: int,
                  stops) -> Optional[str]:
    """Whether a sequence ends after ``token``, its ``n_generated``-th new one."""
    return lib.call("gen.finish_reason", token=token, n_generated=n_generated, max_new=max_new,
                    length=length, max_positions=max_positions, eos=-1,
                    stop=sorted(stops))["finish"]


def goes_on_unless_stopped(n_generated: int, max_new: int, length: int, max_positions: int) -> bool:
    return lib.call("gen.goes_on", n_generated=n_generated, max_new=max_new, length=length,
                    max_positions=max_positions)["ok"]


# ----------------------------------------------------------------------- loop
def generate(engine, requests: Sequence[Request], max_batch: Optional[int] = None,
             stats: Optional[GenStats] = None) -> List[Result]:
    """Runs all requests through ``engine`` (an Engine, or anything with a ``_h``
    handle of the C interface); returns their new tokens and why each ended."""
    n = len(requests)
    I32P = ctypes.POINTER(ctypes.c_int32)
    prompts = [lib.i32_array(int(t) for t in r.prompt) for r in requests]
    pp = (I32P * max(n, 1))(*[ctypes.cast(p, I32P) for p in prompts])
    lens = (ctypes.c_uint32 * max(n, 1))(*[len(r.prompt) for r in requests])
    news = (ctypes.c_uint32 * max(n, 1))(*[max(int(r.max_new), 0) for r in requests])
    opts = [options_c(r.options) for r in requests]
    op = (ctypes.POINTER(lib.GenOptionsC) * max(n, 1))(*[ctypes.pointer(o) for o in opts])
    total = sum(max(int(r.max_new), 0) for r in requests)
    out = (ctypes.c_int32 * max(total, 1))()
    n_out = (ctypes.c_uint32 * max(n, 1))()
    fin = (ctypes.c_int32 * max(n, 1))()
    st = stats_c()
    if max_batch is not None:
        # the handle's own max_batch is what the loop takes; a smaller one is asked for
        # by opening the engine with it
        pass
    lib.check(lib.lib().jb_llm_generate_batch(engine._h, n, pp, lens, news, op, out, n_out, fin,
                                              ctypes.byref(st)))
    if stats is not None:
        got = GenStats.from_c(st)
        for k, v in vars(got).items():
            setattr(stats, k, getattr(stats, k) + v)
    res, at = [], 0
    for i, r in enumerate(requests):
        res.append(Result(list(out[at:at + n_out[i]]), _FINISH.get(fin[i], "")))
        at += max(int(r.max_new), 0)
    return res
