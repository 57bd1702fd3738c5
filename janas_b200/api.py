"""The Python entry point: a thin ctypes layer over the library's C interface
(``include/janas_b200/llm.h``), which follows the reference's
(include/janas/llm.h, src/llm/generate.h).

    llm = janas_b200.open(model_dir, params)                  # jb_llm_open
    tokens, stats = llm.generate(prompt, max_new, options)    # jb_llm_generate
    s = llm.session(options); s.append(prompt); status, token = s.next()   # jb_llm_session_*
    llm.close()                                               # jb_llm_close

``params_default`` is jb_llm_params_default (janas_llm_params_default,
include/janas/llm.h:159), ``n_ctx`` the context of one sequence (struct
janas_llm_params, :76-78), the error codes are the reference's (:43-53),
``GenOptions`` and ``GenStats`` its struct janas_gen_options / janas_gen_stats
(src/llm/generate.h:31-86).  Tokens go in and come out as lists of ids on the
host; there is no tokenizer here.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple, Union

from . import lib
from .lib import (ABI_VERSION, EFAIL, EFULL, EINVAL, ELIMIT, EMODEL, ENOMEM, EOPEN, OK, CacheFull,
                  LLMError)


@dataclass
class LLMParams:
    n_ctx: int = 16384          # context of one sequence, in tokens (the reference's default)
    dtype: str = "bfloat16"     # or "float32": the whole model in true 32-bit
    max_batch: int = 64         # most sequences that run together
    max_tokens: int = 0         # tokens the cache holds in all; 0: n_ctx
    device: str = "cuda:0"


def params_default() -> LLMParams:
    import ctypes
    p = lib.Params()
    lib.lib().jb_llm_params_default(ctypes.byref(p))
    return LLMParams(n_ctx=p.n_ctx, dtype="float32" if p.dtype == lib.F32 else "bfloat16",
                     max_batch=p.max_batch, max_tokens=p.max_tokens, device=f"cuda:{p.device}")


def abi_version() -> int:
    return int(lib.lib().jb_llm_abi_version())


class LLM:
    """An open model.  One thread drives it (include/janas/llm.h:22)."""

    def __init__(self, engine, params: LLMParams):
        self.engine = engine
        self.params = params
        self.last_finish: List[str] = []

    @property
    def n_ctx(self) -> int:
        return self.engine.max_positions

    @property
    def n_vocab(self) -> int:
        return self.engine.vocab_size

    def generate(self, prompt: Sequence[int], max_new: int, options=None):
        """Runs the prompt, then generates up to ``max_new`` tokens, stopping
        after a stop token.  Returns the new tokens and the counters."""
        outs, stats = self.generate_batch([prompt], max_new, options)
        return outs[0], stats

    def generate_batch(self, prompts: Sequence[Sequence[int]],
                       max_new: Union[int, Sequence[int]], options=None):
        """Several prompts of unequal lengths; ``max_new`` and ``options`` are
        one for all or one per prompt.  As many batches run one after another
        as the requests need.  Returns (list of new-token lists, GenStats);
        ``last_finish`` then holds why each ended."""
        from .engine.generate import GenOptions, GenStats, Request, generate
        n = len(prompts)
        news = [max_new] * n if isinstance(max_new, int) else list(max_new)
        if options is None:
            opts = [GenOptions() for _ in range(n)]
        elif isinstance(options, GenOptions):
            opts = [options] * n
        else:
            opts = list(options)
        if len(news) != n or len(opts) != n:
            raise LLMError(EINVAL, "max_new and options: one for all or one per prompt")
        stats = GenStats()
        try:
            res = generate(self.engine, [Request(list(p), m, o)
                                         for p, m, o in zip(prompts, news, opts)], stats=stats)
        except ValueError as e:
            if isinstance(e, LLMError):
                raise
            raise LLMError(EINVAL, str(e)) from None
        self.last_finish = [r.finish for r in res]
        return [r.tokens for r in res], stats

    # ------------------------------------------------------------- sessions
    def session(self, options=None):
        """A sequence of its own on this model, which grows by appended tokens and
        by tokens generated on request (jb_llm_session_create); see
        ``janas_b200.engine.session``.  As many sessions as ``max_batch`` can be
        open at one time; ``close`` gives a session's place and cache pages back."""
        from .engine.session import Session
        try:
            return Session(self.engine, options)
        except ValueError as e:
            if isinstance(e, LLMError):
                raise
            raise LLMError(EINVAL, str(e)) from None

    def sessions_step(self, sessions):
        """Moves several sessions on together in one pass (jb_llm_sessions_step):
        returns (tokens, status), status 0 with a token, 1 when that session's
        context is full."""
        from .engine.session import sessions_step
        return sessions_step(self.engine, list(sessions))

    # ------------------------------------------------- the step function itself
    def slot_new(self) -> int:
        """A place for a sequence in the cache, for callers that drive ``step``
        themselves."""
        return self.engine.new_sequence()

    def slot_free(self, slot: int) -> None:
        self.engine.free_sequence(slot)

    def step(self, entries):
        """One step of the engine: ``entries`` are (slot, tokens, wanted places);
        returns the float32 logits [wanted, vocab] on the device, or None."""
        return self.engine.step(entries)

    def close(self) -> None:
        if self.engine is not None:
            self.engine.close()
        self.engine = None


def open(path: str, params: Optional[LLMParams] = None) -> LLM:
    """Opens a model folder (config.json, model.safetensors)."""
    from .engine import Engine
    p = params or params_default()
    eng = Engine.open(path, dtype=p.dtype, max_tokens=p.max_tokens or p.n_ctx, max_seqs=p.max_batch,
                      device=p.device, n_ctx=p.n_ctx)
    return LLM(eng, p)
