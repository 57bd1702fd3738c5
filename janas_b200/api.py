"""The Python entry point, in the manner of the reference's C interface.

    llm = janas_b200.open(model_dir, params)           # janas_llm_open
    tokens, stats = llm.generate(prompt, max_new, options)   # janas_llm_generate
    s = llm.session(options); s.append(prompt); status, token = s.next()   # janas_llm_session_*
    llm.close()                                        # janas_llm_close

Names follow include/janas/llm.h and src/llm/generate.h: ``params_default``
(janas_llm_params_default, include/janas/llm.h:159), ``n_ctx``
(struct janas_llm_params, :76-78), the error codes (:43-53), ``GenOptions`` and
``GenStats`` (struct janas_gen_options / janas_gen_stats,
src/llm/generate.h:31-86).  Tokens go in and come out as lists of ids on the
host; there is no tokenizer here.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple, Union

ABI_VERSION = 1

OK = 0
EINVAL = -1   # invalid argument
ENOMEM = -2   # out of memory
EOPEN = -3    # model folder missing, unreadable, invalid
EMODEL = -4   # model not supported (architecture)
EFULL = -5    # the context or the cache is full
EFAIL = -8    # internal failure


class LLMError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(message)
        self.code = code


@dataclass
class LLMParams:
    n_ctx: int = 16384          # context of one sequence, in tokens (the reference's default)
    dtype: str = "bfloat16"     # or "float32": the whole model in true 32-bit
    max_batch: int = 64         # most sequences that run together
    max_tokens: int = 0         # tokens the cache holds in all; 0: n_ctx
    device: str = "cuda:0"


def params_default() -> LLMParams:
    return LLMParams()


def abi_version() -> int:
    return ABI_VERSION


class LLM:
    """An open model.  One thread drives it (include/janas/llm.h:22)."""

    def __init__(self, engine, params: LLMParams):
        self.engine = engine
        self.params = params

    @property
    def n_ctx(self) -> int:
        return self.engine.max_positions

    @property
    def n_vocab(self) -> int:
        return self.engine.model.spec.vocab_size

    def generate(self, prompt: Sequence[int], max_new: int, options=None
                 ) -> Tuple[List[int], "GenStats"]:
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
                                         for p, m, o in zip(prompts, news, opts)],
                           max_batch=self.params.max_batch, stats=stats)
        except ValueError as e:
            raise LLMError(EINVAL, str(e)) from None
        self.last_finish = [r.finish for r in res]
        return [r.tokens for r in res], stats

    # ------------------------------------------------------------- sessions
    def session(self, options=None) -> "Session":
        """A sequence of its own on this model, which grows by appended tokens and
        by tokens generated on request (janas_llm_session_create,
        src/llm/generate.h:101-103); see ``janas_b200.engine.session``.  As many
        sessions as ``max_batch`` can be open at one time; ``close`` gives a
        session's place and cache pages back."""
        from .cache import CacheFull
        from .engine.session import Session, SessionError
        try:
            return Session(self.engine, options)
        except (SessionError, ValueError) as e:
            raise LLMError(EINVAL, str(e)) from None
        except (CacheFull, RuntimeError) as e:
            raise LLMError(EFULL, str(e)) from None

    def sessions_step(self, sessions):
        """Moves several sessions on together in one pass
        (janas_llm_sessions_step, src/llm/generate.h:155-158): returns
        (tokens, status), status 0 with a token, 1 when that session's context is
        full."""
        from .cache import CacheFull
        from .engine.session import SessionError, sessions_step
        try:
            return sessions_step(self.engine, list(sessions))
        except SessionError as e:
            raise LLMError(EINVAL, str(e)) from None
        except CacheFull as e:
            raise LLMError(EFULL, str(e)) from None

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
        from .engine import StepEntry, StepError
        from .cache import CacheFull
        try:
            return self.engine.step([e if isinstance(e, StepEntry) else StepEntry(*e)
                                     for e in entries])
        except StepError as e:
            raise LLMError(EINVAL, str(e)) from None
        except CacheFull as e:
            raise LLMError(EFULL, str(e)) from None

    def close(self) -> None:
        self.engine = None


def open(path: str, params: Optional[LLMParams] = None) -> LLM:
    """Opens a model folder (config.json, model.safetensors)."""
    import torch
    from .cache import CacheFull
    from .config import ConfigError
    from .engine import Engine
    from .weights import SafetensorsError, WeightError
    p = params or params_default()
    try:
        eng = Engine.open(path, dtype=p.dtype, max_tokens=p.max_tokens or p.n_ctx,
                          max_seqs=p.max_batch, device=p.device)
    except ConfigError as e:
        code = EMODEL if "not supported" in str(e) else EOPEN
        raise LLMError(code, str(e)) from None
    except (SafetensorsError, WeightError, OSError) as e:
        raise LLMError(EOPEN, str(e)) from None
    except torch.cuda.OutOfMemoryError as e:
        raise LLMError(ENOMEM, str(e)) from None
    except RuntimeError as e:
        # no CUDA device, or the kernel library cannot be built or loaded: there is
        # no other path to fall back to
        raise LLMError(EFAIL, str(e)) from None
    eng.max_positions = min(eng.max_positions, p.n_ctx)
    return LLM(eng, p)
