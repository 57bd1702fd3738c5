"""The engine: a model, its cache, and the one step function.

``Engine.step`` runs a batch of sequences that either all start at their first
token (whole prompts of unequal lengths) or all go on by one token.  It runs
only the tokens it is given, as one batch of rows, against what earlier steps
left in the cache, and returns the logits at the wanted places.  There is no
padding: the rows are the sequences' tokens one after the other, and every
kernel finds a row's sequence and position in small index arrays.

The reference's batched pass has the same contract: pieces {sequence, tokens,
n, pos0} run as one block of rows, every weight read once, each piece attending
over its own sequence's cache, and "each piece's logits are those a pass over
its tokens alone gives" (src/llm/model.h:193-228, src/llm/model.c:878-912).
Arguments are checked before any state is touched (src/llm/model.c:651-655,
675-678).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..cache import Cache, CacheFull
from ..config import config_from_dir
from ..parts import DECODE, EXTEND, PREFILL, LayerCache, StepContext
from ..weights import load_tensors
from .model import DecoderModel

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16,
           "float32": torch.float32, "fp32": torch.float32}


def parse_dtype(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        if name not in (torch.float32, torch.bfloat16):
            raise ValueError("dtype: bfloat16 or float32")
        return name
    try:
        return _DTYPES[str(name)]
    except KeyError:
        raise ValueError(f"dtype {name!r}: bfloat16 or float32") from None


@dataclass
class StepEntry:
    """One sequence's share of a step: its next tokens and the places among
    them (indices into ``tokens``) whose logits are wanted."""

    slot: int
    tokens: Sequence[int]
    want: Sequence[int] = field(default_factory=list)


class StepError(ValueError):
    """A step that cannot run; nothing was changed."""


class Engine:
    def __init__(self, model: DecoderModel, max_tokens: int, max_seqs: Optional[int] = None):
        self.model = model
        self.device = model.device
        self.dtype = model.dtype
        if self.device.type != "cuda":
            raise RuntimeError("janas_b200 runs on a CUDA device only; there is no CPU path")
        if max_seqs is None:
            max_seqs = max(1, min(256, (max_tokens + 63) // 64))
        self.cache = Cache(model.kv_specs(), model.state_specs(), max_tokens, max_seqs,
                           self.dtype, self.device)
        self.max_positions = min(model.spec.max_positions, self.cache.max_tokens)
        model.prepare(self.max_positions)
        self.h2d_bytes = 0       # bytes of step inputs copied to the device so far
        # run-order entry -> (group, index within the group) of the cache it uses
        self._cache_entry: List[Optional[int]] = []
        for e, entry in enumerate(model.spec.run_order):
            src = entry.cache_of if entry.cache_of is not None else e
            self._cache_entry.append(src if src in self.cache.group_of else None)

    # ------------------------------------------------------------ open/close
    @classmethod
    def open(cls, model_dir: str, dtype="bfloat16", max_tokens: int = 4096,
             max_seqs: Optional[int] = None, device: str = "cuda:0") -> "Engine":
        """Reads config.json, picks the model through the registry and loads
        model.safetensors by tensor name."""
        dt = parse_dtype(dtype)
        if not torch.cuda.is_available():
            raise RuntimeError("janas_b200 needs a CUDA device; none is available")
        config = config_from_dir(model_dir)
        model = DecoderModel(config.to_model_spec(), dt, device)
        with torch.cuda.device(model.device):
            model.load(load_tensors(model_dir, model.tensors(), dt))
            eng = cls(model, max_tokens, max_seqs)
        eng.config = config
        return eng

    # ------------------------------------------------------------- sequences
    def new_sequence(self) -> int:
        return self.cache.new_sequence()

    def free_sequence(self, slot: int) -> None:
        self.cache.free_sequence(slot)

    def length(self, slot: int) -> int:
        return int(self.cache.length[slot])

    # ------------------------------------------------------------------ step
    def plan(self, entries: Sequence[StepEntry]):
        """Checks a step and lays out its rows; touches nothing."""
        if not entries:
            raise StepError("a step needs at least one sequence")
        vocab = self.model.spec.vocab_size
        seen = set()
        pos0, lens = [], []
        for ent in entries:
            if not self.cache.slots.live(ent.slot):
                raise StepError(f"slot {ent.slot} is not in use")
            if ent.slot in seen:
                raise StepError(f"slot {ent.slot} appears twice in one step")
            seen.add(ent.slot)
            n = len(ent.tokens)
            if n == 0:
                raise StepError(f"slot {ent.slot}: no tokens")
            p0 = int(self.cache.length[ent.slot])
            if p0 + n > self.max_positions:
                raise StepError(f"slot {ent.slot}: {p0} + {n} tokens exceed the "
                                f"{self.max_positions} positions of the context")
            for w in ent.want:
                if not 0 <= int(w) < n:
                    raise StepError(f"slot {ent.slot}: wanted place {w} is not among "
                                    f"its {n} tokens")
            pos0.append(p0)
            lens.append(n)
        tokens = np.concatenate([np.asarray(ent.tokens, dtype=np.int64) for ent in entries])
        if tokens.min() < 0 or tokens.max() >= vocab:
            raise StepError(f"a token id lies outside the vocabulary of {vocab}")
        pos0a, lena = np.asarray(pos0, dtype=np.int64), np.asarray(lens, dtype=np.int64)
        if (pos0a == 0).all():
            kind = PREFILL
        elif (lena == 1).all():
            kind = DECODE
        else:
            kind = EXTEND
        if not self.model.supports(kind):
            raise StepError("this model cannot append several tokens at once to sequences "
                            "that already hold some (a mixer does not support it)")
        return kind, tokens.astype(np.int32), pos0a, lena

    def step(self, entries: Sequence[StepEntry]) -> Optional[torch.Tensor]:
        """Runs the entries' tokens as one batch.  Returns the float32 logits
        [wanted, vocab] at the wanted places, in the order of the entries and of
        each entry's ``want`` (None when nothing is wanted)."""
        kind, tokens, pos0, lens = self.plan(entries)
        slots = [ent.slot for ent in entries]
        self.cache.reserve(slots, lens.tolist())     # CacheFull leaves everything as it was

        n = int(lens.sum())
        B = len(entries)
        row0 = np.zeros(B + 1, dtype=np.int64)
        np.cumsum(lens, out=row0[1:])
        row_seq = np.repeat(np.arange(B, dtype=np.int32), lens)
        row_pos = (np.arange(n, dtype=np.int64) - np.repeat(row0[:-1], lens)
                   + np.repeat(pos0, lens)).astype(np.int32)
        want = np.asarray([row0[i] + int(w) for i, ent in enumerate(entries) for w in ent.want],
                          dtype=np.int32)
        all_rows = want.size == n and bool((want == np.arange(n)).all())

        # one host buffer, one copy: tokens | row_pos | row_seq | slots | want | block tables
        tables = [self.cache.block_table(g, slots) for g in self.cache.groups]
        parts = [tokens, row_pos, row_seq, np.asarray(slots, dtype=np.int32), want] \
            + [t.reshape(-1) for t in tables]
        sizes = [p.size for p in parts]
        host = torch.from_numpy(np.concatenate(parts)).pin_memory()
        self.h2d_bytes += host.numel() * host.element_size()
        with torch.cuda.device(self.device):
            dev = host.to(self.device, non_blocking=True)
            offs = np.concatenate([[0], np.cumsum(sizes)])
            view = lambda i: dev[int(offs[i]):int(offs[i + 1])]
            bt_dev = {id(g): view(5 + i).view(tables[i].shape)
                      for i, g in enumerate(self.cache.groups)}
            ctx = StepContext(kind=kind, dtype=self.dtype, device=self.device, n_rows=n,
                              n_seqs=B, row_pos=view(1), row_seq=view(2), seq_slot_dev=view(3),
                              seq_slots=slots, seq_pos0=pos0, seq_len=lens, seq_row0=row0,
                              max_pos=int((pos0 + lens).max()) - 1)
            caches = self._layer_caches(bt_dev)
            want_dev = None if all_rows else view(4)
            logits = self.model.forward(ctx, view(0), caches, want_dev)
        self.cache.advance(slots, lens.tolist())
        return logits

    def _layer_caches(self, bt_dev: Dict[int, torch.Tensor]) -> List[LayerCache]:
        out = []
        for e, entry in enumerate(self.model.spec.run_order):
            src = self._cache_entry[e]
            lc = LayerCache(writes=entry.cache_of is None,
                            state=self.cache.mixer_state.get(e))
            if src is not None:
                g = self.cache.group_of[src]
                i = g.index[src]
                lc.k, lc.v, lc.block_table = g.k[i], g.v[i], bt_dev[id(g)]
            out.append(lc)
        return out
