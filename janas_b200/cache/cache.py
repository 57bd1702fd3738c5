"""The cache: paged keys and values per layer group, and per-sequence state.

A sequence lives in a *slot*.  The slot records how many tokens of the sequence
have been computed and owns, in every layer group, the pages that hold its keys
and values.  A page is ``PAGE`` positions of all KV heads of one layer; a group
is the set of run-order entries whose mixers need the same kind of storage (the
same number of KV heads and head size, and either all positions or a window of
them).  Every group has a pool and tensors of its own:

    K, V: [entries of the group, pages, kv_heads, PAGE, head_dim]

A group with a window gives pages back as soon as no later token can see them,
so a long sequence holds only about window / PAGE + 1 pages there.

Beside the pages, every slot has state of fixed size: the sampler's settings and
random state, and whatever fixed-size tensors the model's mixers ask for
(``state_spec``); these are zeroed when a slot is taken.  Qwen3 asks for none.

The reference keeps the same things per sequence in ``struct janas_seq``
(src/llm/model_impl.h:128-171: keys, values, recurrent state), describes layer
groups by per-group geometry arrays (src/llm/model_impl.h:262-274, filled in
src/llm/model_load.c:1113-1146) and reuses a server slot for the next request
(src/server/engine.c:826-838,885-891).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from .pages import PAGE, CacheFull, PagePool, SlotPool, pages_for


@dataclass(frozen=True)
class KVSpec:
    """What a mixer needs stored per position.  ``window`` 0: every position
    stays; otherwise only the last ``window`` positions can be read again."""

    num_kv_heads: int
    head_dim: int
    window: int = 0


@dataclass(frozen=True)
class StateSpec:
    """Fixed-size state a mixer keeps per sequence: a tensor of this shape,
    zero at the sequence's start."""

    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


class KVGroup:
    """The storage of one layer group."""

    def __init__(self, spec: KVSpec, entries: Sequence[int], n_pages: int, n_slots: int,
                 dtype: torch.dtype, device: torch.device):
        self.spec = spec
        self.entries = list(entries)                      # run-order entries stored here
        self.index = {e: i for i, e in enumerate(self.entries)}
        self.pool = PagePool(n_pages, f"cache group {spec}")
        shape = (len(self.entries), n_pages, spec.num_kv_heads, PAGE, spec.head_dim)
        self.k = torch.zeros(shape, dtype=dtype, device=device)
        self.v = torch.zeros(shape, dtype=dtype, device=device)
        # per slot: page of every page index (absolute position // PAGE), -1 once released
        self.pages: List[List[int]] = [[] for _ in range(n_slots)]

    def bytes(self) -> int:
        return 2 * self.k.numel() * self.k.element_size()

    def first_needed_page(self, next_pos: int) -> int:
        """The lowest page index that a token at ``next_pos`` or later can see."""
        if not self.spec.window:
            return 0
        return max(0, next_pos + 1 - self.spec.window) // PAGE

    def extend(self, slot: int, end: int) -> None:
        """Makes room for positions below ``end``."""
        have = self.pages[slot]
        want = pages_for(end)
        if want > len(have):
            have.extend(self.pool.take(want - len(have)))

    def release_unseen(self, slot: int, next_pos: int) -> None:
        have = self.pages[slot]
        first = min(self.first_needed_page(next_pos), len(have))
        gone = [have[i] for i in range(first) if have[i] >= 0]
        if gone:
            self.pool.give_back(gone)
            for i in range(first):
                have[i] = -1

    def free(self, slot: int) -> None:
        self.pool.give_back([p for p in self.pages[slot] if p >= 0])
        self.pages[slot] = []

    def held(self, slot: int) -> int:
        return sum(1 for p in self.pages[slot] if p >= 0)


class Cache:
    """Slots, page groups and per-sequence state for one model on one device.

    ``kv_specs[e]`` / ``state_specs[e]`` are what run-order entry ``e`` needs
    (None for nothing; entries that read another entry's cache have None).
    ``max_tokens`` is the most tokens that live sequences may hold at one time,
    each sequence's count rounded up to a multiple of PAGE; ``max_seqs`` the
    most sequences alive at one time."""

    def __init__(self, kv_specs: Sequence[Optional[KVSpec]],
                 state_specs: Sequence[Optional[StateSpec]], max_tokens: int, max_seqs: int,
                 dtype: torch.dtype, device: torch.device | str):
        if max_tokens <= 0 or max_seqs <= 0:
            raise ValueError("max_tokens and max_seqs must be positive")
        self.device = torch.device(device)
        self.dtype = dtype
        self.max_tokens = pages_for(max_tokens) * PAGE
        self.max_seqs = max_seqs
        n_pages = pages_for(max_tokens)
        self.slots = SlotPool(max_seqs)
        self.length = np.zeros(max_seqs, dtype=np.int64)   # tokens computed, per slot

        by_spec: Dict[KVSpec, List[int]] = {}
        for e, spec in enumerate(kv_specs):
            if spec is not None:
                by_spec.setdefault(spec, []).append(e)
        self.groups: List[KVGroup] = [KVGroup(spec, entries, n_pages, max_seqs, dtype,
                                              self.device)
                                      for spec, entries in by_spec.items()]
        self.group_of: Dict[int, KVGroup] = {e: g for g in self.groups for e in g.entries}

        # fixed-size state per slot
        self.rng = torch.zeros(max_seqs, dtype=torch.int64, device=self.device)
        self.temperature = torch.zeros(max_seqs, dtype=torch.float32, device=self.device)
        self.top_k = torch.zeros(max_seqs, dtype=torch.int32, device=self.device)
        self.top_p = torch.zeros(max_seqs, dtype=torch.float32, device=self.device)
        self.min_p = torch.zeros(max_seqs, dtype=torch.float32, device=self.device)
        self.mixer_state: Dict[int, torch.Tensor] = {
            e: torch.zeros((max_seqs,) + tuple(spec.shape), dtype=spec.dtype, device=self.device)
            for e, spec in enumerate(state_specs) if spec is not None}

    # ------------------------------------------------------------ sequences
    def new_sequence(self) -> int:
        slot = self.slots.take()
        self.length[slot] = 0
        for st in self.mixer_state.values():
            st[slot].zero_()
        return slot

    def free_sequence(self, slot: int) -> None:
        if not self.slots.live(slot):
            raise RuntimeError(f"slot {slot} freed but not in use")
        for g in self.groups:
            g.free(slot)
        self.slots.give_back(slot)
        self.length[slot] = 0

    def can_truncate(self, slot: int, n: int) -> bool:
        """Whether the sequence can go back to its first ``n`` tokens: always to
        none; else only if no mixer keeps a state of its own (which has seen
        everything) and every window group still holds the pages that a token at
        position ``n`` can see."""
        if not self.slots.live(slot) or not 0 <= n <= int(self.length[slot]):
            return False
        if n == 0 or n == int(self.length[slot]):
            return True
        if self.mixer_state:
            return False
        for g in self.groups:
            have = g.pages[slot]
            if any(have[i] < 0 for i in range(g.first_needed_page(n), pages_for(n))):
                return False
        return True

    def truncate(self, slot: int, n: int) -> bool:
        """Keeps the first ``n`` tokens of the sequence and gives back the pages
        beyond them (src/llm/generate.h:160-167: janas_llm_session_truncate).
        False, with nothing changed, where ``can_truncate`` says no."""
        if not self.can_truncate(slot, n):
            return False
        if n == int(self.length[slot]):
            return True
        for g in self.groups:
            have = g.pages[slot]
            keep = pages_for(n)
            gone = [p for p in have[keep:] if p >= 0]
            if gone:
                g.pool.give_back(gone)
            del have[keep:]
        self.length[slot] = n
        if n == 0:
            for st in self.mixer_state.values():
                st[slot].zero_()
        return True

    def set_samplers(self, slots: Sequence[int], options: Sequence) -> None:
        """The sequences' sampling settings (objects with temperature, top_k,
        top_p, min_p and seed); each random sequence starts at its seed
        (src/llm/sample.c:118)."""
        def signed(seed: int) -> int:
            seed &= (1 << 64) - 1
            return seed - (1 << 64) if seed >= (1 << 63) else seed

        idx = torch.tensor(list(slots), dtype=torch.int64, device=self.device)
        put = lambda dst, vals, dt: dst.index_copy_(
            0, idx, torch.tensor(vals, dtype=dt).to(self.device))
        put(self.rng, [signed(int(o.seed)) for o in options], torch.int64)
        put(self.temperature, [float(o.temperature) for o in options], torch.float32)
        put(self.top_k, [int(o.top_k) for o in options], torch.int32)
        put(self.top_p, [float(o.top_p) for o in options], torch.float32)
        put(self.min_p, [float(o.min_p) for o in options], torch.float32)

    # ---------------------------------------------------------------- steps
    def reserve(self, slots: Sequence[int], counts: Sequence[int]) -> None:
        """Makes room for ``counts[i]`` more tokens of ``slots[i]``, for all of
        them or, when the pages do not suffice, for none."""
        taken: List[Tuple[KVGroup, int, int]] = []
        try:
            for slot, n in zip(slots, counts):
                if not self.slots.live(slot):
                    raise RuntimeError(f"slot {slot} is not in use")
                end = int(self.length[slot]) + int(n)
                for g in self.groups:
                    before = len(g.pages[slot])
                    taken.append((g, slot, before))
                    g.extend(slot, end)
        except CacheFull:
            for g, slot, before in taken:
                extra = g.pages[slot][before:]
                if extra:
                    g.pool.give_back(extra)
                    del g.pages[slot][before:]
            raise

    def advance(self, slots: Sequence[int], counts: Sequence[int]) -> None:
        """The step has run: the sequences are longer, and window groups give
        back the pages that no later token can see."""
        for slot, n in zip(slots, counts):
            self.length[slot] += int(n)
            nxt = int(self.length[slot])
            for g in self.groups:
                if g.spec.window:
                    g.release_unseen(slot, nxt)

    def block_table(self, group: KVGroup, slots: Sequence[int]) -> np.ndarray:
        """int32 [len(slots), P]: the page of every page index of each slot
        (-1 where there is none), P a multiple of 8."""
        width = max([len(group.pages[s]) for s in slots] + [1])
        width = (width + 7) // 8 * 8
        bt = np.full((len(slots), width), -1, dtype=np.int32)
        for i, s in enumerate(slots):
            pg = group.pages[s]
            bt[i, :len(pg)] = pg
        return bt

    # ---------------------------------------------------------------- checks
    def tokens_held(self) -> int:
        """Tokens' worth of pages in use in the fullest group."""
        return max([(g.pool.n_pages - g.pool.n_free) * PAGE for g in self.groups] + [0])

    def bytes(self) -> int:
        return sum(g.bytes() for g in self.groups)

    def check(self) -> None:
        """Bookkeeping invariants: no page or slot lost, held twice or free
        twice; pages held only by live slots."""
        self.slots.check()
        for g in self.groups:
            g.pool.check()
            seen = set()
            for slot, pages in enumerate(g.pages):
                if pages and not self.slots.live(slot):
                    raise RuntimeError(f"free slot {slot} still holds pages")
                for p in pages:
                    if p < 0:
                        continue
                    if p in seen:
                        raise RuntimeError(f"page {p} is held twice")
                    seen.add(p)
            if len(seen) != g.pool.n_pages - g.pool.n_free:
                raise RuntimeError("pages held by nobody")
