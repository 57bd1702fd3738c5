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

import os

import numpy as np
import torch

from ..cache import Cache
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
        self.use_graphs = os.environ.get("JANAS_B200_GRAPHS", "1") != "0" and all(
            getattr(b.mixer, "graph_safe", False) for b in model.blocks)
        # captured decode steps by (batch, context bound, sampled, long way), the one
        # used last at the end; the oldest goes when there are more than max_graphs
        self._graphs: Dict[Tuple[int, int, bool, bool], "DecodeGraph"] = {}
        self.max_graphs = 64
        self._graph_pool = None
        self._capture_stream = None
        self._sampler_scratch = None
        self._last_decode = None     # (graph, slots) of the decode step begun last
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
        if self._last_decode is not None and slot in self._last_decode[1]:
            self._last_decode = None    # no step can go on from that step's tokens any more

    def length(self, slot: int) -> int:
        return int(self.cache.length[slot])

    def truncate_sequence(self, slot: int, n: int) -> bool:
        """Keeps the first ``n`` computed tokens of a sequence; False where the
        cache cannot go back there (see ``Cache.truncate``)."""
        if not self.cache.truncate(slot, n):
            return False
        if self._last_decode is not None and slot in self._last_decode[1]:
            self._last_decode = None
        return True

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

    # ---------------------------------------------------------------- decode
    def decode(self, slots: Sequence[int], tokens: Sequence[int], sampled: bool = False,
               big=None) -> np.ndarray:
        """One decode step for sequences that each go on by one token, with the
        choice of the next token on the device; returns the chosen tokens on the
        host.  The step's kernels are the step function's; when every mixer allows
        it they are replayed from a CUDA graph captured for this batch size and
        context bound, else they are launched one by one."""
        return self.decode_end(self.decode_begin(slots, tokens, sampled, big))

    @property
    def decodes_ahead(self) -> bool:
        """Whether ``decode_begin`` takes ``tokens=None``: the step is then fed the
        tokens that the step before it chose, which never leave the device, so it
        can be launched while that step still runs."""
        return self.use_graphs

    def decode_begin(self, slots: Sequence[int], tokens: Optional[Sequence[int]],
                     sampled: bool = False, big=None) -> "PendingDecode":
        """Launches a decode step and returns at once; ``decode_end`` waits for it
        and gives the chosen tokens.  With ``tokens=None`` the sequences go on from
        the tokens chosen by the step begun last, which must have had the same
        slots in the same order.  Steps end in the order in which they began, and
        at most two may be under way."""
        slots = list(slots)
        if tokens is None:
            if not self.use_graphs or self._last_decode is None or self._last_decode[1] != slots:
                raise StepError("a step can go on from the device's own tokens only right "
                                "after a decode step of the same sequences")
            feed = [0] * len(slots)
        else:
            feed = [int(t) for t in tokens]
        entries = [StepEntry(s, [t], [0]) for s, t in zip(slots, feed)]
        if not self.use_graphs:
            logits = self.step(entries)
            return PendingDecode(None, 0, self._sample(logits, slots, sampled, big))
        kind, toks, pos0, lens = self.plan(entries)
        self.cache.reserve(slots, lens.tolist())
        # launch sizes are fixed for positions below ``bound``: a new graph every
        # 256 positions keeps them close to what the step needs
        need = int(pos0.max()) + 1
        bound = min((need + 255) // 256 * 256, self.max_positions)
        # ``big``: some row may keep more candidates than the sampler's short way
        # holds; the graph then sorts all of a row's logits in the engine's scratch
        key = (len(slots), bound, bool(sampled), big is not None and bool(sampled))
        g = self._graphs.pop(key, None)
        if g is None:
            g = DecodeGraph(self, len(slots), bound, bool(sampled), key[3])
            while len(self._graphs) >= max(self.max_graphs, 1):
                # a step of the graph that goes may still be under way
                torch.cuda.current_stream(self.device).synchronize()
                del self._graphs[next(iter(self._graphs))]
            if not self._graphs:
                self._graph_pool = None     # a pool ends with its last graph: take a new one
        self._graphs[key] = g
        before = self._last_decode[0] if tokens is None else None
        pending = g.begin(slots, None if tokens is None else toks, pos0, before)
        self._last_decode = (g, slots)
        self.cache.advance(slots, lens.tolist())
        return pending

    def decode_end(self, pending: "PendingDecode") -> np.ndarray:
        """Waits for a step begun with ``decode_begin``; its chosen tokens."""
        return pending.result()

    def sampler_scratch(self, rows: int):
        """Room for every logit of ``rows`` rows as a sort key and as a probability:
        what the sampler needs for rows that keep more candidates than its short way
        holds (top-k off or large).  One allocation for the engine's life."""
        if self._sampler_scratch is None:
            vocab = self.model.spec.vocab_size
            cap = 1 << (vocab - 1).bit_length()
            n = self.cache.max_seqs
            self._sampler_scratch = (
                torch.empty((n, cap), dtype=torch.int64, device=self.device),
                torch.empty((n, cap), dtype=torch.float32, device=self.device))
        k, p = self._sampler_scratch
        return k[:rows], p[:rows]

    def _sample(self, logits: torch.Tensor, slots: List[int], sampled: bool, big) -> np.ndarray:
        from ..csrc import ops
        if not sampled:
            return ops.sample(logits).cpu().numpy()
        c = self.cache
        row_slot = torch.tensor(slots, dtype=torch.int32).to(self.device, non_blocking=True)
        toks = ops.sample(logits, row_slot=row_slot, temperature=c.temperature, top_k=c.top_k,
                          top_p=c.top_p, min_p=c.min_p, rng=c.rng,
                          big_keys=None if big is None else big[0],
                          big_probs=None if big is None else big[1])
        return toks.cpu().numpy()


class PendingDecode:
    """A decode step under way: ``result()`` waits for it and gives its tokens."""

    def __init__(self, event, n: int, tokens=None):
        self.event, self.n, self.tokens = event, n, tokens
        self.out_host = None

    def result(self) -> np.ndarray:
        if self.tokens is None:
            self.event.synchronize()
            self.tokens = self.out_host.numpy()[:self.n].copy()
        return self.tokens


class DecodeGraph:
    """The decode step of ``batch`` sequences at positions below ``bound``,
    captured once and replayed.

    All that changes from step to step (tokens, positions, slots, block tables)
    lies in a pinned host buffer that is copied to the device before the graph
    runs; the chosen tokens are written where the next step's tokens are read, so
    a step that goes on from them needs nothing from the host but positions and
    block tables, and can be launched while the step before it runs.  There are
    two pinned buffers each way, used in turn: with at most two steps under way,
    the host never writes what a copy still reads, nor reads what a later step
    may already have written.  Launch sizes that depend on the context (the
    attention's chunk count) are fixed at ``bound``; rows whose range is shorter
    leave those chunks at once."""

    def __init__(self, engine: "Engine", batch: int, bound: int, sampled: bool,
                 long_way: bool = False):
        from ..cache.pages import pages_for
        self.engine, self.batch, self.bound, self.sampled = engine, batch, bound, sampled
        self.long_way = long_way
        self.width = (pages_for(bound) + 7) // 8 * 8
        n_groups = len(engine.cache.groups)
        total = 4 * batch + n_groups * batch * self.width
        self.host = [torch.zeros(total, dtype=torch.int32).pin_memory() for _ in range(2)]
        self.out_host = [torch.zeros(batch, dtype=torch.int32).pin_memory() for _ in range(2)]
        self.events = [torch.cuda.Event() for _ in range(2)]
        self.pending: List[Optional[PendingDecode]] = [None, None]
        self.turn = 0
        self.dev = torch.zeros(total, dtype=torch.int32, device=engine.device)
        self.graph: Optional[torch.cuda.CUDAGraph] = None

    def _launch(self) -> None:
        from ..csrc import ops
        eng, B = self.engine, self.batch
        v = lambda i: self.dev[i * B:(i + 1) * B]
        bt = {}
        for gi, g in enumerate(eng.cache.groups):
            a = 4 * B + gi * B * self.width
            bt[id(g)] = self.dev[a:a + B * self.width].view(B, self.width)
        ctx = StepContext(kind=DECODE, dtype=eng.dtype, device=eng.device, n_rows=B, n_seqs=B,
                          row_pos=v(1), row_seq=v(2), seq_slot_dev=v(3), seq_slots=[],
                          seq_pos0=None, seq_len=None, seq_row0=None, max_pos=self.bound - 1)
        logits = eng.model.forward(ctx, v(0), eng._layer_caches(bt), None)
        c = eng.cache
        # the chosen tokens take the place of the tokens the step was fed
        if self.sampled:
            big = eng.sampler_scratch(B) if self.long_way else (None, None)
            ops.sample(logits, out=v(0), row_slot=v(3), temperature=c.temperature,
                       top_k=c.top_k, top_p=c.top_p, min_p=c.min_p, rng=c.rng,
                       big_keys=big[0], big_probs=big[1])
        else:
            ops.sample(logits, out=v(0))

    def begin(self, slots: List[int], tokens: Optional[np.ndarray], pos0: np.ndarray,
              before: Optional["DecodeGraph"]) -> PendingDecode:
        """Copies the step's inputs, runs the step and copies its tokens back,
        all on the current stream, without waiting.  ``tokens`` None: the step is
        fed what the step begun last chose (``before`` is its graph)."""
        eng, B = self.engine, self.batch
        turn = self.turn
        self.turn = 1 - turn
        # the buffers of this turn were last used two steps ago: that step has to be
        # over, and its tokens taken, before they are written again
        if self.pending[turn] is not None:
            self.pending[turn].result()
        host = self.host[turn]
        h = host.numpy()
        if tokens is not None:
            h[0:B] = tokens
        h[B:2 * B] = pos0
        h[2 * B:3 * B] = np.arange(B, dtype=np.int32)
        h[3 * B:4 * B] = slots
        for gi, g in enumerate(eng.cache.groups):
            a = 4 * B + gi * B * self.width
            tab = h[a:a + B * self.width].reshape(B, self.width)
            tab.fill(-1)
            for i, s in enumerate(slots):
                pg = g.pages[s]
                tab[i, :len(pg)] = pg
        from ..csrc import ops
        with torch.cuda.device(eng.device):
            if tokens is not None:
                self.dev.copy_(host, non_blocking=True)
                eng.h2d_bytes += host.numel() * 4
            else:
                if before is not self:
                    self.dev[:B].copy_(before.dev[:B], non_blocking=True)
                self.dev[B:].copy_(host[B:], non_blocking=True)
                eng.h2d_bytes += (host.numel() - B) * 4
            if self.graph is None:
                # the first step runs eagerly (it sizes every scratch buffer and is a
                # real step); the capture that follows records without running
                self._launch()
                self.out_host[turn].copy_(self.dev[:B], non_blocking=True)
                self.events[turn].record()
                torch.cuda.current_stream().synchronize()
                graph = torch.cuda.CUDAGraph()
                if eng._graph_pool is None:
                    eng._graph_pool = torch.cuda.graph_pool_handle()
                if eng._capture_stream is None:
                    eng._capture_stream = torch.cuda.Stream(eng.device)
                before_n = ops.COUNTERS["launches"]
                # capture_begin/capture_end on a stream of the engine's own, not the
                # torch.cuda.graph context: that one collects garbage and empties the
                # allocator's cache first, which gives the last prefill's blocks back
                # to the driver (0.3 s and more after a long prompt, and the next
                # prefill pays for getting them again).  The capture records the
                # kernels without running them, so the tokens just chosen stay.
                side = eng._capture_stream
                side.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(side):
                    graph.capture_begin(pool=eng._graph_pool)
                    try:
                        self._launch()
                    finally:
                        graph.capture_end()
                torch.cuda.current_stream().wait_stream(side)
                self.kernels = ops.COUNTERS["launches"] - before_n   # kernels per replay
                ops.COUNTERS["launches"] = before_n
                self.graph = graph
            else:
                self.graph.replay()
                ops.COUNTERS["launches"] += self.kernels
                self.out_host[turn].copy_(self.dev[:B], non_blocking=True)
                self.events[turn].record()
        pending = PendingDecode(self.events[turn], B)
        pending.out_host = self.out_host[turn]
        self.pending[turn] = pending
        return pending
