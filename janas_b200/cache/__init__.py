"""The cache: slots, paged keys and values per layer group, per-sequence state.

The cache is the library's (``cache/cache.cpp``); the classes here are views of
one, either made on its own (``Cache(...)``: for tests of the bookkeeping, with or
without device storage) or the one an open engine holds (``Engine.cache``).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np

from .. import lib
from ..lib import CacheFull
from ..devmem import as_tensor, dtype_name

PAGE = 64  # positions per page; the library and its kernels use the same number


def pages_for(n_tokens: int) -> int:
    return (n_tokens + PAGE - 1) // PAGE


def _call(method: str, **args):
    """A misuse of the bookkeeping (a page or slot freed twice) is a RuntimeError."""
    try:
        return lib.call(method, **args)
    except CacheFull:
        raise
    except lib.LLMError as e:
        raise RuntimeError(str(e)) from None


@dataclass(frozen=True)
class KVSpec:
    """What a mixer needs stored per position.  ``window`` 0: every position
    stays; otherwise only the last ``window`` positions can be read again."""

    num_kv_heads: int
    head_dim: int
    window: int = 0

    def to_json(self):
        return {"num_kv_heads": self.num_kv_heads, "head_dim": self.head_dim, "window": self.window}


@dataclass(frozen=True)
class StateSpec:
    """Fixed-size state a mixer keeps per sequence: a tensor of this shape, zero at
    the sequence's start."""

    shape: Tuple[int, ...]
    dtype: object = "float32"

    def to_json(self):
        return {"shape": list(self.shape), "dtype": dtype_name(self.dtype)}


class PagePool:
    """The pages of one layer group (``PagePool`` of cache/cache.h), on its own."""

    def __init__(self, n_pages: int, name: str = "cache"):
        try:
            self._id = lib.call("pagepool.new", n=int(n_pages))["id"]
        except lib.LLMError as e:
            raise ValueError(str(e)) from None
        self.n_pages = n_pages

    def _op(self, op, **a):
        return _call("pool.op", id=self._id, op=op, **a)

    @property
    def n_free(self) -> int:
        return self._op("n_free")["n"]

    def take(self, count: int) -> List[int]:
        return self._op("take", count=int(count))["pages"]

    def give_back(self, pages: Sequence[int]) -> None:
        self._op("give_back", pages=[int(p) for p in pages])

    def check(self) -> None:
        self._op("check")

    def __del__(self):
        try:
            lib.call("pool.free", id=self._id)
        except Exception:
            pass


class SlotPool:
    """The slots: one per live sequence (``SlotPool`` of cache/cache.h), on its own."""

    def __init__(self, n_slots: int):
        try:
            self._id = lib.call("slotpool.new", n=int(n_slots))["id"]
        except lib.LLMError as e:
            raise ValueError(str(e)) from None
        self.n_slots = n_slots

    def _op(self, op, **a):
        return _call("pool.op", id=self._id, op=op, **a)

    @property
    def n_free(self) -> int:
        return self._op("n_free")["n"]

    def live(self, slot: int) -> bool:
        return self._op("live", slot=int(slot))["ok"]

    def take(self) -> int:
        return self._op("take")["slot"]

    def give_back(self, slot: int) -> None:
        self._op("give_back", slot=int(slot))

    def check(self) -> None:
        self._op("check")

    def __del__(self):
        try:
            lib.call("pool.free", id=self._id)
        except Exception:
            pass


class _Shape:
    """Stands for a tensor that has a shape and no storage."""

    def __init__(self, shape):
        self.shape = tuple(shape)


class _GroupPool:
    def __init__(self, group: "KVGroup"):
        self._g = group

    @property
    def n_pages(self) -> int:
        return self._g._info()["n_pages"]

    @property
    def n_free(self) -> int:
        return self._g._info()["free_pages"]


class _Pages:
    def __init__(self, group: "KVGroup"):
        self._g = group

    def __getitem__(self, slot: int) -> List[int]:
        return self._g._cache._op("pages", group=self._g.index_in_cache, slot=int(slot))["pages"]


class KVGroup:
    """The storage of one layer group, as the cache describes it."""

    def __init__(self, cache: "Cache", index: int, info: dict):
        self._cache = cache
        self.index_in_cache = index
        self.spec = KVSpec(info["num_kv_heads"], info["head_dim"], info["window"])
        self.entries: List[int] = list(info["entries"])
        self.index = {e: i for i, e in enumerate(self.entries)}
        self.pool = _GroupPool(self)
        self.pages = _Pages(self)
        shape = tuple(info["shape"])
        if info["k"]:
            self.k = as_tensor(info["k"], shape, cache.dtype_name, cache.device_index)
            self.v = as_tensor(info["v"], shape, cache.dtype_name, cache.device_index)
        else:
            self.k = self.v = _Shape(shape)

    def _info(self) -> dict:
        return self._cache._op("describe")["groups"][self.index_in_cache]

    def first_needed_page(self, next_pos: int) -> int:
        """The lowest page index that a token at ``next_pos`` or later can see."""
        if not self.spec.window:
            return 0
        return max(0, next_pos + 1 - self.spec.window) // PAGE

    def held(self, slot: int) -> int:
        return self._cache._op("held", group=self.index_in_cache, slot=int(slot))["held"]


class _Lengths:
    def __init__(self, cache: "Cache"):
        self._c = cache

    def __getitem__(self, slot: int) -> int:
        return self._c._op("length", slot=int(slot))["length"]


class Cache:
    """Slots, page groups and per-sequence state for one model.

    ``kv_specs[e]`` / ``state_specs[e]`` are what run-order entry ``e`` needs (None
    for nothing).  ``device``: "cpu" for bookkeeping without storage, "cuda:N" for a
    cache with its pages and state on that GPU."""

    def __init__(self, kv_specs: Sequence[Optional[KVSpec]] = (),
                 state_specs: Sequence[Optional[StateSpec]] = (), max_tokens: int = 0,
                 max_seqs: int = 0, dtype="float32", device="cpu", _llm: Optional[int] = None):
        self._llm = _llm
        self._id = None
        if _llm is None:
            dev = str(device)
            self.device_index = -1 if dev == "cpu" else int(dev.split(":")[1]) if ":" in dev else 0
            try:
                self._id = lib.call(
                    "cache.new", kv_specs=[None if s is None else s.to_json() for s in kv_specs],
                    state_specs=[None if s is None else s.to_json() for s in state_specs],
                    max_tokens=int(max_tokens), max_seqs=int(max_seqs), dtype=dtype_name(dtype),
                    device=self.device_index)["id"]
            except lib.LLMError as e:
                raise ValueError(str(e)) from None
        else:
            self.device_index = int(device)
        d = self._op("describe")
        self.dtype_name = d["dtype"]
        self.max_tokens = d["max_tokens"]
        self.max_seqs = d["max_seqs"]
        self.groups: List[KVGroup] = [KVGroup(self, i, g) for i, g in enumerate(d["groups"])]
        self.group_of: Dict[int, KVGroup] = {e: g for g in self.groups for e in g.entries}
        self.length = _Lengths(self)
        self.mixer_state: Dict[int, object] = {}
        if self.device_index >= 0:
            for e in d["state_entries"]:
                st = self._op("state", entry=e)
                self.mixer_state[e] = as_tensor(st["ptr"], st["shape"], st["dtype"], self.device_index)

    def _op(self, op: str, **a):
        if self._llm is not None:
            return _call("cache.op", llm=self._llm, op=op, **a)
        return _call("cache.op", id=self._id, op=op, **a)

    # ------------------------------------------------------------ sequences
    def new_sequence(self) -> int:
        return self._op("new_sequence")["slot"]

    def free_sequence(self, slot: int) -> None:
        self._op("free_sequence", slot=int(slot))

    def can_truncate(self, slot: int, n: int) -> bool:
        return self._op("can_truncate", slot=int(slot), n=int(n))["ok"]

    def truncate(self, slot: int, n: int) -> bool:
        return self._op("truncate", slot=int(slot), n=int(n))["ok"]

    def set_samplers(self, slots: Sequence[int], options: Sequence) -> None:
        self._op("set_samplers", slots=[int(s) for s in slots], settings=[
            {"seed": int(o.seed) & (2 ** 64 - 1), "temperature": float(o.temperature),
             "top_k": int(o.top_k), "top_p": float(o.top_p), "min_p": float(o.min_p)}
            for o in options])

    # ---------------------------------------------------------------- steps
    def reserve(self, slots: Sequence[int], counts: Sequence[int]) -> None:
        self._op("reserve", slots=[int(s) for s in slots], counts=[int(c) for c in counts])

    def advance(self, slots: Sequence[int], counts: Sequence[int]) -> None:
        self._op("advance", slots=[int(s) for s in slots], counts=[int(c) for c in counts])

    def block_table(self, group: KVGroup, slots: Sequence[int]) -> np.ndarray:
        r = self._op("block_table", group=group.index_in_cache, slots=[int(s) for s in slots])
        return np.asarray(r["table"], dtype=np.int32).reshape(len(slots), r["width"])

    # ---------------------------------------------------------------- checks
    def tokens_held(self) -> int:
        return self._op("tokens_held")["tokens"]

    def bytes(self) -> int:
        return self._op("describe")["bytes"]

    def check(self) -> None:
        self._op("check")

    def __del__(self):
        if self._id is not None:
            try:
                lib.call("cache.free", id=self._id)
            except Exception:
                pass


__all__ = ["PAGE", "Cache", "CacheFull", "KVGroup", "KVSpec", "PagePool", "SlotPool", "StateSpec",
           "pages_for"]
