"""An open engine: a handle into the library, with the step function, decode steps
and the cache behind Python methods.

The engine itself (model, cache, step function, captured decode steps) is C++
(``engine/engine.cpp``); this class calls the C interface.  ``step`` returns the
logits as a CUDA tensor for callers that go on with PyTorch; everything else
speaks in plain lists and NumPy arrays.
"""
from __future__ import annotations

import ctypes
import json
from dataclasses import dataclass, field
from typing import Any, Dict, List, Mapping, Optional, Sequence

import numpy as np

from .. import lib
from ..cache import Cache, CacheFull
from ..config import ConfigError, ModelSpec, config_from_dict
from ..devmem import dtype_name


def parse_dtype(name) -> str:
    """"bfloat16" or "float32" for a name or a torch dtype."""
    s = dtype_name(name)
    if s not in ("bfloat16", "float32"):
        raise ValueError(f"dtype {name!r}: bfloat16 or float32")
    return s


@dataclass
class StepEntry:
    """One sequence's share of a step: its next tokens and the places among them
    (indices into ``tokens``) whose logits are wanted."""

    slot: int
    tokens: Sequence[int]
    want: Sequence[int] = field(default_factory=list)


class StepError(lib.LLMError, ValueError):
    """A step that cannot run (code EINVAL); nothing was changed.  A step that the
    cache or the context has no room for raises CacheFull (code EFULL)."""

    def __init__(self, message: str):
        lib.LLMError.__init__(self, lib.EINVAL, message)


def _params(dtype, max_tokens: int, max_seqs: Optional[int], device, n_ctx: Optional[int]):
    p = lib.Params()
    lib.lib().jb_llm_params_default(ctypes.byref(p))
    p.dtype = lib.F32 if parse_dtype(dtype) == "float32" else lib.BF16
    p.max_tokens = int(max_tokens)
    if max_seqs is None:
        max_seqs = max(1, min(256, (int(max_tokens) + 63) // 64))
    p.max_batch = int(max_seqs)
    p.n_ctx = int(n_ctx) if n_ctx else max(int(max_tokens), 1)
    s = str(device)
    p.device = int(s.split(":")[1]) if ":" in s else 0
    return p


class PendingDecode:
    """A decode step under way: ``result()`` waits for it and gives its tokens."""

    def __init__(self, engine: "Engine", handle: int, n: int):
        self._engine, self._handle, self.n = engine, handle, n
        self.tokens: Optional[np.ndarray] = None

    def result(self) -> np.ndarray:
        if self.tokens is None:
            out = (ctypes.c_int32 * self.n)()
            lib.check(lib.lib().jb_llm_decode_end(self._engine._h, self._handle, out))
            self.tokens = np.frombuffer(out, dtype=np.int32).copy()
        return self.tokens


class Engine:
    def __init__(self, handle: int):
        self._h = ctypes.c_void_p(handle)
        self._cache: Optional[Cache] = None
        i = self.info()
        self.dtype = i.get("dtype", "bfloat16")
        self.vocab_size = int(lib.lib().jb_llm_n_vocab(self._h))
        self.device_index = i.get("device", 0)
        self.config = config_from_dict(i["config"]) if "config" in i else None
        self.spec = ModelSpec.from_json(i["spec"]) if "spec" in i else None

    # ------------------------------------------------------------ open/close
    @classmethod
    def open(cls, model_dir: str, dtype="bfloat16", max_tokens: int = 4096,
             max_seqs: Optional[int] = None, device: str = "cuda:0",
             n_ctx: Optional[int] = None) -> "Engine":
        """Reads config.json, picks the model through the registry and loads the
        folder's safetensors by tensor name."""
        p = _params(dtype, max_tokens, max_seqs, device, n_ctx)
        h = ctypes.c_void_p()
        lib.check(lib.lib().jb_llm_open(str(model_dir).encode(), ctypes.byref(p), ctypes.byref(h)))
        return cls(h.value)

    @classmethod
    def open_random(cls, config: Mapping[str, Any], seed: int = 0, dtype="bfloat16",
                    max_tokens: int = 4096, max_seqs: Optional[int] = None,
                    device: str = "cuda:0", n_ctx: Optional[int] = None) -> "Engine":
        """A model of the architecture that ``config`` (a config.json as a
        dictionary) names, with weights made at random on the device."""
        p = _params(dtype, max_tokens, max_seqs, device, n_ctx)
        h = ctypes.c_void_p()
        lib.check(lib.lib().jb_llm_open_random(json.dumps(dict(config)).encode(), int(seed),
                                               ctypes.byref(p), ctypes.byref(h)))
        return cls(h.value)

    @classmethod
    def from_spec(cls, spec: ModelSpec, tensors: Optional[Mapping[str, Any]] = None, seed: int = 0,
                  dtype="float32", max_tokens: int = 4096, max_seqs: Optional[int] = None,
                  device: str = "cuda:0") -> "Engine":
        """A model put together from ``spec`` (layers of registered parts and their
        run order); ``tensors``: CUDA tensors by name (copied), else random weights."""
        p = _params(dtype, max_tokens, max_seqs, device, None)
        h = ctypes.c_void_p()
        tj = None
        keep = None
        if tensors is not None:
            keep = {n: t.contiguous() for n, t in tensors.items()}
            tj = json.dumps({n: {"ptr": t.data_ptr(), "dtype": dtype_name(t.dtype),
                                 "shape": list(t.shape)} for n, t in keep.items()}).encode()
            import torch
            torch.cuda.synchronize()
        lib.check(lib.lib().jb_llm_open_spec(json.dumps(spec.to_json()).encode(), tj, int(seed),
                                             ctypes.byref(p), ctypes.byref(h)))
        return cls(h.value)

    def close(self) -> None:
        if self._h is not None and self._h.value:
            lib.lib().jb_llm_close(self._h)
        self._h = None
        self._cache = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def info(self) -> Dict[str, Any]:
        """Sizes, cache and counters of the open model, as the library describes them."""
        text = lib.lib().jb_llm_info(self._h)
        if text is None:
            raise lib.LLMError(lib.EINVAL, lib.last_error())
        return json.loads(text.decode())

    @property
    def max_positions(self) -> int:
        return int(lib.lib().jb_llm_n_ctx(self._h))

    @property
    def cache(self) -> Cache:
        if self._cache is None:
            self._cache = Cache(_llm=self._h.value, device=self.device_index)
        return self._cache

    @property
    def h2d_bytes(self) -> int:
        return self.info()["h2d_bytes"]

    @property
    def stream(self) -> int:
        """The CUDA stream (a cudaStream_t as a number) the engine's work runs on."""
        return lib.lib().jb_llm_stream(self._h) or 0

    def check(self) -> None:
        """Waits for the device; raises when a kernel reported a failed wait."""
        lib.check(lib.lib().jb_llm_check(self._h))

    # switches of the captured decode steps
    def _set(self, **a) -> dict:
        return lib.call("llm.set", llm=self._h.value, **a)

    @property
    def use_graphs(self) -> bool:
        return self._set()["use_graphs"]

    @use_graphs.setter
    def use_graphs(self, on: bool) -> None:
        self._set(use_graphs=bool(on))

    @property
    def n_graphs(self) -> int:
        return self._set()["graphs"]

    def drop_graphs(self) -> None:
        self._set(drop_graphs=True)

    def set_max_graphs(self, n: int) -> None:
        self._set(max_graphs=int(n))

    @property
    def decodes_ahead(self) -> bool:
        return self.use_graphs

    # ------------------------------------------------------------- sequences
    def new_sequence(self) -> int:
        s = ctypes.c_int32()
        lib.check(lib.lib().jb_llm_slot_new(self._h, ctypes.byref(s)))
        return s.value

    def free_sequence(self, slot: int) -> None:
        code = lib.lib().jb_llm_slot_free(self._h, int(slot))
        if code < 0:
            raise RuntimeError(lib.last_error())

    def length(self, slot: int) -> int:
        n = ctypes.c_uint32()
        lib.check(lib.lib().jb_llm_slot_length(self._h, int(slot), ctypes.byref(n)))
        return n.value

    def truncate_sequence(self, slot: int, n: int) -> bool:
        return lib.lib().jb_llm_slot_truncate(self._h, int(slot), int(n)) == 0

    # ------------------------------------------------------------------ step
    def _pieces(self, entries: Sequence[StepEntry]):
        keep = []
        arr = (lib.Piece * max(len(entries), 1))()
        wanted = 0
        for i, e in enumerate(entries):
            if not isinstance(e, StepEntry):
                e = StepEntry(*e)
            toks = lib.i32_array(int(t) for t in e.tokens)
            want = lib.i32_array(int(w) for w in e.want)
            keep += [toks, want]
            arr[i].slot = int(e.slot)
            arr[i].n = len(e.tokens)
            arr[i].tokens = ctypes.cast(toks, ctypes.POINTER(ctypes.c_int32))
            arr[i].n_want = len(e.want)
            arr[i].want = ctypes.cast(want, ctypes.POINTER(ctypes.c_int32))
            wanted += len(e.want)
        return arr, keep, wanted

    def _step(self, entries, out_ptr: int, floats: int) -> None:
        arr, keep, _ = self._pieces(entries)
        code = lib.lib().jb_llm_step(self._h, arr, len(entries), out_ptr, floats)
        if code == lib.EINVAL:
            raise StepError(lib.last_error())
        lib.check(code)

    def step(self, entries: Sequence[StepEntry]):
        """Runs the entries' tokens as one batch.  Returns the float32 logits
        [wanted, vocab] at the wanted places as a CUDA tensor, in the order of the
        entries and of each entry's ``want`` (None when nothing is wanted)."""
        import torch
        entries = [e if isinstance(e, StepEntry) else StepEntry(*e) for e in entries]
        wanted = sum(len(e.want) for e in entries)
        if wanted == 0:
            self._step(entries, None, 0)
            return None
        out = torch.empty((wanted, self.vocab_size), dtype=torch.float32,
                          device=f"cuda:{self.device_index}")
        torch.cuda.current_stream().synchronize()
        self._step(entries, out.data_ptr(), out.numel())
        return out

    def step_numpy(self, entries: Sequence[StepEntry]) -> Optional[np.ndarray]:
        """``step`` with the logits in host memory (no PyTorch needed)."""
        entries = [e if isinstance(e, StepEntry) else StepEntry(*e) for e in entries]
        wanted = sum(len(e.want) for e in entries)
        if wanted == 0:
            self._step(entries, None, 0)
            return None
        out = np.empty((wanted, self.vocab_size), dtype=np.float32)
        self._step(entries, out.ctypes.data, out.size)
        return out

    def step_trace(self, entries: Sequence[StepEntry]) -> List[np.ndarray]:
        """One step (no logits) whose residual stream is copied out after every
        entry of the model's run order: a list of float32 arrays [rows, hidden],
        rows being the entries' tokens one entry after the other.  For finding the
        first layer that goes wrong against a plain implementation; slow."""
        entries = [e if isinstance(e, StepEntry) else StepEntry(*e) for e in entries]
        res = lib.call("llm.step_trace", llm=self._h.value,
                       entries=[{"slot": int(e.slot), "tokens": [int(t) for t in e.tokens]} for e in entries])
        n, hidden = int(res["n_rows"]), int(res["hidden"])
        return [np.asarray(layer, dtype=np.float32).reshape(n, hidden) for layer in res["layers"]]

    # ---------------------------------------------------------------- decode
    def set_sampler(self, slot: int, options) -> None:
        """The sampling settings of one sequence (a GenOptions); the seed restarts
        its random sequence."""
        from .generate import options_c
        o = options_c(options)
        lib.check(lib.lib().jb_llm_slot_sampler(self._h, int(slot), ctypes.byref(o)))

    def decode_begin(self, slots: Sequence[int], tokens: Optional[Sequence[int]],
                     sampled: bool = False) -> PendingDecode:
        """Launches a decode step (one token for each slot, the next token chosen on
        the device) and returns at once; ``tokens=None``: the slots go on from the
        tokens the step begun last chose for them."""
        sl = lib.i32_array(int(s) for s in slots)
        tk = None if tokens is None else lib.i32_array(int(t) for t in tokens)
        h = ctypes.c_void_p()
        code = lib.lib().jb_llm_decode_begin(self._h, sl, len(slots), tk, int(bool(sampled)),
                                             ctypes.byref(h))
        if code == lib.EINVAL:
            raise StepError(lib.last_error())
        lib.check(code)
        return PendingDecode(self, h.value, len(slots))

    def decode_end(self, pending: PendingDecode) -> np.ndarray:
        return pending.result()

    def decode(self, slots: Sequence[int], tokens: Sequence[int], sampled: bool = False) -> np.ndarray:
        return self.decode_end(self.decode_begin(slots, tokens, sampled))
