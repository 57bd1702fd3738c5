"""Layer parts: mixers, feed-forwards, norms, position encodings, blocks.

The parts and their registry are the library's (``parts/*.cpp``).  This module has
two uses.  ``build_part`` builds one part of a registered kind on its own, so that
a test can give it tensors and run it against a plain implementation.  And the
``register_*`` decorators add a part whose code is Python (PyTorch operations on
the engine's stream) under a new kind name: the library then calls it like one of
its own, through the callback interface of ``parts/foreign.cpp``.  Nothing in the
library changes for such a part; it is how tests show that another mixer,
feed-forward, norm or position encoding fits the interfaces.
"""
from __future__ import annotations

import ctypes
import json
import traceback
from dataclasses import dataclass, field
from typing import Any, Dict, List, Mapping, Optional

import numpy as np

from .. import lib
from ..cache import KVSpec, StateSpec
from ..config import ConfigError, PartSpec
from ..devmem import as_tensor, dtype_name
from ..weights import TensorSpec, tensor_list

PREFILL = "prefill"   # every sequence starts at its first token
DECODE = "decode"     # every sequence goes on by one token
EXTEND = "extend"     # anything else (tokens appended to sequences that have some)


def _torch():
    import torch
    return torch


def _device_index(device) -> int:
    s = str(device)
    if s == "cpu":
        return -1
    return int(s.split(":")[1]) if ":" in s else 0


@dataclass
class LayerCache:
    """What a mixer sees of the cache for the run-order entry it runs as."""

    k: Any = None              # [pages, kv_heads, PAGE, head_dim]
    v: Any = None
    block_table: Any = None    # int32 [sequences of the step, P]
    writes: bool = True        # False: read another entry's cache only
    state: Any = None          # [slots, *state shape], indexed by slot

    def to_json(self) -> dict:
        d: Dict[str, Any] = {"writes": bool(self.writes)}
        if self.k is not None:
            d.update(k=self.k.data_ptr(), v=self.v.data_ptr(), n_pages=self.k.shape[0],
                     kv_heads=self.k.shape[1], head_dim=self.k.shape[3],
                     dtype=dtype_name(self.k.dtype))
        if self.block_table is not None:
            d.update(block_table=self.block_table.data_ptr(), bt_stride=self.block_table.shape[1])
        if self.state is not None:
            d.update(state=self.state.data_ptr(), state_shape=list(self.state.shape[1:]),
                     state_dtype=dtype_name(self.state.dtype), n_slots=self.state.shape[0])
        return d


@dataclass
class StepContext:
    """One step: the rows (tokens) it runs and where each belongs.  The ``row_*``
    and ``seq_slot_dev`` tensors are on the device (int32); the ``seq_*`` arrays are
    on the host (empty in a captured decode step)."""

    kind: str
    dtype: Any
    device: Any
    n_rows: int
    n_seqs: int
    row_pos: Any
    row_seq: Any
    seq_slot_dev: Any
    seq_slots: List[int]
    seq_pos0: Any
    seq_len: Any
    seq_row0: Any
    max_pos: int
    hidden: int = 0
    stream: int = 0
    extras: Dict[str, object] = field(default_factory=dict)

    def to_json(self, hidden: int) -> dict:
        lst = lambda a: [] if a is None else [int(x) for x in a]
        return {"kind": self.kind, "dtype": dtype_name(self.dtype), "n_rows": int(self.n_rows),
                "n_seqs": int(self.n_seqs), "hidden": int(hidden),
                "row_pos": self.row_pos.data_ptr(), "row_seq": self.row_seq.data_ptr(),
                "seq_slot": self.seq_slot_dev.data_ptr(), "seq_slots": lst(self.seq_slots),
                "seq_pos0": lst(self.seq_pos0), "seq_len": lst(self.seq_len),
                "seq_row0": lst(self.seq_row0), "max_pos": int(self.max_pos)}


# ------------------------------------------------- parts of the library, alone
class BuiltPart:
    """One part of a registered kind, built on its own (a handle into the library)."""

    def __init__(self, role: str, spec: PartSpec, dtype, device):
        self.role, self.spec, self.dtype, self.device = role, spec, dtype, device
        self._dev = _device_index(device)
        try:
            self._id = lib.call("part.build", role=role, spec=spec.to_json(),
                                dtype=dtype_name(dtype), device=self._dev)["id"]
        except lib.LLMError as e:
            if e.code in (lib.EOPEN, lib.EMODEL):
                raise ConfigError(str(e), e.code) from None
            raise

    def _call(self, method: str, **a) -> dict:
        return lib.call("part." + method, id=self._id, **a)

    def tensors(self, prefix: str) -> Dict[str, TensorSpec]:
        return tensor_list(self._call("tensors", prefix=prefix)["tensors"])

    def load(self, prefix: str, tensors: Mapping[str, Any]) -> None:
        """Takes its tensors (CUDA tensors, float32 or bfloat16); they are copied."""
        want = self.tensors(prefix)
        keep = {n: t.contiguous() for n, t in tensors.items() if n in want}
        self._call("load", prefix=prefix, tensors={
            n: {"ptr": t.data_ptr(), "dtype": dtype_name(t.dtype), "shape": list(t.shape)}
            for n, t in keep.items()})

    def info(self) -> dict:
        return self._call("info")

    def _result(self, r: dict, squeeze: bool = False):
        torch = _torch()
        shape = (r["S"], r["n"], r["m"])
        out = torch.empty(shape, dtype=getattr(torch, r["dtype"]), device=f"cuda:{self._dev}")
        self._call("result", out=out.data_ptr())
        return out[0] if squeeze else out

    def __del__(self):
        try:
            lib.call("part.free", id=self._id)
        except Exception:
            pass

    # ---- norm
    def apply(self, x, out_dtype, delta=None, rows=None):
        """Normalizes the rows of the float32 residual stream ``x`` (see Norm)."""
        torch = _torch()
        torch.cuda.synchronize()
        args: Dict[str, Any] = {"x": x.data_ptr(), "n": x.shape[0], "out_dtype": dtype_name(out_dtype)}
        if delta is not None:
            delta = delta if delta.dim() == 3 else delta.unsqueeze(0)
            delta = delta.contiguous()
            args["delta"] = {"ptr": delta.data_ptr(), "S": delta.shape[0]}
        if rows is not None:
            args["rows"] = {"ptr": rows.data_ptr(), "n": rows.numel()}
        return self._result(self._call("apply", **args), squeeze=True)

    # ---- position encoding, mixer
    def prepare(self, n_positions: int) -> None:
        self._info = self._call("prepare", n_positions=int(n_positions))

    @property
    def position(self) -> "_PositionView":
        return _PositionView(self.info().get("position", {}), self._dev)

    @property
    def n_positions(self) -> int:
        return self.info().get("n_positions", 0)

    @property
    def cos(self):
        i = self.info()
        return as_tensor(i["cos"], (i["n_positions"], i["rotary_dim"] // 2), "float32", self._dev)

    @property
    def sin(self):
        i = self.info()
        return as_tensor(i["sin"], (i["n_positions"], i["rotary_dim"] // 2), "float32", self._dev)

    def kv_spec(self) -> Optional[KVSpec]:
        r = self._call("kv_spec")
        return KVSpec(r["num_kv_heads"], r["head_dim"], r["window"]) if r else None

    def state_spec(self) -> Optional[StateSpec]:
        r = self._call("state_spec")
        return StateSpec(tuple(r["shape"]), r["dtype"]) if r else None

    def supports(self, kind: str) -> bool:
        return self._call("supports", kind=kind)["ok"]

    # ---- mixer, feed-forward
    def forward(self, ctx: StepContext, h, cache: Optional[LayerCache] = None):
        """h: [n, hidden] in the compute dtype -> stack [S, n, hidden] float32."""
        torch = _torch()
        torch.cuda.synchronize()
        h = h.contiguous()
        args = {"ctx": ctx.to_json(h.shape[1]), "h": h.data_ptr()}
        if cache is not None:
            args["cache"] = cache.to_json()
        return self._result(self._call("forward", **args))

    @property
    def FUSED_FROM(self) -> int:
        return self.info()["fused_from"]

    @property
    def FUSED_UP_TO(self) -> int:
        return self.info()["fused_up_to"]


class _PositionView:
    def __init__(self, info: dict, dev: int):
        self._i, self._dev = info, dev

    @property
    def n_positions(self) -> int:
        return self._i.get("n_positions", 0)


def build_part(role: str, spec: PartSpec, dtype, device) -> BuiltPart:
    """One part of the registered kind ``spec.kind``; role: "mixer", "feed_forward",
    "norm" or "position"."""
    return BuiltPart(role, spec, dtype, device)


def registered(role: str) -> List[str]:
    return sorted(lib.call("parts.registered", role=role)["kinds"])


# ------------------------------------------------ parts whose code is Python
class Part:
    """Base of parts written in Python (see ``register_mixer`` and the others)."""

    def __init__(self, spec: PartSpec, dtype, device):
        self.spec, self.dtype, self.device = spec, dtype, device

    def tensors(self, prefix: str) -> Dict[str, TensorSpec]:
        """name -> TensorSpec of every tensor this part reads, below ``prefix``."""
        return {}

    def load(self, prefix: str, tensors: Mapping[str, Any]) -> None:
        """Takes its tensors (on the device, in their resident dtype; the library
        keeps them alive as long as the part lives)."""

    @staticmethod
    def _name(prefix: str, leaf: str) -> str:
        return f"{prefix}.{leaf}" if prefix else leaf


class Norm(Part):
    def apply(self, x, out_dtype, rows=None):
        """x: the float32 residual stream [n, size] (what was pending is added
        already); returns the normalized rows (all, or those ``rows`` names)."""
        raise NotImplementedError


class PositionEncoding(Part):
    """Must offer ``cos`` and ``sin`` (float32 [n_positions, rotary_dim / 2] on the
    device) once ``prepare`` has run, ``rotary_dim`` and ``n_positions``."""

    cos = None
    sin = None
    rotary_dim = 0
    n_positions = 0

    def prepare(self, n_positions: int) -> None:
        pass


class Mixer(Part):
    graph_safe = False

    def kv_spec(self) -> Optional[KVSpec]:
        return None

    def state_spec(self) -> Optional[StateSpec]:
        return None

    def prepare(self, n_positions: int) -> None:
        pass

    def supports(self, kind: str) -> bool:
        return True

    def forward(self, ctx: StepContext, h, cache: LayerCache):
        """h: [n, hidden] in the compute dtype -> [n, hidden] (or a stack [S, n,
        hidden] whose sum it is) float32."""
        raise NotImplementedError


class FeedForward(Part):
    graph_safe = False

    def forward(self, ctx: StepContext, h):
        raise NotImplementedError


_HOSTS: List["_Host"] = []      # kept alive: the library holds their callbacks


class _Host:
    """Serves the library's questions about one registered Python class."""

    def __init__(self, role: str, kind: str, cls: type):
        self.role, self.kind, self.cls = role, kind, cls
        self.instances: Dict[int, Part] = {}
        self.next_id = 1
        self._reply = None
        self.callback = lib.PART_CALLBACK(self._serve)

    def _serve(self, user, method, args_json):
        try:
            out = self._handle(method.decode(), json.loads(args_json.decode()))
        except Exception as e:          # the library turns this into its own failure
            traceback.print_exc()
            out = {"error": f"{type(e).__name__}: {e}"}
        self._reply = ctypes.create_string_buffer(json.dumps(out or {}).encode())
        return ctypes.cast(self._reply, ctypes.c_void_p).value

    def _ctx(self, c: dict) -> StepContext:
        torch = _torch()
        dev = c.get("device", 0)
        n, B = c["n_rows"], c["n_seqs"]
        return StepContext(
            kind=c["kind"], dtype=getattr(torch, c["dtype"]), device=torch.device(f"cuda:{dev}"),
            n_rows=n, n_seqs=B, row_pos=as_tensor(c["row_pos"], (n,), "int32", dev),
            row_seq=as_tensor(c["row_seq"], (n,), "int32", dev),
            seq_slot_dev=as_tensor(c["seq_slot"], (B,), "int32", dev),
            seq_slots=list(c["seq_slots"]), seq_pos0=np.asarray(c["seq_pos0"], dtype=np.int64),
            seq_len=np.asarray(c["seq_len"], dtype=np.int64),
            seq_row0=np.asarray(c["seq_row0"], dtype=np.int64), max_pos=c["max_pos"],
            hidden=c["hidden"], stream=c["stream"])

    def _cache(self, c: dict, dev: int, n_seqs: int) -> LayerCache:
        lc = LayerCache(writes=c.get("writes", True))
        if c.get("k"):
            shape = (c["n_pages"], c["kv_heads"], c["page"], c["head_dim"])
            lc.k = as_tensor(c["k"], shape, c["dtype"], dev)
            lc.v = as_tensor(c["v"], shape, c["dtype"], dev)
        if c.get("block_table"):
            lc.block_table = as_tensor(c["block_table"], (n_seqs, c["bt_stride"]), "int32", dev)
        if c.get("state"):
            lc.state = as_tensor(c["state"], [c["n_slots"]] + list(c["state_shape"]),
                                 c["state_dtype"], dev)
        return lc

    def _handle(self, method: str, a: dict) -> dict:
        torch = _torch()
        if method == "create":
            inst = self.cls(PartSpec.from_json({"kind": a["kind"], "params": a["params"]}),
                            getattr(torch, a["dtype"]), torch.device("cuda:0"))
            i = self.next_id
            self.next_id += 1
            self.instances[i] = inst
            return {"id": i}
        if method == "destroy":
            self.instances.pop(a["id"], None)
            return {}
        inst = self.instances[a["id"]]
        if method == "tensors":
            return {"tensors": [{"name": n, "shape": list(s.shape), "kind": s.kind,
                                 "optional": s.optional}
                                for n, s in inst.tensors(a["prefix"]).items()]}
        if method == "load":
            ts = {n: as_tensor(t["ptr"], t["shape"], t["dtype"]) for n, t in a["tensors"].items()}
            inst.load(a["prefix"], ts)
            return {}
        if method == "kv_spec":
            s = inst.kv_spec()
            return s.to_json() if s is not None else {}
        if method == "state_spec":
            s = inst.state_spec()
            return s.to_json() if s is not None else {}
        if method == "supports":
            return {"ok": bool(inst.supports(a["kind"]))}
        if method == "graph_safe":
            return {"ok": bool(getattr(inst, "graph_safe", False))}
        if method == "prepare":
            inst.prepare(a["n_positions"])
            if self.role != "position":
                return {}
            if inst.cos is None:
                return {"cos": 0, "sin": 0, "rotary_dim": 0, "n_positions": int(inst.n_positions)}
            inst.cos, inst.sin = inst.cos.float().contiguous(), inst.sin.float().contiguous()
            torch.cuda.synchronize()
            return {"cos": inst.cos.data_ptr(), "sin": inst.sin.data_ptr(),
                    "rotary_dim": int(inst.rotary_dim), "n_positions": int(inst.n_positions)}
        if method in ("forward", "apply"):
            c = a["ctx"]
            dev = c.get("device", 0)
            with torch.cuda.stream(torch.cuda.ExternalStream(c["stream"], device=f"cuda:{dev}")):
                if method == "forward":
                    ctx = self._ctx(c)
                    h = as_tensor(a["h"], (ctx.n_rows, ctx.hidden), c["dtype"], dev)
                    out = as_tensor(a["out"], (ctx.n_rows, ctx.hidden), "float32", dev)
                    if self.role == "mixer":
                        res = inst.forward(ctx, h, self._cache(a["cache"], dev, ctx.n_seqs))
                    else:
                        res = inst.forward(ctx, h)
                    res = res.float()
                    out.copy_(res.sum(0) if res.dim() == 3 else res)
                else:
                    size = int(inst.spec.params["size"])
                    x = as_tensor(a["x"], (a["n"], size), "float32", dev)
                    rows = as_tensor(a["rows"], (a["n_out"],), "int32", dev) if a["rows"] else None
                    out = as_tensor(a["out"], (a["n_out"], size), a["out_dtype"], dev)
                    out.copy_(inst.apply(x, getattr(torch, a["out_dtype"]), rows))
            return {}
        raise ValueError(f"no method {method!r}")


def _register(role: str, kind: str):
    def deco(cls: type) -> type:
        host = _Host(role, kind, cls)
        _HOSTS.append(host)
        lib.check(lib.lib().jb_register_part(role.encode(), kind.encode(), host.callback, None))
        cls._host = host
        return cls
    return deco


def register_mixer(kind: str): return _register("mixer", kind)
def register_feed_forward(kind: str): return _register("feed_forward", kind)
def register_norm(kind: str): return _register("norm", kind)
def register_position_encoding(kind: str): return _register("position", kind)


__all__ = ["DECODE", "EXTEND", "PREFILL", "BuiltPart", "FeedForward", "LayerCache", "Mixer", "Norm",
           "Part", "PositionEncoding", "StepContext", "build_part", "register_feed_forward",
           "register_mixer", "register_norm", "register_position_encoding", "registered"]
