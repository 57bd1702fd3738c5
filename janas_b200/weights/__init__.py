"""Weights: what a model folder holds against what a model needs.

The reader, the check (one error for every missing, unexpected, misshapen or
mistyped tensor) and the conversion to resident dtypes are the library's
(``weights/safetensors.cpp``, ``weights/loader.cpp``); this module asks it.  The
random-weights mode that writes a model folder is here: it draws on the host with
PyTorch's generator, one generator per tensor.
"""
from __future__ import annotations

from typing import Dict, List, Mapping, Tuple

import numpy as np

from .. import lib
from .random_init import random_tensor, random_tensors, write_random_model
from .safetensors_io import SafetensorsError, write_safetensors
from .spec import EMBEDDING, INT_TABLE, MATRIX, NORM, TensorSpec


class WeightError(ValueError):
    """The folder's tensors do not match what the model needs."""

    def __init__(self, message: str, detail: Mapping):
        super().__init__(message)
        self.missing: List[str] = list(detail.get("missing", []))
        self.unexpected: List[str] = list(detail.get("unexpected", []))
        self.wrong_shape = [(e["name"], tuple(e["want"]), tuple(e["got"]))
                            for e in detail.get("wrong_shape", [])]
        self.wrong_type = [(e["name"], e["stored"]) for e in detail.get("wrong_type", [])]


def _list_json(expected: Mapping[str, TensorSpec]) -> list:
    return [{"name": n, "shape": list(s.shape), "kind": s.kind, "optional": s.optional}
            for n, s in expected.items()]


def tensor_list(items) -> Dict[str, TensorSpec]:
    """The library's tensor list (JSON) as name -> TensorSpec, in its order."""
    return {t["name"]: TensorSpec(tuple(t["shape"]), t["kind"], t["optional"]) for t in items}


def expected_tensors(spec) -> Dict[str, TensorSpec]:
    """Every tensor a model of this spec reads, by checkpoint name (no device is
    touched)."""
    return tensor_list(lib.call("spec.tensors", spec=spec.to_json())["tensors"])


def list_folder(model_dir: str) -> Dict[str, Tuple[str, Tuple[int, ...]]]:
    """name -> (stored dtype, shape) of every tensor of a model folder; a file that
    is not well-formed raises SafetensorsError."""
    try:
        r = lib.call("checkpoint.list", dir=str(model_dir))
    except lib.LLMError as e:
        raise SafetensorsError(str(e)) from None
    return {t["name"]: (t["dtype"], tuple(t["shape"])) for t in r["tensors"]}


def check_folder(model_dir: str, expected: Mapping[str, TensorSpec]) -> None:
    """Raises ONE WeightError that lists every mismatch between the folder and
    ``expected`` (SafetensorsError for a file that is not well-formed)."""
    try:
        lib.call("weights.check", dir=str(model_dir), tensors=_list_json(expected))
    except lib.LLMError as e:
        detail = getattr(e, "detail", {})
        if detail:
            raise WeightError(str(e), detail) from None
        raise SafetensorsError(str(e)) from None


def resident_dtype(stored: str, kind: str, compute: str) -> str:
    """The dtype ("bfloat16", "float32", "int32") a tensor is kept in on the device."""
    return lib.call("weights.resident", stored=stored, kind=kind, compute=compute)["dtype"]


_NP = {"float32": np.float32, "bfloat16": np.uint16, "int32": np.int32}


def read_tensor(model_dir: str, name: str, dtype: str, shape) -> np.ndarray:
    """The tensor as the engine would keep it (``dtype``: a resident dtype), read by
    the library into host memory.  bfloat16 comes as its 16-bit patterns."""
    out = np.empty(tuple(shape), dtype=_NP[dtype])
    try:
        lib.call("weights.read", dir=str(model_dir), name=name, dtype=dtype,
                 out=out.ctypes.data)
    except lib.LLMError as e:
        raise SafetensorsError(str(e)) from None
    return out


__all__ = ["EMBEDDING", "INT_TABLE", "MATRIX", "NORM", "SafetensorsError", "TensorSpec",
           "WeightError", "check_folder", "expected_tensors", "list_folder", "random_tensor",
           "random_tensors", "read_tensor", "resident_dtype", "tensor_list", "write_random_model",
           "write_safetensors"]
