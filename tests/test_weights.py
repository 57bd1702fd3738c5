"""Weights (no GPU): model folders written and read back, resident dtypes, the one
error that lists every mismatch, malformed files, shards.  The reader and the
checks are the library's own (weights/safetensors.cpp, weights/loader.cpp), reached
through its C interface."""
import json
import os
import struct

import numpy as np
import pytest
import torch

from janas_b200.config import config_from_dict
from janas_b200.weights import (INT_TABLE, MATRIX, NORM, SafetensorsError, TensorSpec, WeightError,
                                check_folder, expected_tensors, list_folder, random_tensors,
                                read_tensor, resident_dtype, write_random_model, write_safetensors)
from tiny import TINY


def folder(tmp_path, name="A", seed=0, dtype=torch.bfloat16):
    d = str(tmp_path / f"m{name}")
    write_random_model(d, config_from_dict(TINY[name]), seed, dtype)
    return d


def bits(t: torch.Tensor) -> np.ndarray:
    return t.view(torch.uint16).numpy() if t.dtype == torch.bfloat16 else t.numpy()


def test_written_folder_reads_back_with_the_library(tmp_path):
    from safetensors.torch import load_file
    d = folder(tmp_path, "B", 1)
    ref = load_file(os.path.join(d, "model.safetensors"))
    exp = expected_tensors(config_from_dict(TINY["B"]).to_model_spec())
    check_folder(d, exp)
    have = list_folder(d)
    assert set(have) == set(ref) == set(exp)
    for k in ref:
        assert have[k] == ("BF16", tuple(ref[k].shape))
        got = read_tensor(d, k, "bfloat16", ref[k].shape)
        assert np.array_equal(got, bits(ref[k])), k
    # widened exactly when the whole model is computed in 32-bit
    wide = read_tensor(d, "model.norm.weight", "float32", ref["model.norm.weight"].shape)
    assert np.array_equal(wide, ref["model.norm.weight"].float().numpy())


def test_random_weights_are_deterministic_and_distributed(tmp_path):
    exp = expected_tensors(config_from_dict(TINY["A"]).to_model_spec())
    a = dict(random_tensors(exp, 0, torch.float32))
    b = dict(random_tensors(exp, 0, torch.float32))
    c = dict(random_tensors(exp, 1, torch.float32))
    assert "lm_head.weight" not in a            # tied: the head is not written
    for k in a:
        assert torch.equal(a[k], b[k])
        assert not torch.equal(a[k], c[k])
    emb = a["model.embed_tokens.weight"]
    assert abs(float(emb.std()) - 0.02) < 0.002 and abs(float(emb.mean())) < 0.002
    n = torch.cat([v.flatten() for k, v in a.items() if "norm" in k])
    assert abs(float(n.mean()) - 1.0) < 0.03 and abs(float(n.std()) - 0.1) < 0.03
    # a tensor's values do not depend on which other tensors exist
    only = dict(random_tensors({"model.norm.weight": exp["model.norm.weight"]}, 0, torch.float32))
    assert torch.equal(only["model.norm.weight"], a["model.norm.weight"])


def test_a_tensor_stored_in_32_bit_stays_so(tmp_path):
    d = folder(tmp_path, "A", 0, torch.float32)
    assert all(dt == "F32" for dt, _ in list_folder(d).values())
    assert resident_dtype("BF16", MATRIX, "bfloat16") == "bfloat16"
    assert resident_dtype("F16", NORM, "bfloat16") == "bfloat16"
    assert resident_dtype("F32", MATRIX, "bfloat16") == "float32"
    assert resident_dtype("BF16", MATRIX, "float32") == "float32"
    assert resident_dtype("I64", INT_TABLE, "bfloat16") == "int32"


def test_half_precision_is_converted_exactly_where_it_fits(tmp_path):
    d = str(tmp_path)
    x = torch.tensor([0.5, -1.25, 3.0e-5, 65504.0, 6.0e-8, 0.0, -0.0], dtype=torch.float16)
    write_safetensors(os.path.join(d, "model.safetensors"), [("x", x)])
    assert np.array_equal(read_tensor(d, "x", "float32", x.shape), x.float().numpy())
    assert np.array_equal(read_tensor(d, "x", "bfloat16", x.shape), bits(x.float().bfloat16()))


def test_one_error_lists_everything(tmp_path):
    d = str(tmp_path / "bad")
    os.makedirs(d)
    cfg = config_from_dict(TINY["A"])
    exp = expected_tensors(cfg.to_model_spec())
    ts = dict(random_tensors(exp, 0, torch.bfloat16))
    del ts["model.layers.0.self_attn.q_norm.weight"]
    del ts["model.layers.1.mlp.down_proj.weight"]
    ts["model.layers.0.self_attn.q_proj.bias"] = torch.zeros(64, dtype=torch.bfloat16)
    ts["model.layers.1.mlp.up_proj.weight"] = torch.zeros(64, 128, dtype=torch.bfloat16)
    ts["model.norm.weight"] = torch.zeros(64, dtype=torch.int32)
    write_safetensors(os.path.join(d, "model.safetensors"), ts.items())
    with pytest.raises(WeightError) as ei:
        check_folder(d, exp)
    e = ei.value
    assert e.missing == ["model.layers.0.self_attn.q_norm.weight",
                         "model.layers.1.mlp.down_proj.weight"]
    assert e.unexpected == ["model.layers.0.self_attn.q_proj.bias"]
    assert e.wrong_shape == [("model.layers.1.mlp.up_proj.weight", (128, 64), (64, 128))]
    assert e.wrong_type == [("model.norm.weight", "I32")]
    msg = str(e)
    for word in ("missing (2)", "unexpected (1)", "wrong shape", "[64, 128]", "expected [128, 64]",
                 "stored as I32"):
        assert word in msg


def test_untied_model_needs_its_head(tmp_path):
    cfg = config_from_dict(TINY["B"])
    exp = expected_tensors(cfg.to_model_spec())
    ts = dict(random_tensors(exp, 0, torch.bfloat16))
    del ts["lm_head.weight"]
    d = str(tmp_path / "nohead")
    os.makedirs(d)
    write_safetensors(os.path.join(d, "model.safetensors"), ts.items())
    with pytest.raises(WeightError, match="lm_head.weight"):
        check_folder(d, exp)


def test_malformed_files(tmp_path):
    d = str(tmp_path)
    p = os.path.join(d, "model.safetensors")
    with pytest.raises(SafetensorsError, match="no model.safetensors"):
        list_folder(d)
    open(p, "wb").write(b"abc")
    with pytest.raises(SafetensorsError, match="too short"):
        list_folder(d)
    open(p, "wb").write(struct.pack("<Q", 1000) + b"{}")
    with pytest.raises(SafetensorsError, match="header length"):
        list_folder(d)
    open(p, "wb").write(struct.pack("<Q", 5) + b"{nope")
    with pytest.raises(SafetensorsError, match="not JSON"):
        list_folder(d)
    hdr = json.dumps({"t": {"dtype": "F32", "shape": [4], "data_offsets": [0, 16]}}).encode()
    open(p, "wb").write(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 8)      # truncated data
    with pytest.raises(SafetensorsError, match="outside the file"):
        list_folder(d)
    hdr = json.dumps({"t": {"dtype": "F32", "shape": [5], "data_offsets": [0, 16]}}).encode()
    open(p, "wb").write(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 16)
    with pytest.raises(SafetensorsError, match="does not match shape"):
        list_folder(d)
    hdr = json.dumps({"t": {"dtype": "F8_E4M3", "shape": [16], "data_offsets": [0, 16]}}).encode()
    open(p, "wb").write(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 16)
    with pytest.raises(SafetensorsError, match="not read"):
        list_folder(d)
    hdr = json.dumps({"t": {"dtype": "F32", "shape": [2 ** 40, 2 ** 40], "data_offsets": [0, 0]}}).encode()
    open(p, "wb").write(struct.pack("<Q", len(hdr)) + hdr)
    with pytest.raises(SafetensorsError, match="does not match shape"):
        list_folder(d)


def test_shards(tmp_path):
    d = str(tmp_path)
    a = {"x": torch.arange(6, dtype=torch.float32).reshape(2, 3)}
    b = {"y": torch.ones(4, dtype=torch.bfloat16), "z": torch.tensor([1, 2, 3], dtype=torch.int64)}
    write_safetensors(os.path.join(d, "model-00001-of-00002.safetensors"), a.items())
    write_safetensors(os.path.join(d, "model-00002-of-00002.safetensors"), b.items())
    json.dump({"weight_map": {"x": "model-00001-of-00002.safetensors",
                              "y": "model-00002-of-00002.safetensors",
                              "z": "model-00002-of-00002.safetensors"}},
              open(os.path.join(d, "model.safetensors.index.json"), "w"))
    exp = {"x": TensorSpec((2, 3)), "y": TensorSpec((4,), NORM), "z": TensorSpec((3,), INT_TABLE)}
    check_folder(d, exp)
    assert list_folder(d) == {"x": ("F32", (2, 3)), "y": ("BF16", (4,)), "z": ("I64", (3,))}
    assert np.array_equal(read_tensor(d, "x", "float32", (2, 3)), a["x"].numpy())
    assert read_tensor(d, "z", "int32", (3,)).tolist() == [1, 2, 3]
    big = {"z": torch.tensor([1, 2 ** 40], dtype=torch.int64)}
    write_safetensors(os.path.join(d, "model-00002-of-00002.safetensors"),
                      list(b.items())[:1] + list(big.items()))
    with pytest.raises(SafetensorsError, match="does not fit int32"):
        read_tensor(d, "z", "int32", (2,))
    # a tensor that the index names and its shard lacks
    json.dump({"weight_map": {"x": "model-00001-of-00002.safetensors",
                              "w": "model-00002-of-00002.safetensors"}},
              open(os.path.join(d, "model.safetensors.index.json"), "w"))
    with pytest.raises(SafetensorsError, match="is not in"):
        list_folder(d)
