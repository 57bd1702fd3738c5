"""Weights: the safetensors reader and writer, the loader's one error, the
random-weights mode (no GPU)."""
import json
import os
import struct

import numpy as np
import pytest
import torch

from janas_b200.config import config_from_dict
from janas_b200.engine import expected_tensors
from janas_b200.weights import (Checkpoint, SafetensorsError, WeightError, load_tensors,
                                random_tensors, resident_dtype, write_random_model,
                                write_safetensors)
from janas_b200.weights.spec import INT_TABLE, MATRIX, NORM, TensorSpec
from tiny import TINY


def folder(tmp_path, name="A", seed=0, dtype=torch.bfloat16):
    d = str(tmp_path / f"m{name}")
    write_random_model(d, config_from_dict(TINY[name]), seed, dtype)
    return d


def test_written_folder_reads_back_with_the_library(tmp_path):
    from safetensors.torch import load_file
    d = folder(tmp_path, "B", 1)
    ref = load_file(os.path.join(d, "model.safetensors"))
    exp = expected_tensors(config_from_dict(TINY["B"]).to_model_spec())
    got = dict(load_tensors(d, exp, torch.bfloat16))
    assert set(got) == set(ref)
    for k in ref:
        assert got[k].dtype == torch.bfloat16
        assert torch.equal(got[k], ref[k]), k
    wide = dict(load_tensors(d, exp, torch.float32))
    assert all(t.dtype == torch.float32 for t in wide.values())
    assert torch.equal(wide["model.norm.weight"], ref["model.norm.weight"].float())


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
    exp = expected_tensors(config_from_dict(TINY["A"]).to_model_spec())
    got = dict(load_tensors(d, exp, torch.bfloat16))
    assert all(t.dtype == torch.float32 for t in got.values())
    assert resident_dtype("BF16", MATRIX, torch.bfloat16) == torch.bfloat16
    assert resident_dtype("F16", NORM, torch.bfloat16) == torch.bfloat16
    assert resident_dtype("F32", MATRIX, torch.bfloat16) == torch.float32
    assert resident_dtype("BF16", MATRIX, torch.float32) == torch.float32
    assert resident_dtype("I64", INT_TABLE, torch.bfloat16) == torch.int32


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
        list(load_tensors(d, exp, torch.bfloat16))
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
        list(load_tensors(d, exp, torch.bfloat16))


def test_malformed_files(tmp_path):
    d = str(tmp_path)
    p = os.path.join(d, "model.safetensors")
    with pytest.raises(SafetensorsError, match="no model.safetensors"):
        Checkpoint(d)
    open(p, "wb").write(b"abc")
    with pytest.raises(SafetensorsError, match="too short"):
        Checkpoint(d)
    open(p, "wb").write(struct.pack("<Q", 1000) + b"{}")
    with pytest.raises(SafetensorsError, match="header length"):
        Checkpoint(d)
    hdr = json.dumps({"t": {"dtype": "F32", "shape": [4], "data_offsets": [0, 16]}}).encode()
    open(p, "wb").write(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 8)      # truncated data
    with pytest.raises(SafetensorsError, match="outside the file"):
        Checkpoint(d)
    hdr = json.dumps({"t": {"dtype": "F32", "shape": [5], "data_offsets": [0, 16]}}).encode()
    open(p, "wb").write(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 16)
    with pytest.raises(SafetensorsError, match="does not match shape"):
        Checkpoint(d)
    hdr = json.dumps({"t": {"dtype": "F8_E4M3", "shape": [16], "data_offsets": [0, 16]}}).encode()
    open(p, "wb").write(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 16)
    with pytest.raises(SafetensorsError, match="not read"):
        Checkpoint(d)


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
    got = dict(load_tensors(d, exp, torch.bfloat16))
    assert torch.equal(got["x"], a["x"]) and got["x"].dtype == torch.float32
    assert got["y"].dtype == torch.bfloat16
    assert got["z"].dtype == torch.int32 and got["z"].tolist() == [1, 2, 3]
