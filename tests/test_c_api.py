"""The library's C interface called through its exported symbols with ctypes, with
structs laid out here by hand (not the package's wrappers): codes, the last-error
text of the calling thread, size-prefixed structs from an older and a newer caller,
and on the GPU the step function, a full cache and generation.  In the manner of
the reference's interface: include/janas/llm.h:43-53 (codes), :71-78 (ABI version,
last error, size first), :159-165 (params_default, open, close)."""
import ctypes
import json
import os
import threading

import numpy as np
import pytest

from helpers import model_dir
from tiny import TINY

OK, EINVAL, EOPEN, EMODEL, EFULL, ESMALL, EFAIL = 0, -1, -3, -4, -5, -7, -8
P = ctypes.c_void_p


class Params(ctypes.Structure):
    _fields_ = [("size", ctypes.c_uint32), ("n_ctx", ctypes.c_uint32), ("max_batch", ctypes.c_uint32),
                ("dtype", ctypes.c_int32), ("device", ctypes.c_int32), ("reserved", ctypes.c_uint32),
                ("max_tokens", ctypes.c_uint64)]


class OldParams(ctypes.Structure):
    """What a caller built against an earlier header would pass: the first fields only."""
    _fields_ = [("size", ctypes.c_uint32), ("n_ctx", ctypes.c_uint32), ("max_batch", ctypes.c_uint32),
                ("dtype", ctypes.c_int32)]


class NewParams(ctypes.Structure):
    """What a caller built against a later header would pass: more than this library knows."""
    _fields_ = Params._fields_ + [("later", ctypes.c_uint64 * 4)]


class Piece(ctypes.Structure):
    _fields_ = [("slot", ctypes.c_int32), ("n", ctypes.c_uint32), ("tokens", ctypes.POINTER(ctypes.c_int32)),
                ("n_want", ctypes.c_uint32), ("want", ctypes.POINTER(ctypes.c_int32))]


class GenOptions(ctypes.Structure):
    _fields_ = [("size", ctypes.c_uint32), ("eos", ctypes.c_int32), ("temperature", ctypes.c_float),
                ("top_k", ctypes.c_int32), ("top_p", ctypes.c_float), ("min_p", ctypes.c_float),
                ("seed", ctypes.c_uint64), ("stop", ctypes.c_int32 * 4), ("n_stop", ctypes.c_int32),
                ("reserved", ctypes.c_uint32)]


class GenStats(ctypes.Structure):
    _fields_ = [("size", ctypes.c_uint32), ("prompt_tokens", ctypes.c_uint32), ("new_tokens", ctypes.c_uint32),
                ("passes", ctypes.c_uint32), ("forced_tokens", ctypes.c_uint32), ("batches", ctypes.c_uint32),
                ("prefill_seconds", ctypes.c_double), ("decode_seconds", ctypes.c_double),
                ("sample_seconds", ctypes.c_double), ("h2d_bytes", ctypes.c_uint64),
                ("d2h_bytes", ctypes.c_uint64)]


@pytest.fixture(scope="module")
def L():
    from janas_b200.csrc import build
    lib = ctypes.CDLL(build.library_path())
    lib.jb_llm_last_error.restype = ctypes.c_char_p
    lib.jb_llm_open.argtypes = [ctypes.c_char_p, P, ctypes.POINTER(P)]
    lib.jb_llm_close.argtypes = [P]
    lib.jb_llm_n_ctx.argtypes = [P]
    lib.jb_llm_n_vocab.argtypes = [P]
    lib.jb_llm_slot_new.argtypes = [P, ctypes.POINTER(ctypes.c_int32)]
    lib.jb_llm_slot_free.argtypes = [P, ctypes.c_int32]
    lib.jb_llm_slot_length.argtypes = [P, ctypes.c_int32, ctypes.POINTER(ctypes.c_uint32)]
    lib.jb_llm_step.argtypes = [P, ctypes.POINTER(Piece), ctypes.c_uint32, P, ctypes.c_uint64]
    lib.jb_llm_generate.argtypes = [P, ctypes.POINTER(ctypes.c_int32), ctypes.c_uint32, ctypes.c_uint32, P,
                                    ctypes.POINTER(ctypes.c_int32), ctypes.POINTER(ctypes.c_uint32),
                                    ctypes.POINTER(ctypes.c_int32), P]
    return lib


def err(L):
    return L.jb_llm_last_error().decode()


def test_version_defaults_and_codes_without_a_device(L, tmp_path):
    assert L.jb_llm_abi_version() == 2
    p = Params()
    L.jb_llm_params_default(ctypes.byref(p))
    assert (p.size, p.n_ctx, p.max_batch, p.dtype, p.device, p.max_tokens) == \
        (ctypes.sizeof(Params), 16384, 64, 0, 0, 0)
    o = GenOptions()
    L.jb_gen_options_default(ctypes.byref(o))
    assert (o.size, o.eos, o.temperature, o.top_k, o.n_stop) == (ctypes.sizeof(GenOptions), -1, 0.0, 0, 0)

    h = P()
    # a folder that is not there
    assert L.jb_llm_open(str(tmp_path / "nothing").encode(), None, ctypes.byref(h)) == EOPEN
    assert "no config.json" in err(L) and not h.value
    # an architecture that is not registered
    d = tmp_path / "llama"
    d.mkdir()
    (d / "config.json").write_text(json.dumps(dict(TINY["A"], architectures=["LlamaForCausalLM"])))
    assert L.jb_llm_open(str(d).encode(), None, ctypes.byref(h)) == EMODEL
    assert "not supported" in err(L) and "Qwen3ForCausalLM" in err(L)
    # a configuration that is refused
    (d / "config.json").write_text(json.dumps(dict(TINY["A"], rope_scaling={"factor": 2})))
    assert L.jb_llm_open(str(d).encode(), None, ctypes.byref(h)) == EOPEN and "rope_scaling" in err(L)
    # weights that do not match: one message lists them all, before any device is touched
    import torch
    from janas_b200.config import config_from_dict
    from janas_b200.weights import expected_tensors, random_tensors, write_safetensors
    (d / "config.json").write_text(json.dumps(TINY["A"]))
    ts = dict(random_tensors(expected_tensors(config_from_dict(TINY["A"]).to_model_spec()), 0, torch.bfloat16))
    del ts["model.norm.weight"]
    ts["extra.bias"] = torch.zeros(3)
    write_safetensors(str(d / "model.safetensors"), ts.items())
    assert L.jb_llm_open(str(d).encode(), None, ctypes.byref(h)) == EOPEN
    assert "missing (1): model.norm.weight" in err(L) and "unexpected (1): extra.bias" in err(L)
    # arguments
    assert L.jb_llm_open(None, None, ctypes.byref(h)) == EINVAL
    bad = Params()
    L.jb_llm_params_default(ctypes.byref(bad))
    bad.size = 0
    assert L.jb_llm_open(str(d).encode(), ctypes.byref(bad), ctypes.byref(h)) == EINVAL and "size" in err(L)
    bad.size, bad.dtype = ctypes.sizeof(Params), 7
    assert L.jb_llm_open(str(d).encode(), ctypes.byref(bad), ctypes.byref(h)) == EINVAL and "dtype" in err(L)
    # structs of other sizes are read as far as both sides know them: the failure is
    # still the folder's, not the struct's
    old = OldParams(ctypes.sizeof(OldParams), 128, 2, 1)
    assert L.jb_llm_open(str(tmp_path / "nothing").encode(), ctypes.byref(old), ctypes.byref(h)) == EOPEN
    new = NewParams()
    L.jb_llm_params_default(ctypes.byref(new))
    new.size = ctypes.sizeof(NewParams)
    assert L.jb_llm_open(str(tmp_path / "nothing").encode(), ctypes.byref(new), ctypes.byref(h)) == EOPEN
    # calls on nothing
    assert L.jb_llm_slot_new(None, ctypes.byref(ctypes.c_int32())) == EINVAL
    L.jb_llm_close(None)


def test_the_last_error_belongs_to_the_thread(L, tmp_path):
    h = P()
    assert L.jb_llm_open(str(tmp_path / "a").encode(), None, ctypes.byref(h)) == EOPEN
    seen = {}

    def other():
        seen["before"] = err(L)
        L.jb_llm_open(None, None, ctypes.byref(P()))
        seen["after"] = err(L)

    t = threading.Thread(target=other)
    t.start()
    t.join()
    assert seen["before"] == "" and "path" in seen["after"]
    assert "no config.json" in err(L)          # this thread's text is untouched


@pytest.mark.gpu
def test_open_step_full_cache_and_generate_through_the_symbols(L):
    import plain_qwen3 as plain
    from helpers import plain_model, rel_err
    c, w = plain_model("B")
    # an older caller's struct: float32, a context of 128, two sequences; the rest by default
    old = OldParams(ctypes.sizeof(OldParams), 128, 2, 1)
    h = P()
    assert L.jb_llm_open(model_dir("B").encode(), ctypes.byref(old), ctypes.byref(h)) == OK, err(L)
    assert L.jb_llm_n_ctx(h) == 128 and L.jb_llm_n_vocab(h) == c["vocab_size"]
    V = c["vocab_size"]

    a, b, third = ctypes.c_int32(), ctypes.c_int32(), ctypes.c_int32()
    assert L.jb_llm_slot_new(h, ctypes.byref(a)) == OK and L.jb_llm_slot_new(h, ctypes.byref(b)) == OK
    assert L.jb_llm_slot_new(h, ctypes.byref(third)) == EFULL and "slots" in err(L)

    toks = [5, 17, 3, 9, 200, 11]
    want = plain.forward(c, w, toks).numpy()
    t = (ctypes.c_int32 * 4)(*toks[:4])
    wn = (ctypes.c_int32 * 2)(0, 3)
    piece = Piece(a.value, 4, t, 2, wn)
    out = np.zeros((2, V), dtype=np.float32)
    # a buffer that is too small is refused before anything runs
    assert L.jb_llm_step(h, ctypes.byref(piece), 1, out.ctypes.data, V) == ESMALL
    n = ctypes.c_uint32(9)
    assert L.jb_llm_slot_length(h, a, ctypes.byref(n)) == OK and n.value == 0
    assert L.jb_llm_step(h, ctypes.byref(piece), 1, out.ctypes.data, out.size) == OK, err(L)
    assert rel_err(out, want[[0, 3]]) <= 5e-6
    # the context (128 positions) has no room for 130 more tokens: EFULL, nothing changed
    long = (ctypes.c_int32 * 130)(*([1] * 130))
    piece2 = Piece(a.value, 130, long, 0, None)
    assert L.jb_llm_step(h, ctypes.byref(piece2), 1, None, 0) == EFULL and "context" in err(L)
    assert L.jb_llm_slot_length(h, a, ctypes.byref(n)) == OK and n.value == 4
    # the cache (128 tokens in all) has no room for 70 tokens of a second sequence
    # beside the 64 that the first holds: EFULL from the pages, nothing changed
    piece3 = Piece(b.value, 70, long, 0, None)
    assert L.jb_llm_step(h, ctypes.byref(piece3), 1, None, 0) == EFULL and "pages" in err(L)
    assert L.jb_llm_slot_length(h, b, ctypes.byref(n)) == OK and n.value == 0
    bad = (ctypes.c_int32 * 1)(V)
    piece4 = Piece(b.value, 1, bad, 0, None)
    assert L.jb_llm_step(h, ctypes.byref(piece4), 1, None, 0) == EINVAL and "vocabulary" in err(L)
    assert L.jb_llm_slot_free(h, a) == OK and L.jb_llm_slot_free(h, b) == OK
    assert L.jb_llm_slot_free(h, a) == EINVAL

    prompt = (ctypes.c_int32 * 5)(*toks[:5])
    got = (ctypes.c_int32 * 6)()
    n_out, fin = ctypes.c_uint32(), ctypes.c_int32()
    st = GenStats()
    st.size = ctypes.sizeof(GenStats)
    assert L.jb_llm_generate(h, prompt, 5, 6, None, got, ctypes.byref(n_out), ctypes.byref(fin),
                             ctypes.byref(st)) == OK, err(L)
    assert list(got[:n_out.value]) == plain.generate(c, w, toks[:5], 6) and fin.value == 2
    assert (st.prompt_tokens, st.new_tokens, st.passes, st.batches) == (5, 6, 5, 1)
    L.jb_llm_close(h)
