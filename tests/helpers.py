"""Helpers shared by the tests: model folders, traces, comparisons."""
import json
import os
import tempfile

import numpy as np
import torch

import plain_qwen3 as plain
from tiny import SEEDS, TINY

_FOLDERS = {}


def model_dir(name: str, stored: torch.dtype = torch.bfloat16) -> str:
    """A temporary model folder for the tiny configuration ``name`` with random
    weights (made once per process)."""
    key = (name, stored)
    if key not in _FOLDERS:
        from janas_b200.config import config_from_dict
        from janas_b200.weights import write_random_model
        d = tempfile.mkdtemp(prefix=f"janas_b200_tiny{name}_")
        write_random_model(d, config_from_dict(TINY[name]), SEEDS[name], stored)
        _FOLDERS[key] = d
    return _FOLDERS[key]


_PLAIN = {}


def plain_model(name: str, stored: torch.dtype = torch.bfloat16):
    key = (name, stored)
    if key not in _PLAIN:
        d = model_dir(name, stored)
        _PLAIN[key] = (plain.read_config(d), plain.read_weights(d))
    return _PLAIN[key]


_PLAIN_LOGITS = {}


def plain_logits(name: str, toks, rounding=None, stored: torch.dtype = torch.bfloat16):
    key = (name, tuple(toks), rounding, stored)
    if key not in _PLAIN_LOGITS:
        c, w = plain_model(name, stored)
        _PLAIN_LOGITS[key] = plain.forward(c, w, list(toks), rounding).numpy()
    return _PLAIN_LOGITS[key]


def rel_err(got: np.ndarray, want: np.ndarray) -> float:
    """Largest absolute difference over the largest wanted magnitude."""
    got, want = np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64)
    assert got.shape == want.shape, (got.shape, want.shape)
    assert np.isfinite(got).all(), "non-finite logits"
    return float(np.abs(got - want).max() / (np.abs(want).max() + 1e-30))


# ---------------------------------------------------------------- traces
def trace_whole(requests):
    """Each request alone and whole, all logits wanted."""
    steps = []
    for i, toks in enumerate(requests):
        steps.append({"step": i, "entries": [{"id": f"r{i}", "tokens": list(toks),
                                              "want": list(range(len(toks)))}],
                      "end": [f"r{i}"]})
    return steps


def trace_tail(requests, tail=32):
    """Each request alone: all but the last ``tail`` tokens in one step, then
    the rest one by one; all logits wanted."""
    steps, k = [], 0
    for i, toks in enumerate(requests):
        toks = list(toks)
        head = max(1, len(toks) - tail)
        steps.append({"step": k, "entries": [{"id": f"r{i}", "tokens": toks[:head],
                                              "want": list(range(head))}], "end": []})
        k += 1
        for j in range(head, len(toks)):
            steps.append({"step": k, "entries": [{"id": f"r{i}", "tokens": [toks[j]],
                                                  "want": [0]}],
                          "end": [f"r{i}"] if j == len(toks) - 1 else []})
            k += 1
        if head == len(toks):
            steps[-1]["end"] = [f"r{i}"]
    return steps


def trace_batches(batches, want_prompt_all=True):
    """``batches``: a list of batches; a batch is a list of (tokens, prompt_len).
    A batch's prompts run in one step, then every request goes on by one token a
    step; a request that has no tokens left ends, the others carry on.  Batches
    run one after the other, so slots and pages are used again."""
    steps, k = [], 0
    for b, batch in enumerate(batches):
        ids = [f"b{b}r{i}" for i in range(len(batch))]
        done = [p for (_, p) in batch]
        ent = [{"id": ids[i], "tokens": list(t[:p]),
                "want": list(range(p)) if want_prompt_all else [p - 1]}
               for i, (t, p) in enumerate(batch)]
        end = [ids[i] for i, (t, p) in enumerate(batch) if p == len(t)]
        steps.append({"step": k, "entries": ent, "end": end})
        k += 1
        while True:
            ent, end = [], []
            for i, (t, p) in enumerate(batch):
                if done[i] < len(t):
                    ent.append({"id": ids[i], "tokens": [t[done[i]]], "want": [0]})
                    done[i] += 1
                    if done[i] == len(t):
                        end.append(ids[i])
            if not ent:
                break
            steps.append({"step": k, "entries": ent, "end": end})
            k += 1
    return steps


def run_trace(engine, steps):
    """Replays ``steps`` in-process; returns {request id: {position: logits}}."""
    from janas_b200.engine import Replayer
    rp = Replayer(engine)
    pos = {}
    out = {}
    for st in steps:
        got = rp.run_step(st)
        r = 0
        for e in st["entries"]:
            base = pos.get(e["id"], 0)
            for w in e["want"]:
                out.setdefault(e["id"], {})[base + w] = got[r]
                r += 1
            pos[e["id"]] = base + len(e["tokens"])
        assert got is None or r == got.shape[0]
    assert not rp.slots, "requests left alive at the end of the trace"
    return out


def write_trace(path, steps):
    with open(path, "w") as f:
        for st in steps:
            f.write(json.dumps(st) + "\n")
