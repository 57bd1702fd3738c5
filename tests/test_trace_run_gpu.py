"""bin/trace_run as a program: a short trace through its command line."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

from helpers import (model_dir, plain_logits, rel_err, trace_batches, write_trace)
from tiny import TINY, tokens

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("dtype,tol", [("float32", 5e-6), ("bfloat16", 2e-2)])
def test_trace_run(tmp_path, dtype, tol):
    rng = np.random.default_rng(21)
    v = TINY["B"]["vocab_size"]
    batch = [(tokens(rng, 40, v), 30), (tokens(rng, 9, v), 2), (tokens(rng, 70, v), 66)]
    steps = trace_batches([batch], want_prompt_all=False)
    steps[1]["entries"][0]["want"] = []            # a step may want nothing of a request
    trace = tmp_path / "trace.jsonl"
    write_trace(trace, steps)
    out = tmp_path / "out"
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model",
                        model_dir("B"), "--dtype", dtype, "--out", str(out), "--max-tokens",
                        "256"], stdin=open(trace), capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stderr[-2000:]
    assert r.stdout.split("\n")[:len(steps)] == [f"done {s['step']}" for s in steps]
    pos = {}
    for st in steps:
        n_want = sum(len(e["want"]) for e in st["entries"])
        path = out / f"{st['step']}.f32"
        if n_want == 0:
            assert not path.exists()
            continue
        got = np.fromfile(path, dtype="<f4").reshape(n_want, v)
        row = 0
        for e in st["entries"]:
            i = int(e["id"][3:])
            base = pos.get(e["id"], 0)
            for w_ in e["want"]:
                want = plain_logits("B", batch[i][0])[base + w_]
                assert rel_err(got[row], want) <= tol, (st["step"], e["id"])
                row += 1
            pos[e["id"]] = base + len(e["tokens"])
