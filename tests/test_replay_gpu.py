"""The engine against the plain implementation under every way of cutting the
work: each request alone and whole; with its last 32 tokens one by one; in
batches of unequal lengths whose shorter requests end earlier, one batch after
another so that slots and pages are used again.  In 32-bit and in bfloat16."""
import numpy as np
import pytest
import torch

from helpers import (model_dir, plain_logits, rel_err, run_trace, trace_batches, trace_tail,
                     trace_whole)
from tiny import TINY, tokens

pytestmark = pytest.mark.gpu

# Largest |difference| over largest |logit| of a request.  Measured on the six
# tiny configurations: float32 up to 1e-6 against the plain model; bfloat16 up to
# 6e-3 against the plain model and 5e-3 against the plain model that rounds at the
# same places; the limits below leave a factor of three to five.
# float32: sums in another order, another exp and sincos.
FP32_TOL = 5e-6
# bfloat16 against the plain implementation that rounds at the same places: what
# is left is an occasional value that rounds the other way (2^-9 of one
# activation) carried through the layers, and the softmax weights, which the
# tensor-core attention rounds to bfloat16 before they meet the values.
BF16_SAME_ROUNDING_TOL = 1.5e-2
# bfloat16 against exact float32: the rounding itself (2^-9 per stored value).
BF16_TOL = 2e-2
# float32 engine against itself under another cut: every kernel adds in an order
# that does not depend on the cut, so the logits are the same bits.
FP32_CUT_TOL = 0.0
# bfloat16 engine against itself under another cut: a prompt's rows go through
# other tile shapes of the tensor-core kernels than a single decoded token.
BF16_CUT_TOL = 1.5e-2

LENGTHS = {"A": [7, 1, 13, 70, 127], "B": [1, 5, 17, 33, 130, 250], "C": [3, 40, 64, 65, 200, 430],
           "D": [1, 31, 64, 129, 300, 500], "E": [2, 63, 128, 257, 600], "F": [1, 9, 65, 190]}


def requests(name):
    rng = np.random.default_rng(100 + ord(name))
    return [tokens(rng, n, TINY[name]["vocab_size"]) for n in LENGTHS[name]]


_ENGINES = {}


def engine(name, dtype, max_tokens=2048):
    from janas_b200.engine import Engine
    key = (name, dtype, max_tokens)
    if key not in _ENGINES:
        _ENGINES[key] = Engine.open(model_dir(name), dtype=dtype, max_tokens=max_tokens)
    return _ENGINES[key]


def check_against_plain(name, dtype, got, reqs, ids):
    for rid, toks in zip(ids, reqs):
        have = np.stack([got[rid][p] for p in range(len(toks))])
        if dtype == "float32":
            e = rel_err(have, plain_logits(name, toks))
            assert e <= FP32_TOL, f"{name} {rid} len {len(toks)}: {e:.3e}"
        else:
            e1 = rel_err(have, plain_logits(name, toks, "bfloat16"))
            e2 = rel_err(have, plain_logits(name, toks))
            assert e1 <= BF16_SAME_ROUNDING_TOL, f"{name} {rid} len {len(toks)}: {e1:.3e}"
            assert e2 <= BF16_TOL, f"{name} {rid} len {len(toks)}: {e2:.3e}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E", "F"])
def test_whole(name, dtype):
    reqs = requests(name)
    eng = engine(name, dtype)
    got = run_trace(eng, trace_whole(reqs))
    check_against_plain(name, dtype, got, reqs, [f"r{i}" for i in range(len(reqs))])
    eng.cache.check()
    assert eng.cache.tokens_held() == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E", "F"])
def test_last_32_one_by_one(name, dtype):
    reqs = requests(name)
    eng = engine(name, dtype)
    whole = run_trace(eng, trace_whole(reqs))
    got = run_trace(eng, trace_tail(reqs, 32))
    ids = [f"r{i}" for i in range(len(reqs))]
    check_against_plain(name, dtype, got, reqs, ids)
    tol = FP32_CUT_TOL if dtype == "float32" else BF16_CUT_TOL
    for rid, toks in zip(ids, reqs):
        a = np.stack([whole[rid][p] for p in range(len(toks))])
        b = np.stack([got[rid][p] for p in range(len(toks))])
        e = rel_err(b, a)
        assert e <= tol, f"{name} {rid}: whole and token-by-token differ by {e:.3e}"
    eng.cache.check()
    assert eng.cache.tokens_held() == 0


def batches_for(name):
    """Two batches of unequal requests; prompts shorter than the requests."""
    rng = np.random.default_rng(200 + ord(name))
    v = TINY[name]["vocab_size"]
    ctx = TINY[name]["max_position_embeddings"]
    shapes = [[(7, 12), (1, 9), (13, 13), (70, 100)],
              [(33, 40), (5, 37), (64, 70), (2, 3), (17, 60)]]
    if ctx >= 256:
        shapes[0].append((130, 160))
        shapes[1].append((200, 250))
    return [[(tokens(rng, total, v), p) for (p, total) in b] for b in shapes]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E", "F"])
def test_unequal_batches_with_slot_reuse(name, dtype):
    from janas_b200.engine import Engine
    batches = batches_for(name)
    # room for one batch at a time only: the second batch has to use again what
    # the first gave back
    need = max(sum((len(t) + 63) // 64 * 64 for t, _ in b) for b in batches)
    eng = Engine.open(model_dir(name), dtype=dtype, max_tokens=need, max_seqs=6)
    got = run_trace(eng, trace_batches(batches))
    eng.cache.check()
    assert eng.cache.tokens_held() == 0
    reqs = [t for b in batches for (t, _) in b]
    ids = [f"b{b}r{i}" for b, batch in enumerate(batches) for i in range(len(batch))]
    check_against_plain(name, dtype, got, reqs, ids)
    # against the same requests alone and whole
    alone = run_trace(engine(name, dtype), trace_whole(reqs))
    tol = FP32_CUT_TOL if dtype == "float32" else BF16_CUT_TOL
    for k, (rid, toks) in enumerate(zip(ids, reqs)):
        a = np.stack([alone[f"r{k}"][p] for p in range(len(toks))])
        b = np.stack([got[rid][p] for p in range(len(toks))])
        e = rel_err(b, a)
        assert e <= tol, f"{name} {rid}: batched and alone differ by {e:.3e}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,seed", [("A", 1), ("B", 2), ("C", 3), ("D", 4), ("E", 5), ("F", 6)])
def test_batches_drawn_at_random(name, seed, dtype):
    """Batches whose sizes, prompt lengths and numbers of decoded tokens are drawn
    from a seeded generator (lengths around the page and chunk edges among them),
    in a cache with just enough room for the largest batch: against the plain
    implementation, and in 32-bit bit for bit against each request alone."""
    from janas_b200.engine import Engine
    c = TINY[name]
    rng = np.random.default_rng(1000 + seed)
    edges = [1, 2, 63, 64, 65, 127, 128, 129, 191, 192, 193, 255, 256, 257]
    cap = min(c["max_position_embeddings"], 420)
    batches = []
    for _ in range(4):
        batch = []
        for _ in range(int(rng.integers(1, 6))):
            total = int(rng.choice(edges)) if rng.random() < 0.5 else int(rng.integers(1, cap + 1))
            total = min(total, cap)
            decoded = int(rng.integers(0, min(total, 40)))      # tokens that come one by one
            batch.append((tokens(rng, total, c["vocab_size"]), total - decoded))
        batches.append(batch)
    need = max(sum((len(t) + 63) // 64 * 64 for t, _ in b) for b in batches)
    eng = Engine.open(model_dir(name), dtype=dtype, max_tokens=need, max_seqs=5)
    got = run_trace(eng, trace_batches(batches))
    eng.cache.check()
    assert eng.cache.tokens_held() == 0
    reqs = [t for b in batches for (t, _) in b]
    ids = [f"b{b}r{i}" for b, batch in enumerate(batches) for i in range(len(batch))]
    check_against_plain(name, dtype, got, reqs, ids)
    if dtype == "float32":
        alone = run_trace(engine(name, dtype), trace_whole(reqs))
        for k, (rid, toks) in enumerate(zip(ids, reqs)):
            a = np.stack([alone[f"r{k}"][p] for p in range(len(toks))])
            b = np.stack([got[rid][p] for p in range(len(toks))])
            assert rel_err(b, a) <= FP32_CUT_TOL, f"{name} {rid}: batched and alone differ"


@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("B", "float32"), ("C", "bfloat16")])
def test_the_residual_stream_after_every_layer_is_the_plain_model_s(name, dtype):
    """``Engine.step_trace`` copies the residual stream out after every layer: a whole
    prompt, then its continuation in a second step from the cache, each against
    the plain model's trace of the same positions.  It is the tool that finds the
    first layer that goes wrong; here every layer is right."""
    import plain_qwen3 as plain
    from helpers import plain_model
    c, w = plain_model(name)
    toks = requests(name)[-1]
    cut = len(toks) - 5
    want = []
    plain.forward(c, w, toks, trace=want)
    eng = engine(name, dtype)
    slot = eng.new_sequence()
    try:
        first = eng.step_trace([(slot, toks[:cut], [])])
        rest = eng.step_trace([(slot, toks[cut:], [])])
    finally:
        eng.free_sequence(slot)
    assert len(first) == len(rest) == c["num_hidden_layers"] == len(want)
    tol = 2e-5 if dtype == "float32" else 3e-2
    for layer, (a, b, x) in enumerate(zip(first, rest, want)):
        x = x.numpy()
        assert a.shape == (cut, c["hidden_size"]) and b.shape == (len(toks) - cut, c["hidden_size"])
        assert rel_err(a, x[:cut]) <= tol, (layer, rel_err(a, x[:cut]))
        assert rel_err(b, x[cut:]) <= tol, (layer, rel_err(b, x[cut:]))
    eng.cache.check()
