"""Generation through the Python entry point against the plain implementation:
greedy and sampled, unequal prompts, stop tokens, more requests than a batch
holds."""
import numpy as np
import pytest
import torch

import plain_qwen3 as plain
from helpers import model_dir, plain_model
from tiny import TINY, tokens

pytestmark = pytest.mark.gpu

PROMPTS = {"A": [7, 1, 13], "B": [1, 5, 17, 33], "C": [3, 70, 40]}


def prompts(name, seed=7):
    rng = np.random.default_rng(seed)
    return [tokens(rng, n, TINY[name]["vocab_size"]) for n in PROMPTS[name]]


_LLM = {}


def llm(name, dtype, max_batch=8):
    import janas_b200
    key = (name, dtype, max_batch)
    if key not in _LLM:
        _LLM[key] = janas_b200.open(model_dir(name), janas_b200.LLMParams(
            n_ctx=256, dtype=dtype, max_batch=max_batch, max_tokens=256 * max_batch))
    return _LLM[key]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_greedy_tokens_are_the_plain_model_s_choice(name, dtype):
    """Every generated token is the plain model's most likely one, up to the
    rounding of the engine's logits: the plain logit of the chosen token is
    within a small margin of the plain maximum."""
    c, w = plain_model(name)
    ps = prompts(name)
    outs, st = llm(name, dtype).generate_batch(ps, 8)
    assert st.new_tokens == 8 * len(ps) and st.passes == 7 and st.batches == 1
    margin = 1e-4 if dtype == "float32" else 3e-2
    for p, o in zip(ps, outs):
        assert len(o) == 8
        lg = plain.forward(c, w, p + o).numpy()
        for j, tok in enumerate(o):
            row = lg[len(p) - 1 + j]
            assert row[tok] >= row.max() - margin * np.abs(row).max(), (name, j)
    if dtype == "float32":      # and exactly the plain generation, token for token
        for p, o in zip(ps, outs):
            assert o == plain.generate(c, w, p, 8)


@pytest.mark.parametrize("name", ["A", "B"])
def test_sampled_tokens_equal_the_plain_sampler_s(name):
    """Temperature 0.8 with per-request seeds, float32: the same tokens as the
    plain model with the plain sampler (the random sequence, the candidates and
    their order are the same; the logits agree to 1e-6)."""
    import janas_b200
    c, w = plain_model(name)
    ps = prompts(name)
    for settings in (dict(temperature=0.8, top_k=20, top_p=0.8), dict(temperature=0.8),
                     dict(temperature=1.3, top_k=5, min_p=0.1)):
        opts = [janas_b200.GenOptions(seed=1 + i, **settings) for i in range(len(ps))]
        outs, st = llm(name, "float32").generate_batch(ps, 8, opts)
        for i, (p, o) in enumerate(zip(ps, outs)):
            want = plain.generate(c, w, p, 8, seed=1 + i, **settings)
            assert o == want, (name, settings, i)


def test_stop_tokens_and_early_ends():
    import janas_b200
    ps = prompts("B")
    m = llm("B", "float32")
    free, _ = m.generate_batch(ps, 10)
    # stop request 1 at its 4th token and request 3 at its 1st
    stop1, stop3 = free[1][3], free[3][0]
    opts = [janas_b200.GenOptions(), janas_b200.GenOptions(eos=stop1),
            janas_b200.GenOptions(), janas_b200.GenOptions(stop=[stop3, 5])]
    outs, st = m.generate_batch(ps, 10, opts)
    first1 = free[1].index(stop1)
    assert outs[1] == free[1][:first1 + 1] and m.last_finish[1] == "stop"
    assert outs[3] == free[3][:1] and m.last_finish[3] == "stop"
    assert outs[0] == free[0] and outs[2] == free[2]       # the others are not disturbed
    assert m.last_finish[0] == "length"
    m.engine.cache.check()
    assert m.engine.cache.tokens_held() == 0


def test_more_requests_than_a_batch_holds():
    rng = np.random.default_rng(11)
    ps = [tokens(rng, n, TINY["A"]["vocab_size"]) for n in (5, 40, 1, 17, 9, 64, 3)]
    news = [6, 3, 9, 1, 6, 4, 0]
    small = llm("A", "float32", max_batch=3)
    outs, st = small.generate_batch(ps, news)
    assert st.batches == 3
    alone = llm("A", "float32")
    for p, n, o in zip(ps, news, outs):
        assert len(o) == n
        assert o == alone.generate(p, n)[0]
    small.engine.cache.check()
    assert small.engine.cache.tokens_held() == 0


def test_context_full_ends_a_sequence():
    import janas_b200
    m = janas_b200.open(model_dir("A"), janas_b200.LLMParams(n_ctx=20, dtype="float32",
                                                            max_batch=2, max_tokens=128))
    rng = np.random.default_rng(12)
    p = tokens(rng, 17, 256)
    out, st = m.generate(p, 50)
    assert len(out) == 4 and m.last_finish == ["context"]     # fed at 17, 18, 19; the 4th has no place
    with pytest.raises(janas_b200.LLMError):
        m.generate(tokens(rng, 21, 256), 5)


def test_long_decoding_stays_with_the_plain_model():
    """300 decoded tokens after a short prompt (pages and chunks are crossed
    while decoding), float32 and bfloat16: the logits along the way, through the
    step function, against the plain model run on the whole sequence."""
    from janas_b200.engine import Engine, StepEntry
    from helpers import rel_err
    name = "C"
    c, w = plain_model(name)
    rng = np.random.default_rng(13)
    toks = tokens(rng, 330, c["vocab_size"])
    want = plain.forward(c, w, toks).numpy()
    for dtype, tol in (("float32", 5e-6), ("bfloat16", 2e-2)):
        eng = Engine.open(model_dir(name), dtype=dtype, max_tokens=512)
        s = eng.new_sequence()
        rows = [eng.step([StepEntry(s, toks[:30], [29])]).cpu().numpy()[0]]
        for t in toks[30:]:
            rows.append(eng.step([StepEntry(s, [t], [0])]).cpu().numpy()[0])
        e = rel_err(np.stack(rows), want[29:])
        assert e <= tol, (dtype, e)
        eng.free_sequence(s)


def test_first_tokens_of_a_sequence():
    """Positions 0, 1, 2 alone: a prompt of one token, then one token at a time."""
    from janas_b200.engine import Engine, StepEntry
    from helpers import rel_err
    for name in "ABC":
        c, w = plain_model(name)
        toks = [3, 1, 4, 1, 5]
        want = plain.forward(c, w, toks).numpy()
        eng = Engine.open(model_dir(name), dtype="float32", max_tokens=64)
        s = eng.new_sequence()
        got = [eng.step([StepEntry(s, [t], [0])]).cpu().numpy()[0] for t in toks]
        assert rel_err(np.stack(got), want) <= 5e-6
        eng.free_sequence(s)


def test_cli_prints_the_same_tokens(tmp_path):
    import subprocess, sys, os
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    c, w = plain_model("A")
    r = subprocess.run([sys.executable, os.path.join(root, "bin", "janas-b200"), model_dir("A"),
                        "--tokens", "5 17 3 200", "--max", "6", "--dtype", "float32",
                        "--ctx", "128", "--stats"], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr
    assert [int(t) for t in r.stdout.split()] == plain.generate(c, w, [5, 17, 3, 200], 6)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replayed_decode_steps_equal_launched_ones(dtype):
    """The decode step replayed from a CUDA graph gives the tokens that the same
    kernels give when launched one by one: greedy and sampled, while sequences
    end at different times (the batch shrinks) and positions cross pages."""
    import janas_b200
    rng = np.random.default_rng(31)
    v = TINY["C"]["vocab_size"]
    ps = [tokens(rng, n, v) for n in (60, 3, 250, 17)]
    news = [40, 12, 30, 70]
    for opts in (None, [janas_b200.GenOptions(temperature=0.9, top_k=30, top_p=0.9, seed=5 + i)
                        for i in range(4)]):
        m = janas_b200.open(model_dir("C"), janas_b200.LLMParams(n_ctx=512, dtype=dtype,
                                                                max_batch=4, max_tokens=2048))
        assert m.engine.use_graphs
        a, _ = m.generate_batch(ps, news, opts)
        assert m.engine.n_graphs >= 3                # several batch sizes were captured
        m.engine.use_graphs = False
        b, _ = m.generate_batch(ps, news, opts)
        assert a == b
        m.engine.cache.check()


def test_old_decode_graphs_are_dropped_and_captured_again():
    """No more than ``max_graphs`` captured steps are kept: the one used longest ago
    goes, and a batch shape that comes back is captured again with the same tokens."""
    import janas_b200
    rng = np.random.default_rng(32)
    v = TINY["B"]["vocab_size"]
    ps = [tokens(rng, n, v) for n in (9, 30, 2, 70)]
    news = [25, 8, 16, 12]
    m = janas_b200.open(model_dir("B"), janas_b200.LLMParams(n_ctx=256, dtype="bfloat16",
                                                            max_batch=4, max_tokens=1024))
    first, _ = m.generate_batch(ps, news)
    shapes = m.engine.n_graphs
    assert shapes >= 3
    m.engine.drop_graphs()
    m.engine.set_max_graphs(2)
    again, _ = m.generate_batch(ps, news)
    assert again == first
    assert m.engine.n_graphs == 2
    third, _ = m.generate_batch(ps, news)       # the first shapes were dropped meanwhile
    assert third == first
    m.engine.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_steps_fed_on_the_device_equal_steps_fed_by_the_host(dtype):
    """A decode step that goes on from the tokens the step before it chose, launched
    while that step runs, chooses what a step fed from the host chooses: greedy
    and sampled, across a page's end and across the context bound at which another
    captured graph takes over (position 256)."""
    import janas_b200
    from janas_b200.engine import Engine, StepEntry
    from janas_b200.engine.engine import StepError
    from janas_b200.engine.generate import GenOptions
    rng = np.random.default_rng(41)
    v = TINY["C"]["vocab_size"]
    ps = [tokens(rng, n, v) for n in (250, 61, 5)]
    runs = {}
    for way in ("host", "device"):
        for sampled in (False, True):
            eng = Engine.open(model_dir("C"), dtype=dtype, max_tokens=1024, max_seqs=4)
            assert eng.decodes_ahead
            slots = [eng.new_sequence() for _ in ps]
            if sampled:
                eng.cache.set_samplers(slots, [GenOptions(temperature=0.8, top_k=20, seed=3 + i)
                                               for i in range(len(ps))])
            logits = eng.step([StepEntry(s, p, [len(p) - 1]) for s, p in zip(slots, ps)])
            toks = logits.argmax(dim=1).cpu().tolist()
            got = []
            if way == "host":
                for _ in range(12):
                    toks = eng.decode(slots, toks, sampled).tolist()
                    got.append(toks)
            else:
                cur = eng.decode_begin(slots, toks, sampled)
                for i in range(12):
                    nxt = eng.decode_begin(slots, None, sampled) if i < 11 else None
                    got.append(eng.decode_end(cur).tolist())
                    cur = nxt
                assert eng.n_graphs == 2            # positions below 256, then from 256 on
                with pytest.raises(StepError):      # other sequences than the last step's
                    eng.decode_begin(slots[:2], None, sampled)
                eng.free_sequence(slots[2])
                with pytest.raises(StepError):      # one of them has ended
                    eng.decode_begin(slots, None, sampled)
                slots = slots[:2]
            assert [eng.length(s) for s in slots] == [len(p) + 12 for p in ps[:len(slots)]]
            runs[way, sampled] = got
            for s in slots:
                eng.free_sequence(s)
            eng.cache.check()
    assert runs["device", False] == runs["host", False]
    assert runs["device", True] == runs["host", True]
    assert runs["host", True] != runs["host", False]
