"""Sessions through the Python entry point against the plain implementation:
turns that go on from the cache, several sessions in one pass, truncation, a
full context; models with and without a window."""
import numpy as np
import pytest

import plain_qwen3 as plain
from helpers import model_dir, plain_model
from tiny import TINY, tokens

pytestmark = pytest.mark.gpu


def open_llm(name, dtype="float32", max_batch=4, n_ctx=256):
    import janas_b200
    return janas_b200.open(model_dir(name), janas_b200.LLMParams(
        n_ctx=n_ctx, dtype=dtype, max_batch=max_batch, max_tokens=n_ctx * max_batch))


@pytest.mark.parametrize("name", ["A", "C", "E"])
def test_turns_go_on_from_the_cache(name):
    """A prompt, a reply, another turn, another reply: every generated token is the
    plain model's choice for the whole sequence so far (float32: exactly), and no
    token is computed twice."""
    c, w = plain_model(name)
    rng = np.random.default_rng(3)
    v = c["vocab_size"]
    m = open_llm(name)
    s = m.session()
    for turn, new in ((tokens(rng, 9, v), 5), (tokens(rng, 70, v), 4), (tokens(rng, 1, v), 3)):
        s.append(turn)
        before = s.computed
        for _ in range(new):
            want = plain.generate(c, w, s.tokens(), 1)[0]
            st, tok = s.next()
            assert (st, tok) == (0, want)
        assert s.computed == s.length - 1 and s.computed > before
    assert s.stats.new_tokens == 12 and s.stats.prompt_tokens == 80 - 3 + 2
    s.close()
    m.engine.cache.check()
    assert m.engine.cache.tokens_held() == 0


def test_session_tokens_are_those_of_generate():
    """Greedy and sampled: a session's tokens are those of ``generate`` with the same
    options (one draw per token from the session's own seed)."""
    import janas_b200
    rng = np.random.default_rng(4)
    m = open_llm("B")
    p = tokens(rng, 12, TINY["B"]["vocab_size"])
    for opts in (janas_b200.GenOptions(), janas_b200.GenOptions(temperature=0.8, top_k=20, seed=11),
                 janas_b200.GenOptions(temperature=1.1, top_p=0.9, seed=5)):
        want, _ = m.generate(p, 10, opts)
        s = m.session(opts)
        s.append(p)
        got = [s.next()[1] for _ in range(10)]
        s.close()
        assert got == want


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_sessions_step_gives_what_each_session_gets_alone(dtype):
    """Three sessions with prompts of unequal lengths, then a turn each on top of
    their replies, moved on together.  In float32 (whose rows do not depend on the
    batch) they are sampled with seeds of their own and get the tokens each gets
    alone.  In bfloat16 rounding differs with the batch, so the sessions choose
    greedily and every token must be the plain model's most likely one for the
    session's sequence so far, up to the rounding of the logits."""
    import janas_b200
    rng = np.random.default_rng(6)
    for name in ("B", "C"):
        c, w = plain_model(name)
        v = TINY[name]["vocab_size"]
        ps = [tokens(rng, n, v) for n in (20, 3, 65)]
        turns = [tokens(rng, n, v) for n in (4, 1, 2)]
        if dtype == "float32":
            opts = [janas_b200.GenOptions(temperature=0.7, top_k=30, seed=21 + i) for i in range(3)]
        else:
            opts = [janas_b200.GenOptions() for _ in range(3)]
        m = open_llm(name, dtype)
        alone = []
        for p, t, o in zip(ps, turns, opts):
            s = m.session(o)
            s.append(p)
            out = [s.next()[1] for _ in range(3)]
            s.append(t)
            out += [s.next()[1] for _ in range(3)]
            alone.append(out)
            s.close()
        ss = [m.session(o) for o in opts]
        for s, p in zip(ss, ps):
            s.append(p)
        got = [[] for _ in ss]
        for it in range(6):
            if it == 3:
                for s, t in zip(ss, turns):
                    s.append(t)
            toks, st = m.sessions_step(ss)
            assert st == [0, 0, 0]
            for g, t in zip(got, toks):
                g.append(t)
        if dtype == "float32":
            assert got == alone
        else:
            for s, p, t, g in zip(ss, ps, turns, got):
                seq = s.tokens()
                assert seq == p + g[:3] + t + g[3:]
                lg = plain.forward(c, w, seq[:-1]).numpy()
                chosen_at = list(range(len(p) - 1, len(p) + 2)) + \
                    list(range(len(p) + 3 + len(t) - 1, len(seq) - 1))
                for at, tok in zip(chosen_at, g):
                    row = lg[at]
                    assert row[tok] >= row.max() - 3e-2 * np.abs(row).max(), (name, at)
        for s in ss:
            s.close()
        m.engine.cache.check()
        assert m.engine.cache.tokens_held() == 0


@pytest.mark.parametrize("name", ["A", "C"])
def test_truncate_and_go_on(name):
    """A reply is cut back and generated again: the same tokens (greedy), on a model
    whose cache can go back and on one with a window whose pages may be gone."""
    c, w = plain_model(name)
    rng = np.random.default_rng(8)
    m = open_llm(name)
    s = m.session()
    p = tokens(rng, 110, c["vocab_size"])     # long enough for the window to let pages go
    s.append(p)
    first = [s.next()[1] for _ in range(8)]
    assert first == plain.generate(c, w, p, 8)
    s.truncate(len(p) + 3)
    assert s.length == len(p) + 3 and s.computed <= len(p) + 2
    again = [s.next()[1] for _ in range(5)]
    assert again == first[3:]
    s.truncate(40)                                     # into the prompt
    want = plain.generate(c, w, p[:40], 4)
    assert [s.next()[1] for _ in range(4)] == want
    s.reset()
    s.append(p[:5])
    assert s.next() == (0, plain.generate(c, w, p[:5], 1)[0])
    s.close()
    m.engine.cache.check()


def test_full_context_and_errors():
    import janas_b200
    m = open_llm("A", n_ctx=20, max_batch=2)
    rng = np.random.default_rng(12)
    s = m.session()
    s.append(tokens(rng, 17, 256))
    out = [s.next() for _ in range(5)]
    assert [st for st, _ in out] == [0, 0, 0, 0, 1]           # as generate: four tokens fit
    t = m.session()
    with pytest.raises(janas_b200.LLMError) as e:
        m.session()                                           # max_batch sessions are open
    assert e.value.code == janas_b200.EFULL
    with pytest.raises(ValueError):
        t.append([1] * 22)
    with pytest.raises(janas_b200.LLMError) as e:
        m.sessions_step([t])                                  # nothing appended yet
    assert e.value.code == janas_b200.EINVAL
    s.close(); t.close()
    m.engine.cache.check()


def test_step_and_slots_through_the_entry_point():
    """``slot_new`` / ``step`` / ``slot_free``: the step function itself, with
    (slot, tokens, wanted places) entries."""
    import janas_b200
    from helpers import rel_err
    c, w = plain_model("B")
    m = open_llm("B")
    toks = [5, 17, 3, 9, 200, 11]
    want = plain.forward(c, w, toks).numpy()
    a = m.slot_new()
    got = m.step([(a, toks[:4], [0, 3])]).cpu().numpy()
    assert rel_err(got, want[[0, 3]]) <= 5e-6
    got = m.step([(a, toks[4:], [1])]).cpu().numpy()          # two more tokens on top
    assert rel_err(got, want[[5]]) <= 5e-6
    with pytest.raises(janas_b200.LLMError) as e:
        m.step([(a, [99999], [0])])
    assert e.value.code == janas_b200.EINVAL
    m.slot_free(a)
    m.engine.cache.check()


def test_cli_chat_goes_on_from_turn_to_turn():
    """``janas-b200 --chat``: two turns on standard input, each reply the plain
    model's continuation of the whole conversation so far."""
    import os, subprocess, sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    c, w = plain_model("A")
    t1, t2 = [5, 17, 3, 200], [9, 1]
    r = subprocess.run([sys.executable, os.path.join(root, "bin", "janas-b200"), model_dir("A"),
                        "--chat", "--max", "5", "--dtype", "float32", "--ctx", "128", "--eos", "-1"],
                       input=" ".join(map(str, t1)) + "\n\nnot ids\n" + " ".join(map(str, t2)) + "\n",
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr
    lines = [[int(t) for t in ln.split()] for ln in r.stdout.splitlines()]
    assert len(lines) == 2 and "invalid literal" in r.stderr
    r1 = plain.generate(c, w, t1, 5)
    assert lines[0] == r1
    assert lines[1] == plain.generate(c, w, t1 + r1 + t2, 5)


@pytest.mark.parametrize("dtype,tol", [("float32", 5e-6), ("bfloat16", 2e-2)])
@pytest.mark.parametrize("name", ["C", "E"])
def test_several_tokens_on_top_of_a_sequence_with_a_window(name, dtype, tol):
    """Steps that append runs of tokens to sequences which hold some, on models whose
    upper or first layers have a window: the window groups have given pages back by
    then, and what every new token can see is still there.  Runs that cross pages
    and the window's width, next to a sequence that goes on by one token and one that
    starts, against the plain model on the whole sequences."""
    from janas_b200.engine import Engine, StepEntry
    from helpers import rel_err
    c, w = plain_model(name)
    rng = np.random.default_rng(17)
    win = c["sliding_window"]
    total = [3 * win + 140, win + 70, 9]
    seqs = [tokens(rng, n, c["vocab_size"]) for n in total]
    want = [plain.forward(c, w, s).numpy() for s in seqs]
    eng = Engine.open(model_dir(name), dtype=dtype, max_tokens=2048, max_seqs=4)
    a, b = eng.new_sequence(), eng.new_sequence()
    done = [0, 0, 0]
    cuts = [[win + 3, 1, 64, win + 60, 5, total[0] - 2 * win - 133], [50, 1, 1, 1, win + 16, 1]]
    third = None
    for it in range(6):
        entries, rows = [], []
        for k, slot in ((0, a), (1, b)):
            n = cuts[k][it]
            entries.append(StepEntry(slot, seqs[k][done[k]:done[k] + n], list(range(n))))
            rows.append((k, done[k], n))
            done[k] += n
        if it == 3:                                   # a third sequence starts meanwhile
            third = eng.new_sequence()
            entries.append(StepEntry(third, seqs[2], list(range(9))))
            rows.append((2, 0, 9))
        got = eng.step(entries).cpu().numpy()
        at = 0
        for k, p0, n in rows:
            e = rel_err(got[at:at + n], want[k][p0:p0 + n])
            assert e <= tol, (name, dtype, it, k, e)
            at += n
    assert done[:2] == total[:2]
    for s in (a, b, third):
        eng.free_sequence(s)
    eng.cache.check()
    assert eng.cache.tokens_held() == 0
