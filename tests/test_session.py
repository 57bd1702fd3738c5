"""Sessions on a stand-in engine: what is fed when, what a full context and a
truncation do, and that several sessions move on together."""
import numpy as np
import pytest

import janas_b200
from janas_b200.engine import session as S
from janas_b200.engine.generate import GenOptions
from standin import StandIn


class FakeEngine(StandIn):
    """The "model" answers token t at position p with (t + p) % 50.  It records the
    steps and checks that every position is fed exactly once, in order."""

    def __init__(self, max_positions=40, extend=True, can_go_back=True):
        super().__init__(max_positions, max_seqs=4, extend=extend)
        self.fed, self.steps = {}, []
        self.can_go_back = can_go_back

    def on_new(self, s):
        self.fed[s] = []

    def truncate(self, s, n):
        if n != 0 and n != self.len[s] and not self.can_go_back:
            return False
        self.len[s] = n
        del self.fed[s][n:]
        return True

    def run(self, entries):
        lens = [len(e["tokens"]) for e in entries]
        pos0 = [self.len[e["slot"]] for e in entries]
        kind = ("prefill" if not any(pos0) else "decode" if all(n == 1 for n in lens)
                else "extend")
        assert kind != "extend" or self.extend
        self.steps.append((kind, lens))
        out = []
        for e in entries:
            slot, toks = e["slot"], e["tokens"]
            assert self.len[slot] + len(toks) <= self.max_positions
            self.fed[slot] += toks
            self.len[slot] += len(toks)
            if e["want"]:
                out.append((toks[-1] + self.len[slot] - 1) % 50)
        return out


def slot_of(eng, session):
    """The stand-in's slot of a session: sessions take slots in the order they were made."""
    return session._slot


def make(eng, options=None):
    before = set(eng.len)
    s = S.Session(eng, options)
    (s._slot,) = set(eng.len) - before
    return s


def expected(hist):
    return (hist[-1] + len(hist) - 1) % 50


def test_turns_feed_every_token_once():
    eng = FakeEngine()
    s = make(eng, GenOptions(seed=9))
    assert eng.seeds == {s._slot: 9}
    with pytest.raises(S.SessionError, match="empty"):
        s.next()
    s.append([3, 4, 5])
    assert (s.length, s.computed) == (3, 0)
    s.prefill()
    assert (s.length, s.computed) == (3, 2) and eng.steps == [("prefill", [2])]
    for _ in range(3):
        want = expected(s.tokens())
        assert s.next() == (S.OK, want)
    assert (s.length, s.computed) == (6, 5)
    s.append([7, 8])                       # a new turn: the last reply token and the turn
    want = expected(s.tokens())
    assert s.next() == (S.OK, want)
    assert eng.steps[-1] == ("extend", [3])
    assert eng.fed[s._slot] == s.tokens()[:-1]           # every token once, in order
    assert s.stats.new_tokens == 4 and s.stats.prompt_tokens == 2 + 2
    s.close()
    assert eng.pool.n_free == 4
    with pytest.raises(S.SessionError, match="closed"):
        s.next()


def test_a_model_that_cannot_extend_goes_token_by_token():
    eng = FakeEngine(extend=False)
    s = make(eng)
    s.append([1, 2, 3])
    s.next()
    s.append([9, 9, 9])
    want = expected(s.tokens())
    assert s.next() == (S.OK, want)
    assert eng.steps[-4:] == [("decode", [1])] * 4
    assert eng.fed[s._slot] == s.tokens()[:-1]


def test_context_full_and_append_limits():
    eng = FakeEngine(max_positions=6)
    s = make(eng)
    with pytest.raises(S.SessionError, match="vocabulary") as e:
        s.append([50])
    assert e.value.code == -1
    with pytest.raises(S.SessionError, match="fit") as e:
        s.append([1] * 8)
    assert e.value.code == -5                # the reference's EFULL
    assert s.length == 0
    s.append([1] * 4)
    out = [s.next() for _ in range(4)]
    # fed at 4 and 5 after the prompt; the third token has no place to be fed
    assert [st for st, _ in out] == [S.OK, S.OK, S.OK, S.FULL] and out[3][1] is None
    assert s.length == 7 and s.computed == 6


def test_truncate_computes_the_last_kept_token_again():
    for can in (True, False):
        eng = FakeEngine(can_go_back=can)
        s = make(eng)
        s.append([5, 6, 7, 8])
        first = [s.next()[1] for _ in range(3)]
        s.truncate(5)                      # the prompt and the first reply token
        assert s.length == 5 and s.computed == (4 if can else 0)
        assert [s.next()[1] for _ in range(2)] == first[1:]
        assert eng.fed[s._slot] == s.tokens()[:-1]
        s.reset()
        assert (s.length, s.computed) == (0, 0)
        with pytest.raises(S.SessionError):
            s.truncate(1)


def test_sessions_move_on_together():
    eng = FakeEngine()
    a, b, c = make(eng), make(eng), make(eng)
    a.append([1, 2, 3]); b.append([4]); c.append([9] * 39 + [1, 2])
    toks, st = S.sessions_step(eng, [a, b, c])
    assert st == [S.OK, S.OK, S.FULL] and toks[2] is None
    assert toks[:2] == [expected([1, 2, 3]), expected([4])]
    assert eng.steps == [("prefill", [3, 1])]
    a.append([6, 6])                       # a goes on with a turn, b by one token
    toks, st = S.sessions_step(eng, [a, b])
    assert eng.steps[-1] == ("extend", [3, 1])
    assert toks == [expected(a.tokens()[:-1]), expected(b.tokens()[:-1])]
    toks, st = S.sessions_step(eng, [b, a])
    assert eng.steps[-1] == ("decode", [1, 1])
    with pytest.raises(S.SessionError, match="twice"):
        S.sessions_step(eng, [a, a])
    other = make(FakeEngine())
    other.append([1])
    with pytest.raises(S.SessionError, match="another engine"):
        S.sessions_step(eng, [a, other])


def test_sessions_driven_at_random_feed_every_position_once_and_in_order():
    """Appends, tokens asked for alone and together, prefills, truncations and
    resets in random order, on an engine that can append runs of tokens, one that
    cannot, and one whose cache cannot go back part of the way: what the engine was
    fed is always the sequence itself, up to its last token but one."""
    rng = np.random.default_rng(5)
    for kind in range(3):
        eng = FakeEngine(max_positions=60, extend=kind != 1, can_go_back=kind != 2)
        ss = [make(eng) for _ in range(3)]
        for it in range(600):
            s = ss[int(rng.integers(3))]
            op = rng.random()
            if op < 0.3:
                room = eng.max_positions + 1 - s.length
                n = int(rng.integers(1, 9))
                if n <= room:
                    s.append([int(t) for t in rng.integers(0, 50, size=n)])
                else:
                    with pytest.raises(S.SessionError):
                        s.append([1] * n)
            elif op < 0.55 and s.length:
                want = expected(s.tokens())
                full = s.length > eng.max_positions        # the last token has no place to be fed
                assert s.next() == ((S.FULL, None) if full else (S.OK, want))
            elif op < 0.7:
                live = [x for x in ss if x.length]
                if live:
                    wants = [expected(x.tokens()) if x.length <= eng.max_positions else None
                             for x in live]
                    toks, st = S.sessions_step(eng, live)
                    assert toks == wants
            elif op < 0.8 and s.length:
                s.prefill()
                assert s.computed >= s.length - 1
            elif op < 0.95 and s.length:
                s.truncate(int(rng.integers(0, s.length + 1)))
            elif op >= 0.95:
                s.reset()
            for x in ss:
                assert x.computed <= max(x.length - 1, 0) or x.computed == x.length == 0
                assert eng.fed[x._slot] == x.tokens()[:x.computed]
        for x in ss:
            x.close()
        assert eng.pool.n_free == 4
