"""The generation loop's decisions, without a device: which requests form a
batch, when a sequence ends, and the whole loop (the library's, engine/generate.cpp)
over a stand-in for the engine."""
import numpy as np
import pytest

from standin import StandIn

import janas_b200
from janas_b200.engine import generate as G
from janas_b200.engine.generate import (FINISH_CONTEXT, FINISH_LENGTH, FINISH_STOP, GenOptions,
                                        Request, finish_reason, plan_batches, tokens_needed)


def test_tokens_needed():
    assert tokens_needed(1, 1, 1000) == 64          # the last new token is never fed back
    assert tokens_needed(64, 1, 1000) == 64
    assert tokens_needed(64, 2, 1000) == 128
    assert tokens_needed(900, 500, 1000) == 1024    # capped by the context, in whole pages


def test_plan_batches():
    assert plan_batches([10] * 5, [5] * 5, 2, 10_000, 1000) == [[0, 1], [2, 3], [4]]
    # the cache holds 256 tokens: 100+30 -> 192, 10+5 -> 64, then full
    assert plan_batches([100, 10, 10, 200], [30, 5, 5, 20], 8, 256, 1000) == [[0, 1], [2], [3]]
    with pytest.raises(janas_b200.CacheFull, match="need"):
        plan_batches([300], [10], 8, 256, 1000)


def test_finish_reason():
    stops = frozenset([7, 9])
    assert finish_reason(7, 1, 10, 5, 100, stops) == FINISH_STOP
    assert finish_reason(3, 10, 10, 5, 100, stops) == FINISH_LENGTH
    assert finish_reason(9, 10, 10, 5, 100, stops) == FINISH_STOP      # stop wins
    assert finish_reason(3, 2, 10, 100, 100, stops) == FINISH_CONTEXT
    assert finish_reason(3, 2, 10, 99, 100, stops) is None


def test_options():
    assert GenOptions(eos=5, stop=[1, 2]).stop_set() == frozenset([1, 2, 5])
    assert GenOptions().stop_set() == frozenset()
    with pytest.raises(ValueError):
        GenOptions(stop=[1, 2, 3, 4, 5]).validate(100)
    with pytest.raises(ValueError):
        GenOptions(top_p=1.5).validate(100)


class FakeEngine(StandIn):
    """Stands in for the engine: the "model" answers token t with (t + 1) % 50,
    and the bookkeeping of slots is checked as the loop goes."""

    def __init__(self, max_positions=40, max_tokens=64 * 4, max_seqs=3, **kw):
        super().__init__(max_positions, max_tokens, max_seqs, **kw)
        self.steps = []

    def run(self, entries):
        self.steps.append([(e["slot"], len(e["tokens"])) for e in entries])
        out = []
        for e in entries:
            assert self.pool.live(e["slot"])
            assert self.len[e["slot"]] + len(e["tokens"]) <= self.max_positions
            self.len[e["slot"]] += len(e["tokens"])
            if e["want"]:
                out.append((e["tokens"][-1] + 1) % 50)
        return out


def run(monkeypatch, eng, reqs, max_batch=None, **kw):
    """The loop takes as many sequences at a time as the stand-in has free slots."""
    res = G.generate(eng, reqs, **kw)
    assert eng.error is None
    return res


def test_loop_unequal_prompts_stops_and_batches(monkeypatch):
    eng = FakeEngine()
    reqs = [Request([1, 2, 3], 5), Request([10], 3, GenOptions(eos=12)),
            Request([20, 21], 0), Request([30] * 38, 10), Request([5], 2, GenOptions(stop=[6]))]
    st = G.GenStats()
    res = run(monkeypatch, eng, reqs, stats=st)
    assert res[0].tokens == [4, 5, 6, 7, 8] and res[0].finish == FINISH_LENGTH
    assert res[1].tokens == [11, 12] and res[1].finish == FINISH_STOP      # the stop token counts
    assert res[2].tokens == [] and res[2].finish == FINISH_LENGTH
    # 38 prompt tokens, context 40: tokens at 38 and 39 are fed, then the context is full
    assert res[3].tokens == [31, 32, 33] and res[3].finish == FINISH_CONTEXT
    assert res[4].tokens == [6] and res[4].finish == FINISH_STOP
    assert eng.pool.n_free == 3 and not eng.len            # every slot came back
    assert st.batches == 2 and st.new_tokens == 11 and st.prompt_tokens == 3 + 1 + 38 + 1
    # first batch: requests 0, 1 (2 has nothing to do); its second request ends first
    assert [len(s) for s in eng.steps[:5]] == [2, 2, 1, 1, 1]
    assert eng.steps[0] == [(eng.steps[0][0][0], 3), (eng.steps[0][1][0], 1)]


def test_loop_refuses_bad_requests(monkeypatch):
    eng = FakeEngine()
    with pytest.raises(janas_b200.LLMError, match="empty") as e:
        run(monkeypatch, eng, [Request([], 3)])
    assert e.value.code == janas_b200.EINVAL
    with pytest.raises(janas_b200.LLMError, match="context") as e:
        run(monkeypatch, eng, [Request([1] * 41, 3)])
    assert e.value.code == janas_b200.ELIMIT
    assert eng.pool.n_free == 3


class AheadEngine(FakeEngine):
    """A stand-in that also takes steps fed by the step before them, as the real
    engine does from its device buffer; it checks the rules of that way."""

    def __init__(self, *a, **kw):
        super().__init__(*a, ahead=True, **kw)
        self.last = None            # (slots, tokens) of the step begun last
        self.under_way = 0
        self.begun = []             # (slots, fed by the host?)
        self.pending = {}

    def on_free(self, s):
        if self.last is not None and s in self.last[0]:
            self.last = None

    def do_decode_begin(self, a):
        slots, tokens = a["slots"], a["tokens"]
        assert self.under_way < 2
        from_host = tokens is not None
        if tokens is None:
            assert self.last is not None and self.last[0] == list(slots)
            tokens = self.last[1]
        self.begun.append((list(slots), from_host))
        out = []
        for s, t in zip(slots, tokens):
            assert self.pool.live(s)
            assert self.len[s] + 1 <= self.max_positions
            self.len[s] += 1
            out.append((t + 1) % 50)
        self.last = (list(slots), out)
        self.under_way += 1
        key = len(self.begun)
        self.pending[key] = out
        return {"pending": key}

    def do_decode_end(self, a):
        self.under_way -= 1
        return {"tokens": self.pending.pop(a["pending"])}


def test_goes_on_unless_stopped_is_finish_reason_with_the_token_left_open():
    for n in range(1, 6):
        for max_new in range(1, 6):
            for length in range(36, 42):
                want = G.finish_reason(7, n, max_new, length, 40, frozenset()) is None
                assert G.goes_on_unless_stopped(n, max_new, length, 40) == want


def test_loop_one_step_ahead_gives_the_same_results(monkeypatch):
    """With an engine that can feed a step the tokens of the step before it, the
    loop launches one step ahead; results, reasons and counts are those of the
    step-by-step loop, and only a stop token costs a step that was not needed."""
    reqs = [Request([1, 2, 3], 5), Request([10], 3, GenOptions(eos=12)),
            Request([20, 21], 0), Request([30] * 38, 10), Request([5], 2, GenOptions(stop=[6])),
            Request([7], 9, GenOptions(stop=[11])), Request([8, 9], 9)]
    plain_eng, eng = FakeEngine(), AheadEngine()
    st0, st = G.GenStats(), G.GenStats()
    want = run(monkeypatch, plain_eng, reqs, stats=st0)
    res = run(monkeypatch, eng, reqs, stats=st)
    assert [(r.tokens, r.finish) for r in res] == [(r.tokens, r.finish) for r in want]
    assert eng.pool.n_free == 3 and not eng.len and eng.under_way == 0
    assert (st.new_tokens, st.batches, st.prompt_tokens) == \
        (st0.new_tokens, st0.batches, st0.prompt_tokens)
    # request 5, the last of its batch by then, draws its stop token while the step
    # after it is under way: that one step was not needed.  Where others go on, a
    # stopped sequence costs a row of a step that runs anyway.
    assert st.passes == len(eng.begun) == st0.passes + 1
    assert any(not from_host for _, from_host in eng.begun)      # steps were fed on the device


def test_loop_one_step_ahead_on_requests_drawn_at_random(monkeypatch):
    """Many small workloads (prompt lengths, limits, stop tokens, contexts that
    fill up, batches that shrink): with and without steps launched ahead, the same
    tokens and reasons; every slot comes back; at most one step more per batch."""
    rng = np.random.default_rng(2026)
    for case in range(150):
        ctx = int(rng.integers(8, 41))
        reqs = []
        for _ in range(int(rng.integers(1, 8))):
            n = int(rng.integers(1, ctx + 1))
            stop = [int(t) for t in rng.integers(0, 50, size=int(rng.integers(0, 4)))]
            eos = int(rng.integers(0, 50)) if rng.random() < 0.5 else -1
            reqs.append(Request([int(t) for t in rng.integers(0, 50, size=n)],
                                int(rng.integers(0, 12)), GenOptions(eos=eos, stop=stop)))
        max_batch = int(rng.integers(1, 4))
        a = FakeEngine(max_positions=ctx, max_seqs=max_batch)
        b = AheadEngine(max_positions=ctx, max_seqs=max_batch)
        sa, sb = G.GenStats(), G.GenStats()
        want = run(monkeypatch, a, reqs, stats=sa)
        got = run(monkeypatch, b, reqs, stats=sb)
        assert [(r.tokens, r.finish) for r in got] == [(r.tokens, r.finish) for r in want], case
        assert b.pool.n_free == max_batch and not b.len and b.under_way == 0
        a.close(); b.close()
        assert sb.new_tokens == sa.new_tokens and sb.batches == sa.batches
        assert sa.passes <= sb.passes <= sa.passes + sa.batches


def test_batches_are_planned_against_what_is_free_now(monkeypatch):
    """Slots and pages held by others (open sessions, a caller's own slots) are not
    the loop's to plan with: it cuts batches by the free slots and the free tokens of
    the moment, and with nothing free it fails as a full cache before taking anything."""
    import ctypes
    from janas_b200 import lib
    eng = FakeEngine(max_seqs=3)
    held = ctypes.c_int32()
    lib.check(lib.lib().jb_llm_slot_new(eng._h, ctypes.byref(held)))       # someone holds a slot
    reqs = [Request([1, 2], 3), Request([3], 3), Request([4, 5, 6], 3)]
    st = G.GenStats()
    res = run(monkeypatch, eng, reqs, stats=st)
    assert [r.tokens for r in res] == [[3, 4, 5], [4, 5, 6], [7, 8, 9]]
    assert st.batches == 2 and [len(s) for s in eng.steps[:1]] == [2]      # two at a time, not three
    assert eng.pool.n_free == 2 and eng.pool.live(held.value)              # the held slot is untouched
    eng.max_tokens = 64                                                    # room for one sequence
    st = G.GenStats()
    run(monkeypatch, eng, reqs, stats=st)
    assert st.batches == 3
    eng.max_tokens = 0
    with pytest.raises(janas_b200.CacheFull):
        run(monkeypatch, eng, reqs)
    eng.max_tokens = 256
    others = [ctypes.c_int32(), ctypes.c_int32()]
    for o in others:
        lib.check(lib.lib().jb_llm_slot_new(eng._h, ctypes.byref(o)))
    with pytest.raises(janas_b200.CacheFull) as e:                         # no slot is free
        run(monkeypatch, eng, reqs)
    assert e.value.code == janas_b200.EFULL
    assert eng.pool.n_free == 0
    for o in [held] + others:
        lib.check(lib.lib().jb_llm_slot_free(eng._h, o.value))
    assert eng.pool.n_free == 3 and not eng.len
