"""Requests drawn at random, generated in batches of whatever else is there, with
sessions that hold slots and pages in between: in float32 every request's tokens
are exactly those it gets when it is generated alone, and the cache's books stay
right (no slot or page lost, held twice or freed twice)."""
import numpy as np
import pytest

from helpers import model_dir
from tiny import TINY, tokens

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name", ["A", "C"])
def test_random_batches_give_every_request_the_tokens_it_gets_alone(name):
    import janas_b200
    rng = np.random.default_rng(5)
    vocab = TINY[name]["vocab_size"]
    llm = janas_b200.open(model_dir(name), janas_b200.LLMParams(
        n_ctx=256, dtype="float32", max_batch=6, max_tokens=6 * 256))
    alone = {}

    def solo(p, n, eos):
        key = (tuple(p), n, eos)
        if key not in alone:
            alone[key] = llm.generate_batch([p], n, [janas_b200.GenOptions(eos=eos)])[0][0]
        return alone[key]

    sessions, checked = [], 0
    for _ in range(40):
        n_req = int(rng.integers(1, 15))                # often more than one batch holds
        ps = [tokens(rng, int(rng.integers(1, 120)), vocab) for _ in range(n_req)]
        n_new = int(rng.integers(1, 40))
        eos = [int(rng.integers(0, vocab)) if rng.random() < 0.5 else -1 for _ in range(n_req)]
        if rng.random() < 0.3 and len(sessions) < 3:    # a session that holds a slot and pages
            s = llm.session()
            s.append(tokens(rng, int(rng.integers(1, 60)), vocab))
            s.prefill()
            sessions.append(s)
        if rng.random() < 0.2 and sessions:
            sessions.pop(int(rng.integers(0, len(sessions)))).close()
        outs, _ = llm.generate_batch(ps, n_new, [janas_b200.GenOptions(eos=e) for e in eos])
        for p, o, e in zip(ps, outs, eos):
            assert o == solo(p, n_new, e)
            checked += 1
        llm.engine.cache.check()
    for s in sessions:
        s.close()
    llm.engine.cache.check()
    assert checked > 200
    llm.close()
