"""Failures that must be seen, not survived in silence: a kernel's bounded wait that
runs out, a sampler row that needs more room than the short way has, a captured
decode step replayed after the temporaries' pool has grown."""
import numpy as np
import pytest
import torch

import plain_qwen3 as plain
from helpers import model_dir, plain_model
from tiny import TINY, tokens

pytestmark = pytest.mark.gpu


def test_a_bounded_wait_that_runs_out_is_reported_and_cleared():
    """A kernel waits, with the tensor-core products' own wait and a limit of a
    millisecond, on a barrier that nothing ever arrives at.  It returns, leaves its
    code in the products' error word, and harms nothing: the word reads 9 once and 0
    after; an open engine reports the failure as EFAIL at its next check and is
    usable again after it; the next product is right.  (No kernel of the library
    waits without a limit, and nothing here faults.)"""
    import janas_b200
    from janas_b200 import lib
    from janas_b200.csrc import ops
    assert ops.gemm_tc_error() == 0
    assert lib.call("kernels.wait_selftest", limit_cycles=2_000_000)["code"] == 0
    assert ops.gemm_tc_error() == 9
    assert ops.gemm_tc_error() == 0          # reading clears it

    m = janas_b200.open(model_dir("D"), janas_b200.LLMParams(n_ctx=128, max_batch=2, max_tokens=256))
    first, _ = m.generate([5, 6, 7], 4)
    assert lib.call("kernels.wait_selftest", limit_cycles=2_000_000)["code"] == 0
    with pytest.raises(janas_b200.LLMError) as e:
        m.generate([5, 6, 7], 4)             # the loop checks where it has the tokens anyway
    assert e.value.code == janas_b200.EFAIL and "code 9" in str(e.value)
    again, _ = m.generate([5, 6, 7], 4)      # the word is clear again, the engine as before
    assert again == first
    m.engine.cache.check()
    assert m.engine.cache.tokens_held() == 0
    m.close()

    a = (torch.randn(40, 256) * 0.3).bfloat16()
    w = (torch.randn(300, 256) * 0.1).bfloat16()
    got = ops.linear(a.cuda(), w.cuda()).sum(0).cpu()
    want = a.float() @ w.float().T
    assert (got - want).abs().max() <= 2e-3 * want.abs().max() and ops.gemm_tc_error() == 0


def test_the_sampler_says_when_a_row_needs_the_long_way():
    from janas_b200.csrc import ops
    L = ops.lib()
    assert L.jb_sample_needs_big(151936, 20) == 0
    assert L.jb_sample_needs_big(151936, 0) == 1 and L.jb_sample_needs_big(151936, 65) == 1
    assert L.jb_sample_needs_big(262144, 64) == 0
    assert L.jb_sample_needs_big(262145, 20) == 1      # more chunks than the merge holds
    assert L.jb_sample_needs_big(10, 20) == 1          # top_k not below the vocabulary
    # the kernel's own answer for such a row without scratch is -1, never a wrong token
    V = 300_000
    logits = torch.randn(2, V, device="cuda")
    temp = torch.full((2,), 0.8, device="cuda")
    topk = torch.full((2,), 20, dtype=torch.int32, device="cuda")
    z = torch.zeros(2, device="cuda")
    rng = torch.zeros(2, dtype=torch.int64, device="cuda")
    out = ops.sample(logits, temperature=temp, top_k=topk, top_p=z, min_p=z, rng=rng)
    assert out.tolist() == [-1, -1]


def test_a_vocabulary_beyond_the_short_way_samples_through_the_graph():
    """300,000 tokens: with top_k 20 every row still needs all its candidates sorted
    (its 74 chunks' lists do not fit the merge).  The engine sees that from the
    vocabulary, gives the sampler its scratch inside the captured decode step, and
    draws the plain sampler's tokens."""
    import tempfile
    import janas_b200
    from janas_b200.config import config_from_dict
    from janas_b200.weights import write_random_model
    cfg = dict(TINY["A"], vocab_size=300_000, num_hidden_layers=1)
    with tempfile.TemporaryDirectory() as d:
        write_random_model(d, config_from_dict(cfg), 3)
        c, w = plain.read_config(d), plain.read_weights(d)
        m = janas_b200.open(d, janas_b200.LLMParams(n_ctx=64, dtype="float32", max_batch=2,
                                                    max_tokens=128))
        rng = np.random.default_rng(1)
        ps = [tokens(rng, 5, 300_000), tokens(rng, 2, 300_000)]
        opts = [janas_b200.GenOptions(temperature=0.8, top_k=20, seed=4 + i) for i in range(2)]
        assert m.engine.use_graphs
        outs, st = m.generate_batch(ps, 5, opts)
        assert m.engine.n_graphs >= 1
        for i, (p, o) in enumerate(zip(ps, outs)):
            assert all(0 <= t < 300_000 for t in o)
            assert o == plain.generate(c, w, p, 5, temperature=0.8, top_k=20, seed=4 + i)
        # and through sessions, which choose the way per step
        s = m.session(opts[0])
        s.append(ps[0])
        assert [s.next()[1] for _ in range(5)] == outs[0]
        s.close()
        m.close()


def test_captured_steps_stay_right_after_the_temporaries_grow():
    """A decode step is captured while the pool of temporaries is small; then a long
    prompt makes the pool take much more; then the captured step is replayed.  The
    pool keeps every buffer it ever handed out while captured steps exist, so the
    replay's addresses are still its own: the same tokens as before."""
    import janas_b200
    rng = np.random.default_rng(8)
    v = TINY["E"]["vocab_size"]
    for dtype in ("float32", "bfloat16"):
        m = janas_b200.open(model_dir("E"), janas_b200.LLMParams(n_ctx=640, dtype=dtype, max_batch=3,
                                                                 max_tokens=2048))
        ps = [tokens(rng, n, v) for n in (9, 30)]
        first, _ = m.generate_batch(ps, 12)
        graphs = m.engine.n_graphs
        before = m.engine.info()["pool_bytes"]
        long_out, _ = m.generate([int(t) for t in rng.integers(0, v, size=600)], 3)
        assert m.engine.info()["pool_bytes"] > before
        again, _ = m.generate_batch(ps, 12)
        assert again == first
        assert m.engine.n_graphs >= graphs
        m.engine.check()
        m.close()
