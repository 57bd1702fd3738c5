"""The engine at the layer sizes of Qwen3-4B (hidden 2560, 32 heads in 8 groups of
head size 128, feed-forward 9728; 2 of its 36 layers, a vocabulary of 40,003 so that
the head's product runs in several waves and ends in a ragged tile) under the three
ways of cutting the work, in 32-bit and in bfloat16: each request alone and whole;
with its last 32 tokens one by one; in unequal batches, one after another in a cache
with room for one.  The tiny configurations of the other tests reach neither the
many-token tiles of the tensor-core product, nor prefill attention over more than
three chunks, nor the norm's sum over a dozen partial sums; these sizes do.

The reference checks the same on its real model: blocks against token by token
(tests/llm_eval.c:169-232) and alone against batched (tests/multiseq_check.c:143-232).

The plain implementation computes every row of every request (one pass per request
on the host) but the logits of sampled positions only: the first and last, the
edges of pages and chunks, and a few drawn at random.
"""
import numpy as np
import pytest
import torch

import plain_qwen3 as plain
from helpers import rel_err, run_trace, trace_batches

pytestmark = pytest.mark.gpu

WIDE = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=2,
    hidden_size=2560, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
    intermediate_size=9728, vocab_size=40003, rope_theta=1e6, rms_norm_eps=1e-6,
    tie_word_embeddings=True, max_position_embeddings=8192)
LENGTHS = [40, 300, 1100, 2048]

# Largest |difference| over the largest |logit| of a request's compared rows,
# measured on a B200 (the figures in the comments), with a factor of about three.
FP32_TOL = 2e-5            # 32-bit engine against the plain model: 5.1e-6 (sums of 9,728 terms in another order)
FP32_CUT_TOL = 0.0         # 32-bit engine, another cut: the same bits
BF16_TOL = 3e-2            # bfloat16 engine against the 32-bit engine: 9.7e-3
BF16_PLAIN_TOL = 2.5e-2    # bfloat16 engine against the plain model that rounds at the same places: 7.7e-3
BF16_CUT_TOL = 2.5e-2      # bfloat16 engine, another cut (other tiles, other partial sums): 8.0e-3

_STATE = {}


def folder():
    if "dir" not in _STATE:
        import tempfile
        from janas_b200.config import config_from_dict
        from janas_b200.weights import write_random_model
        d = tempfile.mkdtemp(prefix="janas_b200_wide_")
        write_random_model(d, config_from_dict(WIDE), 7)
        _STATE["dir"] = d
    return _STATE["dir"]


def requests():
    rng = np.random.default_rng(77)
    return [rng.integers(0, WIDE["vocab_size"], size=n).tolist() for n in LENGTHS]


def rows_of(n):
    """Positions of a request of n tokens whose logits are compared."""
    rng = np.random.default_rng(n)
    edges = [0, 1, 63, 64, 65, 127, 128, 129, 255, 256, 1023, 1024, 1025, 2047]
    rows = {r for r in edges if r < n} | {n - 1} | set(range(max(0, n - 32), n))
    rows |= {int(r) for r in rng.integers(0, n, size=8)}
    return sorted(rows)


def plain_rows(i, rounding=None):
    key = ("plain", i, rounding)
    if key not in _STATE:
        if "weights" not in _STATE:
            _STATE["weights"] = (plain.read_config(folder()), plain.read_weights(folder()))
        c, w = _STATE["weights"]
        toks = requests()[i]
        torch.set_num_threads(8)        # 1.4 TFLOP in all; the comparisons here leave room for
        try:                            # what the order of a library's sums may differ by
            _STATE[key] = plain.forward(c, w, toks, rounding, rows=rows_of(len(toks))).numpy()
        finally:
            torch.set_num_threads(1)
    return _STATE[key]


def engine(dtype, max_tokens=2048 + 64, max_seqs=1):
    from janas_b200.engine import Engine
    return Engine.open(folder(), dtype=dtype, max_tokens=max_tokens, max_seqs=max_seqs, n_ctx=8192)


def whole(eng):
    """Each request alone and whole: {request: logits of its compared rows}."""
    from janas_b200.engine import StepEntry
    out = {}
    for i, toks in enumerate(requests()):
        s = eng.new_sequence()
        out[i] = eng.step_numpy([StepEntry(s, toks, rows_of(len(toks)))])
        eng.free_sequence(s)
    return out


def tail(eng, last=32):
    """All but the last 32 tokens in one step, then those one by one."""
    from janas_b200.engine import StepEntry
    out = {}
    for i, toks in enumerate(requests()):
        n = len(toks)
        head = max(1, n - last)
        rows = rows_of(n)
        s = eng.new_sequence()
        got = {}
        first = eng.step_numpy([StepEntry(s, toks[:head], [r for r in rows if r < head])])
        for r, lg in zip([r for r in rows if r < head], first):
            got[r] = lg
        for p in range(head, n):
            got[p] = eng.step_numpy([StepEntry(s, [toks[p]], [0])])[0]
        eng.free_sequence(s)
        out[i] = np.stack([got[r] for r in rows])
    return out


def batched(dtype):
    """Two batches of unequal requests (prompts of 30, 250, 1000 and 1900 tokens,
    the rest of each request one token a step, the shorter ones ending earlier), one
    after the other in a cache that holds one batch: the second uses again what the
    first gave back."""
    reqs = requests()
    prompts = [30, 250, 1000, 1900]
    batches = [[(reqs[0], prompts[0]), (reqs[3], prompts[3])], [(reqs[2], prompts[2]), (reqs[1], prompts[1])]]
    ids = {0: "b0r0", 3: "b0r1", 2: "b1r0", 1: "b1r1"}
    need = max(sum((len(t) + 63) // 64 * 64 for t, _ in b) for b in batches)
    eng = engine(dtype, max_tokens=need, max_seqs=2)
    got = run_trace(eng, trace_batches(batches, want_prompt_all=False))
    eng.cache.check()
    assert eng.cache.tokens_held() == 0
    eng.check()
    eng.close()
    out = {}
    for i, rid in ids.items():
        # compared: the prompt's last row and every row that came one by one
        rows = [r for r in rows_of(len(reqs[i])) if r >= prompts[i] - 1]
        out[i] = (rows, np.stack([got[rid][r] for r in rows]))
    return out


def pick(full_rows, logits, rows):
    at = {r: k for k, r in enumerate(full_rows)}
    return np.stack([logits[at[r]] for r in rows])


@pytest.fixture(scope="module")
def runs():
    """Every way of cutting, once per dtype."""
    r = {}
    for dtype in ("float32", "bfloat16"):
        eng = engine(dtype)
        r[dtype, "whole"] = whole(eng)
        r[dtype, "tail"] = tail(eng)
        eng.cache.check()
        assert eng.cache.tokens_held() == 0
        eng.check()                 # no tensor-core wait ran out on the way
        eng.close()
        r[dtype, "batched"] = batched(dtype)
    return r


def test_float32_whole_requests_equal_the_plain_model(runs):
    worst = 0.0
    for i in range(len(LENGTHS)):
        e = rel_err(runs["float32", "whole"][i], plain_rows(i))
        worst = max(worst, e)
        assert e <= FP32_TOL, f"request {i} ({LENGTHS[i]} tokens): {e:.3e}"
    print(f"float32 against plain: {worst:.3e}")


def test_float32_is_the_same_bits_however_the_work_is_cut(runs):
    for i, n in enumerate(LENGTHS):
        a = runs["float32", "whole"][i]
        assert rel_err(runs["float32", "tail"][i], a) <= FP32_CUT_TOL, f"request {i}: tail"
        rows, b = runs["float32", "batched"][i]
        assert rel_err(b, pick(rows_of(n), a, rows)) <= FP32_CUT_TOL, f"request {i}: batched"


def test_bfloat16_whole_requests(runs):
    w32, wp = 0.0, 0.0
    for i in range(len(LENGTHS)):
        e = rel_err(runs["bfloat16", "whole"][i], runs["float32", "whole"][i])
        w32 = max(w32, e)
        assert e <= BF16_TOL, f"request {i} ({LENGTHS[i]} tokens) against 32-bit: {e:.3e}"
    for i in (0, 1, 3):
        e = rel_err(runs["bfloat16", "whole"][i], plain_rows(i, "bfloat16"))
        wp = max(wp, e)
        assert e <= BF16_PLAIN_TOL, f"request {i} against the plain model that rounds: {e:.3e}"
    print(f"bfloat16 against float32: {w32:.3e}; against plain with rounding: {wp:.3e}")


def test_bfloat16_under_other_cuts(runs):
    worst = 0.0
    for i, n in enumerate(LENGTHS):
        a = runs["bfloat16", "whole"][i]
        e = rel_err(runs["bfloat16", "tail"][i], a)
        rows, b = runs["bfloat16", "batched"][i]
        e2 = rel_err(b, pick(rows_of(n), a, rows))
        worst = max(worst, e, e2)
        assert e <= BF16_CUT_TOL, f"request {i}: tail {e:.3e}"
        assert e2 <= BF16_CUT_TOL, f"request {i}: batched {e2:.3e}"
        # and the other cuts against the 32-bit engine too
        assert rel_err(runs["bfloat16", "tail"][i], runs["float32", "whole"][i]) <= BF16_TOL
    print(f"bfloat16, other cuts against whole: {worst:.3e}")


# ------------------------------------------------------------------ the products' tiles
@pytest.mark.parametrize("tile", [128, 160, 192, 224, 256])
def test_every_tile_width_of_the_many_token_product(tile):
    """Each of the five token-tile widths of the tensor-core product over many
    tokens, forced, for the plain product (with k cut in two as well) and for the
    fused gate-up-SwiGLU product; the library says which width ran."""
    from janas_b200.csrc import ops
    L = ops.lib()
    g = torch.Generator().manual_seed(tile)
    n, m, k = 600, 1100, 2560
    a = (torch.randn(n, k, generator=g) * 0.5).bfloat16()
    w = (torch.randn(m, k, generator=g) * 0.05).bfloat16()
    gu = (torch.randn(2 * 640, k, generator=g) * 0.05).bfloat16()
    want = a.float() @ w.float().T
    z = a.float() @ gu.float().T
    want_act = (z[:, :640] / (1 + torch.exp(-z[:, :640])) * z[:, 640:])
    assert L.jb_gemm_tc_force_tile(tile) == 0
    try:
        for splits in (1, 2):
            got = ops.linear(a.cuda(), w.cuda(), splits=splits).sum(0).cpu()
            assert L.jb_gemm_tc_last_tile() == tile
            assert (got - want).abs().max() <= 2e-3 * want.abs().max()
        act = ops.linear_swiglu(a.cuda(), gu.cuda()).float().cpu()
        assert L.jb_gemm_tc_last_tile() == tile
        assert (act - want_act).abs().max() <= 2 ** -7 * want_act.abs().max()
    finally:
        L.jb_gemm_tc_force_tile(0)
    assert ops.gemm_tc_error() == 0
    assert L.jb_gemm_tc_force_tile(100) == -1


# ------------------------------------------------------------------ long prefill attention
def attention_rows(q, k, v, rows):
    """Causal GQA attention for the sampled rows of one sequence, row by row: head h
    reads KV head h / (heads / kv_heads), scores (q . k) / sqrt(head size), weights
    exp(s - max) over their sum (src/llm/attention.c:574-588,874-875,1012)."""
    n, nh, hd = q.shape
    group = nh // k.shape[1]
    out = torch.zeros(len(rows), nh, hd, dtype=torch.float64)
    for i, r in enumerate(rows):
        for h in range(nh):
            s = (k[:r + 1, h // group].double() @ q[r, h].double()) / np.sqrt(hd)
            wgt = torch.exp(s - s.max())
            out[i, h] = (wgt[:, None] * v[:r + 1, h // group].double()).sum(0) / wgt.sum()
    return out.float()


@pytest.mark.parametrize("n", [2048, 8192])
def test_prefill_attention_over_many_chunks(n):
    """The tensor-core prefill attention at 32 heads in 8 groups of 128 values over
    2,048 and 8,192 positions (16 and 64 chunks of keys), against the formula on
    sampled rows; one query and one key far back are scaled so that a far key's
    weight stands out among thousands."""
    from janas_b200.csrc import ops
    nh, nkv, hd = 32, 8, 128
    g = torch.Generator().manual_seed(n)
    q = torch.randn(n, nh, hd, generator=g).bfloat16()
    k = torch.randn(n, nkv, hd, generator=g).bfloat16()
    v = torch.randn(n, nkv, hd, generator=g).bfloat16()
    far, near = 5, n - 3
    k[far] = q[near, ::4]                 # every group's first head finds position 5: score sqrt(128) there
    pages = (n + 63) // 64
    kc = torch.zeros(pages, nkv, 64, hd, dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    perm = torch.randperm(pages, generator=g)             # the sequence's pages lie scattered
    for p in range(pages):
        a, b = p * 64, min(n, p * 64 + 64)
        kc[perm[p], :, :b - a] = k[a:b].transpose(0, 1)
        vc[perm[p], :, :b - a] = v[a:b].transpose(0, 1)
    bt = perm.to(torch.int32)[None, :].contiguous()
    pad = (-bt.shape[1]) % 8
    if pad:
        bt = torch.cat([bt, torch.full((1, pad), -1, dtype=torch.int32)], dim=1)
    pos = torch.arange(n, dtype=torch.int32)
    seq = torch.zeros(n, dtype=torch.int32)
    per = ops.attention_block_positions(nh, nkv)
    blocks = ops.attention_blocks(np.array([0]), np.array([0]), np.array([n]), per, torch.device("cuda:0"))
    chunks = (n - 1) // ops.attention_chunk() + 1
    got = ops.attention(q.cuda(), kc.cuda(), vc.cuda(), pos.cuda(), seq.cuda(), bt.cuda(), 0,
                        1.0 / np.sqrt(hd), chunks, blocks=blocks).float().cpu()
    assert ops.attn_tc_error() == 0
    rng = np.random.default_rng(n)
    rows = sorted({0, 1, 127, 128, 129, n // 2, near, n - 1} | {int(r) for r in rng.integers(0, n, size=6)})
    want = attention_rows(q.float(), k.float(), v.float(), rows)
    err = (got[rows] - want).abs().max()
    assert err <= 2e-2 * want.abs().max(), float(err / want.abs().max())
    # the far key carries most of that row's weight: leaving it out would be seen
    wrong = attention_rows(q.float(), torch.cat([k[:far], k[far:far + 1] * 0, k[far + 1:]]).float(), v.float(), [near])
    assert (wrong - want[rows.index(near)]).abs().max() > 0.2 * want.abs().max()
