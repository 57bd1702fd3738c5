"""The plain implementation itself (no GPU): against vectors computed by the
reference's own C code where that compiles alone (tests/golden), and against
its own invariants."""
import json
import os

import numpy as np
import pytest
import torch

import plain_qwen3 as plain
from helpers import plain_logits, plain_model
from tiny import TINY, tokens

GOLDEN = json.load(open(os.path.join(os.path.dirname(__file__), "golden",
                                     "reference_vectors.json")))


class LCG:
    """The generator of tests/golden/make_golden.py's driver."""

    def __init__(self, seed):
        self.s = seed

    def next(self):
        self.s = (self.s * 6364136223846793005 + 1442695040888963407) & ((1 << 64) - 1)
        return float(self.s >> 11) * (1.0 / 9007199254740992.0)


def golden_rows():
    g = LCG(12345)
    rows = np.zeros((12, 300), dtype=np.float32)
    for r in range(12):
        for i in range(300):
            rows[r, i] = np.float32((g.next() - 0.5) * 8.0)
    rows[3, 17] = rows[3, 5] = 6.0
    rows[4, 100] = rows[4, 101] = rows[4, 102] = 3.5
    return rows


SETTINGS = [(0.0, 0, 0.0, 0.0, 1), (0.8, 20, 0.8, 0.0, 1), (0.7, 0, 0.0, 0.0, 7),
            (1.0, 5, 0.0, 0.0, 42), (1.5, 0, 0.9, 0.05, 3), (0.3, 50, 1.0, 0.2, 99),
            (2.0, 3, 0.5, 0.0, 18446744073709551615)]


def test_sampler_matches_the_reference_sampler():
    rows = golden_rows()
    for (t, k, p, mp, seed), want in zip(SETTINGS, GOLDEN["sampler"]):
        rng, got = seed, []
        for rep in range(3):
            for r in range(12):
                tok, rng = plain.sample(rows[r], t, k, p, mp, rng)
                got.append(tok)
        assert got == want, (t, k, p, mp, seed)


def test_rope_angles_match_the_reference_math():
    bases, nrot = [10000.0, 1000000.0, 50000.0], [16, 32, 128]
    for b, pos, i, cs, sn in GOLDEN["rope"]:
        c, s = plain.rope_table([pos], nrot[b], bases[b])
        assert abs(float(c[0, i]) - cs) <= 1e-7 and abs(float(s[0, i]) - sn) <= 1e-7, (b, pos, i)


def test_silu_matches_the_reference_math():
    g = LCG(777)
    for want in GOLDEN["silu_mul"]:
        a = np.float32((g.next() - 0.5) * 24.0)
        u = np.float32((g.next() - 0.5) * 4.0)
        x = torch.tensor([a], dtype=torch.float32)
        got = float((x / (1.0 + torch.exp(-x)) * float(u))[0])
        assert abs(got - want) <= 2e-6 * max(1.0, abs(want))


def test_rms_norm_matches_the_reference_norm():
    """plain.rms_norm against the reference's rms_norm (an inline function of its
    model header, compiled alone): bit for bit, or within one unit in the last
    place where the square root's rounding differs."""
    for case in GOLDEN["rms_norm"]:
        n, step = case["n"], case["step"]
        g = LCG(case["seed"])
        x, w = np.zeros(n, dtype=np.float32), np.zeros(n, dtype=np.float32)
        for i in range(n):
            x[i] = np.float32((g.next() - 0.5) * 8.0)
            w[i] = np.float32(1.0 + (g.next() - 0.5) * 0.4)
        got = plain.rms_norm(torch.from_numpy(x), torch.from_numpy(w),
                             float(np.float32(case["eps"]))).numpy()[::step]
        want = np.asarray(case["out"], dtype=np.float32)
        assert got.shape == want.shape
        assert np.abs(got - want).max() <= 2.0 ** -23 * np.abs(want).max(), n


def test_attention_matches_the_reference_attention():
    """plain.attention against the reference's own attention code (janas_attn_run
    with float scores, compiled alone: tests/golden/make_golden.py) on keys and
    values that its eight-bit cache holds exactly: grouped heads of 16, 48 and 128
    values, sequences run in blocks of 50 tokens, rows at the blocks' and the
    windows' edges."""
    for case in GOLDEN["attention"]:
        nh, nkv, hd, n, window = (case[k] for k in ("nh", "nkv", "hd", "n", "window"))
        g = LCG(case["seed"])
        q = np.array([np.float32((g.next() - 0.5) * 4.0) for _ in range(n * nh * hd)],
                     dtype=np.float32).reshape(n, nh, hd)
        k = np.zeros((n, nkv, hd), dtype=np.float32)
        v = np.zeros((n, nkv, hd), dtype=np.float32)
        for h in range(nkv):
            for t in range(n):
                ks = np.float32(0.004 + 0.008 * g.next())
                vs = np.float32(0.004 + 0.008 * g.next())
                for d in range(hd):
                    k[t, h, d] = np.float32(int(g.next() * 255.0) - 127) * ks
                    v[t, h, d] = np.float32(int(g.next() * 255.0) - 127) * vs
        out = plain.attention(torch.from_numpy(q), torch.from_numpy(k), torch.from_numpy(v), window)
        step = hd // 16
        for row, want in case["rows"].items():
            want = np.asarray(want, dtype=np.float64).reshape(nh, 16)
            got = out[int(row)].double().numpy()[:, ::step]
            err = np.abs(got - want).max() / np.abs(want).max()
            assert err <= 2e-6, (nh, nkv, hd, window, row, err)
        if window:      # the window does matter at the rows that were compared
            full = plain.attention(torch.from_numpy(q), torch.from_numpy(k), torch.from_numpy(v), 0)
            last = max(int(r) for r in case["rows"])
            assert (full[last] - out[last]).abs().max() > 1e-3


def test_whole_model_against_the_reference_model_code():
    """plain.forward against the logits that the reference's own forward pass wrote
    for a tiny random Qwen3 (tests/golden/make_model_golden.py: its tools, run on a
    CPU, on weights that its eight-bit type holds exactly).  The reference rounds
    activations and cached keys and values to eight bits, so the two agree to a few
    hundredths of the largest logit, not more.  That is enough to tell the structure:
    the same comparison with two norms' weights exchanged, gate and up exchanged,
    another rotation base or the KV heads paired the other way is off by ten times
    as much and more."""
    golden = os.path.join(os.path.dirname(__file__), "golden")
    import importlib.util
    spec = importlib.util.spec_from_file_location("tiny_q8_model",
                                                  os.path.join(golden, "tiny_q8_model.py"))
    tiny = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(tiny)
    ref = json.load(open(os.path.join(golden, "reference_model_logits.json")))
    pos = ref["positions"]
    want = np.asarray(ref["logits"], dtype=np.float32)
    c = dict(tiny.CONFIG)
    w = {h: torch.from_numpy(a.copy()) for _, h, a, _, _ in tiny.tensors()}

    def off(config, weights):
        got = plain.forward(config, weights, tiny.TOKENS).numpy()[pos]
        return got, np.abs(got - want).max(axis=1) / np.abs(want).max(axis=1)

    got, err = off(c, w)
    assert err.max() <= 6e-2 and err.mean() <= 4e-2, err
    assert np.corrcoef(got.ravel(), want.ravel())[0, 1] >= 0.999
    assert (got.argmax(1) == want.argmax(1)).mean() >= 0.75

    def exchanged(a, b):
        wrong = dict(w)
        for l in range(c["num_hidden_layers"]):
            x, y = f"model.layers.{l}.{a}", f"model.layers.{l}.{b}"
            wrong[x], wrong[y] = w[y], w[x]
        return off(c, wrong)[1]

    late = [i for i, p in enumerate(pos) if p >= 7]        # rows that see several positions
    assert exchanged("self_attn.q_norm.weight", "self_attn.k_norm.weight")[late].min() >= 0.2
    assert exchanged("input_layernorm.weight", "post_attention_layernorm.weight").min() >= 0.5
    assert exchanged("mlp.gate_proj.weight", "mlp.up_proj.weight").min() >= 0.5
    assert off(dict(c, rope_theta=1e6), w)[1][late].min() >= 0.25
    wrong = dict(w)
    half = c["head_dim"]
    for l in range(c["num_hidden_layers"]):
        k = f"model.layers.{l}.self_attn.k_proj.weight"
        wrong[k] = torch.cat([w[k][half:], w[k][:half]])          # the two KV heads exchanged
    assert off(c, wrong)[1][1:].min() >= 0.5


def test_splitmix_and_greedy():
    s, z = plain.splitmix64(0)
    assert (s, z) == (0x9E3779B97F4A7C15, 0xE220A8397B1DCDAF)     # the published first output
    row = np.array([1.0, 5.0, 5.0, -2.0], dtype=np.float32)
    assert plain.sample(row, 0.0, 0, 0, 0, 5) == (1, 5)            # first maximum, state untouched
    a = [plain.sample(row, 1.0, 0, 0, 0, 9)[0] for _ in range(3)]
    assert len(set(a)) == 1                                          # same seed, same draw


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_a_prefix_has_the_same_logits(name):
    rng = np.random.default_rng(3)
    toks = tokens(rng, 90, TINY[name]["vocab_size"])
    whole = plain_logits(name, toks)
    part = plain_logits(name, toks[:41])
    assert np.abs(whole[:41] - part).max() <= 1e-5


def test_window_hides_old_positions():
    """With a window of 37, changing token 0 must not change the top layers' view
    beyond what the full layers carry; with all layers windowed it changes nothing."""
    c, w = plain_model("C")
    c2 = dict(c, layer_types=["sliding_attention"] * 4)
    rng = np.random.default_rng(4)
    toks = tokens(rng, 120, c["vocab_size"])
    other = [(toks[0] + 1) % c["vocab_size"]] + toks[1:]
    a = plain.forward(c2, w, toks).numpy()
    b = plain.forward(c2, w, other).numpy()
    # 4 layers of window 37 reach back 4 * 36 = 144 positions at most: position 119
    # is reached; so cut the reach with a window of 20: 4 * 19 = 76 < 119
    c3 = dict(c2, sliding_window=20)
    a = plain.forward(c3, w, toks).numpy()
    b = plain.forward(c3, w, other).numpy()
    assert np.abs(a[0] - b[0]).max() > 1e-4
    assert np.abs(a[100:] - b[100:]).max() == 0.0


def test_attention_picks_the_key_that_stands_out():
    n, hd = 50, 16
    q = torch.zeros(n, 2, hd)
    k = torch.zeros(n, 1, hd)
    v = torch.randn(n, 1, hd)
    q[:, :, 0] = 40.0
    k[7, 0, 0] = 40.0          # one score of 400 among zeros
    out = plain.attention(q, k, v, 0)
    assert torch.allclose(out[30, 1], v[7, 0], atol=1e-6)
    assert torch.allclose(out[3, 0], v[:4, 0].mean(0), atol=1e-6)    # before it: uniform
    win = plain.attention(q, k, v, 10)
    assert torch.allclose(win[30, 0], v[21:31, 0].mean(0), atol=1e-6)  # outside the window
    assert torch.allclose(win[16, 0], v[7, 0], atol=1e-6)               # its edge: 16 + 1 - 10 = 7
