"""Each part of a layer alone, built from a PartSpec through the registry, and
a model put together from parts that are not Qwen3's: a toy mixer with state of
its own, a layer that runs twice, a layer that reads another layer's cache, a
layer without position encoding.  None of this changes a file of the framework.
"""
import math
from typing import Dict, Mapping, Optional

import numpy as np
import pytest
import torch

import plain_qwen3 as plain

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


def build(role, spec, dtype=torch.float32):
    from janas_b200.parts import build_part
    return build_part(role, spec, dtype, DEV)


def give(part, prefix, seed=0, dtype=torch.float32):
    """Random tensors for a part, loaded; returns them as float32 on the host."""
    from janas_b200.weights import random_tensors
    ts = {n: t for n, t in random_tensors(part.tensors(prefix), seed, dtype)}
    part.load(prefix, {n: t.to(DEV) for n, t in ts.items()})
    return {n: t.float() for n, t in ts.items()}


def context(pos0s, lens, dtype=torch.float32):
    from janas_b200.parts import DECODE, EXTEND, PREFILL, StepContext
    pos0, lens = np.asarray(pos0s), np.asarray(lens)
    n, B = int(lens.sum()), len(lens)
    row0 = np.concatenate([[0], np.cumsum(lens)])
    row_seq = np.repeat(np.arange(B), lens).astype(np.int32)
    row_pos = np.concatenate([np.arange(p, p + l) for p, l in zip(pos0, lens)]).astype(np.int32)
    kind = PREFILL if (pos0 == 0).all() else DECODE if (lens == 1).all() else EXTEND
    return StepContext(kind=kind, dtype=dtype, device=DEV, n_rows=n, n_seqs=B,
                       row_pos=torch.from_numpy(row_pos).to(DEV),
                       row_seq=torch.from_numpy(row_seq).to(DEV),
                       seq_slot_dev=torch.arange(B, dtype=torch.int32, device=DEV),
                       seq_slots=list(range(B)), seq_pos0=pos0, seq_len=lens, seq_row0=row0,
                       max_pos=int((pos0 + lens).max()) - 1)


def test_norm_part():
    from janas_b200.config import PartSpec
    norm = build("norm", PartSpec("rmsnorm", {"size": 200, "eps": 1e-4}))
    w = give(norm, "some.norm")
    assert list(w) == ["some.norm.weight"]
    x = torch.randn(9, 200) * 2
    got = norm.apply(x.to(DEV), torch.float32).cpu()
    want = plain.rms_norm(x, w["some.norm.weight"], 1e-4)
    assert (got - want).abs().max() <= 2e-6 * want.abs().max()


def test_rope_part():
    from janas_b200.config import PartSpec
    rope = build("position", PartSpec("rope_neox", {"rotary_dim": 80, "theta": 12345.0,
                                                    "max_positions": 5000}))
    rope.prepare(300)
    assert rope.cos.shape == (300, 40)
    rope.prepare(100)                    # never shrinks
    assert rope.n_positions == 300
    c, s = plain.rope_table(range(300), 80, 12345.0)
    assert torch.equal(rope.cos.cpu(), c) and torch.equal(rope.sin.cpu(), s)
    rope.prepare(10 ** 6)                # no more positions than the model has
    assert rope.n_positions == 5000


def test_swiglu_part():
    from janas_b200.config import PartSpec
    ffn = build("feed_forward", PartSpec("swiglu", {"hidden_size": 72, "intermediate_size": 200}))
    w = give(ffn, "mlp", seed=3)
    h = torch.randn(11, 72)
    got = ffn.forward(context([0], [11]), h.to(DEV)).sum(0).cpu()
    want = plain.swiglu(h, w, "mlp.", None)
    assert (got - want).abs().max() <= 3e-6 * want.abs().max()


@pytest.mark.parametrize("rows,hidden,inter", [(40, 72, 200), (100, 72, 200), (700, 72, 200),
                                               (8, 1024, 136)])
def test_swiglu_part_bfloat16(rows, hidden, inter, monkeypatch):
    """Many rows, or few rows whose product would not be cut along k: gate, up and
    the activation in one tensor-core kernel; else the product, then the activation
    kernel.  All against the plain feed-forward with the activation rounded to
    bfloat16."""
    from janas_b200.config import PartSpec
    from janas_b200.csrc import ops
    ffn = build("feed_forward", PartSpec("swiglu", {"hidden_size": hidden,
                                                    "intermediate_size": inter}), torch.bfloat16)
    w = give(ffn, "mlp", seed=3, dtype=torch.bfloat16)
    h = torch.randn(rows, hidden).bfloat16()
    h[3] *= 40.0                          # gates far from zero on both sides
    got = ffn.forward(context([0], [rows], torch.bfloat16), h.to(DEV)).sum(0).cpu()
    assert ops.gemm_tc_error() == 0
    uncut = ops.linear_parts(rows, 2 * inter, hidden) == 1
    assert ffn.info()["fused_last"] == (rows >= ffn.FUSED_FROM or
                                         (rows <= ffn.FUSED_UP_TO and uncut))
    assert uncut == (hidden == 72)          # the cases cover both
    want = plain.swiglu(h.float(), w, "mlp.", "bfloat16")
    err = (got - want).abs().max(dim=1).values                    # row by row: row 3 is large
    assert bool((err <= 2 ** -7 * want.abs().max(dim=1).values).all())


@pytest.mark.parametrize("window,qk_norm,rope", [(0, True, True), (20, True, True),
                                                 (0, False, True), (0, True, False)])
def test_attention_part(window, qk_norm, rope):
    """The attention mixer alone over its own little cache: a whole prompt, then
    tokens one by one, against the plain attention layer on the whole sequence."""
    from janas_b200.cache import Cache
    from janas_b200.config import PartSpec
    from janas_b200.parts import LayerCache
    nh, nkv, hd, dm, n = 6, 3, 32, 72, 90
    pos = PartSpec("rope_neox", {"rotary_dim": hd, "theta": 1e4, "max_positions": 512}) \
        if rope else PartSpec("none")
    att = build("mixer", PartSpec("gqa_attention", {
        "hidden_size": dm, "num_heads": nh, "num_kv_heads": nkv, "head_dim": hd,
        "qk_norm_eps": 1e-5 if qk_norm else None, "window": window, "position": pos}))
    w = give(att, "attn", seed=5)
    att.prepare(512)
    cache = Cache([att.kv_spec()], [None], 256, 2, torch.float32, DEV)
    s = cache.new_sequence()
    g = cache.groups[0]
    x = torch.randn(n, dm)

    def run(p0, cnt):
        cache.reserve([s], [cnt])
        bt = torch.from_numpy(cache.block_table(g, [s])).to(DEV)
        lc = LayerCache(k=g.k[0], v=g.v[0], block_table=bt)
        out = att.forward(context([p0], [cnt]), x[p0:p0 + cnt].contiguous().to(DEV), lc)
        cache.advance([s], [cnt])
        return out.sum(0).cpu()

    got = torch.cat([run(0, 70)] + [run(p, 1) for p in range(70, n)])
    # the plain layer, with the options switched the same way
    c = dict(num_attention_heads=nh, num_key_value_heads=nkv, head_dim=hd, rms_norm_eps=1e-5,
             rope_theta=1e4)
    ww = dict(w)
    if not qk_norm:
        ww["attn.q_norm.weight"] = ww["attn.k_norm.weight"] = None
    q = (x @ ww["attn.q_proj.weight"].T).view(n, nh, hd)
    k = (x @ ww["attn.k_proj.weight"].T).view(n, nkv, hd)
    v = (x @ ww["attn.v_proj.weight"].T).view(n, nkv, hd)
    if qk_norm:
        q = plain.rms_norm(q, ww["attn.q_norm.weight"], 1e-5)
        k = plain.rms_norm(k, ww["attn.k_norm.weight"], 1e-5)
    if rope:
        cs, sn = plain.rope_table(range(n), hd, 1e4)
        q, k = plain.rope_neox(q, cs, sn), plain.rope_neox(k, cs, sn)
    want = plain.attention(q, k, v, window).reshape(n, nh * hd) @ ww["attn.o_proj.weight"].T
    assert (got - want).abs().max() <= 5e-6 * want.abs().max()


def test_a_toy_position_encoding_is_registered_and_used_by_the_attention_part():
    """Another position encoding, defined here: angles that grow linearly with the
    pair's index (no powers of a base), given to the attention mixer by name.
    Nothing in the framework knows it."""
    from janas_b200.cache import Cache
    from janas_b200.config import PartSpec
    from janas_b200.parts import LayerCache, PositionEncoding, register_position_encoding

    @register_position_encoding("toy_linear_angles")
    class LinearAngles(PositionEncoding):
        last = None         # the instance the library built last, for the test to ask

        def __init__(self, spec, dtype, device):
            super().__init__(spec, dtype, device)
            self.rotary_dim = int(spec.params["rotary_dim"])
            self.step = float(spec.params["step"])
            self.cos = self.sin = None
            LinearAngles.last = self

        def table(self, n):
            half = self.rotary_dim // 2
            ang = (torch.arange(n, dtype=torch.float64)[:, None] * self.step *
                   torch.arange(1, half + 1, dtype=torch.float64)[None, :])
            return torch.cos(ang).float(), torch.sin(ang).float()

        def prepare(self, n_positions):
            if self.cos is None or self.cos.shape[0] < n_positions:
                c, s = self.table(n_positions)
                self.cos, self.sin = c.to(self.device), s.to(self.device)

        @property
        def n_positions(self):
            return 0 if self.cos is None else self.cos.shape[0]

    nh, nkv, hd, dm, n = 4, 2, 64, 40, 75
    pos = PartSpec("toy_linear_angles", {"rotary_dim": hd, "step": 0.013})
    att = build("mixer", PartSpec("gqa_attention", {
        "hidden_size": dm, "num_heads": nh, "num_kv_heads": nkv, "head_dim": hd,
        "qk_norm_eps": 1e-6, "window": 0, "position": pos}))
    w = give(att, "attn", seed=11)
    att.prepare(128)
    cache = Cache([att.kv_spec()], [None], 128, 1, torch.float32, DEV)
    s = cache.new_sequence()
    g = cache.groups[0]
    x = torch.randn(n, dm)

    def run(p0, cnt):
        cache.reserve([s], [cnt])
        bt = torch.from_numpy(cache.block_table(g, [s])).to(DEV)
        lc = LayerCache(k=g.k[0], v=g.v[0], block_table=bt)
        out = att.forward(context([p0], [cnt]), x[p0:p0 + cnt].contiguous().to(DEV), lc)
        cache.advance([s], [cnt])
        return out.sum(0).cpu()

    got = torch.cat([run(0, 60)] + [run(p, 1) for p in range(60, n)])
    q = plain.rms_norm((x @ w["attn.q_proj.weight"].T).view(n, nh, hd), w["attn.q_norm.weight"], 1e-6)
    k = plain.rms_norm((x @ w["attn.k_proj.weight"].T).view(n, nkv, hd), w["attn.k_norm.weight"], 1e-6)
    v = (x @ w["attn.v_proj.weight"].T).view(n, nkv, hd)
    cs, sn = LinearAngles.last.table(n)
    q, k = plain.rope_neox(q, cs, sn), plain.rope_neox(k, cs, sn)
    want = plain.attention(q, k, v, 0).reshape(n, nh * hd) @ w["attn.o_proj.weight"].T
    assert (got - want).abs().max() <= 5e-6 * want.abs().max()
    # and it does turn the heads: without it the answer is another
    bare = plain.attention(plain.rms_norm((x @ w["attn.q_proj.weight"].T).view(n, nh, hd),
                                          w["attn.q_norm.weight"], 1e-6),
                           plain.rms_norm((x @ w["attn.k_proj.weight"].T).view(n, nkv, hd),
                                          w["attn.k_norm.weight"], 1e-6), v, 0)
    bare = bare.reshape(n, nh * hd) @ w["attn.o_proj.weight"].T
    assert (bare - want).abs().max() > 1e-3 * want.abs().max()


# ------------------------------------------------------------------ toy parts
def register_toys():
    """A mixer whose output is the running mean of its inputs (its state: the
    running sum and the count), and a feed-forward that routes every token to one
    of two scalings.  Written with library tensor operations: they are test toys,
    not product code."""
    from janas_b200.cache import StateSpec
    from janas_b200.parts import FeedForward, Mixer, register_feed_forward, register_mixer
    from janas_b200.weights import NORM, TensorSpec

    @register_mixer("toy_running_mean")
    class RunningMean(Mixer):
        def __init__(self, spec, dtype, device):
            super().__init__(spec, dtype, device)
            self.size = int(spec.params["size"])
            self.gain = None

        def tensors(self, prefix):
            return {self._name(prefix, "gain"): TensorSpec((self.size,), NORM)}

        def load(self, prefix, tensors):
            self.gain = tensors[self._name(prefix, "gain")].float()

        def state_spec(self):
            return StateSpec((self.size + 1,))          # the sum, and the count

        def forward(self, ctx, h, cache):
            out = torch.empty((ctx.n_rows, self.size), dtype=torch.float32, device=h.device)
            for i, slot in enumerate(ctx.seq_slots):
                a, b = int(ctx.seq_row0[i]), int(ctx.seq_row0[i + 1])
                st = cache.state[slot]
                sums = st[:-1] + torch.cumsum(h[a:b].float(), dim=0)
                counts = st[-1] + torch.arange(1, b - a + 1, device=h.device)
                out[a:b] = sums / counts[:, None] * self.gain
                st[:-1] = sums[-1]
                st[-1] = counts[-1]
            return out.unsqueeze(0)

    @register_feed_forward("toy_two_way")
    class TwoWay(FeedForward):
        def __init__(self, spec, dtype, device):
            super().__init__(spec, dtype, device)
            self.scales = spec.params["scales"]

        def forward(self, ctx, h):
            h = h.float()
            way = (h[:, 0] > 0).float()[:, None]          # the router: the sign of one channel
            return (h * (way * self.scales[0] + (1 - way) * self.scales[1])).unsqueeze(0)


def toy_spec():
    from janas_b200.config import LayerSpec, ModelSpec, PartSpec, RunEntry
    dm = 48
    norm = PartSpec("rmsnorm", {"size": dm, "eps": 1e-5})
    att = lambda pos: PartSpec("gqa_attention", {
        "hidden_size": dm, "num_heads": 3, "num_kv_heads": 1, "head_dim": 16, "qk_norm_eps": 1e-5,
        "window": 0, "position": pos})
    rope = PartSpec("rope_neox", {"rotary_dim": 16, "theta": 1e4, "max_positions": 256})
    swiglu = PartSpec("swiglu", {"hidden_size": dm, "intermediate_size": 80})
    layers = (
        LayerSpec("prenorm", PartSpec("toy_running_mean", {"size": dm}), swiglu, norm, norm,
                  "toy.layers.0", mixer_name="mix"),
        LayerSpec("prenorm", att(rope), PartSpec("toy_two_way", {"scales": (0.5, -0.25)}), norm,
                  norm, "toy.layers.1"),
        LayerSpec("prenorm", att(PartSpec("none")), swiglu, norm, norm, "toy.layers.2"),
    )
    # layer 0 runs twice (two states), layer 1 twice: the second time on the first's cache
    order = (RunEntry(0), RunEntry(1), RunEntry(2), RunEntry(0), RunEntry(1, cache_of=1))
    return ModelSpec(architecture="Toy", hidden_size=dm, vocab_size=97, max_positions=256,
                     layers=layers, run_order=order, final_norm=norm, tie_embeddings=True,
                     embedding_name="toy.embed.weight", final_norm_name="toy.norm")


def toy_plain(w, toks):
    """The toy model on a whole sequence, with plain operations."""
    n = len(toks)
    x = plain.embedding(w["toy.embed.weight"], toks)

    def mean_layer(x):
        h = plain.rms_norm(x, w["toy.layers.0.input_layernorm.weight"], 1e-5)
        m = torch.cumsum(h, 0) / torch.arange(1, n + 1)[:, None] * w["toy.layers.0.mix.gain"]
        x = x + m
        h = plain.rms_norm(x, w["toy.layers.0.post_attention_layernorm.weight"], 1e-5)
        return x + plain.swiglu(h, w, "toy.layers.0.mlp.", None)

    def attn(x, p, rope, kv=None):
        h = plain.rms_norm(x, w[p + "input_layernorm.weight"], 1e-5)
        q = (h @ w[p + "self_attn.q_proj.weight"].T).view(n, 3, 16)
        k = (h @ w[p + "self_attn.k_proj.weight"].T).view(n, 1, 16)
        v = (h @ w[p + "self_attn.v_proj.weight"].T).view(n, 1, 16)
        q = plain.rms_norm(q, w[p + "self_attn.q_norm.weight"], 1e-5)
        k = plain.rms_norm(k, w[p + "self_attn.k_norm.weight"], 1e-5)
        if rope:
            cs, sn = plain.rope_table(range(n), 16, 1e4)
            q, k = plain.rope_neox(q, cs, sn), plain.rope_neox(k, cs, sn)
        if kv is not None:
            k, v = kv
        a = plain.attention(q, k, v, 0).reshape(n, 48) @ w[p + "self_attn.o_proj.weight"].T
        return x + a, (k, v)

    def two_way(x, p):
        h = plain.rms_norm(x, w[p + "post_attention_layernorm.weight"], 1e-5)
        way = (h[:, 0] > 0).float()[:, None]
        return x + h * (way * 0.5 + (1 - way) * -0.25)

    x = mean_layer(x)
    x, kv1 = attn(x, "toy.layers.1.", True)
    x = two_way(x, "toy.layers.1.")
    x, _ = attn(x, "toy.layers.2.", False)
    h = plain.rms_norm(x, w["toy.layers.2.post_attention_layernorm.weight"], 1e-5)
    x = x + plain.swiglu(h, w, "toy.layers.2.mlp.", None)
    x = mean_layer(x)
    x, _ = attn(x, "toy.layers.1.", True, kv=kv1)
    x = two_way(x, "toy.layers.1.")
    return plain.rms_norm(x, w["toy.norm.weight"], 1e-5) @ w["toy.embed.weight"].T


def test_a_model_of_toy_parts_is_registered_built_and_stepped():
    from janas_b200.engine import Engine, expected_tensors
    from janas_b200.weights import random_tensors
    from helpers import rel_err, run_trace, trace_batches, trace_tail, trace_whole
    register_toys()
    spec = toy_spec()
    names = expected_tensors(spec)
    assert "toy.layers.0.mix.gain" in names and "toy.layers.1.self_attn.q_proj.weight" in names
    assert not any("layers.1.mlp" in n for n in names)         # the toy feed-forward has no tensors
    ts = dict(random_tensors(names, 9, torch.float32))
    eng = Engine.from_spec(spec, {n: t.to(DEV) for n, t in ts.items()}, dtype="float32",
                           max_tokens=1024, max_seqs=4)
    assert not eng.use_graphs               # the toys do not say that they can be captured
    # the cache: entries 1 and 2 share a group (same KV shape), entry 4 reads entry 1's,
    # entries 0 and 3 have a state each
    assert len(eng.cache.groups) == 1 and eng.cache.groups[0].entries == [1, 2]
    assert sorted(eng.cache.mixer_state) == [0, 3]
    rng = np.random.default_rng(1)
    reqs = [rng.integers(0, 97, size=n).tolist() for n in (5, 70, 33, 140)]
    want = [toy_plain(ts, r).numpy() for r in reqs]
    whole = run_trace(eng, trace_whole(reqs))
    tail = run_trace(eng, trace_tail(reqs, 32))
    batched = run_trace(eng, trace_batches([[(reqs[0], 2), (reqs[1], 40), (reqs[3], 100)],
                                            [(reqs[2], 33), (reqs[3], 7)]]))
    for i, r in enumerate(reqs):
        a = np.stack([whole[f"r{i}"][p] for p in range(len(r))])
        assert rel_err(a, want[i]) <= 1e-5, i
        b = np.stack([tail[f"r{i}"][p] for p in range(len(r))])
        assert rel_err(b, a) <= 2e-6, i                         # the toy's cumsum is not bitwise
    for rid, i in (("b0r0", 0), ("b0r1", 1), ("b0r2", 3), ("b1r0", 2), ("b1r1", 3)):
        b = np.stack([batched[rid][p] for p in range(len(reqs[i]))])
        assert rel_err(b, want[i]) <= 1e-5, rid
    eng.cache.check()


def test_a_toy_norm_is_registered_and_used_in_every_place_a_norm_stands():
    """Another norm, defined here: a layer norm (mean taken off, a weight and a
    bias), as the norm before the mixer, before the feed-forward and before the
    head of a two-layer model.  Nothing in the framework knows it."""
    from janas_b200.config import LayerSpec, ModelSpec, PartSpec, RunEntry
    from janas_b200.engine import Engine, expected_tensors
    from janas_b200.parts import Norm, register_norm
    from janas_b200.weights import NORM, TensorSpec, random_tensors
    from helpers import rel_err, run_trace, trace_tail, trace_whole

    @register_norm("toy_layer_norm")
    class LayerNorm(Norm):
        def __init__(self, spec, dtype, device):
            super().__init__(spec, dtype, device)
            self.size, self.eps = int(spec.params["size"]), float(spec.params["eps"])

        def tensors(self, prefix):
            return {self._name(prefix, "weight"): TensorSpec((self.size,), NORM),
                    self._name(prefix, "bias"): TensorSpec((self.size,), NORM)}

        def load(self, prefix, tensors):
            self.w = tensors[self._name(prefix, "weight")].float()
            self.b = tensors[self._name(prefix, "bias")].float()

        def apply(self, x, out_dtype, rows=None):
            if rows is not None:
                x = x[rows.long()]
            c = x - x.mean(1, keepdim=True)
            return (c / torch.sqrt(c.pow(2).mean(1, keepdim=True) + self.eps) * self.w + self.b).to(out_dtype)

    dm = 40
    norm = PartSpec("toy_layer_norm", {"size": dm, "eps": 1e-4})
    rope = PartSpec("rope_neox", {"rotary_dim": 16, "theta": 1e4, "max_positions": 128})
    att = PartSpec("gqa_attention", {"hidden_size": dm, "num_heads": 2, "num_kv_heads": 1, "head_dim": 16,
                                     "qk_norm_eps": 1e-5, "window": 0, "position": rope})
    ffn = PartSpec("swiglu", {"hidden_size": dm, "intermediate_size": 56})
    layers = tuple(LayerSpec("prenorm", att, ffn, norm, norm, f"t.layers.{i}") for i in range(2))
    spec = ModelSpec(architecture="ToyNorm", hidden_size=dm, vocab_size=61, max_positions=128, layers=layers,
                     run_order=(RunEntry(0), RunEntry(1)), final_norm=norm, tie_embeddings=True,
                     embedding_name="t.embed.weight", final_norm_name="t.norm")
    names = expected_tensors(spec)
    assert "t.layers.1.post_attention_layernorm.bias" in names and "t.norm.bias" in names
    w = dict(random_tensors(names, 3, torch.float32))
    eng = Engine.from_spec(spec, {n: t.to(DEV) for n, t in w.items()}, dtype="float32", max_tokens=512,
                           max_seqs=2)

    def ln(x, p):
        c = x - x.mean(1, keepdim=True)
        return c / torch.sqrt(c.pow(2).mean(1, keepdim=True) + 1e-4) * w[p + ".weight"] + w[p + ".bias"]

    def plain_model(toks):
        n = len(toks)
        x = plain.embedding(w["t.embed.weight"], toks)
        for i in range(2):
            p = f"t.layers.{i}."
            h = ln(x, p + "input_layernorm")
            q = plain.rms_norm((h @ w[p + "self_attn.q_proj.weight"].T).view(n, 2, 16),
                               w[p + "self_attn.q_norm.weight"], 1e-5)
            k = plain.rms_norm((h @ w[p + "self_attn.k_proj.weight"].T).view(n, 1, 16),
                               w[p + "self_attn.k_norm.weight"], 1e-5)
            v = (h @ w[p + "self_attn.v_proj.weight"].T).view(n, 1, 16)
            cs, sn = plain.rope_table(range(n), 16, 1e4)
            q, k = plain.rope_neox(q, cs, sn), plain.rope_neox(k, cs, sn)
            x = x + plain.attention(q, k, v, 0).reshape(n, 32) @ w[p + "self_attn.o_proj.weight"].T
            x = x + plain.swiglu(ln(x, p + "post_attention_layernorm"), w, p + "mlp.", None)
        return ln(x, "t.norm") @ w["t.embed.weight"].T

    rng = np.random.default_rng(2)
    reqs = [rng.integers(0, 61, size=n).tolist() for n in (9, 50)]
    whole = run_trace(eng, trace_whole(reqs))
    tail = run_trace(eng, trace_tail(reqs, 32))
    for i, r in enumerate(reqs):
        want = plain_model(r).numpy()
        a = np.stack([whole[f"r{i}"][p] for p in range(len(r))])
        b = np.stack([tail[f"r{i}"][p] for p in range(len(r))])
        assert rel_err(a, want) <= 1e-5 and rel_err(b, want) <= 1e-5, i
    eng.cache.check()
