"""A plain, slow implementation of the Qwen3 dense decoder, for comparison.

Whole sequences, no cache, one function for each part, float32 on the CPU.  It
shares no code with ``janas_b200``: it reads ``config.json`` with ``json`` and
the weights with the ``safetensors`` package, and every function restates a
formula of the reference, cited as file:line within prabanta-dev/janas.

The reference's own model code cannot run a float32 or bfloat16 model: its loader
accepts quantized weight types alone (src/llm/model_load.c:68-71), quantizes
activations and the cache to eight bits (src/llm/model_attn.c:42-48,115-145) and
wants sizes that are multiples of 256 (src/llm/model_load.c:827-830).  So this
file is compared with the reference in two ways (``tests/golden/``,
``tests/test_plain.py``).  Part by part, exactly: what of the reference compiles
alone here (its sampler, its math functions, its RMSNorm, and its attention with
float scores over keys and values that its eight-bit cache holds exactly) gives
the same tokens, the same bits or agrees to 1e-6.  And whole, loosely: a tiny
random Qwen3 whose matrices its eight-bit weight type holds exactly went through
its own tools (gguf2jns, llm_eval) on the CPU; ``forward`` below agrees with the
logits it wrote to a few hundredths of the largest (what its eight-bit
activations cost), while a wrong pairing of heads, exchanged norms or another
rotation are off by ten times as much.

``rounding="bfloat16"`` rounds the activations to bfloat16 at the places where a
bfloat16 engine stores them (norm outputs, q/k/v after RoPE, the attention
output, the activated gate, and optionally the softmax weights); the sums stay
in float32.  ``rounding=None`` is the exact float32 model.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

MASK64 = (1 << 64) - 1


# --------------------------------------------------------------------- reading
def read_config(model_dir: str) -> Dict:
    with open(os.path.join(model_dir, "config.json"), "r", encoding="utf-8") as f:
        c = json.load(f)
    # tools/hf2gguf.c:262-265: head_dim defaults to hidden/heads, tied to false
    c.setdefault("head_dim", c["hidden_size"] // c["num_attention_heads"])
    if c["head_dim"] is None:
        c["head_dim"] = c["hidden_size"] // c["num_attention_heads"]
    c.setdefault("tie_word_embeddings", False)
    n = c["num_hidden_layers"]
    if c.get("layer_types") is None:
        if c.get("use_sliding_window"):
            first = c.get("max_window_layers") or 0
            c["layer_types"] = ["sliding_attention" if i >= first else "full_attention"
                                for i in range(n)]
        else:
            c["layer_types"] = ["full_attention"] * n
    return c


def read_weights(model_dir: str) -> Dict[str, torch.Tensor]:
    from safetensors.torch import load_file
    w = load_file(os.path.join(model_dir, "model.safetensors"))
    return {k: v.to(torch.float32) for k, v in w.items()}


def _round(x: torch.Tensor, rounding: Optional[str]) -> torch.Tensor:
    if rounding is None:
        return x
    assert rounding == "bfloat16"
    return x.to(torch.bfloat16).to(torch.float32)


# ----------------------------------------------------------------------- parts
def embedding(table: torch.Tensor, tokens: Sequence[int]) -> torch.Tensor:
    """x[j, :] = E[token_j, :], no scaling (src/llm/model.c:78-91,658-667)."""
    return table[torch.tensor(list(tokens), dtype=torch.long)].clone()


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """Sum of squares in double, scale = 1/sqrtf((float)(ss/n) + eps),
    out = (x*scale)*w (src/llm/model_impl.h:635-644)."""
    n = x.shape[-1]
    ss = (x.double() * x.double()).sum(dim=-1, keepdim=True)
    mean = (ss / n).to(torch.float32)
    scale = 1.0 / torch.sqrt(mean + torch.tensor(eps, dtype=torch.float32))
    return (x * scale) * w


def rope_table(positions: Sequence[int], n_rot: int, base: float):
    """theta(p, i) = (float)p * powf(base, -2 i / n_rot); cos and sin of it
    (src/llm/model.c:100-113).  The reference's powf is a double computation
    rounded once (src/llm/jmath.c:131-134) and its sincos is evaluated in
    double (src/llm/jmath.c:163-200)."""
    half = n_rot // 2
    expo = np.float32(-2.0) * np.arange(half, dtype=np.float32) / np.float32(n_rot)
    inv = np.power(np.float64(np.float32(base)), expo.astype(np.float64)).astype(np.float32)
    pos = np.asarray(list(positions), dtype=np.float32)
    theta = (pos[:, None] * inv[None, :]).astype(np.float32)
    cs = np.cos(theta.astype(np.float64)).astype(np.float32)
    sn = np.sin(theta.astype(np.float64)).astype(np.float32)
    return torch.from_numpy(cs), torch.from_numpy(sn)


def rope_neox(v: torch.Tensor, cs: torch.Tensor, sn: torch.Tensor) -> torch.Tensor:
    """Pairs (i, i + half): v[i] = a cos - b sin, v[i+half] = a sin + b cos
    (src/llm/model_attn.c:31-39).  v: [tokens, heads, n_rot]; cs, sn:
    [tokens, half]."""
    half = v.shape[-1] // 2
    a, b = v[..., :half], v[..., half:]
    c, s = cs[:, None, :], sn[:, None, :]
    return torch.cat([a * c - b * s, a * s + b * c], dim=-1)


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, window: int,
              rounding: Optional[str] = None, round_weights: bool = False) -> torch.Tensor:
    """Causal GQA attention of one whole sequence.

    Head h uses KV head h / (heads / kv_heads) (src/llm/attention.c:874-875);
    score = (q . k) / sqrt(head_dim) (src/llm/attention.c:1012); token j sees
    t <= j (src/llm/attention.c:659-662,734) and, with a window, only
    t >= j + 1 - window (src/llm/attention.c:736-739); weights
    exp(s - max), 0 where s - max < -80, divided by their sum
    (src/llm/attention.c:574-588,870-910).
    q: [n, heads, hd]; k, v: [n, kv_heads, hd] -> [n, heads, hd]."""
    n, nh, hd = q.shape
    nkv = k.shape[1]
    group = nh // nkv
    scale = np.float32(1.0) / np.sqrt(np.float32(hd))
    out = torch.zeros_like(q)
    j = torch.arange(n)[:, None]
    t = torch.arange(n)[None, :]
    visible = t <= j
    if window:
        visible &= t >= j + 1 - window
    for h in range(nh):
        kh = h // group
        s = (q[:, h, :] @ k[:, kh, :].T) * float(scale)
        s = s.masked_fill(~visible, float("-inf"))
        m = s.max(dim=-1, keepdim=True).values
        d = s - m
        w = torch.where(d < -80.0, torch.zeros_like(d), torch.exp(d))
        w = torch.where(visible, w, torch.zeros_like(w))
        denom = w.sum(dim=-1, keepdim=True)
        if round_weights:
            w = _round(w, rounding)
        out[:, h, :] = (w @ v[:, kh, :]) / denom
    return out


def attention_layer(x: torch.Tensor, positions: Sequence[int], w: Dict[str, torch.Tensor],
                    prefix: str, c: Dict, window: int, rounding: Optional[str],
                    round_weights: bool) -> torch.Tensor:
    """q, k, v products without biases, per-head q_norm/k_norm before RoPE with
    the model's eps, RoPE, attention, output product
    (src/llm/model_attn.c:75-146,224-285)."""
    n = x.shape[0]
    nh, nkv, hd = c["num_attention_heads"], c["num_key_value_heads"], c["head_dim"]
    q = (x @ w[prefix + "q_proj.weight"].T).view(n, nh, hd)
    k = (x @ w[prefix + "k_proj.weight"].T).view(n, nkv, hd)
    v = (x @ w[prefix + "v_proj.weight"].T).view(n, nkv, hd)
    q = rms_norm(q, w[prefix + "q_norm.weight"], c["rms_norm_eps"])
    k = rms_norm(k, w[prefix + "k_norm.weight"], c["rms_norm_eps"])
    cs, sn = rope_table(positions, hd, c["rope_theta"])
    q = _round(rope_neox(q, cs, sn), rounding)
    k = _round(rope_neox(k, cs, sn), rounding)
    v = _round(v, rounding)
    a = _round(attention(q, k, v, window, rounding, round_weights), rounding)
    return a.reshape(n, nh * hd) @ w[prefix + "o_proj.weight"].T


def swiglu(x: torch.Tensor, w: Dict[str, torch.Tensor], prefix: str,
           rounding: Optional[str]) -> torch.Tensor:
    """h = SiLU(gate) * up = gate / (1 + e^-gate) * up, then the down product
    (src/llm/vmath.h:64-68, src/llm/model_ffn.c:147-154)."""
    g = x @ w[prefix + "gate_proj.weight"].T
    u = x @ w[prefix + "up_proj.weight"].T
    h = _round(g / (1.0 + torch.exp(-g)) * u, rounding)
    return h @ w[prefix + "down_proj.weight"].T


def forward(c: Dict, w: Dict[str, torch.Tensor], tokens: Sequence[int],
            rounding: Optional[str] = None, round_weights: bool = False,
            trace: Optional[List[torch.Tensor]] = None,
            rows: Optional[Sequence[int]] = None) -> torch.Tensor:
    """Logits [len(tokens), vocab] of one whole sequence from position 0 (with
    ``rows``: of those positions only; the layers still see every token).

    Pre-norm blocks: x += Attn(RMSNorm(x)); x += FFN(RMSNorm(x))
    (src/llm/model.c:743-796); then the final norm and the head, which is the
    embedding table when the model ties them (src/llm/model.c:827-866,
    src/llm/model_load.c:1004-1007)."""
    eps = c["rms_norm_eps"]
    x = embedding(w["model.embed_tokens.weight"], tokens)
    positions = list(range(len(tokens)))
    for i in range(c["num_hidden_layers"]):
        p = f"model.layers.{i}."
        window = c["sliding_window"] if c["layer_types"][i] == "sliding_attention" else 0
        h = _round(rms_norm(x, w[p + "input_layernorm.weight"], eps), rounding)
        x = x + attention_layer(h, positions, w, p + "self_attn.", c, window, rounding,
                                round_weights)
        h = _round(rms_norm(x, w[p + "post_attention_layernorm.weight"], eps), rounding)
        x = x + swiglu(h, w, p + "mlp.", rounding)
        if trace is not None:
            trace.append(x.clone())
    if rows is not None:
        x = x[list(rows)]
    h = _round(rms_norm(x, w["model.norm.weight"], eps), rounding)
    head = w.get("lm_head.weight")
    if head is None:
        assert c["tie_word_embeddings"], "no lm_head.weight and the model does not tie"
        head = w["model.embed_tokens.weight"]
    return h @ head.T


# -------------------------------------------------------------------- sampling
SPLITMIX_STEP = 0x9E3779B97F4A7C15


def splitmix64(state: int):
    """One step of the counter generator: returns (new state, number)
    (src/llm/sample.c:133-139)."""
    state = (state + SPLITMIX_STEP) & MASK64
    z = state
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & MASK64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & MASK64
    return state, z ^ (z >> 31)


def argmax_first(row: np.ndarray) -> int:
    """The first index of the largest value (src/llm/sample.c:141-148)."""
    return int(np.argmax(row))


def sample(row: np.ndarray, temperature: float, top_k: int, top_p: float, min_p: float,
           rng_state: int):
    """One pick from a row of logits: returns (token, new rng state).

    temperature <= 0: the first maximum, no random number is used.  Otherwise
    the candidates are the logits not below max - 30 T, the top_k largest of
    them when 0 < top_k < vocab (equal logits: the lower id first), sorted;
    p_i = exp((l_i - l_0) / T); top_p keeps the shortest prefix whose mass
    reaches top_p * sum; min_p drops what is below min_p * p_0; one splitmix64
    number picks by walking the prefix (src/llm/sample.c:283-342)."""
    row = np.asarray(row, dtype=np.float32)
    if temperature <= 0:
        return argmax_first(row), rng_state
    t = np.float32(temperature)
    mx = row[argmax_first(row)]
    floor = np.float32(mx - np.float32(30.0) * t)
    ids = np.nonzero(row >= floor)[0]
    order = ids[np.lexsort((ids, -row[ids].astype(np.float64)))]   # falling logit, rising id
    nv = row.shape[0]
    k = top_k if 0 < top_k < nv else nv
    order = order[:k]
    top = row[order[0]]
    p = np.exp(((row[order] - top) / t).astype(np.float32)).astype(np.float32)
    csum = np.cumsum(p.astype(np.float64))          # added one by one, in order
    total = float(csum[-1])
    nc = len(p)
    if 0 < top_p < 1:
        lim = float(np.float32(top_p)) * total
        # the shortest prefix whose mass reaches lim (at least one candidate)
        kk = int(np.searchsorted(csum, lim, side="left")) + 1
        kk = min(max(kk, 1), nc)
        nc, total = kk, float(csum[kk - 1])
    if min_p > 0:
        lim = np.float32(min_p) * p[0]
        below = np.nonzero(p[1:nc] < lim)[0]
        kk = int(below[0]) + 1 if below.size else nc
        for i in range(kk, nc):
            total -= float(p[i])
        nc = kk
    rng_state, z = splitmix64(rng_state)
    u = float(z >> 11) * (2.0 ** -53) * total
    for i in range(nc - 1):
        u -= float(p[i])
        if u < 0:
            return int(order[i]), rng_state
    return int(order[nc - 1]), rng_state


def generate(c: Dict, w: Dict[str, torch.Tensor], prompt: Sequence[int], max_new: int,
             temperature: float = 0.0, top_k: int = 0, top_p: float = 0.0,
             min_p: float = 0.0, seed: int = 0, stop: Sequence[int] = (),
             rounding: Optional[str] = None) -> List[int]:
    """The prompt, then up to max_new tokens, stopping after a stop token
    (which is part of the output) (src/llm/generate.c:1116-1144,699-707).  The
    random sequence starts at the seed (src/llm/sample.c:118)."""
    seq = list(prompt)
    out: List[int] = []
    rng = seed & MASK64
    for _ in range(max_new):
        logits = forward(c, w, seq, rounding)[-1].numpy()
        tok, rng = sample(logits, temperature, top_k, top_p, min_p, rng)
        out.append(tok)
        seq.append(tok)
        if tok in stop:
            break
    return out
