"""A tiny random Qwen3 model whose matrices are exactly what the reference's
eight-bit weight type (Q8_0: blocks of 32 signed bytes times one half-precision
scale) holds, so that the reference's own model code and a float32
implementation can run the same weights.  The numbers come from splitmix64 over
element indices, so that they are the same wherever this file runs.

Used by make_model_golden.py (which writes the model as a GGUF file for the
reference's tools) and by tests/test_plain.py (which gives the same weights to
the plain implementation)."""
import numpy as np

CONFIG = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=2, hidden_size=256,
    num_attention_heads=4, num_key_value_heads=2, head_dim=64, intermediate_size=512,
    vocab_size=320, rope_theta=10000.0, rms_norm_eps=1e-6, tie_word_embeddings=True,
    max_position_embeddings=512, layer_types=["full_attention", "full_attention"])
# the reference's model code wants widths that are multiples of 256
# (src/llm/model_load.c:827-830); heads * head_dim = 256 too

TOKENS = [17, 3, 300, 5, 5, 211, 0, 319, 42, 7, 99, 150, 23, 8, 250, 64, 1, 77, 310, 12,
          200, 31, 6, 180, 45, 290, 11, 2, 133, 58, 270, 9, 101, 36, 222, 14, 301, 66, 4, 190]


def uniform(stream: int, n: int) -> np.ndarray:
    """n numbers in [0, 1): splitmix64 of stream * 2^40 + index."""
    with np.errstate(over="ignore"):
        z = np.arange(n, dtype=np.uint64) + np.uint64(stream << 40)
        z = z * np.uint64(0x9E3779B97F4A7C15) + np.uint64(0x9E3779B97F4A7C15)
        z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        z = z ^ (z >> np.uint64(31))
    return (z >> np.uint64(11)).astype(np.float64) * (1.0 / 9007199254740992.0)


def q8_0_matrix(stream: int, rows: int, cols: int, std: float = 0.02):
    """Bytes in -127 .. 127 and a scale per block of 32: the float32 weights
    [rows, cols] and the blocks as the file holds them (scale, then 32 bytes)."""
    q = (np.floor(uniform(2 * stream, rows * cols) * 255.0) - 127.0).astype(np.int8)
    q = q.reshape(rows, cols // 32, 32)
    d = ((0.6 + 0.8 * uniform(2 * stream + 1, rows * cols // 32)) * std / 73.0)
    d = d.astype(np.float16).reshape(rows, cols // 32)
    w = (q.astype(np.float32) * d.astype(np.float32)[..., None]).reshape(rows, cols)
    raw = np.zeros((rows, cols // 32, 34), dtype=np.uint8)
    raw[..., :2] = d.view(np.uint8).reshape(rows, cols // 32, 2)
    raw[..., 2:] = q.view(np.uint8)
    return w, raw.tobytes()


def norm_vector(stream: int, n: int) -> np.ndarray:
    """Norm weights between 0.5 and 1.5: far enough from one to matter."""
    return (1.0 + (uniform(2 * stream, n) - 0.5)).astype(np.float32)


def tensors(c=CONFIG):
    """[(GGUF name, checkpoint name, float32 array, bytes in the file, Q8_0?)] in the
    file's order (names: src/llm/model_load.c:403-503,999-1007)."""
    L, dm, ff, V = c["num_hidden_layers"], c["hidden_size"], c["intermediate_size"], c["vocab_size"]
    qd, kvd = c["num_attention_heads"] * c["head_dim"], c["num_key_value_heads"] * c["head_dim"]
    out, stream = [], [0]

    def matrix(g, h, rows, cols):
        # the layers' matrices are larger than a trained model's would be, so that what
        # the layers add to the residual stream shows in the logits beside the
        # embedding's own share
        stream[0] += 1
        w, raw = q8_0_matrix(stream[0], rows, cols, 0.02 if g == "token_embd.weight" else 0.05)
        out.append((g, h, w, raw, True))

    def vector(g, h, n):
        stream[0] += 1
        w = norm_vector(stream[0], n)
        out.append((g, h, w, w.tobytes(), False))

    matrix("token_embd.weight", "model.embed_tokens.weight", V, dm)
    vector("output_norm.weight", "model.norm.weight", dm)
    for l in range(L):
        g, h = f"blk.{l}.", f"model.layers.{l}."
        vector(g + "attn_norm.weight", h + "input_layernorm.weight", dm)
        matrix(g + "attn_q.weight", h + "self_attn.q_proj.weight", qd, dm)
        matrix(g + "attn_k.weight", h + "self_attn.k_proj.weight", kvd, dm)
        matrix(g + "attn_v.weight", h + "self_attn.v_proj.weight", kvd, dm)
        matrix(g + "attn_output.weight", h + "self_attn.o_proj.weight", dm, qd)
        vector(g + "attn_q_norm.weight", h + "self_attn.q_norm.weight", c["head_dim"])
        vector(g + "attn_k_norm.weight", h + "self_attn.k_norm.weight", c["head_dim"])
        vector(g + "ffn_norm.weight", h + "post_attention_layernorm.weight", dm)
        matrix(g + "ffn_gate.weight", h + "mlp.gate_proj.weight", ff, dm)
        matrix(g + "ffn_up.weight", h + "mlp.up_proj.weight", ff, dm)
        matrix(g + "ffn_down.weight", h + "mlp.down_proj.weight", dm, ff)
    return out
