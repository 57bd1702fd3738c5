"""The tiny configurations the tests use.  They differ in every size and
option: layers, width, heads and groups, head size, feed-forward width,
vocabulary, rope base, eps, tied or separate head, context, window."""
import numpy as np

# 2 layers, heads * head_dim == hidden, tied, no window
TINY_A = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3",
    num_hidden_layers=2, hidden_size=64, num_attention_heads=4, num_key_value_heads=2,
    head_dim=16, intermediate_size=128, vocab_size=256, rope_theta=10000.0,
    rms_norm_eps=1e-6, tie_word_embeddings=True, max_position_embeddings=128)

# 3 layers, GQA ratio 3, heads * head_dim != hidden, separate head, no size a power of two
TINY_B = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3",
    num_hidden_layers=3, hidden_size=96, num_attention_heads=6, num_key_value_heads=2,
    head_dim=32, intermediate_size=224, vocab_size=384, rope_theta=1e6,
    rms_norm_eps=1e-5, tie_word_embeddings=False, max_position_embeddings=256)

# 4 layers, the upper two with a sliding window that is no multiple of anything;
# one KV head (ratio 5), head size 48, long context
TINY_C = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3",
    num_hidden_layers=4, hidden_size=80, num_attention_heads=5, num_key_value_heads=1,
    head_dim=48, intermediate_size=136, vocab_size=331, rope_theta=50000.0,
    rms_norm_eps=3e-6, tie_word_embeddings=True, max_position_embeddings=1024,
    use_sliding_window=True, sliding_window=37, max_window_layers=2)

TINY = {"A": TINY_A, "B": TINY_B, "C": TINY_C}
SEEDS = {"A": 0, "B": 1, "C": 2}


def tokens(rng: np.random.Generator, n: int, vocab: int):
    return rng.integers(0, vocab, size=n).tolist()
