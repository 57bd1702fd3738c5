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

# head size 64: the tensor-core attention kernels with one 64-value block per head;
# GQA ratio 4, untied, eps and rope base different again
TINY_D = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3",
    num_hidden_layers=2, hidden_size=128, num_attention_heads=4, num_key_value_heads=1,
    head_dim=64, intermediate_size=200, vocab_size=500, rope_theta=300000.0,
    rms_norm_eps=2e-6, tie_word_embeddings=False, max_position_embeddings=512)

# head size 128 as in the full-size models, 3 KV heads of 2 query heads, a window on
# the first layer only (given as layer_types), vocabulary no multiple of 8
TINY_E = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3",
    num_hidden_layers=3, hidden_size=104, num_attention_heads=6, num_key_value_heads=3,
    head_dim=128, intermediate_size=264, vocab_size=777, rope_theta=1e6,
    rms_norm_eps=1e-6, tie_word_embeddings=True, max_position_embeddings=640,
    use_sliding_window=True, sliding_window=150,
    layer_types=["sliding_attention", "full_attention", "full_attention"])

# sizes that are multiples of nothing: width 50 (rows of 100 bytes: the tensor-core
# product refuses them and the plain one takes over), as many KV heads as heads
TINY_F = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3",
    num_hidden_layers=2, hidden_size=50, num_attention_heads=3, num_key_value_heads=3,
    head_dim=16, intermediate_size=90, vocab_size=123, rope_theta=7777.0,
    rms_norm_eps=1e-4, tie_word_embeddings=True, max_position_embeddings=200)

TINY = {"A": TINY_A, "B": TINY_B, "C": TINY_C, "D": TINY_D, "E": TINY_E, "F": TINY_F}
SEEDS = {"A": 0, "B": 1, "C": 2, "D": 3, "E": 4, "F": 5}


def tokens(rng: np.random.Generator, n: int, vocab: int):
    return rng.integers(0, vocab, size=n).tolist()
