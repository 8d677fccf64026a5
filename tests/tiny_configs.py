"""The two tiny Qwen3 configurations the tests use; they differ in every size and
option: layers, hidden width, heads and groups, head size (q width equal to / different
from the hidden width), intermediate width, vocabulary (no powers of two in B's widths),
rope_theta, rms_norm_eps, tied / untied head, cache page size and context length."""


def _config(**sizes):
    base = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", hidden_act="silu",
                attention_bias=False, attention_dropout=0.0, use_sliding_window=False,
                sliding_window=None, rope_scaling=None, torch_dtype="bfloat16")
    base.update(sizes)
    return base


TINY_A = _config(num_hidden_layers=2, hidden_size=64, num_attention_heads=4, num_key_value_heads=2,
                 head_dim=16, intermediate_size=128, vocab_size=256, rope_theta=10000.0,
                 rms_norm_eps=1e-6, tie_word_embeddings=True, max_position_embeddings=128)
TINY_A_SEED, TINY_A_PAGE = 0, 16

TINY_B = _config(num_hidden_layers=3, hidden_size=96, num_attention_heads=6, num_key_value_heads=2,
                 head_dim=32, intermediate_size=256, vocab_size=512, rope_theta=1000000.0,
                 rms_norm_eps=1e-5, tie_word_embeddings=False, max_position_embeddings=256)
TINY_B_SEED, TINY_B_PAGE = 1, 8

# A third shape with sizes that are no power of two anywhere, for replay tests.
TINY_C = _config(num_hidden_layers=2, hidden_size=80, num_attention_heads=6, num_key_value_heads=3,
                 head_dim=48, intermediate_size=200, vocab_size=331, rope_theta=50000.0,
                 rms_norm_eps=3e-6, tie_word_embeddings=False, max_position_embeddings=640)
TINY_C_SEED, TINY_C_PAGE = 2, 16

ALL = {"a": (TINY_A, TINY_A_SEED, TINY_A_PAGE), "b": (TINY_B, TINY_B_SEED, TINY_B_PAGE),
       "c": (TINY_C, TINY_C_SEED, TINY_C_PAGE)}
