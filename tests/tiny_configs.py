"""The tiny configurations of the tests.  A and B are the two the benchmark description names; they
differ in every size and option.  C adds what A and B lack: a sliding window on some layers, a
group of four query heads per key/value head, and a head size (48) that is no power of two."""

from zephyr_b200.config import Qwen3Config

TINY = {
    "A": dict(seed=0, page_size=4, config=dict(
        vocab_size=256, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
        num_key_value_heads=2, head_dim=16, max_position_embeddings=128, rms_norm_eps=1e-6, rope_theta=10000.0,
        tie_word_embeddings=True, layer_windows=(0, 0))),
    "B": dict(seed=1, page_size=8, config=dict(
        vocab_size=311, hidden_size=96, intermediate_size=200, num_hidden_layers=3, num_attention_heads=6,
        num_key_value_heads=3, head_dim=32, max_position_embeddings=256, rms_norm_eps=1e-5, rope_theta=1000000.0,
        tie_word_embeddings=False, layer_windows=(0, 0, 0))),
    "C": dict(seed=2, page_size=16, config=dict(
        vocab_size=199, hidden_size=80, intermediate_size=144, num_hidden_layers=3, num_attention_heads=8,
        num_key_value_heads=2, head_dim=48, max_position_embeddings=256, rms_norm_eps=3e-6, rope_theta=500000.0,
        tie_word_embeddings=False, layer_windows=(0, 24, 24))),
}


def tiny_config(name: str) -> Qwen3Config:
    return Qwen3Config(**TINY[name]["config"])
