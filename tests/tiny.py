"""The small configurations the tests run, as config.json dictionaries.

A and B are the two tiny Qwen2 shapes of the benchmark description; they differ in every
size and option. C and D add what A and B leave out: a sliding window on the upper
layers, head sizes of 48 and 64, and more query heads per group.
"""

from __future__ import annotations

import torch

from mercury_b200.config import config_from_dict
from mercury_b200.weights import random_tensors

TINY_A = {
    "architectures": ["Qwen2ForCausalLM"], "num_hidden_layers": 2, "hidden_size": 64,
    "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 16,
    "intermediate_size": 128, "vocab_size": 256, "rope_theta": 10000.0, "rms_norm_eps": 1e-6,
    "tie_word_embeddings": True, "use_sliding_window": False, "max_position_embeddings": 2048,
}
TINY_B = {
    "architectures": ["Qwen2ForCausalLM"], "num_hidden_layers": 3, "hidden_size": 96,
    "num_attention_heads": 3, "num_key_value_heads": 1, "head_dim": 32,
    "intermediate_size": 320, "vocab_size": 384, "rope_theta": 1000000.0, "rms_norm_eps": 1e-5,
    "tie_word_embeddings": False, "use_sliding_window": False, "max_position_embeddings": 4096,
}
TINY_C = {
    "architectures": ["Qwen2ForCausalLM"], "num_hidden_layers": 3, "hidden_size": 80,
    "num_attention_heads": 6, "num_key_value_heads": 2, "head_dim": 48,
    "intermediate_size": 200, "vocab_size": 331, "rope_theta": 50000.0, "rms_norm_eps": 3e-6,
    "tie_word_embeddings": False, "use_sliding_window": True, "sliding_window": 24,
    "max_window_layers": 1, "max_position_embeddings": 1024,
}
TINY_D = {
    "architectures": ["Qwen2ForCausalLM"], "num_hidden_layers": 2, "hidden_size": 112,
    "num_attention_heads": 7, "num_key_value_heads": 1, "head_dim": 64,
    "intermediate_size": 176, "vocab_size": 515, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6,
    "tie_word_embeddings": True, "use_sliding_window": False, "max_position_embeddings": 2048,
}
TINY_E = {   # one KV head under 32 query heads, head size 80 (no tensor-core attention), pages of 64
    "architectures": ["Qwen2ForCausalLM"], "num_hidden_layers": 2, "hidden_size": 160,
    "num_attention_heads": 32, "num_key_value_heads": 1, "head_dim": 80,
    "intermediate_size": 272, "vocab_size": 1000, "rope_theta": 100000.0, "rms_norm_eps": 1e-5,
    "tie_word_embeddings": False, "use_sliding_window": False, "max_position_embeddings": 2048,
}
PAGE_SIZE = {"A": 16, "B": 8, "C": 16, "D": 32, "E": 64}
SEED = {"A": 0, "B": 1, "C": 2, "D": 3, "E": 4}
RAW = {"A": TINY_A, "B": TINY_B, "C": TINY_C, "D": TINY_D, "E": TINY_E}


def tiny_model(name: str, std: float | None = None):
    """(raw config dictionary, typed config, {name: bfloat16 tensor})."""
    raw = RAW[name]
    _entry, config = config_from_dict(raw)
    tensors = random_tensors(config, SEED[name], torch.bfloat16, std)
    return raw, config, tensors


def random_tokens(count: int, vocab: int, seed: int) -> list[int]:
    gen = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (count,), generator=gen).tolist()
