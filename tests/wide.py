"""Models of real layer widths for the GPU tests: the sizes of Qwen2.5-0.5B, 1.5B and 7B
with two layers, random weights, and the plain implementation as their oracle, run in
float64 on the GPU (the same plain PyTorch functions, only where the weights lie differs)."""

from __future__ import annotations

from functools import lru_cache

import numpy as np
import torch

from mercury_b200.config import config_from_dict
from mercury_b200.weights import random_tensors
from plain_qwen2 import plain_logits_at
from tiny import random_tokens

_COMMON = {"architectures": ["Qwen2ForCausalLM"], "num_hidden_layers": 2, "rope_theta": 1000000.0,
           "rms_norm_eps": 1e-6, "max_position_embeddings": 32768}
WIDTHS = {
    "0.5B": {**_COMMON, "hidden_size": 896, "num_attention_heads": 14, "num_key_value_heads": 2,
             "head_dim": 64, "intermediate_size": 4864, "vocab_size": 151936,
             "tie_word_embeddings": True},
    "1.5B": {**_COMMON, "hidden_size": 1536, "num_attention_heads": 12, "num_key_value_heads": 2,
             "head_dim": 128, "intermediate_size": 8960, "vocab_size": 151936,
             "tie_word_embeddings": True},
    "7B": {**_COMMON, "hidden_size": 3584, "num_attention_heads": 28, "num_key_value_heads": 4,
           "head_dim": 128, "intermediate_size": 18944, "vocab_size": 152064,
           "tie_word_embeddings": False},
}
SHARPEN = 2.0   # q and k projections are scaled so that attention is not nearly uniform


@lru_cache(maxsize=None)
def model(name: str):
    """(raw config dictionary, typed config, {name: bfloat16 tensor on the CPU})."""
    raw = WIDTHS[name]
    _entry, config = config_from_dict(raw)
    tensors = random_tensors(config, 7, torch.bfloat16)
    for key in tensors:
        if "q_proj" in key or "k_proj" in key:
            tensors[key] = (tensors[key].float() * SHARPEN).to(torch.bfloat16)
    return raw, config, tensors


_ORACLE_WEIGHTS: dict[str, dict] = {}


def oracle_weights(name: str) -> dict:
    """The model's weights in float64 on the GPU, one model at a time (7B widths take 12 GB)."""
    if name not in _ORACLE_WEIGHTS:
        _ORACLE_WEIGHTS.clear()
        torch.cuda.empty_cache()
        _raw, _config, tensors = model(name)
        _ORACLE_WEIGHTS[name] = {k: v.to("cuda", torch.float64) for k, v in tensors.items()}
    return _ORACLE_WEIGHTS[name]


def tokens_for(name: str, length: int, seed: int) -> list[int]:
    return random_tokens(length, WIDTHS[name]["vocab_size"], seed)


@lru_cache(maxsize=4096)
def oracle_rows(name: str, length: int, seed: int, rows: tuple[int, ...]) -> np.ndarray:
    """float64 logits [len(rows), vocab] of the sequence `tokens_for(name, length, seed)` at
    the positions `rows`."""
    with torch.inference_mode():
        out = plain_logits_at(WIDTHS[name], oracle_weights(name), tokens_for(name, length, seed), rows)
    return out.cpu().numpy()


def relative_error(got: np.ndarray, want: np.ndarray) -> float:
    """Largest |difference| as a fraction of the largest |logit| wanted."""
    return float(np.abs(got.astype(np.float64) - want).max() / np.abs(want).max())
