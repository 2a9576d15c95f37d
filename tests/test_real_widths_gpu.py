"""The layer sizes of Qwen2.5-0.5B and 1.5B (full widths, head sizes 64 and 128, the real
vocabulary, two layers to keep the CPU oracle quick) through replay in 32-bit and in
bfloat16: whole, the last tokens one by one, and mixed with reused pages. These are the
sizes the tensor-core attention, the few-token products and the decode graphs serve."""

from __future__ import annotations

from functools import lru_cache

import pytest
import torch

import replay_cases
import replay_check
from mercury_b200.config import config_from_dict
from mercury_b200.weights import random_tensors
from plain_qwen2 import plain_logits
from tiny import random_tokens

pytestmark = pytest.mark.gpu

WIDTHS = {
    "0.5B": {"architectures": ["Qwen2ForCausalLM"], "num_hidden_layers": 2, "hidden_size": 896,
             "num_attention_heads": 14, "num_key_value_heads": 2, "head_dim": 64,
             "intermediate_size": 4864, "vocab_size": 151936, "rope_theta": 1000000.0,
             "rms_norm_eps": 1e-6, "tie_word_embeddings": True, "max_position_embeddings": 32768},
    "1.5B": {"architectures": ["Qwen2ForCausalLM"], "num_hidden_layers": 2, "hidden_size": 1536,
             "num_attention_heads": 12, "num_key_value_heads": 2, "head_dim": 128,
             "intermediate_size": 8960, "vocab_size": 151936, "rope_theta": 1000000.0,
             "rms_norm_eps": 1e-6, "tie_word_embeddings": True, "max_position_embeddings": 32768},
}
LENGTHS = (150, 70, 97, 40, 130)
MAX_TOKENS = 384
# bfloat16 at these widths: the plain PyTorch twin of the kernels (float32 arithmetic,
# bfloat16 storage between kernels, run on the CPU through the same step function) is
# itself off from the float64 oracle by up to 1.3e-2 (0.5B widths) and 2.3e-2 (1.5B widths)
# of the largest logit on these requests: rounding to 8 bits grows with the width and the
# maximum is taken over a vocabulary of 151936. The engine is held to 1.75 times the twin's
# worst figure; the tiny models keep 2e-2.
BF16_TOLERANCE = 4e-2


@lru_cache(maxsize=None)
def model(name):
    raw = WIDTHS[name]
    _entry, config = config_from_dict(raw)
    tensors = random_tensors(config, 7, torch.bfloat16)
    for key in tensors:            # sharpen attention as the tiny tests do
        if "q_proj" in key or "k_proj" in key:
            tensors[key] = (tensors[key].float() * 2.0).to(torch.bfloat16)
    return raw, config, tensors


@lru_cache(maxsize=None)
def requests_and_oracle(name):
    raw, _config, tensors = model(name)
    requests = {f"r{i}": random_tokens(n, raw["vocab_size"], 200 + i) for i, n in enumerate(LENGTHS)}
    want = {rid: plain_logits(raw, tensors, toks).numpy() for rid, toks in requests.items()}
    return requests, want


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("name", ["0.5B", "1.5B"])
def test_real_widths(name, dtype, monkeypatch):
    from mercury_b200.engine.runner import ModelRunner

    raw, config, tensors = model(name)
    requests, want = requests_and_oracle(name)
    monkeypatch.setattr(replay_check, "oracle", lambda _n, _l: want)
    monkeypatch.setitem(replay_check.RAW, name, raw)
    for mode in ("whole", "decode_tail", "mixed"):
        builder = getattr(replay_cases, mode)
        steps, rows = builder(requests, MAX_TOKENS, seed=5) if mode == "mixed" else builder(requests)
        runner = ModelRunner(config=config, tensors=tensors, dtype=dtype, device="cuda", page_size=16,
                             num_pages=MAX_TOKENS // 16, max_seqs=4, max_step_tokens=MAX_TOKENS,
                             max_model_len=MAX_TOKENS)
        replay_check.run_and_check(runner, name, LENGTHS, steps, rows, dtype,
                                   BF16_TOLERANCE if dtype == torch.bfloat16 else None)
