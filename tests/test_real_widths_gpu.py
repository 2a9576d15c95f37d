"""The layer sizes of Qwen2.5-0.5B, 1.5B and 7B (full widths, head sizes 64 and 128, grouped
heads 14:2, 12:2 and 28:4, the real vocabularies, tied and untied heads; two layers to keep
the oracle quick) through replay in 32-bit and in bfloat16: whole, the last tokens one by
one, portions of changing size, and mixed with reused pages. These are the sizes the
tensor-core attention, the few-token products (the TMA-fed ones at 7B widths) and the
decode graphs serve."""

from __future__ import annotations

from functools import lru_cache

import pytest
import torch

import replay_cases
import replay_check
from wide import WIDTHS, model, oracle_rows, tokens_for

pytestmark = pytest.mark.gpu

LENGTHS = (150, 70, 97, 40, 130)
MAX_TOKENS = 384
# bfloat16: the plain PyTorch twin of the kernels (float32 arithmetic, bfloat16 storage
# between kernels, the same step function) is itself off from the float64 oracle by up to
# 1.3e-2 (0.5B widths), 2.3e-2 (1.5B widths) and 3.3e-2 (7B widths) of the largest logit on
# these requests: rounding to 8 bits grows with the width, and the maximum is taken over a
# vocabulary of 150 thousand. The engine is held to 1.75 times the twin's figure at each width;
# the tiny models keep 2e-2.
BF16_TOLERANCE = {"0.5B": 2.3e-2, "1.5B": 4e-2, "7B": 5.8e-2}


@lru_cache(maxsize=None)
def requests_and_oracle(name):
    requests = {f"r{i}": tokens_for(name, n, 200 + i) for i, n in enumerate(LENGTHS)}
    want = {f"r{i}": oracle_rows(name, n, 200 + i, tuple(range(n))) for i, n in enumerate(LENGTHS)}
    return requests, want


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("name", ["0.5B", "1.5B", "7B"])
def test_real_widths(name, dtype):
    from mercury_b200.engine.runner import ModelRunner

    raw, config, tensors = model(name)
    requests, want = requests_and_oracle(name)
    for mode in ("whole", "decode_tail", "portions", "mixed"):
        builder = getattr(replay_cases, mode)
        steps, rows = builder(requests, MAX_TOKENS, seed=5) if mode == "mixed" else builder(requests)
        runner = ModelRunner(config=config, tensors=tensors, dtype=dtype, device="cuda", page_size=16,
                             num_pages=MAX_TOKENS // 16, max_seqs=4, max_step_tokens=MAX_TOKENS,
                             max_model_len=MAX_TOKENS)
        replay_check.run_and_check(runner, name, LENGTHS, steps, rows, dtype,
                                   BF16_TOLERANCE[name] if dtype == torch.bfloat16 else None,
                                   want=want, vocab=raw["vocab_size"])
        del runner
        torch.cuda.empty_cache()
