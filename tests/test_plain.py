"""The plain implementation itself: properties its formulas must have, and the golden
comparison with the reference's own CPU model (tests/golden/)."""

from __future__ import annotations

import json
from pathlib import Path

import numpy as np
import pytest
import torch

import plain_qwen2 as P
from tiny import RAW, random_tokens, tiny_model

GOLDEN = Path(__file__).resolve().parent / "golden"


def test_rotate_half_and_relative_positions():
    x = torch.arange(8.0)
    assert P.plain_rotate_half(x).tolist() == [-4, -5, -6, -7, 0, 1, 2, 3]
    gen = torch.Generator().manual_seed(0)
    q = torch.randn(1, 1, 32, generator=gen, dtype=torch.float64)
    k = torch.randn(1, 1, 32, generator=gen, dtype=torch.float64)
    def score(pq, pk):
        a = P.plain_rope(q, P.plain_rope_angles(torch.tensor([pq]), 32, 1e4))
        b = P.plain_rope(k, P.plain_rope_angles(torch.tensor([pk]), 32, 1e4))
        return float((a * b).sum())
    assert abs(score(10, 3) - score(107, 100)) < 1e-4   # angles are float32, as in the reference


def test_later_tokens_do_not_change_earlier_logits():
    raw, _cfg, tensors = tiny_model("B")
    tokens = random_tokens(30, raw["vocab_size"], 3)
    full = P.plain_logits(raw, tensors, tokens)
    head = P.plain_logits(raw, tensors, tokens[:12])
    assert torch.allclose(full[:12], head, atol=1e-12)


def test_window_hides_old_keys_only_in_windowed_layers():
    raw, _cfg, tensors = tiny_model("C")           # window 24 from layer 1 on
    tokens = random_tokens(60, raw["vocab_size"], 4)
    changed = [(t + 1) % raw["vocab_size"] for t in tokens[:5]] + tokens[5:]
    a = P.plain_logits(raw, tensors, tokens)
    b = P.plain_logits(raw, tensors, changed)
    assert not torch.allclose(a[40], b[40])        # layer 0 still sees everything
    q = torch.randn(40, 2, 16, dtype=torch.float64)
    k, v = torch.randn(40, 1, 16, dtype=torch.float64), torch.randn(40, 1, 16, dtype=torch.float64)
    v2 = v.clone()
    v2[:10] += 1.0
    assert torch.equal(P.plain_attention(q, k, v, 0.25, 8)[20:], P.plain_attention(q, k, v2, 0.25, 8)[20:])
    assert not torch.equal(P.plain_attention(q, k, v, 0.25, 0)[20:], P.plain_attention(q, k, v2, 0.25, 0)[20:])


def test_sampling_rules():
    logits = torch.tensor([0.0, 3.0, 3.0, 1.0])
    assert P.plain_sample(logits, 0.0, 1.0, 0.9) == 1           # greedy, lowest index on ties
    probs = P.plain_probabilities(logits, 1.0, 0.5)
    assert probs[0] == 0 and probs[3] == 0 and abs(float(probs.sum()) - 1) < 1e-12
    assert P.plain_sample(logits, 1.0, 1.0, 0.0) == 0 and P.plain_sample(logits, 1.0, 1.0, 0.9999) == 3
    us = [P.plain_uniform(7, i) for i in range(2000)]
    assert all(0 <= u < 1 for u in us) and abs(sum(us) / 2000 - 0.5) < 0.03
    assert P.plain_uniform(7, 0) != P.plain_uniform(8, 0)


@pytest.mark.parametrize("name", ["A", "B", "D", "E"])
def test_plain_matches_the_reference_model(name):
    """Logits the reference's own Qwen2ForCausalLM produced on the CPU in float32 for the
    same random weights (made once by tests/golden/make_golden.py, stored as float32)."""
    meta = json.loads((GOLDEN / f"tiny_{name}.json").read_text())
    want = np.fromfile(GOLDEN / f"tiny_{name}.f32", dtype="<f4").reshape(meta["shape"])
    raw, _cfg, tensors = tiny_model(name)
    assert raw == meta["config"]
    got = P.plain_logits(raw, tensors, meta["tokens"], dtype=torch.float64).numpy()
    err = np.abs(got - want).max() / np.abs(want).max()
    assert err < 1e-5, err
