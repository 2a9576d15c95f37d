"""Run a trace through `mercury_b200.trace_run.replay` and compare every written row with
the plain implementation's whole-sequence logits."""

from __future__ import annotations

import json
import tempfile
from functools import lru_cache
from pathlib import Path

import numpy as np
import torch

from mercury_b200.trace_run import replay
from plain_qwen2 import plain_logits
from tiny import RAW, random_tokens, tiny_model

# max |difference| allowed, as a fraction of the largest |logit| of the request.
# float32: kernels and oracle differ only in the order of float32 sums.
# bfloat16: activations and weights rounded to 8 bits of mantissa between kernels.
TOLERANCE = {torch.float32: 3e-5, torch.bfloat16: 2e-2}

SHARPEN = 4.0   # q and k projections are scaled so that attention is not nearly uniform


@lru_cache(maxsize=None)
def sharpened_model(name: str):
    raw, config, tensors = tiny_model(name)
    for key in tensors:
        if "q_proj" in key or "k_proj" in key:
            tensors[key] = (tensors[key].float() * SHARPEN).to(torch.bfloat16)
    return raw, config, tensors


@lru_cache(maxsize=None)
def requests_for(name: str, lengths: tuple[int, ...]) -> dict:
    vocab = RAW[name]["vocab_size"]
    return {f"r{i}": random_tokens(n, vocab, 100 + i) for i, n in enumerate(lengths)}


@lru_cache(maxsize=None)
def oracle(name: str, lengths: tuple[int, ...]) -> dict:
    raw, _config, tensors = sharpened_model(name)
    return {rid: plain_logits(raw, tensors, tokens).numpy()
            for rid, tokens in requests_for(name, lengths).items()}


def run_and_check(runner, name, lengths, steps, rows, dtype, tolerance=None) -> float:
    """Replays `steps` on `runner`; returns the worst relative error seen."""
    tolerance = TOLERANCE[dtype] if tolerance is None else tolerance
    want = oracle(name, lengths)
    vocab = RAW[name]["vocab_size"]
    worst = 0.0
    with tempfile.TemporaryDirectory() as tmp:
        done = []
        replay(runner, [json.dumps(s) for s in steps], Path(tmp), done.append)
        assert done == [f"done {s['step']}" for s in steps]
        for step, expected in rows.items():
            path = Path(tmp) / f"{step}.f32"
            if not expected:
                assert not path.exists()
                continue
            got = np.fromfile(path, dtype="<f4").reshape(len(expected), vocab)
            for row, (rid, pos) in enumerate(expected):
                ref = want[rid][pos]
                err = float(np.abs(got[row].astype(np.float64) - ref).max() / np.abs(want[rid]).max())
                assert np.isfinite(got[row]).all(), f"step {step} {rid}@{pos}: non-finite logits"
                assert err <= tolerance, (
                    f"step {step}: request {rid} position {pos}: relative error {err:.3e} "
                    f"exceeds {tolerance:.0e}")
                worst = max(worst, err)
    assert not runner.cache.live, "a finished request still holds pages"
    runner.cache.check_invariants()
    assert runner.cache.leaked_pages() == 0
    return worst
