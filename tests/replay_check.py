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
from tiny import PAGE_SIZE, RAW, random_tokens, tiny_model

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
def requests_with_shared_prefix(name: str, lengths: tuple[int, ...], shared: int) -> dict:
    """Like `requests_for`, but each request of the second half begins with the first
    `shared` tokens of its counterpart in the first half (which, in a replay that admits
    them in order, has finished or is well under way by then)."""
    requests = {rid: list(tokens) for rid, tokens in requests_for(name, lengths).items()}
    names = list(requests)
    half = len(names) // 2
    for before, rid in zip(names[:half], names[half:]):
        n = min(shared, len(requests[rid]) - 1, len(requests[before]))
        requests[rid][:n] = requests[before][:n]
    return requests


def shared_prefix_case(name: str) -> tuple[int, tuple[int, ...], int]:
    """(shared tokens, request lengths, pool size in tokens) of the shared-prefix replay of
    a tiny model: two pages and five tokens shared, every request long enough to hold them
    before its tail, and a pool that holds about half of what the requests need together."""
    shared = 2 * PAGE_SIZE[name] + 5
    lengths = tuple(shared + 34 + extra for extra in (3, 40, 17, 58, 9, 26))
    return shared, lengths, 256 if PAGE_SIZE[name] <= 16 else 512


@lru_cache(maxsize=None)
def oracle_shared(name: str, lengths: tuple[int, ...], shared: int) -> dict:
    raw, _config, tensors = sharpened_model(name)
    return {rid: plain_logits(raw, tensors, tokens).numpy()
            for rid, tokens in requests_with_shared_prefix(name, lengths, shared).items()}


@lru_cache(maxsize=None)
def oracle(name: str, lengths: tuple[int, ...]) -> dict:
    raw, _config, tensors = sharpened_model(name)
    return {rid: plain_logits(raw, tensors, tokens).numpy()
            for rid, tokens in requests_for(name, lengths).items()}


def run_and_check(runner, name, lengths, steps, rows, dtype, tolerance=None, want=None,
                  vocab=None, replay_options=None) -> float:
    """Replays `steps` on `runner`; returns the worst relative error seen. `want` maps a
    request id to its whole-sequence logits (default: the tiny model `name` through the
    plain implementation)."""
    tolerance = TOLERANCE[dtype] if tolerance is None else tolerance
    want = oracle(name, lengths) if want is None else want
    vocab = RAW[name]["vocab_size"] if vocab is None else vocab
    scale = {rid: float(np.abs(w).max()) for rid, w in want.items()}
    worst = 0.0
    with tempfile.TemporaryDirectory() as tmp:
        done = []
        replay(runner, [json.dumps(s) for s in steps], Path(tmp), done.append,
               **(replay_options or {}))
        assert done == [f"done {s['step']}" for s in steps]
        for step, expected in rows.items():
            path = Path(tmp) / f"{step}.f32"
            if not expected:
                assert not path.exists()
                continue
            got = np.fromfile(path, dtype="<f4").reshape(len(expected), vocab)
            for row, (rid, pos) in enumerate(expected):
                ref = want[rid][pos]
                err = float(np.abs(got[row].astype(np.float64) - ref).max() / scale[rid])
                assert np.isfinite(got[row]).all(), f"step {step} {rid}@{pos}: non-finite logits"
                assert err <= tolerance, (
                    f"step {step}: request {rid} position {pos}: relative error {err:.3e} "
                    f"exceeds {tolerance:.0e}")
                worst = max(worst, err)
    assert not runner.cache.live, "a finished request still holds pages"
    runner.cache.check_invariants()
    assert runner.cache.leaked_pages() == 0
    return worst
