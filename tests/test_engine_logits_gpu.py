"""What the engine samples from, tapped step by step on the GPU, in 32-bit and in bfloat16:
the logits of every generated token against the plain implementation, under a cold cache, a
warm prefix cache, a pool so small that requests are preempted and recomputed, and each of
the three admission policies; pages are poisoned with NaN whenever they change hands. And
three of the random engine scenarios of the CPU suite on the GPU's own kernels."""

from __future__ import annotations

import numpy as np
import pytest
import torch

from plain_qwen2 import plain_generate, plain_logits
from test_engine_fuzz import play, scenario
from tiny import PAGE_SIZE, RAW, random_tokens, tiny_model

pytestmark = pytest.mark.gpu

TOLERANCE = {"float32": 3e-5, "bfloat16": 2e-2}


def make_engine(name, dtype="float32", num_blocks=64, policy="fcfs", max_running=4, chunk=24,
                budget=64, model_len=192, lookahead=True, prefix_caching=True):
    from mercury_b200 import Engine, EngineConfig
    from mercury_b200.engine.runner import ModelRunner

    _raw, config, tensors = tiny_model(name)
    page = PAGE_SIZE[name]
    runner = ModelRunner(config=config, tensors=tensors,
                         dtype=torch.float32 if dtype == "float32" else torch.bfloat16,
                         device="cuda", page_size=page, num_pages=num_blocks, max_seqs=max_running,
                         max_step_tokens=budget, max_model_len=model_len, poison_pages=True)
    cfg = EngineConfig(model="(memory)", dtype=dtype, block_size=page, num_blocks=num_blocks,
                       max_running=max_running, max_batched_tokens=budget, prefill_chunk=chunk,
                       max_model_len=model_len, policy=policy, debug_invariants=True,
                       lookahead=lookahead, prefix_caching=prefix_caching)
    return Engine(cfg, runner=runner)


def generate_tapped(engine, prompts, max_tokens):
    """Tokens per prompt, and for each (prompt, output index) the logits row it was
    sampled from (the last one seen, if a request was recomputed after a preemption)."""
    from mercury_b200 import SamplingParams

    rows: dict[tuple[int, int], np.ndarray] = {}
    names = {f"gen-{engine._submitted + i}": i for i in range(len(prompts))}

    def tap(requests, logits):
        data = logits.float().cpu().numpy()
        for row, r in enumerate(requests):
            rows[(names[r.rid], len(r.out))] = data[row].copy()

    engine.tap = tap
    try:
        outs = engine.generate(prompts, SamplingParams(), max_tokens)
    finally:
        engine.tap = None
    return outs, rows


def check_against_plain(raw, tensors, prompts, outs, rows, tolerance, what):
    """Every tapped row against the plain implementation's logits for the engine's own
    tokens; a token other than the plain argmax is allowed only where the two candidates'
    true logits lie within the tolerance of each other."""
    for i, (prompt, out) in enumerate(zip(prompts, outs)):
        want = plain_logits(raw, tensors, prompt + out).numpy()
        scale = float(np.abs(want).max())
        for index, token in enumerate(out):
            ref = want[len(prompt) + index - 1]
            got = rows[(i, index)]
            assert np.isfinite(got).all(), f"{what}: request {i} output {index}: non-finite logits"
            err = float(np.abs(got - ref).max()) / scale
            assert err <= tolerance, f"{what}: request {i} output {index}: relative error {err:.2e}"
            assert float(ref.max() - ref[token]) <= 2 * tolerance * scale, (
                f"{what}: request {i} output {index}: token {token} is not (nearly) the best")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_logits_under_cold_and_warm_cache_preemption_and_policies(dtype):
    name = "A"
    raw, _cfg, tensors = tiny_model(name)
    shared = random_tokens(48, 256, 77)
    prompts = [shared + random_tokens(n, 256, 80 + n) for n in (3, 20, 9, 31)]
    tol = TOLERANCE[dtype]
    engine = make_engine(name, dtype)
    cold, rows = generate_tapped(engine, prompts, 10)
    check_against_plain(raw, tensors, prompts, cold, rows, tol, "cold cache")
    hits = engine.cache.stats["hit_tokens"]
    warm, rows = generate_tapped(engine, prompts, 10)
    assert engine.cache.stats["hit_tokens"] >= hits + 4 * 48, "the second pass was meant to hit"
    check_against_plain(raw, tensors, prompts, warm, rows, tol, "warm cache")
    for policy in ("lpm", "lpm_aging"):
        outs, rows = generate_tapped(make_engine(name, dtype, policy=policy), prompts, 10)
        check_against_plain(raw, tensors, prompts, outs, rows, tol, policy)
    tight = make_engine(name, dtype, num_blocks=13)
    outs, rows = generate_tapped(tight, prompts, 10)
    assert tight.sched.stats["preemptions"] > 0, "the pool was meant to run out"
    check_against_plain(raw, tensors, prompts, outs, rows, tol, "small pool")
    assert tight.leaked_pages() == 0
    if dtype == "float32":
        want = [plain_generate(raw, tensors, p, 10) for p in prompts]
        assert cold == want and warm == want and outs == want


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", [1, 4, 7])
def test_random_scenarios_on_the_gpu(seed, dtype):
    """Scenarios of the CPU suite (arrivals over time, small pools, policies, portions,
    end-of-sequence tokens, sampling, aborts) on the CUDA kernels: launching ahead changes
    no token, and in 32-bit the greedy requests give the plain implementation's tokens."""
    sc = scenario(seed)
    aborts = sc[-1]

    def factory(name, lookahead, **engine_args):
        return make_engine(name, dtype, lookahead=lookahead, **engine_args)

    plain, _ = play(False, *sc, factory=factory)
    ahead, _engine = play(True, *sc, factory=factory)
    for i in plain:
        if i in aborts:
            short, long_ = sorted((plain[i]["tokens"], ahead[i]["tokens"]), key=len)
            assert long_[:len(short)] == short
        else:
            assert ahead[i] == plain[i], f"request {i}"
    if dtype != "float32":
        return
    name, prompts, limits, params, _arrive, _args, eos, _aborts = sc
    raw, _config, tensors = tiny_model(name)
    for i, p in enumerate(params):
        if not p.greedy or i in aborts:
            continue
        want = plain_generate(raw, tensors, prompts[i], limits[i])
        if not p.ignore_eos:
            ends = [j for j, token in enumerate(want) if token in eos]
            want = want[:ends[0] + 1] if ends else want
        assert ahead[i]["tokens"] == want, f"request {i}"
