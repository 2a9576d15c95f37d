"""Generation through the Python entry point on the GPU: greedy and sampled tokens against
the plain implementation; batching, a warm prefix cache, forced preemption and every
policy must not change a request's tokens."""

from __future__ import annotations

import json
import subprocess
import sys
from pathlib import Path

import pytest
import torch

from plain_qwen2 import plain_generate, plain_logits
from tiny import PAGE_SIZE, RAW, random_tokens, tiny_model

pytestmark = pytest.mark.gpu


def make_engine(name, dtype="float32", num_blocks=64, policy="fcfs", max_running=4, chunk=24,
                budget=64, model_len=192, lookahead=True):
    from mercury_b200 import Engine, EngineConfig
    from mercury_b200.engine.runner import ModelRunner

    _raw, config, tensors = tiny_model(name)
    page = PAGE_SIZE[name]
    runner = ModelRunner(config=config, tensors=tensors,
                         dtype=torch.float32 if dtype == "float32" else torch.bfloat16,
                         device="cuda", page_size=page, num_pages=num_blocks, max_seqs=max_running,
                         max_step_tokens=budget, max_model_len=model_len)
    cfg = EngineConfig(model="(memory)", dtype=dtype, block_size=page, num_blocks=num_blocks,
                       max_running=max_running, max_batched_tokens=budget, prefill_chunk=chunk,
                       max_model_len=model_len, policy=policy, debug_invariants=True,
                       lookahead=lookahead)
    return Engine(cfg, runner=runner)


def prompts_for(name, lengths=(5, 17, 33, 60, 44)):
    return [random_tokens(n, RAW[name]["vocab_size"], 40 + i) for i, n in enumerate(lengths)]


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_greedy_generation_equals_plain(name):
    from mercury_b200 import SamplingParams

    raw, _cfg, tensors = tiny_model(name)
    prompts = prompts_for(name)
    engine = make_engine(name)
    outs = engine.generate(prompts, SamplingParams(), max_tokens=8)
    assert outs == [plain_generate(raw, tensors, p, 8) for p in prompts]
    assert engine.leaked_pages() == 0


def test_bfloat16_greedy_tokens_are_near_best():
    """In bfloat16 a close second may win; each chosen token's true logit must be within
    the bfloat16 tolerance of the best, given the engine's own earlier tokens."""
    from mercury_b200 import SamplingParams

    raw, _cfg, tensors = tiny_model("B")
    prompts = prompts_for("B")
    outs = make_engine("B", "bfloat16").generate(prompts, SamplingParams(), max_tokens=6)
    for prompt, out in zip(prompts, outs):
        logits = plain_logits(raw, tensors, prompt + out)
        for i, token in enumerate(out):
            row = logits[len(prompt) + i - 1]
            assert float(row.max() - row[token]) <= 2e-2 * float(logits.abs().max())


def test_sampled_generation_equals_plain_and_ignores_batching():
    from mercury_b200 import SamplingParams

    raw, _cfg, tensors = tiny_model("B")
    prompts = prompts_for("B", (1, 9, 24, 40))
    params = [SamplingParams(temperature=0.7, seed=11 + i) for i in range(4)]
    together = make_engine("B").generate(prompts, params, max_tokens=6)
    alone = [make_engine("B", max_running=1).generate([p], [q], max_tokens=6)[0]
             for p, q in zip(prompts, params)]
    assert together == alone
    want = [plain_generate(raw, tensors, p, 6, temperature=0.7, seed=11 + i)
            for i, p in enumerate(prompts)]
    assert together == want
    nucleus = make_engine("B").generate(prompts[:2], SamplingParams(temperature=1.0, top_p=0.3, seed=5), 6)
    assert nucleus == [plain_generate(raw, tensors, p, 6, temperature=1.0, top_p=0.3, seed=5)
                       for p in prompts[:2]]


def test_warm_prefix_cache_preemption_and_policies_keep_the_tokens():
    from mercury_b200 import SamplingParams

    raw, _cfg, tensors = tiny_model("A")
    shared = random_tokens(48, 256, 77)
    prompts = [shared + random_tokens(n, 256, 80 + n) for n in (3, 20, 9, 31)]
    want = [plain_generate(raw, tensors, p, 10) for p in prompts]
    engine = make_engine("A")
    assert engine.generate(prompts, SamplingParams(), 10) == want
    hits_before = engine.cache.stats["hit_tokens"]
    assert engine.generate(prompts, SamplingParams(), 10) == want      # warm cache
    assert engine.cache.stats["hit_tokens"] > hits_before
    for policy in ("lpm", "lpm_aging"):
        assert make_engine("A", policy=policy).generate(prompts, SamplingParams(), 10) == want
    tight = make_engine("A", num_blocks=13, model_len=192)
    assert tight.generate(prompts, SamplingParams(), 10) == want
    assert tight.sched.stats["preemptions"] > 0, "the pool was meant to run out"
    assert tight.leaked_pages() == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_launching_ahead_changes_no_token_on_the_device(dtype):
    """The step after the one in flight takes its token ids from the device (patch_tokens):
    same tokens and same reasons to end as with every step read back first, with requests
    ending by length at different times and one ending on an end-of-sequence token."""
    from mercury_b200 import SamplingParams

    name = "B"
    prompts = prompts_for(name, (5, 17, 33, 60, 44, 9))
    limits = [12, 3, 9, 1, 7, 15]

    def run(lookahead, eos):
        engine = make_engine(name, dtype, lookahead=lookahead)
        engine.eos_ids = set(eos)
        got = {i: [[], None] for i in range(len(prompts))}

        def sink_for(i):
            def sink(event):
                if event.kind == "token":
                    got[i][0].append(event.token)
                elif event.kind == "done":
                    got[i][1] = event.finish_reason
            return sink

        for i, (prompt, limit) in enumerate(zip(prompts, limits)):
            engine.submit(f"r{i}", prompt, limit, sink_for(i), SamplingParams(), arrival=float(i))
        engine.run_until_idle()
        assert engine.leaked_pages() == 0
        return [tuple(map(tuple, [got[i][0]])) + (got[i][1],) for i in range(len(prompts))], engine

    plain, _ = run(False, ())
    ahead, engine = run(True, ())
    assert ahead == plain and engine.metrics.counters["steps_launched_ahead"] > 5
    eos = plain[5][0][2]                       # the third token of the longest output
    stopped, _ = run(False, (eos,))
    assert stopped[5][1] == "stop"
    ahead, engine = run(True, (eos,))
    assert ahead == stopped and engine.metrics.counters["surplus_tokens"] >= 1


def test_refusals_and_events():
    from mercury_b200 import SamplingParams

    engine = make_engine("A")
    events = []
    engine.submit("empty", [], 4, events.append)
    engine.submit("long", [1] * 190, 10, events.append)
    engine.submit("alien", [1, 999], 4, events.append)
    assert [e.kind for e in events] == ["error"] * 3
    with pytest.raises(ValueError):
        engine.generate([[1, 2], []], SamplingParams(), 4)
    engine.run_until_idle()
    events.clear()
    engine.submit("ok", [1, 2, 3], 3, events.append, SamplingParams())
    engine.run_until_idle()
    assert [e.kind for e in events] == ["token", "token", "token", "done"]
    assert events[-1].finish_reason == "length" and [e.index for e in events[:3]] == [0, 1, 2]


def test_command_line(tmp_path):
    """python -m mercury_b200.generate with --random-weights, as a user would run it."""
    raw, _cfg, tensors = tiny_model("B")
    config = tmp_path / "config.json"
    config.write_text(json.dumps(raw))
    root = Path(__file__).resolve().parent.parent
    done = subprocess.run(
        [sys.executable, "-m", "mercury_b200.generate", "--model", str(tmp_path / "model"),
         "--random-weights", str(config), "--seed", "1", "--prompt-ids", "5,17,3,99",
         "--prompt-ids", "7 8 9", "--max-tokens", "5", "--dtype", "float32", "--block-size", "8",
         "--num-blocks", "32", "--max-running", "2", "--max-batched-tokens", "32"],
        capture_output=True, text=True, cwd=root, timeout=600)
    assert done.returncode == 0, done.stderr
    lines = [json.loads(line) for line in done.stdout.strip().splitlines()]
    assert [len(l["output_ids"]) for l in lines] == [5, 5]
    assert lines[0]["output_ids"] == plain_generate(raw, tensors, [5, 17, 3, 99], 5)
