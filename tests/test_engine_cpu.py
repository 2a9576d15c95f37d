"""The engine loop on the CPU (PyTorch kernel twins): launching a step ahead of reading the
step in front must not change any request's tokens, whatever ends the requests (length, an
end-of-sequence token met on the way, an abort), however few pages there are."""

from __future__ import annotations

import pytest
import torch

from kernel_twins import TorchOps
from plain_qwen2 import plain_generate
from tiny import PAGE_SIZE, RAW, random_tokens, tiny_model


def make_engine(name, lookahead, num_blocks=64, policy="fcfs", max_running=4, chunk=24,
                budget=64, model_len=192, prefix_caching=True):
    from mercury_b200 import Engine, EngineConfig
    from mercury_b200.engine.runner import ModelRunner

    _raw, config, tensors = tiny_model(name)
    page = PAGE_SIZE[name]
    runner = ModelRunner(config=config, tensors=tensors, dtype=torch.float32, device="cpu",
                         page_size=page, num_pages=num_blocks, max_seqs=max_running,
                         max_step_tokens=budget, max_model_len=model_len, ops=TorchOps())
    cfg = EngineConfig(model="(memory)", device="cpu", dtype="float32", block_size=page,
                       num_blocks=num_blocks, max_running=max_running, max_batched_tokens=budget,
                       prefill_chunk=chunk, max_model_len=model_len, policy=policy,
                       debug_invariants=True, lookahead=lookahead, prefix_caching=prefix_caching)
    return Engine(cfg, runner=runner)


def run(engine, prompts, max_tokens, eos=(), params=None):
    """Submit everything, step until idle; per request its tokens and why it ended."""
    from mercury_b200 import SamplingParams

    engine.eos_ids = set(eos)
    got = {i: {"tokens": [], "index": [], "reason": None} for i in range(len(prompts))}

    def sink_for(i):
        def sink(event):
            if event.kind == "token":
                got[i]["tokens"].append(event.token)
                got[i]["index"].append(event.index)
            elif event.kind == "done":
                got[i]["reason"] = event.finish_reason
        return sink

    for i, (prompt, limit) in enumerate(zip(prompts, max_tokens)):
        engine.submit(f"r{i}", prompt, limit, sink_for(i),
                      params[i] if params else SamplingParams(), arrival=float(i))
    engine.run_until_idle()
    assert engine.leaked_pages() == 0
    for entry in got.values():
        assert entry["index"] == list(range(len(entry["tokens"])))
        assert -1 not in entry["tokens"]
    return [(got[i]["tokens"], got[i]["reason"]) for i in range(len(prompts))]


@pytest.mark.parametrize("name", ["A", "B"])
def test_launching_ahead_changes_no_token(name):
    raw, _config, tensors = tiny_model(name)
    vocab = RAW[name]["vocab_size"]
    prompts = [random_tokens(n, vocab, 60 + i) for i, n in enumerate((5, 17, 33, 60, 44, 9))]
    limits = [12, 3, 9, 1, 7, 15]
    want = [plain_generate(raw, tensors, p, n) for p, n in zip(prompts, limits)]
    sync = run(make_engine(name, False), prompts, limits)
    assert [t for t, _ in sync] == want and all(reason == "length" for _t, reason in sync)
    engine = make_engine(name, True)
    assert run(engine, prompts, limits) == sync
    assert engine.metrics.counters["steps_launched_ahead"] > 5

    # an end-of-sequence token met on the way: the third token of the longest output
    eos = want[5][2]
    stopped = run(make_engine(name, False), prompts, limits, eos=[eos])
    assert stopped[5][1] == "stop" and stopped[5][0] == want[5][:want[5].index(eos) + 1]
    engine = make_engine(name, True)
    assert run(engine, prompts, limits, eos=[eos]) == stopped
    assert engine.metrics.counters["surplus_tokens"] >= 1     # the price of finding out late


def test_launching_ahead_with_few_pages_sampling_and_every_policy():
    from mercury_b200 import SamplingParams

    name = "A"
    raw, _config, tensors = tiny_model(name)
    shared = random_tokens(48, 256, 77)
    prompts = [shared + random_tokens(n, 256, 80 + n) for n in (3, 20, 9, 31, 14)]
    limits = [10, 6, 10, 4, 8]
    params = [SamplingParams(temperature=0.8, seed=3 + i) if i % 2 else SamplingParams()
              for i in range(5)]
    base = run(make_engine(name, False), prompts, limits, params=params)
    for kwargs in ({}, {"policy": "lpm"}, {"policy": "lpm_aging"}, {"num_blocks": 13},
                   {"max_running": 2}, {"prefix_caching": False}, {"chunk": 7, "budget": 16}):
        engine = make_engine(name, True, **kwargs)
        assert run(engine, prompts, limits, params=params) == base, kwargs
        assert engine.metrics.counters["steps_launched_ahead"] > 0, kwargs
    tight = make_engine(name, True, num_blocks=13)
    run(tight, prompts, limits, params=params)
    assert tight.sched.stats["preemptions"] > 0, "the pool was meant to run out"


def test_abort_while_a_step_is_under_way():
    name = "B"
    vocab = RAW[name]["vocab_size"]
    prompts = [random_tokens(n, vocab, 90 + i) for i, n in enumerate((12, 30, 21))]
    engine = make_engine(name, True)
    events = {i: [] for i in range(3)}
    for i, prompt in enumerate(prompts):
        engine.submit(f"r{i}", prompt, 20, events[i].append, arrival=float(i))
    for _ in range(6):
        engine.step()
    assert engine._flight is not None, "a step was meant to be under way"
    engine.abort("r1")
    engine.run_until_idle()
    assert events[1][-1].kind == "done" and events[1][-1].finish_reason == "abort"
    assert all(e.token != -1 for i in events for e in events[i] if e.kind == "token")
    assert [len([e for e in events[i] if e.kind == "token"]) for i in (0, 2)] == [20, 20]
    assert engine.leaked_pages() == 0 and not engine.sched.has_work()
    aborted = [r for r in engine.metrics.finished if r["rid"] == "r1"][0]
    assert aborted["output_tokens"] == len([e for e in events[1] if e.kind == "token"])


def test_a_refused_generate_call_leaves_nothing_queued():
    name = "A"
    vocab = RAW[name]["vocab_size"]
    engine = make_engine(name, True)
    good = random_tokens(9, vocab, 5)
    with pytest.raises(ValueError, match="outside the vocabulary"):
        engine.generate([good, [vocab + 3]], max_tokens=4)
    assert not engine._commands and not engine._sinks
    # the engine goes on as if the refused call had not been made
    tokens = engine.generate([good], max_tokens=4)
    assert len(tokens) == 1 and len(tokens[0]) == 4
    assert engine.metrics.counters["finished_requests"] == 1
    assert engine.leaked_pages() == 0


def test_a_name_in_use_is_refused():
    name = "A"
    vocab = RAW[name]["vocab_size"]
    engine = make_engine(name, True)
    first, second = [], []
    engine.submit("same", random_tokens(7, vocab, 1), 3, first.append)
    engine.submit("same", random_tokens(5, vocab, 2), 3, second.append)
    assert [e.kind for e in second] == ["error"] and "still under way" in second[0].message
    engine.run_until_idle()
    assert [e.kind for e in first] == ["token"] * 3 + ["done"]
    # once it has ended the name is free again
    engine.submit("same", random_tokens(5, vocab, 2), 2, second.append)
    engine.run_until_idle()
    assert [e.kind for e in second] == ["error", "token", "token", "done"]
    assert engine.leaked_pages() == 0


def test_a_sink_that_raises_loses_its_request_not_the_loop():
    """mercury/engine.py:259-262: the request whose sink raised is aborted (its pages go
    back, its done-event is not delivered to the broken sink), the others finish."""
    from mercury_b200 import SamplingParams

    engine = make_engine("A", True)
    prompts = [random_tokens(n, 256, 90 + n) for n in (9, 21, 14)]
    good = {0: [], 2: []}
    seen = []

    def bad_sink(event):
        seen.append(event.kind)
        if event.kind == "token" and len([k for k in seen if k == "token"]) == 2:
            raise RuntimeError("the client went away")

    def sink_for(i):
        return lambda event: good[i].append(event.token if event.kind == "token" else event.finish_reason)

    engine.submit("r0", prompts[0], 6, sink_for(0), SamplingParams(), arrival=0.0)
    engine.submit("r1", prompts[1], 6, bad_sink, SamplingParams(), arrival=1.0)
    engine.submit("r2", prompts[2], 6, sink_for(2), SamplingParams(), arrival=2.0)
    engine.run_until_idle()
    raw, _config, tensors = tiny_model("A")
    for i in (0, 2):
        assert good[i] == plain_generate(raw, tensors, prompts[i], 6) + ["length"]
    assert seen.count("token") == 2, "no event may reach a sink after it raised"
    assert engine.metrics.counters["aborted_requests"] == 1
    assert engine.leaked_pages() == 0 and not engine.sched.has_work()
    assert [r["finish_reason"] for r in engine.metrics.finished if r["rid"] == "r1"] == ["abort"]
