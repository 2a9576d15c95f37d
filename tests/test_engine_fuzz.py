"""Random scenarios on the CPU (PyTorch kernel twins): requests that arrive over time, small
pools, every policy, portions of every size, end-of-sequence tokens, sampling and aborts.
Launching a step ahead must change no request's tokens or ending, greedy requests must give
the plain implementation's tokens, no page may leak, and no stand-in may reach a sink."""

from __future__ import annotations

import random

import pytest

from plain_qwen2 import plain_generate
from test_engine_cpu import make_engine
from tiny import PAGE_SIZE, RAW, random_tokens, tiny_model


def scenario(seed: int):
    from mercury_b200 import SamplingParams

    rng = random.Random(seed)
    name = rng.choice(["A", "B", "C"])
    vocab, page = RAW[name]["vocab_size"], PAGE_SIZE[name]
    count = rng.randint(2, 9)
    shared = random_tokens(rng.randint(0, 40), vocab, seed * 7 + 1)
    prompts, limits, params, arrive = [], [], [], []
    for i in range(count):
        own = random_tokens(rng.randint(1, 50), vocab, seed * 100 + i)
        prompts.append(shared + own if rng.random() < 0.5 else own)
        limits.append(rng.randint(1, 14))
        params.append(SamplingParams(temperature=rng.choice([0.0, 0.0, 0.7, 1.3]),
                                     top_p=rng.choice([1.0, 0.9]), seed=rng.randint(0, 99),
                                     ignore_eos=rng.random() < 0.2))
        arrive.append(rng.randint(0, 12))
    longest = max(len(p) + n for p, n in zip(prompts, limits))
    model_len = max(64, -(-longest // page) * page)
    least = model_len // page
    engine_args = dict(
        num_blocks=rng.choice([least, least + 2, least * 2, 64 + least]),
        policy=rng.choice(["fcfs", "lpm", "lpm_aging"]), max_running=rng.choice([1, 2, 4, 4]),
        chunk=rng.choice([2, 5, 16, 24, 64]), budget=rng.choice([8, 16, 64]),
        model_len=model_len, prefix_caching=rng.random() < 0.7)
    eos = set(rng.sample(range(vocab), rng.choice([0, 0, 8, 40])))
    aborts = {rng.randrange(count): rng.randint(0, 15)} if rng.random() < 0.3 else {}
    return name, prompts, limits, params, arrive, engine_args, eos, aborts


def play(lookahead, name, prompts, limits, params, arrive, engine_args, eos, aborts,
         factory=make_engine):
    """Requests are submitted (and aborted) at their step numbers; per request its tokens
    and how it ended, and the engine."""
    engine = factory(name, lookahead, **engine_args)
    engine.eos_ids = set(eos)
    got = {i: {"tokens": [], "index": [], "end": None} for i in range(len(prompts))}

    def sink_for(i):
        def sink(event):
            assert got[i]["end"] is None, "an event after the request's end"
            if event.kind == "token":
                got[i]["tokens"].append(event.token)
                got[i]["index"].append(event.index)
            elif event.kind in ("done", "error"):
                got[i]["end"] = event.finish_reason or event.message
        return sink

    waiting = sorted(range(len(prompts)), key=lambda i: arrive[i])
    tick = 0
    while waiting or engine.sched.has_work() or engine._commands or engine._flight is not None:
        while waiting and arrive[waiting[0]] <= tick:
            i = waiting.pop(0)
            engine.submit(f"r{i}", prompts[i], limits[i], sink_for(i), params[i],
                          arrival=float(arrive[i]))
        for i, when in aborts.items():
            if when == tick:
                engine.abort(f"r{i}")
        engine.step()
        tick += 1
        assert tick < 3000, "the engine does not come to an end"
    assert engine.leaked_pages() == 0
    engine.cache.check_invariants()
    for entry in got.values():
        assert entry["end"] is not None
        assert entry["index"] == list(range(len(entry["tokens"])))
        assert -1 not in entry["tokens"]
    return got, engine


SEEDS = list(range(10))


@pytest.mark.parametrize("seed", SEEDS)
def test_random_scenarios_with_and_without_launching_ahead(seed):
    sc = scenario(seed)
    aborts = sc[-1]
    plain, _ = play(False, *sc)
    ahead, _engine = play(True, *sc)
    for i in plain:
        if i in aborts:
            # the abort meets the request at another point of its life: one output is a
            # prefix of the other
            short, long_ = sorted((plain[i]["tokens"], ahead[i]["tokens"]), key=len)
            assert long_[:len(short)] == short
        else:
            assert ahead[i] == plain[i], f"request {i}"
    # greedy requests against the plain implementation (whole sequences, no cache)
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


def test_the_scenarios_cover_what_they_are_meant_to():
    ahead = preempted = stopped = aborted = sampled = 0
    for seed in SEEDS:
        sc = scenario(seed)
        got, engine = play(True, *sc)
        ahead += engine.metrics.counters["steps_launched_ahead"]
        preempted += engine.sched.stats["preemptions"]
        stopped += sum(1 for e in got.values() if e["end"] == "stop")
        aborted += sum(1 for e in got.values() if e["end"] == "abort")
        sampled += sum(1 for p in sc[3] if not p.greedy)
    assert ahead > 20 and preempted > 0 and stopped > 0 and aborted > 0 and sampled > 0, (
        ahead, preempted, stopped, aborted, sampled)
