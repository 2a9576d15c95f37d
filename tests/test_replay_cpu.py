"""The replay program's logic without a GPU: the same traces as the GPU tests, run through
the step function on top of the PyTorch kernel twins. This checks the batch layout, the
block tables, page reuse and the window bookkeeping; the kernels are checked on the GPU."""

from __future__ import annotations

import pytest
import torch

import replay_cases
from kernel_twins import TorchOps
from replay_check import (oracle_shared, requests_for, requests_with_shared_prefix, run_and_check,
                          shared_prefix_case, sharpened_model)
from tiny import PAGE_SIZE, RAW

LENGTHS = {"A": (37, 70, 129, 45), "B": (33, 64, 150, 41), "C": (50, 131, 65, 90),
           "D": (35, 120, 64, 47), "E": (70, 33, 100, 51)}


def make_runner(name, num_tokens=320, poison=True):
    from mercury_b200.engine.runner import ModelRunner

    _raw, config, tensors = sharpened_model(name)
    page = PAGE_SIZE[name]
    return ModelRunner(config=config, tensors=tensors, dtype=torch.float32, device="cpu",
                       page_size=page, num_pages=num_tokens // page, max_seqs=4,
                       max_step_tokens=num_tokens, max_model_len=num_tokens, ops=TorchOps(),
                       poison_pages=poison)


@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
@pytest.mark.parametrize("mode", ["whole", "decode_tail", "portions", "mixed"])
def test_replay_logic(name, mode):
    lengths = LENGTHS[name]
    requests = requests_for(name, lengths)
    builder = getattr(replay_cases, mode)
    steps, rows = builder(requests, 320, seed=2) if mode == "mixed" else builder(requests)
    run_and_check(make_runner(name), name, lengths, steps, rows, torch.float32)


@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
def test_replay_logic_with_cached_prefixes(name):
    """The requests of the second half begin with two pages and a bit of a request of the
    first half and, with prefix caching, start on that request's pages, which are still in
    the pool (given back, or still held); the pool is small enough for cached pages to be
    taken away again."""
    shared, lengths, pool = shared_prefix_case(name)
    requests = requests_with_shared_prefix(name, lengths, shared)
    steps, rows = replay_cases.mixed(requests, pool, seed=4, max_live=2, first_portion=shared + 3)
    runner = make_runner(name, pool)
    run_and_check(runner, name, lengths, steps, rows, torch.float32,
                  want=oracle_shared(name, lengths, shared), replay_options={"prefix_caching": True})
    assert runner.cache.stats["hit_tokens"] >= 2 * PAGE_SIZE[name], "no request started on cached pages"
    assert sum(pool.evictions for pool in runner.cache.pools) > 0, "no cached page was ever evicted"
