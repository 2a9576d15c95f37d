"""Replay on the GPU, in 32-bit and in bfloat16: each request whole; most of it in one step
and the last 32 tokens one by one; portions of changing size down to two tokens; mixed,
up to four live requests with so few pages that they are used again; and mixed with
requests that start on the cached pages of an earlier request's equal prefix. Every written
row is compared with the plain implementation. Every runner here poisons its pages: a page
is filled with NaN whenever it changes hands, so a key read from beyond a sequence's length
or from a page's earlier owner shows as a non-finite logit."""

from __future__ import annotations

import json
import os
import subprocess
import sys
import tempfile
from pathlib import Path

import numpy as np
import pytest
import torch

import replay_cases
from replay_check import (TOLERANCE, oracle, oracle_shared, requests_for,
                          requests_with_shared_prefix, run_and_check, shared_prefix_case,
                          sharpened_model)
from tiny import PAGE_SIZE, RAW

pytestmark = pytest.mark.gpu

LENGTHS = {"A": (37, 70, 129, 200, 45, 96, 161), "B": (33, 64, 150, 41, 97, 208, 80),
           "C": (50, 131, 65, 190, 77, 40, 100), "D": (35, 120, 64, 201, 90, 47, 133),
           "E": (70, 33, 140, 90, 51)}
MAX_TOKENS = 512   # 8 pages of 64: the seven requests need far more, so pages come back


def make_runner(name, dtype, num_tokens=MAX_TOKENS):
    from mercury_b200.engine.runner import ModelRunner

    _raw, config, tensors = sharpened_model(name)
    page = PAGE_SIZE[name]
    return ModelRunner(config=config, tensors=tensors, dtype=dtype, device="cuda", page_size=page,
                       num_pages=num_tokens // page, max_seqs=4, max_step_tokens=num_tokens,
                       max_model_len=min(num_tokens, RAW[name]["max_position_embeddings"]),
                       poison_pages=True)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
@pytest.mark.parametrize("mode", ["whole", "decode_tail", "portions", "mixed"])
def test_replay_matches_plain(name, dtype, mode):
    lengths = LENGTHS[name]
    requests = requests_for(name, lengths)
    if mode == "whole":
        steps, rows = replay_cases.whole(requests)
    elif mode == "decode_tail":
        steps, rows = replay_cases.decode_tail(requests)
    elif mode == "portions":
        steps, rows = replay_cases.portions(requests)
    else:
        steps, rows = replay_cases.mixed(requests, MAX_TOKENS, seed=3)
    runner = make_runner(name, dtype)
    run_and_check(runner, name, lengths, steps, rows, dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
def test_replay_on_cached_prefixes(name, dtype):
    """Mixed replay with prefix caching: the requests of the second half begin with two
    pages and a bit of a request of the first half and start on its pages, which are still
    in the pool; positions behind a cached prefix keep their rotation and their logits. The
    pool is small enough for cached pages to be evicted and written anew."""
    shared, lengths, pool = shared_prefix_case(name)
    requests = requests_with_shared_prefix(name, lengths, shared)
    steps, rows = replay_cases.mixed(requests, pool, seed=4, max_live=2, first_portion=shared + 3)
    runner = make_runner(name, dtype, pool)
    run_and_check(runner, name, lengths, steps, rows, dtype,
                  want=oracle_shared(name, lengths, shared), replay_options={"prefix_caching": True})
    assert runner.cache.stats["hit_tokens"] >= 2 * PAGE_SIZE[name], "no request started on cached pages"
    assert sum(p.evictions for p in runner.cache.pools) > 0, "no cached page was ever evicted"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
def test_long_decoding(dtype):
    """One request decoded token by token over many pages, after a two-token start."""
    name, lengths = "A", (300,)
    requests = requests_for(name, lengths)
    steps, rows = replay_cases.decode_tail(requests, tail=298)
    runner = make_runner(name, dtype)
    run_and_check(runner, name, lengths, steps, rows, dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_first_tokens(name, dtype):
    """The first positions of a sequence, one token per step from the very first."""
    lengths = (6, 1, 2, 3)
    requests = requests_for(name, lengths)
    steps, rows = replay_cases.decode_tail(requests, tail=64)
    runner = make_runner(name, dtype)
    run_and_check(runner, name, lengths, steps, rows, dtype)


def test_weights_stored_in_32_bit_stay_so_in_the_bfloat16_engine():
    """A checkpoint stored in float32, run by the bfloat16 engine: the weights stay 32-bit,
    the products fall to the kernels that take such weights, and the result is at least as
    close to the oracle as with bfloat16 weights."""
    from mercury_b200.engine.runner import ModelRunner

    name, lengths = "B", LENGTHS["B"][:4]
    _raw, config, tensors = sharpened_model(name)
    wide = {k: v.float() for k, v in tensors.items()}
    requests = requests_for(name, lengths)
    steps, rows = replay_cases.mixed(requests, 512, seed=2)
    page = PAGE_SIZE[name]
    runner = ModelRunner(config=config, tensors=wide, dtype=torch.bfloat16, device="cuda",
                         page_size=page, num_pages=512 // page, max_seqs=4, max_step_tokens=512,
                         max_model_len=512, poison_pages=True)
    mixer = runner.model.blocks[0].mixer
    assert mixer.qkv_weight.dtype == torch.float32 and runner.model.embedding.table.dtype == torch.float32
    assert next(iter(runner.kv_layers.values()))[0].dtype == torch.bfloat16
    run_and_check(runner, name, lengths, steps, rows, torch.bfloat16)


@pytest.mark.parametrize("switches", [(), ("--prefix-caching", "--poison-pages")],
                         ids=["plain", "prefix+poison"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(dtype, switches, tmp_path):
    """The program itself, as a user runs it: a model folder, steps on standard input."""
    from mercury_b200.weights import write_random_model

    name = "B"
    _raw, config, tensors = sharpened_model(name)
    folder = tmp_path / "model"
    write_random_model(folder, config, seed=0)
    from safetensors.torch import save_file

    save_file({k: v.contiguous() for k, v in tensors.items()}, str(folder / "model.safetensors"))
    lengths = LENGTHS[name][:4]
    requests = requests_for(name, lengths)
    steps, rows = replay_cases.mixed(requests, 512, seed=1)
    root = Path(__file__).resolve().parent.parent
    out = tmp_path / "out"
    done = subprocess.run(
        [str(root / "bin" / "trace_run"), "--model", str(folder), "--dtype", dtype, "--out",
         str(out), "--max-tokens", "512", "--block-size", str(PAGE_SIZE[name]), *switches],
        input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True,
        timeout=600)
    assert done.returncode == 0, done.stderr
    assert done.stdout.split("\n")[:-1] == [f"done {s['step']}" for s in steps]
    want = oracle(name, LENGTHS[name])
    tol = TOLERANCE[torch.float32 if dtype == "float32" else torch.bfloat16]
    for step, expected in rows.items():
        got = np.fromfile(out / f"{step}.f32", dtype="<f4").reshape(len(expected), -1)
        for row, (rid, pos) in enumerate(expected):
            err = np.abs(got[row] - want[rid][pos]).max() / np.abs(want[rid]).max()
            assert err <= tol, (step, rid, pos, err)
