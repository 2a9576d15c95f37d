"""bench.py's arithmetic and the parts of its contract that need no GPU."""

from __future__ import annotations

import json
import subprocess
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))


def test_bytes_and_flops_of_the_benchmark_model():
    import bench

    cfg = bench.QWEN25_05B
    numbers = bench.model_numbers(cfg)
    # per layer: q/k/v [1152, 896] + bias, o [896, 896], gate/up [9728, 896], down [896, 4864],
    # two norm weights; once: the head [151936, 896] and the final norm; two bytes each
    layer = 1152 * 896 + 1152 + 896 * 896 + 9728 * 896 + 896 * 4864 + 2 * 896
    assert numbers["weight_bytes"] == 2 * (24 * layer + 151936 * 896 + 896)
    # keys and values of one token: 24 layers x 2 KV heads x 64 x 2 tensors x 2 bytes
    assert numbers["kv_bytes_per_token"] == 24 * 2 * 64 * 2 * 2
    per_token = 2 * 24 * (1152 * 896 + 896 * 896 + 3 * 4864 * 896)
    assert numbers["gemm_flops_per_token"] == per_token
    # causal attention over T tokens: T^2 / 2 (query, key) pairs, 4 d flops each, per query head
    assert numbers["attn_flops"](2048) == 2 * 2048 * 2048 * 14 * 64 * 24


def test_more_than_one_gpu_is_refused_with_one_line_and_exit_code_two():
    done = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--gpus", "2"],
                          capture_output=True, text=True, timeout=120)
    assert done.returncode == 2
    assert len(done.stdout.strip().splitlines()) == 1


@pytest.mark.skipif(torch.cuda.is_available(), reason="with a GPU this would time the reference")
def test_the_reference_arm_answers_in_one_json_line_without_a_gpu():
    done = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference",
                           "--steps", "2", "--warmup", "1"], capture_output=True, text=True,
                          timeout=300)
    assert done.returncode == 0
    lines = done.stdout.strip().splitlines()
    assert len(lines) == 1
    record = json.loads(lines[0])
    assert record["impl"] == "reference"
    assert "value" in record or isinstance(record.get("unavailable"), str)


def test_both_arms_name_the_same_metric_and_config():
    import bench

    config = bench.bench_config("measured")
    assert len(config) <= 20 and all(not isinstance(v, (list, dict)) for v in config.values())
    assert config["layers"] == 24 and config["global_batch"] == 8 and config["seq_len"] == 2048
    assert "batch 8" in bench.METRIC


def test_class_costs_add_up_to_the_step():
    """The per-class bytes of a decode step sum to the step's bytes (weights once, the cache
    of the live requests), and the per-class flops of a prompt step to the step's flops."""
    import bench

    cfg = bench.QWEN25_05B
    numbers = bench.model_numbers(cfg)
    costs = bench.class_costs(cfg, 8, 2048, 2048)
    decode = costs["decode"]
    weights_and_cache = sum(decode[k][1] for k in ("q/k/v product", "attention", "residual product",
                                                    "gated product", "product"))
    norms = 2 * (24 * 2 * 896 + 896)
    assert weights_and_cache + norms == numbers["weight_bytes"] + 8 * 2048 * numbers["kv_bytes_per_token"]
    prefill = costs["prefill"]
    flops = sum(prefill[k][1] for k in ("q/k/v product", "attention", "residual product", "gated product"))
    assert flops == 2048 * numbers["gemm_flops_per_token"] + numbers["attn_flops"](2048)
