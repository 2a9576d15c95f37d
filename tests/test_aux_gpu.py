"""The engine's aids for looking at itself, on the GPU: a bounded wait that runs out, the
checked build of the kernels, per-kernel-class timing, automatic sizing of the page pool,
and scratch memory that captured graphs still use after it was outgrown."""

from __future__ import annotations

import json
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

from plain_qwen2 import plain_generate, plain_logits
from tiny import PAGE_SIZE, RAW, random_tokens, tiny_model

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def test_a_wait_that_runs_out_is_reported_and_the_next_launch_is_right():
    """The tcgen05 product with the bytes of its first k-block announced and never sent, and
    a wait limit of about a millisecond: every role gives up in bounded time, the error
    word is set, `check_errors` raises, the output is left alone, and an ordinary launch on
    the same stream right after it computes the right product."""
    from mercury_b200.kernels import library
    from mercury_b200.kernels.library import KernelError
    from mercury_b200.kernels.ops import CudaOps

    ops = CudaOps("cuda", gemm="tcgen05")
    lib = library.load()
    gen = torch.Generator().manual_seed(3)
    x = torch.randn((300, 896), generator=gen).bfloat16().cuda()
    w = (torch.randn((200, 896), generator=gen) * 0.1).bfloat16().cuda()
    out = torch.full((300, 200), 7.0, dtype=torch.bfloat16, device="cuda")
    error = ops._error_word()
    rc = lib.mb_gemm_tcgen05_withheld(x.data_ptr(), w.data_ptr(), out.data_ptr(), 300, 200, 896,
                                      error.data_ptr(), 2_000_000,
                                      torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    ops._tc_pending = True
    with pytest.raises(KernelError, match="gave up waiting"):
        ops.check_errors()
    assert bool((out == 7.0).all()), "a product that gave up must not write its output"
    ops.linear(x, w, None, out)
    ops.check_errors()
    want = x.double() @ w.double().T
    assert float((out.double() - want).abs().max() / want.abs().max()) <= 5e-3


def test_checked_build_reports_bad_indices_and_runs_a_replay_clean():
    env = dict(os.environ, MERCURY_B200_BOUNDS_CHECK="1")
    done = subprocess.run([sys.executable, str(ROOT / "tests" / "checked_build_case.py")],
                          capture_output=True, text=True, env=env, timeout=900)
    assert done.returncode == 0, done.stderr[-3000:]
    out = json.loads(done.stdout.strip().splitlines()[-1])
    assert out["checked"] is True
    assert out["replay_float32"] <= 3e-5 and out["replay_bfloat16"] <= 2e-2
    assert out["good"] == "not reported" and out["good_again"] == "not reported"
    assert "a page number beyond the pool: 10 (limit 8)" in out["page"]
    assert "a block-table column beyond the table: 4 (limit 4)" in out["column"]
    assert "a position beyond the rotation tables: 64 (limit 64)" in out["position"]
    assert "a token id outside the vocabulary: 1000 (limit 300)" in out["token"]


def _engine(name, dtype="bfloat16", **more):
    from mercury_b200 import Engine, EngineConfig
    from mercury_b200.engine.runner import ModelRunner

    _raw, config, tensors = tiny_model(name)
    page = PAGE_SIZE[name]
    runner = ModelRunner(config=config, tensors=tensors,
                         dtype=torch.float32 if dtype == "float32" else torch.bfloat16, device="cuda",
                         page_size=page, num_pages=64, max_seqs=4, max_step_tokens=64, max_model_len=192)
    cfg = EngineConfig(model="(memory)", dtype=dtype, block_size=page, num_blocks=64, max_running=4,
                       max_batched_tokens=64, prefill_chunk=24, max_model_len=192, **more)
    return Engine(cfg, runner=runner)


def test_kernel_classes_are_timed_on_request():
    from mercury_b200 import SamplingParams

    prompts = [random_tokens(n, RAW["D"]["vocab_size"], 60 + n) for n in (9, 30, 17)]
    plain = _engine("D").generate(prompts, SamplingParams(), 6)
    engine = _engine("D", time_kernels=True)
    assert engine.generate(prompts, SamplingParams(), 6) == plain
    records = list(engine.metrics.steps)
    assert records and all(r.kernel_ms for r in records)
    classes = set().union(*(r.kernel_ms for r in records))
    assert {"embedding", "norm", "attention", "residual product", "gated product",
            "product"} <= classes, classes
    assert classes & {"q/k/v product", "q/k/v + rotary + store"}, classes
    assert all(ms > 0 for r in records for ms in r.kernel_ms.values())
    summary = engine.metrics.summary()
    assert summary["kernel_ms"]["attention"] > 0 and 0 <= summary["prepare_share"] < 1
    assert engine.runner.graph_replays == 0, "timed steps run eagerly"


def test_command_line_sizes_the_pool_itself(tmp_path):
    """--num-blocks -1: the pool takes what is left of the device after the weights."""
    raw, _cfg, tensors = tiny_model("B")
    config = tmp_path / "config.json"
    config.write_text(json.dumps(raw))
    done = subprocess.run(
        [sys.executable, "-m", "mercury_b200.generate", "--model", str(tmp_path / "model"),
         "--random-weights", str(config), "--seed", "1", "--prompt-ids", "5,17,3,99",
         "--max-tokens", "5", "--dtype", "float32", "--block-size", "8", "--num-blocks", "-1",
         "--max-running", "2", "--max-batched-tokens", "32", "--max-model-len", "64"],
        capture_output=True, text=True, cwd=ROOT, timeout=600)
    assert done.returncode == 0, done.stderr[-3000:]
    line = [l for l in done.stderr.splitlines() if "autosized to" in l]
    assert line and int(line[0].split("autosized to")[1].split()[0]) >= 8
    assert json.loads(done.stdout.strip().splitlines()[-1])["output_ids"] == \
        plain_generate(raw, tensors, [5, 17, 3, 99], 5)


def test_outgrown_scratch_stays_alive_for_captured_graphs():
    """A captured decode step holds the address of the attention's scratch memory. A later
    step that needs more gets a new buffer; the old one must stay allocated, or a tensor
    that took its place would be overwritten by (and would corrupt) the next replay."""
    from mercury_b200.engine.batch import StepEntry
    from mercury_b200.engine.runner import ModelRunner

    raw, config, tensors = tiny_model("A")
    runner = ModelRunner(config=config, tensors=tensors, dtype=torch.float32, device="cuda",
                         page_size=16, num_pages=32, max_seqs=2, max_step_tokens=128, max_model_len=256)
    runner.ops.decode_splits = 4                       # the split merge goes through scratch
    tokens = random_tokens(140, 256, 9)
    want = plain_logits(raw, tensors, tokens)
    seq = runner.open("s")
    runner.step([StepEntry(seq, tokens[:100], [])])
    scale = float(want.abs().max())

    def decode(position):
        got = runner.step([StepEntry(seq, [tokens[position]], [0])])[0].double().cpu()
        return float((got - want[position]).abs().max()) / scale

    assert decode(100) <= 3e-5 and decode(101) <= 3e-5      # captured, replayed
    assert runner.graph_replays == 2
    old = runner.ops._scratch
    assert old is not None
    address, size = old.data_ptr(), old.numel()
    del old
    runner.ops._scratch_for(2 * size)                       # a later step needs more
    assert runner.ops._scratch.data_ptr() != address
    squatters = [torch.full((size,), float("nan"), device="cuda") for _ in range(4)]
    assert all(t.data_ptr() != address for t in squatters), "the outgrown scratch was given back"
    assert decode(102) <= 3e-5 and decode(103) <= 3e-5
    assert all(bool(torch.isnan(t).all()) for t in squatters)
